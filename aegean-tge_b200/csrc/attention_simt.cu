// Paged causal attention on the CUDA cores, any head size, float32 arithmetic.
//
// One warp per (token, query head).  Keys are visited in position order with a
// running maximum, so a row's result depends only on its own keys, never on
// the batch it arrives in or on how its request was cut into portions.  It is
// the attention of the whole float32 path and of head sizes the tensor-core
// kernel was not compiled for.
//
// Per query head h at position p (reference: src/cpu/scalar/attention_scalar.cpp:48-115,
// src/models/qwen2.cpp:1243-1304): kv head = h / group; for t in [first, p]:
// s_t = dot(q, K_t) * scale (dot first, scale after); softmax over s; out = sum w_t V_t.
// The causal mask is the loop bound; `window` > 0 additionally drops keys older
// than p - window + 1.  Values may have a size of their own (`value_dim`), and a head may have a sink: a learned
// score `sink[h]` that joins the softmax's denominator once, unscaled, with no key and no value behind it.
// With a window and `pool` > 0 the query also sees, in the same softmax, one pooled key and value for every
// block of `pool` positions that lies wholly before its window (block b if b*pool + pool - 1 <= p - window); they
// are read from pages of their own, entry b where position b would be, and visited before the tokens.
// `dist_bias` [heads, span] (float32): a learned bias added to the scaled score of the key at distance n, entry
// min(n, span - 1) of the head's row.
#include "common.cuh"

namespace {

constexpr int MAX_PER_LANE = 8;  // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(128) attention_simt_kernel(
    const T* __restrict__ q, int q_stride, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
    const int* __restrict__ block_table, int max_pages, int num_pages, int page_size,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token, T* __restrict__ out, int out_stride,
    int heads, int kv_heads, int head_dim, int value_dim, int v_pitch, const float* __restrict__ sink, float scale, int window,
    int pool, const T* __restrict__ kp_pages, const T* __restrict__ vp_pages, const int* __restrict__ pool_table,
    int pool_max_pages, int pool_num_pages, const float* __restrict__ dist_bias, int dist_span, int* status) {
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * 4 + warp;
  if (h >= heads) return;
  const int group = heads / kv_heads;
  // a learned bias by distance, unscaled: row h of [heads, span], distances from span - 1 on share the last entry
  const float* bias_row = dist_bias != nullptr ? dist_bias + (size_t)h * dist_span : nullptr;
  const int kvh = h / group;
  const int pos = positions[t];
  const int seq = seq_of_token[t];
  const int* table = block_table + (size_t)seq * max_pages;

  float qv[MAX_PER_LANE], acc[MAX_PER_LANE];
  const T* qrow = q + (size_t)t * q_stride + (size_t)h * head_dim;
#pragma unroll
  for (int i = 0; i < MAX_PER_LANE; ++i) {
    const int d = lane + 32 * i;
    qv[i] = d < head_dim ? to_float<T>(qrow[d]) : 0.0f;
    acc[i] = 0.0f;
  }
  float m = -INFINITY, l = 0.0f;
  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  if (pool > 0 && window > 0) {
    const int seen = first / pool;                       // blocks that end at or before pos - window
    const int* ptable = pool_table + (size_t)seq * pool_max_pages;
    for (int entry = 0; entry < seen; ++entry) {
      const int page_index = entry / page_size;
      const int page = page_index < pool_max_pages ? ptable[page_index] : -1;
      if (page < 0 || page >= pool_num_pages) {
        if (lane == 0) atomicOr(status, TGE_STATUS_BAD_PAGE);
        break;
      }
      const T* krow = kp_pages + (((size_t)page * kv_heads + kvh) * page_size + entry % page_size) * head_dim;
      const T* vrow = vp_pages + (((size_t)page * kv_heads + kvh) * page_size + entry % page_size) * value_dim;
      float dot = 0.0f;
#pragma unroll
      for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) dot = fmaf(qv[i], to_float<T>(krow[d]), dot);
      }
      dot = warp_sum(dot);
      const float s = dot * scale;
      const float m_new = fmaxf(m, s);
      const float corr = expf(m - m_new);
      const float p = expf(s - m_new);
      l = l * corr + p;
#pragma unroll
      for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < value_dim) acc[i] = fmaf(p, to_float<T>(vrow[d]), acc[i] * corr);
      }
      m = m_new;
    }
  }
  for (int page_index = first / page_size; page_index * page_size <= pos; ++page_index) {
    const int page = page_index < max_pages ? table[page_index] : -1;
    if (page < 0 || page >= num_pages) {
      if (lane == 0) atomicOr(status, TGE_STATUS_BAD_PAGE);
      break;
    }
    const size_t base = ((size_t)page * kv_heads + kvh) * page_size * head_dim;
    const size_t vbase = ((size_t)page * kv_heads + kvh) * page_size * v_pitch;   // v_pitch: numbers between two values' starts
    const int lo = max(first - page_index * page_size, 0);
    const int hi = min(pos - page_index * page_size, page_size - 1);
    for (int slot = lo; slot <= hi; ++slot) {
      const T* krow = k_pages + base + (size_t)slot * head_dim;
      const T* vrow = v_pages + vbase + (size_t)slot * v_pitch;
      float dot = 0.0f;
#pragma unroll
      for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) dot = fmaf(qv[i], to_float<T>(krow[d]), dot);
      }
      dot = warp_sum(dot);
      float s = dot * scale;
      if (bias_row != nullptr) s += bias_row[min(pos - (page_index * page_size + slot), dist_span - 1)];
      const float m_new = fmaxf(m, s);
      const float corr = expf(m - m_new);  // exp(-inf) = 0 on the first key
      const float p = expf(s - m_new);
      l = l * corr + p;
#pragma unroll
      for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < value_dim) acc[i] = fmaf(p, to_float<T>(vrow[d]), acc[i] * corr);
      }
      m = m_new;
    }
  }
  if (sink != nullptr) {
    // the sink enters like one more key whose value is zero
    const float s = sink[h];
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new);
    l = l * corr + expf(s - m_new);
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) acc[i] *= corr;
  }
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
  T* orow = out + (size_t)t * out_stride + (size_t)h * value_dim;
#pragma unroll
  for (int i = 0; i < MAX_PER_LANE; ++i) {
    const int d = lane + 32 * i;
    if (d < value_dim) orow[d] = from_float<T>(acc[i] * inv);
  }
}

// For the tensor-core path: a walk over the pooled entries a query sees (scores in base-2 units, s = q . k * scale *
// log2 e, running maximum and sum as in the kernel above), then the merge with the states that the tensor-core
// kernels left for the window's key runs (partial_o [runs, tokens, heads, value_dim], partial_ml [runs, tokens, heads, 2]: unnormalised sums,
// maxima in base-2 units, denominators), the runs that hold keys visible to the row in run order, and the row's
// output.  One warp per (token, head): the pooled state never leaves its registers.
template <typename T>
__global__ void __launch_bounds__(128) attention_pooled_merge_kernel(
    const T* __restrict__ q, int q_stride, const T* __restrict__ kp_pages, const T* __restrict__ vp_pages,
    const int* __restrict__ pool_table, int pool_max_pages, int pool_num_pages, int page_size,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token, const float* __restrict__ partial_o,
    const float* __restrict__ partial_ml, int total_tokens, int num_runs, int run_tokens, T* __restrict__ out,
    int out_stride, int heads, int kv_heads, int head_dim, int value_dim, float scale_log2, int window, int pool,
    const float* __restrict__ sink, int* status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * 4 + warp;
  if (h >= heads) return;
  const int kvh = h / (heads / kv_heads);
  const int pos = positions[t];
  const int seq = seq_of_token[t];
  const int first = pos - window + 1 > 0 ? pos - window + 1 : 0;
  const int seen = first / pool;
  float qv[MAX_PER_LANE], acc[MAX_PER_LANE];
  const T* qrow = q + (size_t)t * q_stride + (size_t)h * head_dim;
#pragma unroll
  for (int i = 0; i < MAX_PER_LANE; ++i) {
    const int d = lane + 32 * i;
    qv[i] = d < head_dim ? to_float<T>(qrow[d]) : 0.0f;
    acc[i] = 0.0f;
  }
  float m = -INFINITY, l = 0.0f;
  const int* ptable = pool_table + (size_t)seq * pool_max_pages;
  for (int entry = 0; entry < seen; ++entry) {
    const int page_index = entry / page_size;
    const int page = page_index < pool_max_pages ? ptable[page_index] : -1;
    if (page < 0 || page >= pool_num_pages) {
      if (lane == 0) atomicOr(status, TGE_STATUS_BAD_PAGE);
      break;
    }
    const T* krow = kp_pages + (((size_t)page * kv_heads + kvh) * page_size + entry % page_size) * head_dim;
    const T* vrow = vp_pages + (((size_t)page * kv_heads + kvh) * page_size + entry % page_size) * value_dim;
    float dot = 0.0f;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int d = lane + 32 * i;
      if (d < head_dim) dot = fmaf(qv[i], to_float<T>(krow[d]), dot);
    }
    const float s = warp_sum(dot) * scale_log2;
    const float m_new = fmaxf(m, s);
    const float corr = exp2f(m - m_new);
    const float w = exp2f(s - m_new);
    l = l * corr + w;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int d = lane + 32 * i;
      if (d < value_dim) acc[i] = fmaf(w, to_float<T>(vrow[d]), acc[i] * corr);
    }
    m = m_new;
  }
  const int run_lo = first / run_tokens;
  const int run_hi = min(pos / run_tokens, num_runs - 1);
  for (int run = run_lo; run <= run_hi; ++run) {
    const size_t slot = ((size_t)run * total_tokens + t) * heads + h;
    const float2 ml = *reinterpret_cast<const float2*>(partial_ml + slot * 2);
    if (ml.x == -INFINITY) continue;
    const float m_new = fmaxf(m, ml.x);
    const float mine = exp2f(m - m_new), theirs = exp2f(ml.x - m_new);
    l = l * mine + ml.y * theirs;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int d = lane + 32 * i;
      if (d < value_dim) acc[i] = fmaf(partial_o[slot * value_dim + d], theirs, acc[i] * mine);
    }
    m = m_new;
  }
  if (sink != nullptr) l += exp2f(sink[h] * 1.4426950408889634f - (m == -INFINITY ? 0.0f : m));
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
  T* orow = out + (size_t)t * out_stride + (size_t)h * value_dim;
#pragma unroll
  for (int i = 0; i < MAX_PER_LANE; ++i) {
    const int d = lane + 32 * i;
    if (d < value_dim) orow[d] = from_float<T>(acc[i] * inv);
  }
}

}  // namespace

TGE_API int tge_attention_simt(const void* q, int q_stride, const void* k_pages, const void* v_pages,
                               const int* block_table, int max_pages, int num_pages, int page_size,
                               const int* positions, const int* seq_of_token, void* out, int out_stride, int tokens,
                               int heads, int kv_heads, int head_dim, int value_dim, const float* sink, float scale,
                               int window, int is_bf16, int pool, const void* kp_pages, const void* vp_pages,
                               const int* pool_table, int pool_max_pages, int pool_num_pages, int v_pitch,
                               const float* dist_bias, int dist_span, int* status, cudaStream_t stream) {
  // v_pitch: numbers between the starts of two positions' values in `v_pages` (0: value_dim, values packed).  A cache
  // whose values are the leading part of its keys passes the keys' pages twice and the keys' size here.
  if (v_pitch == 0) v_pitch = value_dim;
  TGE_REQUIRE(v_pitch >= value_dim, "attention: a value pitch of %d is less than the values' size %d", v_pitch, value_dim);
  TGE_REQUIRE(pool == 0 || v_pitch == value_dim, "attention: pooled blocks go with packed values");
  TGE_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
              "attention: heads %d must be a positive multiple of kv heads %d", heads, kv_heads);
  TGE_REQUIRE(head_dim > 0 && head_dim <= 32 * MAX_PER_LANE, "attention: head_dim %d outside (0, %d]", head_dim,
              32 * MAX_PER_LANE);
  TGE_REQUIRE(value_dim > 0 && value_dim <= 32 * MAX_PER_LANE, "attention: value_dim %d outside (0, %d]", value_dim,
              32 * MAX_PER_LANE);
  TGE_REQUIRE(page_size > 0 && max_pages > 0 && num_pages > 0, "attention: bad page geometry");
  TGE_REQUIRE(window >= 0, "attention: negative window");
  TGE_REQUIRE(dist_bias == nullptr || dist_span > 0, "attention: a bias by distance needs its span");
  TGE_REQUIRE(pool >= 0 && (pool == 0 || (window > 0 && kp_pages != nullptr && vp_pages != nullptr && pool_table != nullptr &&
                                          pool_max_pages > 0 && pool_num_pages > 0)),
              "attention: pooled blocks need a window, their pages and their table");
  if (tokens == 0) return 0;
  dim3 grid(tokens, (heads + 3) / 4);
  if (is_bf16)
    attention_simt_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table,
        max_pages, num_pages, page_size, positions, seq_of_token, (__nv_bfloat16*)out, out_stride, heads, kv_heads,
        head_dim, value_dim, v_pitch, sink, scale, window, pool, (const __nv_bfloat16*)kp_pages, (const __nv_bfloat16*)vp_pages,
        pool_table, pool_max_pages, pool_num_pages, dist_bias, dist_span, status);
  else
    attention_simt_kernel<float><<<grid, 128, 0, stream>>>(
        (const float*)q, q_stride, (const float*)k_pages, (const float*)v_pages, block_table, max_pages, num_pages,
        page_size, positions, seq_of_token, (float*)out, out_stride, heads, kv_heads, head_dim, value_dim, v_pitch, sink, scale,
        window, pool, (const float*)kp_pages, (const float*)vp_pages, pool_table, pool_max_pages, pool_num_pages, dist_bias,
        dist_span, status);
  return tge_launched("attention_simt", 1);
}

TGE_API int tge_attention_pooled_merge(const void* q, int q_stride, const void* kp_pages, const void* vp_pages,
                                       const int* pool_table, int pool_max_pages, int pool_num_pages, int page_size,
                                       const int* positions, const int* seq_of_token, const float* partial_o,
                                       const float* partial_ml, int num_runs, int run_tokens, void* out, int out_stride,
                                       int tokens, int heads, int kv_heads, int head_dim, int value_dim, float scale,
                                       int window, int pool, const float* sink, int is_bf16, int* status,
                                       cudaStream_t stream) {
  TGE_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0, "attention: heads %d, kv heads %d", heads, kv_heads);
  TGE_REQUIRE(head_dim > 0 && head_dim <= 32 * MAX_PER_LANE && value_dim > 0 && value_dim <= 32 * MAX_PER_LANE,
              "attention: head sizes %d and %d outside (0, %d]", head_dim, value_dim, 32 * MAX_PER_LANE);
  TGE_REQUIRE(window > 0 && pool > 0 && page_size > 0 && pool_max_pages > 0 && pool_num_pages > 0,
              "attention: pooled blocks need a window, their size and their pages");
  TGE_REQUIRE(num_runs > 0 && run_tokens > 0 && partial_o != nullptr && partial_ml != nullptr,
              "attention: the merge needs the key runs' states");
  if (tokens == 0) return 0;
  dim3 grid(tokens, (heads + 3) / 4);
  const float scale_log2 = scale * 1.4426950408889634f;
  if (is_bf16)
    tge_launch(attention_pooled_merge_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)q, q_stride,
               (const __nv_bfloat16*)kp_pages, (const __nv_bfloat16*)vp_pages, pool_table, pool_max_pages, pool_num_pages,
               page_size, positions, seq_of_token, partial_o, partial_ml, tokens, num_runs, run_tokens, (__nv_bfloat16*)out,
               out_stride, heads, kv_heads, head_dim, value_dim, scale_log2, window, pool, sink, status);
  else
    tge_launch(attention_pooled_merge_kernel<float>, grid, dim3(128), 0, stream, (const float*)q, q_stride,
               (const float*)kp_pages, (const float*)vp_pages, pool_table, pool_max_pages, pool_num_pages, page_size, positions,
               seq_of_token, partial_o, partial_ml, tokens, num_runs, run_tokens, (float*)out, out_stride, heads, kv_heads,
               head_dim, value_dim, scale_log2, window, pool, sink, status);
  return tge_launched("attention_pooled_merge", 1);
}
