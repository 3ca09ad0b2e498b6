// Kernels of attention over a latent cache.
//
// What a token keeps is one latent vector c (kv_rank numbers, RMS-normed) and one rotated key part shared by all
// heads (rot numbers): a single cache entry [c | kr].  Head n's key is [Wuk_n c | kr] and its value Wuv_n c, so with
// queries carried into the latent space, q~_n = Wuk_n^T q_n, the scores are q~_n . c + qr_n . kr and the output is
// Wuv_n (sum_j p_j c_j): attention with ONE key/value head whose keys are the entries and whose values are the
// entries' first kv_rank numbers.  The paged attention kernels do that part; this file holds what surrounds it:
//
//  * latent_prepare     - from the float32 rows of the first product, [query latent | kv latent | shared key part |
//                         gate logits]: the RMS norm of the query latent (to the run dtype), the RMS norm of the kv
//                         latent and the rotation of the shared key part, both written into the token's cache entry,
//                         and the logistic gate (float32).
//  * head_linear        - a product per head, out[t, n, :] = W_n x[t, n, :] (queries into the latent space, attended
//                         latents to values), optionally times a gate per head or per element.
//  * rotate_interleaved - rotation of neighbouring pairs (2i, 2i+1) by position * frequency_i, from cos/sin tables,
//                         over `rot_dims` numbers of a run from a given place on; the rest is copied.
//
// Long prompt portions go another way: many queries meet every key, so it pays to give every head its own keys and
// values again, [Wuk_n c | kr] and Wuv_n c, in pages of the step's own, and to run ordinary attention with as many
// key/value heads as heads (smaller rows per head, the fastest kernels).  For that:
//
//  * latent_gather      - the latents of every position the step's requests hold, from their cache entries into dense
//                         rows (the product's input), and the shared key part into every head's key rows.
//  * latent_scatter     - the product's output, [heads x dim | heads x vdim] per position, into the key and value pages.
//  * gate_rows          - the logistic gate on the attended rows, per head or per element.
//
// Norm statistics, angles (tables), the gate and every accumulation are float32.
#include "common.cuh"

namespace {

// One number of a run after the rotation of neighbouring pairs; `e` indexes the run, `x` points at its start.
__device__ __forceinline__ float rotated_pair_element(const float* x, int e, int rot_dims, const float* cos_row,
                                                      const float* sin_row) {
  if (e >= rot_dims) return x[e];
  const int pair = e >> 1;
  const float c = cos_row[pair], s = sin_row[pair];
  return (e & 1) ? fmaf(x[e], c, x[e - 1] * s) : fmaf(x[e], c, -x[e + 1] * s);
}

template <typename T>
__global__ void __launch_bounds__(256) latent_prepare_kernel(
    const float* __restrict__ raw, long long ld_raw, int q_rank, int kv_rank, int rot, int gate_n, int has_kv,
    const float* __restrict__ q_weight, const float* __restrict__ kv_weight, float eps, const float* __restrict__ cos_table,
    const float* __restrict__ sin_table, int rot_dims, int max_positions, const int* __restrict__ positions,
    const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int max_pages, int num_pages, int page_size,
    T* __restrict__ pages, T* __restrict__ q_latent, float* __restrict__ gate, int* status) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const float* row = raw + (size_t)t * ld_raw;
  // the query latent
  float ss = 0.0f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
  ss = block_sum(ss, scratch);
  const float inv_q = 1.0f / sqrtf(ss / (float)q_rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
    q_latent[(size_t)t * q_rank + i] = from_float<T>(row[i] * inv_q * q_weight[i]);
  int column = q_rank;
  if (has_kv) {
    const float* c = row + column;
    const float* kr = c + kv_rank;
    column += kv_rank + rot;
    float sc = 0.0f;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) sc = fmaf(c[i], c[i], sc);
    sc = block_sum(sc, scratch);
    if (pages != nullptr) {
      const float inv_c = 1.0f / sqrtf(sc / (float)kv_rank + eps);
      const int pos = positions[t];
      const int page_index = pos / page_size;
      const int page = (pos >= 0 && page_index < max_pages) ? block_table[(size_t)seq_of_token[t] * max_pages + page_index] : -1;
      if (pos < 0 || pos >= max_positions || page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicOr(status, pos < 0 || pos >= max_positions ? TGE_STATUS_BAD_ROW : TGE_STATUS_BAD_PAGE);
      } else {
        T* entry = pages + ((size_t)page * page_size + (pos % page_size)) * (size_t)(kv_rank + rot);
        for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) entry[i] = from_float<T>(c[i] * inv_c * kv_weight[i]);
        const float* cos_row = cos_table + (size_t)pos * (rot_dims / 2);
        const float* sin_row = sin_table + (size_t)pos * (rot_dims / 2);
        for (int base = 0; base < rot; base += 256) {
          const int e = base + threadIdx.x;
          if (e < rot) entry[kv_rank + e] = from_float<T>(rotated_pair_element(kr, e, rot_dims, cos_row, sin_row));
        }
      }
    }
  }
  const float* z = row + column;
  for (int i = threadIdx.x; i < gate_n; i += blockDim.x) gate[(size_t)t * gate_n + i] = 1.0f / (1.0f + expf(-z[i]));
}

constexpr int HL_BM = 32, HL_BN = 32, HL_BK = 32;
constexpr int HL_ROWS_MAX_TOKENS = 16;     // steps of up to this many tokens take the kernel that walks the rows

// out[t, n, j] = gate * sum_k x[t, n, k] * w[n, j, k]; a block owns 32 tokens x 32 outputs of one head, a thread a
// 2 x 2 patch, every output accumulated over k in ascending order (so a row's result does not depend on the batch).
template <typename T>
__global__ void __launch_bounds__(256) head_linear_kernel(
    const T* __restrict__ x, long long x_row, long long x_head, const T* __restrict__ w, T* __restrict__ out,
    long long out_row, long long out_head, const float* __restrict__ gate, int gate_mode, long long gate_row, int tokens,
    int n_out, int k_in) {
  __shared__ float xs[HL_BM][HL_BK + 1];
  __shared__ float ws[HL_BN][HL_BK + 1];
  pdl_trigger();
  pdl_wait();
  const int head = blockIdx.y;
  const int t0 = blockIdx.x * HL_BM, j0 = blockIdx.z * HL_BN;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const T* wh = w + (size_t)head * n_out * k_in;
  float acc[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};
  for (int k0 = 0; k0 < k_in; k0 += HL_BK) {
    for (int idx = threadIdx.x; idx < HL_BM * HL_BK; idx += 256) {
      const int r = idx / HL_BK, c = idx - r * HL_BK;
      const int t = t0 + r, k = k0 + c;
      xs[r][c] = (t < tokens && k < k_in) ? to_float<T>(x[(size_t)t * x_row + (size_t)head * x_head + k]) : 0.0f;
      const int j = j0 + r;
      ws[r][c] = (j < n_out && k < k_in) ? to_float<T>(wh[(size_t)j * k_in + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll 8
    for (int c = 0; c < HL_BK; ++c) {
      const float a0 = xs[ty * 2][c], a1 = xs[ty * 2 + 1][c];
      const float b0 = ws[tx * 2][c], b1 = ws[tx * 2 + 1][c];
      acc[0][0] = fmaf(a0, b0, acc[0][0]);
      acc[0][1] = fmaf(a0, b1, acc[0][1]);
      acc[1][0] = fmaf(a1, b0, acc[1][0]);
      acc[1][1] = fmaf(a1, b1, acc[1][1]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    const int t = t0 + ty * 2 + a;
    if (t >= tokens) continue;
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      const int j = j0 + tx * 2 + b;
      if (j >= n_out) continue;
      float v = acc[a][b];
      if (gate_mode == 1) v *= gate[(size_t)t * gate_row + head];
      else if (gate_mode == 2) v *= gate[(size_t)t * gate_row + (size_t)head * n_out + j];
      out[(size_t)t * out_row + (size_t)head * out_head + j] = from_float<T>(v);
    }
  }
}

// The same product for a step of few tokens: a warp owns one output of one head and walks the tokens four at a time,
// every lane the numbers lane, lane + 32, ... of the rows, the lanes' sums meeting in a butterfly; the order of a row's
// sum depends on k_in alone.
template <typename T>
__global__ void __launch_bounds__(256) head_linear_rows_kernel(
    const T* __restrict__ x, long long x_row, long long x_head, const T* __restrict__ w, T* __restrict__ out,
    long long out_row, long long out_head, const float* __restrict__ gate, int gate_mode, long long gate_row, int tokens,
    int n_out, int k_in) {
  pdl_trigger();
  pdl_wait();
  const int head = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.y * 8 + warp;
  if (j >= n_out) return;
  const T* wrow = w + ((size_t)head * n_out + j) * k_in;
  for (int t0 = 0; t0 < tokens; t0 += 4) {
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int k = lane; k < k_in; k += 32) {
      const float wk = to_float<T>(wrow[k]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = t0 + i < tokens ? t0 + i : tokens - 1;
        acc[i] = fmaf(to_float<T>(x[(size_t)t * x_row + (size_t)head * x_head + k]), wk, acc[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float v = warp_sum(acc[i]);
      const int t = t0 + i;
      if (lane == 0 && t < tokens) {
        if (gate_mode == 1) v *= gate[(size_t)t * gate_row + head];
        else if (gate_mode == 2) v *= gate[(size_t)t * gate_row + (size_t)head * n_out + j];
        out[(size_t)t * out_row + (size_t)head * out_head + j] = from_float<T>(v);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) rotate_interleaved_kernel(
    const T* __restrict__ src, long long src_row, long long src_head, T* __restrict__ dst, long long dst_row,
    long long dst_head, const float* __restrict__ cos_table, const float* __restrict__ sin_table, int rot_dims,
    int max_positions, const int* __restrict__ positions, int tokens, int heads, int width, int first, int* status) {
  pdl_trigger();
  pdl_wait();
  const long long total = (long long)tokens * heads * width;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int e = (int)(idx % width);
    const int head = (int)((idx / width) % heads);
    const int t = (int)(idx / ((long long)width * heads));
    const int pos = positions[t];
    if (pos < 0 || pos >= max_positions) {
      atomicOr(status, TGE_STATUS_BAD_ROW);
      continue;
    }
    const T* run = src + (size_t)t * src_row + (size_t)head * src_head;
    float v = to_float<T>(run[e]);
    if (e >= first && e < first + rot_dims) {
      const int pair = (e - first) >> 1;
      const float c = cos_table[(size_t)pos * (rot_dims / 2) + pair], s = sin_table[(size_t)pos * (rot_dims / 2) + pair];
      v = ((e - first) & 1) ? fmaf(v, c, to_float<T>(run[e - 1]) * s) : fmaf(v, c, -to_float<T>(run[e + 1]) * s);
    }
    dst[(size_t)t * dst_row + (size_t)head * dst_head + e] = from_float<T>(v);
  }
}

// The same on pairs of bfloat16 (every size, stride and the first rotated place even, rows on 4 bytes): a thread owns
// one pair, so a rotated pair is read once.
__global__ void __launch_bounds__(256) rotate_interleaved_pairs_kernel(
    const __nv_bfloat16* __restrict__ src, long long src_row, long long src_head, __nv_bfloat16* __restrict__ dst,
    long long dst_row, long long dst_head, const float* __restrict__ cos_table, const float* __restrict__ sin_table,
    int rot_dims, int max_positions, const int* __restrict__ positions, int tokens, int heads, int width, int first,
    int* status) {
  pdl_trigger();
  pdl_wait();
  const int half = width >> 1;
  const long long per_token = (long long)heads * half;
  const long long total = (long long)tokens * per_token;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / per_token);
    const int rest = (int)(idx - (long long)t * per_token);
    const int head = rest / half;
    const int e = 2 * (rest - head * half);
    const int pos = positions[t];
    if (pos < 0 || pos >= max_positions) {
      atomicOr(status, TGE_STATUS_BAD_ROW);
      continue;
    }
    float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + (size_t)t * src_row + (size_t)head * src_head + e));
    if (e >= first && e < first + rot_dims) {
      const int pair = (e - first) >> 1;
      const float c = cos_table[(size_t)pos * (rot_dims / 2) + pair], s = sin_table[(size_t)pos * (rot_dims / 2) + pair];
      v = make_float2(fmaf(v.x, c, -v.y * s), fmaf(v.y, c, v.x * s));
    }
    *reinterpret_cast<__nv_bfloat162*>(dst + (size_t)t * dst_row + (size_t)head * dst_head + e) = __floats2bfloat162_rn(v.x, v.y);
  }
}

// One block per position slot of the step's own pages: slot r = page * page_size + offset; page p belongs to request
// page_seq[p] and is its page_idx[p]-th.  Positions beyond what the request holds give zeros.
template <typename T>
__global__ void __launch_bounds__(128) latent_gather_kernel(
    const T* __restrict__ pages, const int* __restrict__ table, int max_pages, int num_pages, const int* __restrict__ page_seq,
    const int* __restrict__ page_idx, const int* __restrict__ ctx_len, int page_size, int kv_rank, int rot, int heads, int per,
    T* __restrict__ latents, T* __restrict__ keys, int* status) {
  pdl_trigger();
  pdl_wait();
  const int slot = blockIdx.x, p = slot / page_size, off = slot % page_size;
  const int seq = page_seq[p], index = page_idx[p];
  const bool held = index * page_size + off < ctx_len[seq];
  const T* entry = nullptr;
  if (held) {
    const int real = index < max_pages ? table[(size_t)seq * max_pages + index] : -1;
    if (real < 0 || real >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, TGE_STATUS_BAD_ROW);
    } else {
      entry = pages + ((size_t)real * page_size + off) * (kv_rank + rot);
    }
  }
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x)
    latents[(size_t)slot * kv_rank + i] = entry ? entry[i] : from_float<T>(0.0f);
  const int dim = per - rot;
  for (int i = threadIdx.x; i < heads * rot; i += blockDim.x) {
    const int n = i / rot, d = i % rot;
    keys[(((size_t)p * heads + n) * page_size + off) * per + dim + d] = entry ? entry[kv_rank + d] : from_float<T>(0.0f);
  }
}

// expanded: [slots, ld] = per position [heads x dim plain key parts | heads x vdim values]; keys [pages, heads,
// page_size, dim + rot], values [pages, heads, page_size, vdim].
template <typename T>
__global__ void __launch_bounds__(256) latent_scatter_kernel(const T* __restrict__ expanded, long long ld, int page_size,
                                                             int heads, int dim, int per, int vdim, T* __restrict__ keys,
                                                             T* __restrict__ values) {
  pdl_trigger();
  pdl_wait();
  const int slot = blockIdx.x, p = slot / page_size, off = slot % page_size;
  const T* row = expanded + (size_t)slot * ld;
  for (int i = threadIdx.x; i < heads * dim; i += blockDim.x) {
    const int n = i / dim, d = i % dim;
    keys[(((size_t)p * heads + n) * page_size + off) * per + d] = row[i];
  }
  const T* vrow = row + (size_t)heads * dim;
  for (int i = threadIdx.x; i < heads * vdim; i += blockDim.x) {
    const int n = i / vdim, d = i % vdim;
    values[(((size_t)p * heads + n) * page_size + off) * vdim + d] = vrow[i];
  }
}

// x[t, n, j] *= gate[t, n] (mode 1) or gate[t, n * vdim + j] (mode 2), in place.
template <typename T>
__global__ void __launch_bounds__(256) gate_rows_kernel(T* __restrict__ x, long long x_row, const float* __restrict__ gate,
                                                        long long gate_row, int mode, int heads, int vdim) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < heads * vdim; i += blockDim.x) {
    const float g = gate[(size_t)t * gate_row + (mode == 1 ? i / vdim : i)];
    x[(size_t)t * x_row + i] = from_float<T>(to_float<T>(x[(size_t)t * x_row + i]) * g);
  }
}

}  // namespace

// raw: float32 [tokens, ld_raw] = [q_rank | (kv_rank | rot, when has_kv) | gate_n].  pages: [num_pages, page_size,
// kv_rank + rot] in the run dtype, or null (the entries are another layer's, or nothing is to be stored).
// cos/sin: float32 [max_positions, rot_dims / 2].  q_latent: run dtype [tokens, q_rank]; gate: float32 [tokens, gate_n].
TGE_API int tge_latent_prepare(const float* raw, long long ld_raw, int q_rank, int kv_rank, int rot, int gate_n, int has_kv,
                               const float* q_weight, const float* kv_weight, float eps, const float* cos_table,
                               const float* sin_table, int rot_dims, int max_positions, const int* positions,
                               const int* seq_of_token, const int* block_table, int max_pages, int num_pages,
                               int page_size, void* pages, void* q_latent, float* gate, int is_bf16, int tokens,
                               int* status, cudaStream_t stream) {
  TGE_REQUIRE(tokens >= 0 && q_rank > 0 && gate_n >= 0, "latent_prepare: bad shape");
  TGE_REQUIRE(!has_kv || (kv_rank > 0 && rot >= 0 && rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= rot),
              "latent_prepare: %d rotated numbers of %d (an even count within the shared key part)", rot_dims, rot);
  TGE_REQUIRE(ld_raw >= q_rank + (has_kv ? kv_rank + rot : 0) + gate_n, "latent_prepare: rows of %lld hold less than they should", ld_raw);
  TGE_REQUIRE(!has_kv || pages == nullptr || (page_size > 0 && max_pages > 0 && num_pages > 0 && block_table != nullptr &&
                                              (rot_dims == 0 || (cos_table != nullptr && sin_table != nullptr))),
              "latent_prepare: storing needs the page geometry and the rotation's tables");
  if (tokens == 0) return 0;
  if (is_bf16)
    tge_launch(latent_prepare_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, raw, ld_raw, q_rank, kv_rank, rot,
               gate_n, has_kv, q_weight, kv_weight, eps, cos_table, sin_table, rot_dims, max_positions, positions,
               seq_of_token, block_table, max_pages, num_pages, page_size, (__nv_bfloat16*)pages, (__nv_bfloat16*)q_latent,
               gate, status);
  else
    tge_launch(latent_prepare_kernel<float>, dim3(tokens), dim3(256), 0, stream, raw, ld_raw, q_rank, kv_rank, rot, gate_n,
               has_kv, q_weight, kv_weight, eps, cos_table, sin_table, rot_dims, max_positions, positions, seq_of_token,
               block_table, max_pages, num_pages, page_size, (float*)pages, (float*)q_latent, gate, status);
  return tge_launched("latent_prepare", 1);
}

// x: rows of `x_row` elements, head n's input at x + n * x_head (k_in numbers); w: [heads, n_out, k_in]; out likewise
// with out_row / out_head.  gate_mode 0: none; 1: gate[t * gate_row + n]; 2: gate[t * gate_row + n * n_out + j].
TGE_API int tge_head_linear(const void* x, long long x_row, long long x_head, const void* w, void* out, long long out_row,
                            long long out_head, const float* gate, int gate_mode, long long gate_row, int tokens, int heads,
                            int n_out, int k_in, int is_bf16, cudaStream_t stream) {
  TGE_REQUIRE(tokens >= 0 && heads > 0 && n_out > 0 && k_in > 0, "head_linear: bad shape");
  TGE_REQUIRE(gate_mode >= 0 && gate_mode <= 2 && (gate_mode == 0 || gate != nullptr), "head_linear: gate mode %d", gate_mode);
  TGE_REQUIRE(heads <= 65535 && (n_out + HL_BN - 1) / HL_BN <= 65535, "head_linear: too many heads or outputs for one launch");
  if (tokens == 0) return 0;
  if (tokens <= HL_ROWS_MAX_TOKENS) {
    dim3 small(heads, (n_out + 7) / 8);
    if (is_bf16)
      tge_launch(head_linear_rows_kernel<__nv_bfloat16>, small, dim3(256), 0, stream, (const __nv_bfloat16*)x, x_row, x_head,
                 (const __nv_bfloat16*)w, (__nv_bfloat16*)out, out_row, out_head, gate, gate_mode, gate_row, tokens, n_out, k_in);
    else
      tge_launch(head_linear_rows_kernel<float>, small, dim3(256), 0, stream, (const float*)x, x_row, x_head, (const float*)w,
                 (float*)out, out_row, out_head, gate, gate_mode, gate_row, tokens, n_out, k_in);
    return tge_launched("head_linear", 1);
  }
  dim3 grid((tokens + HL_BM - 1) / HL_BM, heads, (n_out + HL_BN - 1) / HL_BN);
  if (is_bf16)
    tge_launch(head_linear_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)x, x_row, x_head,
               (const __nv_bfloat16*)w, (__nv_bfloat16*)out, out_row, out_head, gate, gate_mode, gate_row, tokens, n_out, k_in);
  else
    tge_launch(head_linear_kernel<float>, grid, dim3(256), 0, stream, (const float*)x, x_row, x_head, (const float*)w,
               (float*)out, out_row, out_head, gate, gate_mode, gate_row, tokens, n_out, k_in);
  return tge_launched("head_linear", 1);
}

// src / dst: runs of `width` numbers per (token, head), at t * row + n * head (elements), two buffers.  The rotated
// numbers are those from `first` on; the others are copied.
TGE_API int tge_rotate_interleaved(const void* src, long long src_row, long long src_head, void* dst, long long dst_row,
                                   long long dst_head, const float* cos_table, const float* sin_table, int rot_dims,
                                   int max_positions, const int* positions, int tokens, int heads, int width, int first,
                                   int is_bf16, int* status, cudaStream_t stream) {
  TGE_REQUIRE(tokens >= 0 && heads > 0 && width > 0, "rotate_interleaved: bad shape");
  TGE_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && first >= 0 && first + rot_dims <= width,
              "rotate_interleaved: %d rotated numbers from %d on of %d", rot_dims, first, width);
  TGE_REQUIRE(src != dst, "rotate_interleaved: a pair's second number is read after its first is written; give two buffers");
  if (tokens == 0) return 0;
  const long long total = (long long)tokens * heads * width;
  const int blocks = (int)((total + 255) / 256 > 65535 * 16 ? 65535 * 16 : (total + 255) / 256);
  if (is_bf16 && ((width | first | src_row | src_head | dst_row | dst_head) & 1) == 0 && (((uintptr_t)src | (uintptr_t)dst) & 3) == 0) {
    const int pair_blocks = (int)((total / 2 + 255) / 256 > 148 * 16 ? 148 * 16 : (total / 2 + 255) / 256);
    tge_launch(rotate_interleaved_pairs_kernel, dim3(pair_blocks), dim3(256), 0, stream, (const __nv_bfloat16*)src, src_row,
               src_head, (__nv_bfloat16*)dst, dst_row, dst_head, cos_table, sin_table, rot_dims, max_positions, positions, tokens,
               heads, width, first, status);
    return tge_launched("rotate_interleaved", 1);
  }
  if (is_bf16)
    tge_launch(rotate_interleaved_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)src,
               src_row, src_head, (__nv_bfloat16*)dst, dst_row, dst_head, cos_table, sin_table, rot_dims, max_positions,
               positions, tokens, heads, width, first, status);
  else
    tge_launch(rotate_interleaved_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)src, src_row, src_head,
               (float*)dst, dst_row, dst_head, cos_table, sin_table, rot_dims, max_positions, positions, tokens, heads, width,
               first, status);
  return tge_launched("rotate_interleaved", 1);
}

// pages: the cache [num_pages, page_size, kv_rank + rot] found through table [seqs, max_pages]; the step's own pages:
// own_pages of page_size slots, page p being request page_seq[p]'s page_idx[p]-th; ctx_len [seqs]: positions held.
// latents: [own_pages * page_size, kv_rank]; keys: [own_pages, heads, page_size, per] (only the last `rot` numbers of
// a row are written here).
TGE_API int tge_latent_gather(const void* pages, const int* table, int max_pages, int num_pages, const int* page_seq,
                              const int* page_idx, const int* ctx_len, int own_pages, int page_size, int kv_rank, int rot,
                              int heads, int per, void* latents, void* keys, int is_bf16, int* status, cudaStream_t stream) {
  TGE_REQUIRE(own_pages >= 0 && page_size > 0 && kv_rank > 0 && rot >= 0 && heads > 0 && per >= rot && max_pages > 0 && num_pages > 0,
              "latent_gather: bad shape");
  if (own_pages == 0) return 0;
  if (is_bf16)
    tge_launch(latent_gather_kernel<__nv_bfloat16>, dim3(own_pages * page_size), dim3(128), 0, stream, (const __nv_bfloat16*)pages,
               table, max_pages, num_pages, page_seq, page_idx, ctx_len, page_size, kv_rank, rot, heads, per,
               (__nv_bfloat16*)latents, (__nv_bfloat16*)keys, status);
  else
    tge_launch(latent_gather_kernel<float>, dim3(own_pages * page_size), dim3(128), 0, stream, (const float*)pages, table,
               max_pages, num_pages, page_seq, page_idx, ctx_len, page_size, kv_rank, rot, heads, per, (float*)latents,
               (float*)keys, status);
  return tge_launched("latent_gather", 1);
}

TGE_API int tge_latent_scatter(const void* expanded, long long ld, int own_pages, int page_size, int heads, int dim, int per,
                               int vdim, void* keys, void* values, int is_bf16, cudaStream_t stream) {
  TGE_REQUIRE(own_pages >= 0 && page_size > 0 && heads > 0 && dim >= 0 && per >= dim && vdim > 0 &&
              ld >= (long long)heads * (dim + vdim), "latent_scatter: bad shape");
  if (own_pages == 0) return 0;
  if (is_bf16)
    tge_launch(latent_scatter_kernel<__nv_bfloat16>, dim3(own_pages * page_size), dim3(256), 0, stream,
               (const __nv_bfloat16*)expanded, ld, page_size, heads, dim, per, vdim, (__nv_bfloat16*)keys, (__nv_bfloat16*)values);
  else
    tge_launch(latent_scatter_kernel<float>, dim3(own_pages * page_size), dim3(256), 0, stream, (const float*)expanded, ld,
               page_size, heads, dim, per, vdim, (float*)keys, (float*)values);
  return tge_launched("latent_scatter", 1);
}

TGE_API int tge_gate_rows(void* x, long long x_row, const float* gate, long long gate_row, int mode, int tokens, int heads,
                          int vdim, int is_bf16, cudaStream_t stream) {
  TGE_REQUIRE(tokens >= 0 && heads > 0 && vdim > 0 && (mode == 1 || mode == 2) && gate != nullptr, "gate_rows: bad shape");
  if (tokens == 0) return 0;
  if (is_bf16)
    tge_launch(gate_rows_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, (__nv_bfloat16*)x, x_row, gate, gate_row,
               mode, heads, vdim);
  else
    tge_launch(gate_rows_kernel<float>, dim3(tokens), dim3(256), 0, stream, (float*)x, x_row, gate, gate_row, mode, heads, vdim);
  return tge_launched("gate_rows", 1);
}
