// Kernels of mixers whose state is a matrix per head that every token decays, corrects and reads, and of the parts
// around them:
//
//  * gated_prepare    - after the mixer's one input product: a short causal convolution over time (with or without a
//                       bias) and SiLU on a run of channels, the unit norm of q and k per head, the decay and the write
//                       strength of every head, as the recurrence takes them (float32);
//  * conv_tail_update - the convolution's last taps-1 inputs of every request, kept for the next step;
//  * gated_rule_scan  - S <- a_t S; u = b_t (v_t - [S^T k_t]); S <- S + k_t u^T; o_t = S^T q_t (+ d v_t), token by token,
//                       the state float32 in a per-request slot.  With the bracket it is the gated delta rule, without it
//                       the state-space recurrence (k = B, q = C, b = the step size, a = exp(-A dt));
//  * norm_scale_add   - x += alpha * y / rms(y) * w: a branch's output normalised over the width and added into the stream;
//  * qk_temp_store    - after an attention's q/k product: the per-head norm of q and k, the queries' temperature by
//                       position, and the store of the keys and of the values, which are the keys as projected;
//  * gated_clamp_act  - a = min(g, L) sigmoid(alpha min(g, L)) (clamp(u, -L, L) + 1) from interleaved (g, u) rows;
//  * concat_rows      - [x | x0] in the products' number format.
//
// Statistics, decays, step sizes, gates and the state are float32 in both number formats.
#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_g(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sigmoid_g(float z) { return 1.0f / (1.0f + expf(-z)); }
// log(1 + exp(z)) without overflow
__device__ __forceinline__ float softplus_g(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }

constexpr int GP_MAX_TAPS = 16;

// One convolved and activated channel of token t.  `raw` row t holds the step's inputs; inputs from before the portion
// come from the request's tail [taps-1, channels] (oldest first), zeros for a request that starts.
__device__ __forceinline__ float conv_channel(const float* __restrict__ raw, long long ld, int conv_off, int c, int t,
                                              int first, const float* __restrict__ tail, int channels,
                                              const float* __restrict__ w, const float* __restrict__ bias, int taps) {
  float acc = bias != nullptr ? bias[c] : 0.0f;
  const int keep = taps - 1;
  for (int j = 0; j < taps; ++j) {
    const int at = t - keep + j;                       // the token this tap reads
    float u;
    if (at >= first) u = raw[(size_t)at * ld + conv_off + c];
    else u = tail[(size_t)(keep + at - first) * channels + c];
    acc = fmaf(w[(size_t)c * taps + j], u, acc);
  }
  return silu_g(acc);
}

// mode 0 (delta): raw = [q | k | v | gate | b | a], q and k of `groups` heads x dim, v of heads x vdim; q, k, v convolved.
//   qk[t, g] = (unit(q) dim^-1/2, unit(k)), v[t, h], gates[t, h] = (exp(-exp(A_h) softplus(a + dt_bias_h)), sigmoid(b)).
// mode 1 (state space): raw = [z | x | B | C | dt], x of heads x vdim, B and C of `groups` x dim; x, B, C convolved.
//   qk[t, g] = (C, B), v[t, h] = x, gates[t, h] = (exp(-exp(A_h) dt), dt) with dt = softplus(dt + dt_bias_h).
// One block per token (several for a step of few tokens); its warps take the units (q/k groups, value heads) in turn.
__global__ void __launch_bounds__(128) gated_prepare_kernel(
    const float* __restrict__ raw, long long ld, int mode, int groups, int heads, int dim, int vdim, int taps,
    const float* __restrict__ conv_w, const float* __restrict__ conv_b, const float* __restrict__ tails,
    const int* __restrict__ slots, const int* __restrict__ q_start, const int* __restrict__ seq_of_token,
    const float* __restrict__ a_log, const float* __restrict__ dt_bias, float unit_eps, float q_scale,
    float* __restrict__ qk, float* __restrict__ v, float* __restrict__ gates) {
  pdl_trigger();
  const int t = blockIdx.x;
  const int seq = seq_of_token[t];
  const int first = q_start[seq];
  const int slot = slots[seq];
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int qk_width = groups * dim, v_width = heads * vdim;
  const int channels = 2 * qk_width + v_width;
  // where the convolved run starts, and where q (or C), k (or B) and v (or x) lie inside it
  const int conv_off = mode == 0 ? 0 : v_width;
  const int q_at = mode == 0 ? 0 : v_width + qk_width;      // C comes after B
  const int k_at = mode == 0 ? qk_width : v_width;
  const int v_at = mode == 0 ? 2 * qk_width : 0;
  const float* tail = tails != nullptr ? tails + (size_t)slot * (taps - 1) * channels : nullptr;
  // the units (q/k groups, value heads) are shared out over the blocks of a token: one block for a long step, several
  // for a step of few tokens, which would otherwise leave most of the device idle
  for (int unit = blockIdx.y * warps + warp; unit < groups + heads; unit += gridDim.y * warps) {
    if (unit < groups) {
      float* dst = qk + ((size_t)t * groups + unit) * 2 * dim;
      for (int which = 0; which < 2; ++which) {
        const int at = (which == 0 ? q_at : k_at) + unit * dim;
        float sum = 0.0f;
        for (int i = lane; i < dim; i += 32) {
          const float value = conv_channel(raw, ld, conv_off, at + i, t, first, tail, channels, conv_w, conv_b, taps);
          dst[which * dim + i] = value;
          sum = fmaf(value, value, sum);
        }
        if (mode == 0) {
          sum = warp_sum(sum);
          const float factor = (which == 0 ? q_scale : 1.0f) / sqrtf(sum + unit_eps);
          for (int i = lane; i < dim; i += 32) dst[which * dim + i] *= factor;     // each lane its own elements
        }
      }
    } else {
      const int h = unit - groups;
      for (int i = lane; i < vdim; i += 32)
        v[(size_t)t * v_width + h * vdim + i] =
            conv_channel(raw, ld, conv_off, v_at + h * vdim + i, t, first, tail, channels, conv_w, conv_b, taps);
    }
  }
  for (int h = blockIdx.y == 0 ? threadIdx.x : heads; h < heads; h += blockDim.x) {
    const float* row = raw + (size_t)t * ld;
    float decay, strength;
    if (mode == 0) {
      const float b = row[channels + v_width + h], a = row[channels + v_width + heads + h];
      decay = expf(-expf(a_log[h]) * softplus_g(a + dt_bias[h]));
      strength = sigmoid_g(b);
    } else {
      const float dt = softplus_g(row[v_width + channels + h] + dt_bias[h]);
      decay = expf(-expf(a_log[h]) * dt);
      strength = dt;
    }
    gates[((size_t)t * heads + h) * 2] = decay;
    gates[((size_t)t * heads + h) * 2 + 1] = strength;
  }
}

// The convolution's tail after the step: the last taps-1 inputs of each request, oldest first.  One thread per
// (request, channel) reads what it needs before it writes, so a portion shorter than the tail shifts it.
__global__ void conv_tail_update_kernel(const float* __restrict__ raw, long long ld, int conv_off, float* __restrict__ tails,
                                        const int* __restrict__ slots, const int* __restrict__ q_start, int taps,
                                        int channels) {
  pdl_trigger();
  pdl_wait();
  const int seq = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int keep = taps - 1;
  const int first = q_start[seq], n = q_start[seq + 1] - first;
  if (n <= 0 || keep <= 0) return;
  float* mine = tails + (size_t)slots[seq] * keep * channels + c;
  float old[GP_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < GP_MAX_TAPS; ++j) old[j] = j < keep ? mine[(size_t)j * channels] : 0.0f;
#pragma unroll
  for (int j = 0; j < GP_MAX_TAPS; ++j) {
    if (j < keep) {
      const int at = n + j;                                // in (old tail, then this step's rows)
      mine[(size_t)j * channels] = at < keep ? old[at] : raw[(size_t)(first + at - keep) * ld + conv_off + c];
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// The recurrence, token by token.  Columns of the state do not interact: column j of S needs k, q, the head's two
// gates and v_j only.  Eight lanes share a column, each holding ROWS of its rows in registers (row r * 8 + part), so a
// warp owns four columns and the two sums over the rows (S^T k and S^T q) are three butterfly steps each.  The next
// token's q, k, v and gates are loaded while this token's arithmetic runs.  Grid: (column tiles, heads, requests).
constexpr int GR_WARPS = 4;
constexpr int GR_COLS = GR_WARPS * 4;       // columns of a block

template <int ROWS, bool DELTA>
__global__ void __launch_bounds__(GR_WARPS * 32) gated_rule_scan_kernel(
    const float* __restrict__ qk, const float* __restrict__ v, const float* __restrict__ gates,
    const float* __restrict__ skip, int heads, int groups, int dim, int vdim, float* __restrict__ state,
    const int* __restrict__ slots, const int* __restrict__ q_start, float* __restrict__ out) {
  pdl_trigger();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int part = lane & 7;
  const int head = blockIdx.y, seq = blockIdx.z;
  const int group = head / (heads / groups);
  const int column = blockIdx.x * GR_COLS + warp * 4 + (lane >> 3);
  const bool live = column < vdim;
  const int first = q_start[seq], last = q_start[seq + 1];
  const int slot = slots[seq];
  const float d_skip = skip != nullptr ? skip[head] : 0.0f;
  pdl_wait();
  if (first >= last) return;
  float* mine = state + (((size_t)slot * heads + head) * dim) * vdim + column;
  float s[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int i = r * 8 + part;
    s[r] = (live && i < dim) ? mine[(size_t)i * vdim] : 0.0f;
  }
  float qn[ROWS], kn[ROWS], vn, an, bn;
  auto fetch = [&](int t) {
    const float* src = qk + ((size_t)t * groups + group) * 2 * dim;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int i = r * 8 + part;
      qn[r] = i < dim ? src[i] : 0.0f;
      kn[r] = i < dim ? src[dim + i] : 0.0f;
    }
    vn = live ? v[((size_t)t * heads + head) * vdim + column] : 0.0f;
    const float2 g = *reinterpret_cast<const float2*>(gates + ((size_t)t * heads + head) * 2);
    an = g.x;
    bn = g.y;
  };
  fetch(first);
  for (int t = first; t < last; ++t) {
    float q[ROWS], k[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) { q[r] = qn[r]; k[r] = kn[r]; }
    const float value = vn, a = an, b = bn;
    if (t + 1 < last) fetch(t + 1);
    float seen = 0.0f;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      s[r] *= a;
      if (DELTA) seen = fmaf(s[r], k[r], seen);
    }
    if (DELTA) {
      seen += __shfl_xor_sync(0xffffffffu, seen, 1);
      seen += __shfl_xor_sync(0xffffffffu, seen, 2);
      seen += __shfl_xor_sync(0xffffffffu, seen, 4);
    }
    const float u = b * (value - seen);
    float acc = 0.0f;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      s[r] = fmaf(k[r], u, s[r]);
      acc = fmaf(s[r], q[r], acc);
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
    if (live && part == 0) out[((size_t)t * heads + head) * vdim + column] = fmaf(d_skip, value, acc);
  }
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int i = r * 8 + part;
    if (live && i < dim) mine[(size_t)i * vdim] = s[r];
  }
}

// The same recurrence for portions of several tokens and keys of 32, 64, 128 or 256 numbers.  q, k, v and the gates of
// 16 tokens (8 with keys of 256) are copied into shared memory ahead of the arithmetic (cp.async, two buffers), so a
// token's step waits for shared memory and one butterfly, not for the L2.  A lane holds the ROWS consecutive rows
// part * ROWS .. of TWO neighbouring columns (its q and k serve both), read as 16-byte units; the parts' runs are four
// floats apart in banks.  Both sums over the rows are taken of the decayed OLD state, S^T k and S^T q, together with
// k . q, in one butterfly: the token's output is (a S)^T q + u (k . q), and only u stands between this token's state
// and the next one's.  PARTS lanes (8 or 16) share a column pair: with 16 a block of four warps owns 16 columns, a
// head is spread over twice as many warps, and each warp has half the arithmetic between two butterflies.

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

template <int ROWS, int PARTS, bool DELTA>
__global__ void __launch_bounds__(GR_WARPS * 32) gated_rule_scan_staged_kernel(
    const float* __restrict__ qk, const float* __restrict__ v, const float* __restrict__ gates,
    const float* __restrict__ skip, int heads, int groups, int vdim, float* __restrict__ state,
    const int* __restrict__ slots, const int* __restrict__ q_start, float* __restrict__ out) {
  constexpr int DIM = ROWS * PARTS;
  constexpr int GS_COLS = GR_WARPS * 2 * (32 / PARTS); // columns of a block
  constexpr int PITCH = ROWS + 4;                      // floats between two parts' runs
  constexpr int VEC = 2 * PARTS * PITCH;               // q then k of one token
  constexpr int GS_TOKENS = VEC > 320 ? 8 : 16;        // tokens per buffer: both buffers within 48 KB
  __shared__ __align__(16) float qk_s[2][GS_TOKENS][VEC];
  __shared__ float v_s[2][GS_TOKENS][GS_COLS];
  __shared__ __align__(8) float g_s[2][GS_TOKENS][2];
  pdl_trigger();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int part = lane & (PARTS - 1);
  const int head = blockIdx.y, seq = blockIdx.z;
  const int group = head / (heads / groups);
  const int local = (warp * (32 / PARTS) + lane / PARTS) * 2;      // the first of the lane's two columns, inside the block
  const int column = blockIdx.x * GS_COLS + local;
  const bool live0 = column < vdim, live1 = column + 1 < vdim;
  const int first = q_start[seq], last = q_start[seq + 1];
  const int slot = slots[seq];
  const float d_skip = skip != nullptr ? skip[head] : 0.0f;
  pdl_wait();
  if (first >= last) return;
  float* mine = state + (((size_t)slot * heads + head) * DIM) * vdim + column;
  float s0[ROWS], s1[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    s0[r] = live0 ? mine[(size_t)(part * ROWS + r) * vdim] : 0.0f;
    s1[r] = live1 ? mine[(size_t)(part * ROWS + r) * vdim + 1] : 0.0f;
  }

  auto stage = [&](int buffer, int base) {
    const int count = min(GS_TOKENS, last - base);
    // q and k: 2 * DIM floats per token in units of four; unit u of a token covers rows 4u .. 4u + 3 of q (then of k)
    for (int e = threadIdx.x; e < count * (2 * DIM / 4); e += blockDim.x) {
      const int n = e / (2 * DIM / 4), u = e - n * (2 * DIM / 4);
      const int which = u / (DIM / 4), row = (u - which * (DIM / 4)) * 4;
      cp_async16(&qk_s[buffer][n][which * PARTS * PITCH + (row / ROWS) * PITCH + row % ROWS],
                 qk + ((size_t)(base + n) * groups + group) * 2 * DIM + which * DIM + row);
    }
    for (int e = threadIdx.x; e < count * GS_COLS; e += blockDim.x) {
      const int n = e / GS_COLS, c = e - n * GS_COLS;
      if (blockIdx.x * GS_COLS + c < vdim)
        cp_async4(&v_s[buffer][n][c], v + ((size_t)(base + n) * heads + head) * vdim + blockIdx.x * GS_COLS + c);
    }
    for (int e = threadIdx.x; e < count * 2; e += blockDim.x)
      cp_async4(&g_s[buffer][e >> 1][e & 1], gates + ((size_t)(base + (e >> 1)) * heads + head) * 2 + (e & 1));
    cp_async_commit();
  };

  stage(0, first);
  int buffer = 0;
  for (int base = first; base < last; base += GS_TOKENS, buffer ^= 1) {
    if (base + GS_TOKENS < last) {
      stage(buffer ^ 1, base + GS_TOKENS);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int count = min(GS_TOKENS, last - base);
    float q[ROWS], k[ROWS], next_value0, next_value1, next_a, next_b;
    auto fetch = [&](int n) {
      next_value0 = live0 ? v_s[buffer][n][local] : 0.0f;
      next_value1 = live1 ? v_s[buffer][n][local + 1] : 0.0f;
      next_a = g_s[buffer][n][0];
      next_b = g_s[buffer][n][1];
      const float4* qv = reinterpret_cast<const float4*>(&qk_s[buffer][n][part * PITCH]);
      const float4* kv = reinterpret_cast<const float4*>(&qk_s[buffer][n][PARTS * PITCH + part * PITCH]);
#pragma unroll
      for (int r = 0; r < ROWS; r += 4) {
        const float4 qq = qv[r / 4], kk = kv[r / 4];
        q[r] = qq.x; q[r + 1] = qq.y; q[r + 2] = qq.z; q[r + 3] = qq.w;
        k[r] = kk.x; k[r + 1] = kk.y; k[r + 2] = kk.z; k[r + 3] = kk.w;
      }
    };
    fetch(0);
#pragma unroll 2
    for (int n = 0; n < count; ++n) {
      const float value0 = next_value0, value1 = next_value1, a = next_a, b = next_b;
      float seen0[2] = {0.0f, 0.0f}, seen1[2] = {0.0f, 0.0f}, read0[2] = {0.0f, 0.0f}, read1[2] = {0.0f, 0.0f};
      float kq[2] = {0.0f, 0.0f};
      float kr[ROWS];
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        s0[r] *= a;
        s1[r] *= a;
        kr[r] = k[r];
        if (DELTA) {
          seen0[r & 1] = fmaf(s0[r], k[r], seen0[r & 1]);
          seen1[r & 1] = fmaf(s1[r], k[r], seen1[r & 1]);
        }
        read0[r & 1] = fmaf(s0[r], q[r], read0[r & 1]);
        read1[r & 1] = fmaf(s1[r], q[r], read1[r & 1]);
        kq[r & 1] = fmaf(k[r], q[r], kq[r & 1]);
      }
      if (n + 1 < count) fetch(n + 1);                 // the next token's q and k, while the sums cross the lanes
      float p0 = seen0[0] + seen0[1], p1 = seen1[0] + seen1[1];
      float o0 = read0[0] + read0[1], o1 = read1[0] + read1[1], dot = kq[0] + kq[1];
#pragma unroll
      for (int step = 1; step < PARTS; step <<= 1) {
        if (DELTA) {
          p0 += __shfl_xor_sync(0xffffffffu, p0, step);
          p1 += __shfl_xor_sync(0xffffffffu, p1, step);
        }
        o0 += __shfl_xor_sync(0xffffffffu, o0, step);
        o1 += __shfl_xor_sync(0xffffffffu, o1, step);
        dot += __shfl_xor_sync(0xffffffffu, dot, step);
      }
      const float u0 = b * (value0 - p0), u1 = b * (value1 - p1);
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        s0[r] = fmaf(kr[r], u0, s0[r]);
        s1[r] = fmaf(kr[r], u1, s1[r]);
      }
      if (part == 0) {
        float* dst = out + ((size_t)(base + n) * heads + head) * vdim + column;
        if (live0) dst[0] = fmaf(d_skip, value0, fmaf(u0, dot, o0));
        if (live1) dst[1] = fmaf(d_skip, value1, fmaf(u1, dot, o1));
      }
    }
    __syncthreads();                                   // the buffer is copied into again two rounds on
  }
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    if (live0) mine[(size_t)(part * ROWS + r) * vdim] = s0[r];
    if (live1) mine[(size_t)(part * ROWS + r) * vdim + 1] = s1[r];
  }
}

template <bool DELTA>
int launch_gated_rule_scan(const float* qk, const float* v, const float* gates, const float* skip, int heads, int groups,
                           int dim, int vdim, float* state, const int* slots, const int* q_start, float* out, int num_seqs,
                           bool portions, cudaStream_t stream) {
  const dim3 grid((vdim + GR_COLS - 1) / GR_COLS, heads, num_seqs), block(GR_WARPS * 32);
  if (portions && (dim == 32 || dim == 64 || dim == 128 || dim == 256) && (uintptr_t)qk % 16 == 0) {
    // eight lanes to a column pair at keys of 32 and 128, sixteen at 64 and 256 (measured at 2,048 tokens, 28 heads:
    // keys of 128: 960 us with eight, 1,036 with sixteen; keys of 64: 657 with eight, 494 with sixteen)
    const int parts = (dim == 64 || dim == 256) ? 16 : 8;
    const int cols = GR_WARPS * 2 * (32 / parts);
    const dim3 grid((vdim + cols - 1) / cols, heads, num_seqs);
#define TGE_GS_CASE(R, P)                                                                                                  \
  if (dim == R * P && parts == P) {                                                                                       \
    tge_launch(gated_rule_scan_staged_kernel<R, P, DELTA>, grid, block, 0, stream, qk, v, gates, skip, heads, groups, vdim, \
               state, slots, q_start, out);                                                                               \
    return tge_launched("gated_rule_scan_staged", 1);                                                                     \
  }
    TGE_GS_CASE(4, 8) TGE_GS_CASE(16, 8) TGE_GS_CASE(4, 16) TGE_GS_CASE(16, 16)
#undef TGE_GS_CASE
  }
  const int rows = (dim + 7) / 8;
#define TGE_GR_CASE(R)                                                                                                  \
  if (rows <= R) {                                                                                                     \
    tge_launch(gated_rule_scan_kernel<R, DELTA>, grid, block, 0, stream, qk, v, gates, skip, heads, groups, dim, vdim, \
               state, slots, q_start, out);                                                                            \
    return tge_launched("gated_rule_scan", 1);                                                                         \
  }
  TGE_GR_CASE(2) TGE_GR_CASE(4) TGE_GR_CASE(6) TGE_GR_CASE(8) TGE_GR_CASE(12) TGE_GR_CASE(16) TGE_GR_CASE(24) TGE_GR_CASE(32)
#undef TGE_GR_CASE
  tge_set_error("gated_rule_scan: keys of %d numbers (up to 256)", dim);
  return -1;
}

// x[t] += alpha * y[t] / sqrt(mean(y[t]^2) + eps) * w; one block per token.
__global__ void __launch_bounds__(256) norm_scale_add_kernel(float* __restrict__ x, const float* __restrict__ y, long long ldy,
                                                             const float* __restrict__ weight, int width, float alpha,
                                                             float eps) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const float* src = y + (size_t)blockIdx.x * ldy;
  float sum = 0.0f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) sum = fmaf(src[i], src[i], sum);
  const float factor = alpha / sqrtf(block_sum(sum, scratch) / (float)width + eps);
  float* dst = x + (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = fmaf(src[i] * factor, weight[i], dst[i]);
}

// After the q/k product of an attention whose values are its keys as projected.  Row t holds [q | k] (heads and
// kv_heads of head_dim).  The values' pages get k as it arrives; then q and k are normalised per head (a null weight:
// left as they are), q is multiplied by 1 + coef ln(floor((p + 1) / every) + 1), q is rewritten in place and k goes to
// its pages.  One block per token, a warp per head.
template <typename T>
__global__ void __launch_bounds__(256) qk_temp_store_kernel(
    T* __restrict__ qk, int row_stride, const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
    float temp_coef, int temp_every, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ block_table, int max_pages, T* __restrict__ k_pages, T* __restrict__ v_pages, int num_pages,
    int page_size, int heads, int kv_heads, int head_dim, int store_kv, int* status) {
  pdl_trigger();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int seq = seq_of_token[t];
  size_t base = 0;
  bool store = store_kv != 0;
  if (store) {
    const int page_index = pos / page_size;
    const int page = (pos >= 0 && page_index < max_pages) ? block_table[(size_t)seq * max_pages + page_index] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, TGE_STATUS_BAD_PAGE);
      store = false;
    } else {
      base = ((size_t)page * kv_heads * page_size + (pos % page_size)) * head_dim;
    }
  }
  const float temperature = temp_every > 0 ? 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f) : 1.0f;
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  T* row = qk + (size_t)t * row_stride;
  for (int unit = warp; unit < heads + kv_heads; unit += warps) {
    const bool is_q = unit < heads;
    T* src = row + (size_t)unit * head_dim;
    const float* weight = is_q ? q_weight : k_weight;
    const size_t at = base + (size_t)(unit - heads) * page_size * head_dim;
    float sum = 0.0f;
    for (int d = lane; d < head_dim; d += 32) {
      const float value = to_float<T>(src[d]);
      sum = fmaf(value, value, sum);
      if (!is_q && store) v_pages[at + d] = src[d];
    }
    float factor = is_q ? temperature : 1.0f;
    if (weight != nullptr) factor *= 1.0f / sqrtf(warp_sum(sum) / (float)head_dim + eps);
    for (int d = lane; d < head_dim; d += 32) {
      const T value = from_float<T>(to_float<T>(src[d]) * factor * (weight != nullptr ? weight[d] : 1.0f));
      if (is_q) src[d] = value;
      else if (store) k_pages[at + d] = value;
    }
  }
}

// rows [T, 2 * inner] float32 with (g_i, u_i) side by side -> out [T, inner]:
// g <- min(g, L); u <- clamp(u, -L, L); out = g sigmoid(alpha g) (u + offset).
template <typename T>
__global__ void __launch_bounds__(256) gated_clamp_act_kernel(const float* __restrict__ rows, long long ld, T* __restrict__ out,
                                                              long long ld_out, int tokens, int inner, float limit,
                                                              float alpha, float offset) {
  pdl_trigger();
  pdl_wait();
  const long long count = (long long)tokens * inner;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(e / inner), i = (int)(e - (long long)t * inner);
    const float2 gu = *reinterpret_cast<const float2*>(rows + (size_t)t * ld + 2 * (size_t)i);
    const float g = fminf(gu.x, limit);
    const float u = fminf(fmaxf(gu.y, -limit), limit);
    out[(size_t)t * ld_out + i] = from_float<T>(g * sigmoid_g(alpha * g) * (u + offset));
  }
}

// out[t] = [a[t] | b[t]] in the products' number format.
template <typename T>
__global__ void __launch_bounds__(256) concat_rows_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                          T* __restrict__ out, int tokens, int width) {
  pdl_trigger();
  pdl_wait();
  const long long count = (long long)tokens * 2 * width;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (long long)gridDim.x * blockDim.x) {
    const long long t = e / (2 * width);
    const int i = (int)(e - t * 2 * width);
    out[e] = from_float<T>(i < width ? a[t * width + i] : b[t * width + i - width]);
  }
}

unsigned blocks_for(long long count, int threads) {
  const long long blocks = (count + threads - 1) / threads;
  return (unsigned)(blocks < 1 ? 1 : (blocks > 65535 * 8 ? 65535 * 8 : blocks));
}

}  // namespace

TGE_API int tge_gated_prepare(const float* raw, long long ld, int mode, int groups, int heads, int dim, int vdim, int taps,
                              const float* conv_w, const float* conv_b, float* tails, const int* slots, const int* q_start,
                              const int* seq_of_token, const float* a_log, const float* dt_bias, float unit_eps,
                              float q_scale, float* qk, float* v, float* gates, int tokens, int num_seqs,
                              cudaStream_t stream) {
  TGE_REQUIRE(mode == 0 || mode == 1, "gated_prepare: mode %d", mode);
  TGE_REQUIRE(groups > 0 && heads > 0 && heads % groups == 0 && dim > 0 && vdim > 0,
              "gated_prepare: %d heads on %d groups of %d, values of %d", heads, groups, dim, vdim);
  TGE_REQUIRE(taps >= 1 && taps <= GP_MAX_TAPS && conv_w != nullptr, "gated_prepare: %d taps (1 to %d)", taps, GP_MAX_TAPS);
  TGE_REQUIRE(taps == 1 || tails != nullptr, "gated_prepare: a convolution over time needs the requests' tails");
  const long long need = 2LL * groups * dim + (long long)heads * vdim * (mode == 0 ? 2 : 2) + (mode == 0 ? 2 : 1) * heads;
  TGE_REQUIRE(ld >= need, "gated_prepare: rows of %lld numbers, %lld needed", ld, need);
  if (tokens == 0) return 0;
  const int slices = tokens >= 256 ? 1 : (groups + heads + 3) / 4;
  tge_launch(gated_prepare_kernel, dim3(tokens, slices), dim3(128), 0, stream, raw, ld, mode, groups, heads, dim, vdim, taps, conv_w,
             conv_b, (const float*)tails, slots, q_start, seq_of_token, a_log, dt_bias, unit_eps, q_scale, qk, v, gates);
  int rc = tge_launched("gated_prepare", 1);
  if (rc < 0 || taps == 1) return rc;
  const int channels = 2 * groups * dim + heads * vdim;
  tge_launch(conv_tail_update_kernel, dim3((channels + 127) / 128, num_seqs), dim3(128), 0, stream, raw, ld,
             mode == 0 ? 0 : heads * vdim, tails, slots, q_start, taps, channels);
  rc = tge_launched("conv_tail_update", 2);
  return rc;
}

TGE_API int tge_gated_rule_scan(const float* qk, const float* v, const float* gates, const float* skip, int delta, int heads,
                                int groups, int dim, int vdim, float* state, const int* slots, const int* q_start, float* out,
                                int num_seqs, int tokens, cudaStream_t stream) {
  TGE_REQUIRE(groups > 0 && heads > 0 && heads % groups == 0 && dim > 0 && vdim > 0 && dim <= 256,
              "gated_rule_scan: %d heads on %d groups, keys of %d (up to 256), values of %d", heads, groups, dim, vdim);
  TGE_REQUIRE(num_seqs >= 0 && num_seqs <= 65535 && heads <= 65535, "gated_rule_scan: %d requests in a step", num_seqs);
  if (num_seqs == 0 || tokens == 0) return 0;
  if (delta)
    return launch_gated_rule_scan<true>(qk, v, gates, skip, heads, groups, dim, vdim, state, slots, q_start, out, num_seqs,
                                        tokens > num_seqs, stream);
  return launch_gated_rule_scan<false>(qk, v, gates, skip, heads, groups, dim, vdim, state, slots, q_start, out, num_seqs,
                                       tokens > num_seqs, stream);
}

TGE_API int tge_norm_scale_add(float* x, const float* y, long long ldy, const float* weight, int tokens, int width, float alpha,
                               float eps, cudaStream_t stream) {
  TGE_REQUIRE(tokens >= 0 && width > 0 && ldy >= width && eps > 0.0f, "norm_scale_add: bad shape");
  if (tokens == 0) return 0;
  tge_launch(norm_scale_add_kernel, dim3(tokens), dim3(256), 0, stream, x, y, ldy, weight, width, alpha, eps);
  return tge_launched("norm_scale_add", 1);
}

TGE_API int tge_qk_temp_store(void* qk, int is_bf16, int row_stride, const float* q_weight, const float* k_weight, float eps,
                              float temp_coef, int temp_every, const int* positions, const int* seq_of_token,
                              const int* block_table, int max_pages, void* k_pages, void* v_pages, int num_pages, int page_size,
                              int tokens, int heads, int kv_heads, int head_dim, int store_kv, int* status, cudaStream_t stream) {
  TGE_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && head_dim > 0, "qk_temp_store: bad sizes");
  TGE_REQUIRE(row_stride >= (heads + kv_heads) * head_dim, "qk_temp_store: rows of %d numbers do not hold q and k", row_stride);
  TGE_REQUIRE(eps > 0.0f || (q_weight == nullptr && k_weight == nullptr), "qk_temp_store: eps must be positive");
  TGE_REQUIRE(temp_every >= 0, "qk_temp_store: a temperature every %d positions", temp_every);
  TGE_REQUIRE(!store_kv || (page_size > 0 && max_pages > 0 && num_pages > 0 && k_pages && v_pages && block_table),
              "qk_temp_store: bad page geometry");
  if (tokens == 0) return 0;
  if (is_bf16)
    tge_launch(qk_temp_store_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, (__nv_bfloat16*)qk, row_stride, q_weight,
               k_weight, eps, temp_coef, temp_every, positions, seq_of_token, block_table, max_pages, (__nv_bfloat16*)k_pages,
               (__nv_bfloat16*)v_pages, num_pages, page_size, heads, kv_heads, head_dim, store_kv, status);
  else
    tge_launch(qk_temp_store_kernel<float>, dim3(tokens), dim3(256), 0, stream, (float*)qk, row_stride, q_weight, k_weight, eps,
               temp_coef, temp_every, positions, seq_of_token, block_table, max_pages, (float*)k_pages, (float*)v_pages,
               num_pages, page_size, heads, kv_heads, head_dim, store_kv, status);
  return tge_launched("qk_temp_store", 1);
}

TGE_API int tge_gated_clamp_act(const float* rows, long long ld, void* out, long long ld_out, int is_bf16, int tokens, int inner,
                                float limit, float alpha, float offset, cudaStream_t stream) {
  TGE_REQUIRE(tokens >= 0 && inner > 0 && ld >= 2LL * inner && ld % 2 == 0 && ld_out >= inner && limit > 0.0f,
              "gated_clamp_act: bad shape");
  TGE_REQUIRE((uintptr_t)rows % 8 == 0, "gated_clamp_act: rows must start on 8 bytes");
  if (tokens == 0) return 0;
  const unsigned blocks = blocks_for((long long)tokens * inner, 256);
  if (is_bf16)
    tge_launch(gated_clamp_act_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, rows, ld, (__nv_bfloat16*)out, ld_out,
               tokens, inner, limit, alpha, offset);
  else
    tge_launch(gated_clamp_act_kernel<float>, dim3(blocks), dim3(256), 0, stream, rows, ld, (float*)out, ld_out, tokens, inner,
               limit, alpha, offset);
  return tge_launched("gated_clamp_act", 1);
}

TGE_API int tge_concat_rows(const float* a, const float* b, void* out, int is_bf16, int tokens, int width, cudaStream_t stream) {
  TGE_REQUIRE(tokens >= 0 && width > 0, "concat_rows: bad shape");
  if (tokens == 0) return 0;
  const unsigned blocks = blocks_for((long long)tokens * 2 * width, 256);
  if (is_bf16)
    tge_launch(concat_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, a, b, (__nv_bfloat16*)out, tokens, width);
  else
    tge_launch(concat_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, a, b, (float*)out, tokens, width);
  return tge_launched("concat_rows", 1);
}
