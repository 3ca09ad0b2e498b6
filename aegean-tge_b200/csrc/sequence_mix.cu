// Kernels of the mixers that carry a fixed-size state from token to token, and of the layers around them:
//
//  * decay_scan       - linear attention with a fixed decay per head: S_t = c S_(t-1) + k_t v_t^T, o_t = S_t^T q_t,
//                       the state in float32 in a per-request slot, q and k activated, rotated and scaled on the way in.
//                       Three kernels, chosen by the longest portion of a step: token by token (single tokens, short
//                       portions), chunks of 32 tokens (any key size up to 256), chunks of 64 with register tiles and
//                       asynchronous copies (keys up to 128), the last also in segments that share one long portion out
//                       over the device (decay_segment_carry between its two launches); decay_prepare readies q and k
//                       once per step for the chunked ones;
//  * gated_norm       - RMS norm over groups of a row (a head, or all heads together), times an activated gate;
//  * conv_norm_rope_store / conv_state_update - a short causal convolution over time on every channel of q, k and v
//                       (its last taps-1 inputs kept per request), the per-head norm of q and k, their rotation, and
//                       the store of k and v into their pages;
//  * pool_kv          - the mean key and mean value of every block of P positions that a step completes;
//  * scale_add_norm   - the layer that normalises after the sum: x <- rms(a x + y) g;
//  * to_run_dtype     - float32 rows in the format the products read.
//
// All statistics, states, angles and sums are float32 in both number formats; what is bfloat16 in the
// bfloat16 path is the projections these kernels read and the rows they hand to the next product.
#include <stdlib.h>

#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

// ---------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void to_run_dtype_kernel(const float* __restrict__ x, T* __restrict__ out, size_t count) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) out[i] = from_float<T>(x[i]);
}

// x[r, :] <- rms(alpha x[r, :] + y[r, :]) * weight, in place; `copy` (may be null) receives the same row in T.
template <typename T>
__global__ void __launch_bounds__(256) scale_add_norm_kernel(float* __restrict__ x, const float* __restrict__ y,
                                                             long long ldy, const float* __restrict__ weight,
                                                             T* __restrict__ copy, int hidden, float alpha, float eps) {
  __shared__ float scratch[32];
  float* row = x + (size_t)blockIdx.x * hidden;
  const float* add = y + (size_t)blockIdx.x * ldy;
  float sum = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = fmaf(alpha, row[i], add[i]);
    sum = fmaf(v, v, sum);
  }
  sum = block_sum(sum, scratch);
  const float scale = 1.0f / sqrtf(sum / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = fmaf(alpha, row[i], add[i]) * scale * weight[i];
    row[i] = v;
    if (copy != nullptr) copy[(size_t)blockIdx.x * hidden + i] = from_float<T>(v);
  }
}

// The same with 16-byte accesses and the row held in registers between the two passes: rows of a multiple of four
// elements, at most sixteen per thread.
__device__ __forceinline__ void store_quad(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
__device__ __forceinline__ void store_quad(__nv_bfloat16* dst, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 packed;
  packed.x = *reinterpret_cast<const uint32_t*>(&lo);
  packed.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = packed;
}

template <typename T>
__global__ void __launch_bounds__(1024) scale_add_norm_vec_kernel(float* __restrict__ x, const float* __restrict__ y,
                                                                  long long ldy, const float* __restrict__ weight,
                                                                  T* __restrict__ copy, int hidden, float alpha, float eps) {
  __shared__ float scratch[32];
  pdl_trigger();
  const int quads = hidden >> 2;
  float4 gain[4], value[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {                  // constants of the model: before the wait
    const int i = threadIdx.x + k * blockDim.x;
    gain[k] = i < quads ? reinterpret_cast<const float4*>(weight)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();
  float4* row = reinterpret_cast<float4*>(x + (size_t)blockIdx.x * hidden);
  const float4* add = reinterpret_cast<const float4*>(y + (size_t)blockIdx.x * ldy);
  float sum = 0.0f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < quads) {
      const float4 a = row[i], b = add[i];
      v = make_float4(fmaf(alpha, a.x, b.x), fmaf(alpha, a.y, b.y), fmaf(alpha, a.z, b.z), fmaf(alpha, a.w, b.w));
    }
    value[k] = v;
    sum = fmaf(v.x, v.x, sum); sum = fmaf(v.y, v.y, sum); sum = fmaf(v.z, v.z, sum); sum = fmaf(v.w, v.w, sum);
  }
  sum = block_sum(sum, scratch);
  const float scale = 1.0f / sqrtf(sum / (float)hidden + eps);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < quads) {
      const float4 v = make_float4(value[k].x * scale * gain[k].x, value[k].y * scale * gain[k].y,
                                   value[k].z * scale * gain[k].z, value[k].w * scale * gain[k].w);
      row[i] = v;
      if (copy != nullptr) store_quad(copy + (size_t)blockIdx.x * hidden + 4 * (size_t)i, v);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// Linear attention with a decay per head.  A block owns 32 columns of one head's state for one request and walks
// the request's tokens of this step in order, SCAN_TOKENS at a time: the block prepares their q and k (activation,
// rotation, scale) in shared memory, every thread then updates its rows of its column token by token and adds up
// its share of o, and the four row groups' shares are summed in a fixed order.  Columns of the state do not
// interact, so the grid is (column tiles, heads, requests) and a result depends on nothing but the request's own
// tokens in their order.
constexpr int SCAN_TOKENS = 8;
constexpr int SCAN_WARPS = 4;

template <typename T, int ROWS, int TOKENS>
__global__ void __launch_bounds__(SCAN_WARPS * 32) decay_scan_kernel(
    const T* __restrict__ rows, long long ld, int q_off, int k_off, int v_off, int heads, int dim, int vdim,
    int activation, const float* __restrict__ cos_table, const float* __restrict__ sin_table, int table_positions,
    int rotary, float k_scale, const float* __restrict__ decay, float* __restrict__ state,
    const int* __restrict__ slots, const int* __restrict__ q_start, const int* __restrict__ positions,
    float* __restrict__ out, int* status) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float shared[];
  float* qs = shared;                                   // [TOKENS][dim]
  float* ks = qs + TOKENS * dim;                   // [TOKENS][dim]
  float* partial = ks + TOKENS * dim;              // [SCAN_WARPS][TOKENS][32]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int head = blockIdx.y, seq = blockIdx.z;
  const int column = blockIdx.x * 32 + lane;
  const bool live = column < vdim;
  const int first = q_start[seq], last = q_start[seq + 1];
  if (first >= last) return;
  const int slot = slots[seq];
  const float c = decay[head];
  const int half = rotary >> 1;
  float* mine = state + (((size_t)slot * heads + head) * dim) * vdim + column;
  float s[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int i = warp * ROWS + r;
    s[r] = (live && i < dim) ? mine[(size_t)i * vdim] : 0.0f;
  }
  for (int base = first; base < last; base += TOKENS) {
    const int count = min(TOKENS, last - base);
    // q and k of these tokens as the recurrence takes them
    for (int e = threadIdx.x; e < count * dim; e += blockDim.x) {
      const int n = e / dim, i = e - n * dim;
      const T* row = rows + (size_t)(base + n) * ld;
      float q = to_float<T>(row[q_off + head * dim + i]);
      float k = to_float<T>(row[k_off + head * dim + i]);
      if (activation) { q = silu_f(q); k = silu_f(k); }
      if (i < rotary) {
        const int other = i < half ? i + half : i - half;
        float q2 = to_float<T>(row[q_off + head * dim + other]);
        float k2 = to_float<T>(row[k_off + head * dim + other]);
        if (activation) { q2 = silu_f(q2); k2 = silu_f(k2); }
        int position = positions[base + n];
        if (position < 0 || position >= table_positions) {
          atomicOr(status, TGE_STATUS_BAD_ROW);
          position = 0;
        }
        const float cs = cos_table[(size_t)position * half + (i < half ? i : i - half)];
        const float sn = sin_table[(size_t)position * half + (i < half ? i : i - half)];
        // the pair (u, v) = (element i, element i + half) becomes (u cos - v sin, v cos + u sin)
        q = i < half ? q * cs - q2 * sn : q * cs + q2 * sn;
        k = i < half ? k * cs - k2 * sn : k * cs + k2 * sn;
      }
      qs[e] = q;
      ks[e] = k * k_scale;
    }
    float v[TOKENS];
#pragma unroll
    for (int n = 0; n < TOKENS; ++n) {
      float value = 0.0f;
      if (live && n < count) {
        value = to_float<T>(rows[(size_t)(base + n) * ld + v_off + head * vdim + column]);
        if (activation) value = silu_f(value);
      }
      v[n] = value;
    }
    __syncthreads();
#pragma unroll
    for (int n = 0; n < TOKENS; ++n) {
      float acc = 0.0f;
      if (n < count) {
        const float* qn = qs + n * dim + warp * ROWS;
        const float* kn = ks + n * dim + warp * ROWS;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          if (warp * ROWS + r < dim) {
            s[r] = fmaf(kn[r], v[n], c * s[r]);
            acc = fmaf(s[r], qn[r], acc);
          }
        }
      }
      partial[(warp * TOKENS + n) * 32 + lane] = acc;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < count * 32; e += blockDim.x) {
      const int n = e >> 5, l = e & 31;
      float total = 0.0f;
#pragma unroll
      for (int w = 0; w < SCAN_WARPS; ++w) total += partial[(w * TOKENS + n) * 32 + l];
      const int col = blockIdx.x * 32 + l;
      if (col < vdim) out[(size_t)(base + n) * heads * vdim + head * vdim + col] = total;
    }
    // the next round writes qs/ks before its first barrier, and partial after it: a barrier here keeps the
    // sums above apart from both
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int i = warp * ROWS + r;
    if (live && i < dim) mine[(size_t)i * vdim] = s[r];
  }
}

// q and k as the recurrence takes them (activation, rotation, the factor on k), float32 [tokens, heads, 2, dim]: once
// per step for the chunked kernels, whose blocks (one per run of state columns) would each redo it otherwise.
template <typename T>
__global__ void __launch_bounds__(128) decay_prepare_kernel(
    const T* __restrict__ rows, long long ld, int q_off, int k_off, int heads, int dim, int activation,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, int table_positions, int rotary,
    float k_scale, const int* __restrict__ positions, float* __restrict__ prepared, int* status) {
  const int t = blockIdx.x, head = blockIdx.y;
  const int half = rotary >> 1;
  const T* row = rows + (size_t)t * ld;
  int position = positions[t];
  if (rotary > 0 && (position < 0 || position >= table_positions)) {
    if (threadIdx.x == 0) atomicOr(status, TGE_STATUS_BAD_ROW);
    position = 0;
  }
  float* dst = prepared + ((size_t)t * heads + head) * 2 * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float q = to_float<T>(row[q_off + head * dim + i]);
    float k = to_float<T>(row[k_off + head * dim + i]);
    if (activation) { q = silu_f(q); k = silu_f(k); }
    if (i < rotary) {
      const int other = i < half ? i + half : i - half;
      float q2 = to_float<T>(row[q_off + head * dim + other]);
      float k2 = to_float<T>(row[k_off + head * dim + other]);
      if (activation) { q2 = silu_f(q2); k2 = silu_f(k2); }
      const float cs = cos_table[(size_t)position * half + (i < half ? i : i - half)];
      const float sn = sin_table[(size_t)position * half + (i < half ? i : i - half)];
      // the pair (u, v) = (element i, element i + half) becomes (u cos - v sin, v cos + u sin)
      q = i < half ? q * cs - q2 * sn : q * cs + q2 * sn;
      k = i < half ? k * cs - k2 * sn : k * cs + k2 * sn;
    }
    dst[i] = q;
    dst[dim + i] = k * k_scale;
  }
}

// The same recurrence for portions of many tokens, CHUNK tokens at a time.  With S the state before a chunk of n
// tokens, c the head's decay and t, j places in the chunk:
//   o_t   = c^(t+1) S^T q_t + sum_(j <= t) c^(t-j) (q_t . k_j) v_j
//   S_new = c^n S + sum_j k_j (c^(n-1-j) v_j)^T
// so a chunk is three small products on the CUDA cores (scores, readout, state update), all float32, instead of n
// dependent steps.  Only non-negative powers of c occur, so a small decay loses nothing.  A block owns 32 columns of
// one head's state for one request, as in the token-by-token kernel; the state stays in shared memory between
// chunks.  A row's result differs from the token-by-token kernel's by rounding only.
constexpr int CHUNK = 32;
constexpr int CHUNK_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(CHUNK_THREADS) decay_scan_chunked_kernel(
    const T* __restrict__ rows, long long ld, const float* __restrict__ prepared, int v_off, int heads, int dim, int vdim,
    int activation, const float* __restrict__ decay, float* __restrict__ state, const int* __restrict__ slots,
    const int* __restrict__ q_start, float* __restrict__ out) {
  extern __shared__ __align__(16) float shared[];
  const int ldq = dim + 1;
  float* Qs = shared;                         // [CHUNK][dim + 1]
  float* Ks = Qs + CHUNK * ldq;               // [CHUNK][dim + 1]
  float* Vs = Ks + CHUNK * ldq;               // [CHUNK][32]
  float* Vd = Vs + CHUNK * 32;                // [CHUNK][32]   v_j * c^(n-1-j)
  float* As = Vd + CHUNK * 32;                // [CHUNK (j)][CHUNK + 1 (t)]   c^(t-j) q_t . k_j
  float* Ss = As + CHUNK * (CHUNK + 1);       // [dim][32]
  float* pw = Ss + dim * 32;                  // c^0 .. c^CHUNK
  const int tid = threadIdx.x;
  const int head = blockIdx.y, seq = blockIdx.z;
  const int column0 = blockIdx.x * 32;
  const int first = q_start[seq], last = q_start[seq + 1];
  if (first >= last) return;
  const int slot = slots[seq];
  const float c = decay[head];
  float* mine = state + (((size_t)slot * heads + head) * dim) * vdim;
  if (tid <= CHUNK) pw[tid] = (float)pow((double)c, (double)tid);      // each power rounded once
  for (int e = tid; e < dim * 32; e += CHUNK_THREADS) {
    const int i = e >> 5, col = column0 + (e & 31);
    Ss[e] = col < vdim ? mine[(size_t)i * vdim + col] : 0.0f;
  }
  const int t_of = tid >> 3, quad = (tid & 7) * 4;      // a thread's row (or row group) and its four columns
  for (int base = first; base < last; base += CHUNK) {
    const int n = min(CHUNK, last - base);
    __syncthreads();                                     // the powers and the state are there; the last chunk is done with Ks, Vd
    for (int e = tid; e < CHUNK * dim; e += CHUNK_THREADS) {
      const int t = e / dim, i = e - t * dim;
      float q = 0.0f, k = 0.0f;
      if (t < n) {
        const float* src = prepared + ((size_t)(base + t) * heads + head) * 2 * dim;
        q = src[i];
        k = src[dim + i];
      }
      Qs[t * ldq + i] = q;
      Ks[t * ldq + i] = k;
    }
    for (int e = tid; e < CHUNK * 32; e += CHUNK_THREADS) {
      const int t = e >> 5, col = column0 + (e & 31);
      float v = 0.0f;
      if (t < n && col < vdim) {
        v = to_float<T>(rows[(size_t)(base + t) * ld + v_off + head * vdim + col]);
        if (activation) v = silu_f(v);
      }
      Vs[e] = v;
      Vd[e] = t < n ? v * pw[n - 1 - t] : 0.0f;
    }
    __syncthreads();
    // scores of the chunk, decayed: row t, columns quad .. quad + 3, at or below the diagonal
    if (quad <= t_of) {
      float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
      const float* qrow = Qs + t_of * ldq;
      const float* krow = Ks + quad * ldq;
#pragma unroll 8
      for (int i = 0; i < dim; ++i) {
        const float q = qrow[i];
        a0 = fmaf(q, krow[i], a0);
        a1 = fmaf(q, krow[ldq + i], a1);
        a2 = fmaf(q, krow[2 * ldq + i], a2);
        a3 = fmaf(q, krow[3 * ldq + i], a3);
      }
      if (quad <= t_of) As[quad * (CHUNK + 1) + t_of] = a0 * pw[t_of - quad];
      if (quad + 1 <= t_of) As[(quad + 1) * (CHUNK + 1) + t_of] = a1 * pw[t_of - quad - 1];
      if (quad + 2 <= t_of) As[(quad + 2) * (CHUNK + 1) + t_of] = a2 * pw[t_of - quad - 2];
      if (quad + 3 <= t_of) As[(quad + 3) * (CHUNK + 1) + t_of] = a3 * pw[t_of - quad - 3];
    }
    __syncthreads();
    // readout: row t, four of the block's columns
    {
      float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
      const float* qrow = Qs + t_of * ldq;
#pragma unroll 8
      for (int i = 0; i < dim; ++i) {
        const float q = qrow[i];
        const float4 s4 = *reinterpret_cast<const float4*>(Ss + i * 32 + quad);
        o0 = fmaf(q, s4.x, o0); o1 = fmaf(q, s4.y, o1); o2 = fmaf(q, s4.z, o2); o3 = fmaf(q, s4.w, o3);
      }
      const float carried = pw[t_of + 1];
      o0 *= carried; o1 *= carried; o2 *= carried; o3 *= carried;
#pragma unroll 4
      for (int j = 0; j <= t_of; ++j) {
        const float a = As[j * (CHUNK + 1) + t_of];
        const float4 v4 = *reinterpret_cast<const float4*>(Vs + j * 32 + quad);
        o0 = fmaf(a, v4.x, o0); o1 = fmaf(a, v4.y, o1); o2 = fmaf(a, v4.z, o2); o3 = fmaf(a, v4.w, o3);
      }
      if (t_of < n) {
        float* dst = out + (size_t)(base + t_of) * heads * vdim + (size_t)head * vdim + column0 + quad;
        const int room = vdim - column0 - quad;
        if (room > 0) dst[0] = o0;
        if (room > 1) dst[1] = o1;
        if (room > 2) dst[2] = o2;
        if (room > 3) dst[3] = o3;
      }
    }
    __syncthreads();
    // state: rows t_of, t_of + 32, ... of the block's four columns
    {
      float acc[8][4];
#pragma unroll
      for (int r = 0; r < 8; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.0f;
#pragma unroll 2
      for (int j = 0; j < n; ++j) {
        const float4 v4 = *reinterpret_cast<const float4*>(Vd + j * 32 + quad);
        const float* krow = Ks + j * ldq + t_of;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          if (t_of + 32 * r < dim) {
            const float k = krow[32 * r];
            acc[r][0] = fmaf(k, v4.x, acc[r][0]); acc[r][1] = fmaf(k, v4.y, acc[r][1]);
            acc[r][2] = fmaf(k, v4.z, acc[r][2]); acc[r][3] = fmaf(k, v4.w, acc[r][3]);
          }
        }
      }
      const float kept = pw[n];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int i = t_of + 32 * r;
        if (i < dim) {
          float4* cell = reinterpret_cast<float4*>(Ss + i * 32 + quad);
          float4 s4 = *cell;
          s4.x = fmaf(kept, s4.x, acc[r][0]); s4.y = fmaf(kept, s4.y, acc[r][1]);
          s4.z = fmaf(kept, s4.z, acc[r][2]); s4.w = fmaf(kept, s4.w, acc[r][3]);
          *cell = s4;
        }
      }
    }
  }
  __syncthreads();
  for (int e = tid; e < dim * 32; e += CHUNK_THREADS) {
    const int i = e >> 5, col = column0 + (e & 31);
    if (col < vdim) mine[(size_t)i * vdim + col] = Ss[e];
  }
}

// The chunked kernel for keys of up to 128 elements: chunks of 64 tokens, 64 columns of the state per block, and
// every thread a 4 x 4 (state: 8 x 4) tile of each product's result, so that a pair of 16-byte reads from shared
// memory feeds sixteen multiply-adds.  q and k are kept transposed ([element][token]) for that.
constexpr int WIDE = 64;                 // tokens per chunk and columns per block
constexpr int WIDE_LD = WIDE + 4;        // row stride of the transposed tiles: 16-byte aligned
constexpr int SEGMENT = 256;             // tokens per segment when one portion is shared out over many blocks

__device__ __forceinline__ void copy16_async(float* dst_shared, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst_shared)), "l"(src));
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void copies_wait() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

// MODE 0: a block walks a request's whole portion from the state in its slot and leaves the new state there.
// One long prompt then keeps only heads x (vdim / 64) blocks busy, so such steps cut every portion into segments
// of `segment` tokens and run three launches: MODE 1 (a block per segment: the segment's own contribution to the
// state, from zero, into `carry[segment]`), `decay_segment_carry_kernel` (per request, in order: carry[k] <- the
// state the segment starts from, state <- c^len state + contribution; the last one goes to the slot), MODE 2 (a
// block per segment: the readout, from carry[segment]).  blockIdx.z counts segments over all requests of the step.
template <typename T, int MODE>
__global__ void __launch_bounds__(256) decay_scan_wide_kernel(
    const T* __restrict__ rows, long long ld, const float* __restrict__ prepared, int v_off, int heads, int dim, int vdim,
    int activation, const float* __restrict__ decay, float* __restrict__ state, const int* __restrict__ slots,
    const int* __restrict__ q_start, float* __restrict__ out, float* __restrict__ carry, int num_seqs, int segment) {
  extern __shared__ __align__(16) float shared[];
  float* Qt = shared;                         // [dim][WIDE_LD]   q, element-major
  float* Kt = Qt + dim * WIDE_LD;             // [dim][WIDE_LD]   k, element-major
  float* Vs = Kt + dim * WIDE_LD;             // [WIDE][WIDE]
  float* Vd = Vs + WIDE * WIDE;               // [WIDE][WIDE]     v_j * c^(n-1-j)
  float* As = Vd + WIDE * WIDE;               // [WIDE (j)][WIDE_LD (t)]   c^(t-j) q_t . k_j
  float* Ss = As + WIDE * WIDE_LD;            // [dim][WIDE]
  float* pw = Ss + dim * WIDE;                // c^0 .. c^WIDE
  float* stage = pw + WIDE + 4;               // [WIDE][2 dim]: the next chunk's q and k on their way in (dim % 4 == 0)
  const int tid = threadIdx.x;
  const int head = blockIdx.y;
  const int column0 = blockIdx.x * WIDE;
  int seq = -1, first = 0, last = 0;
  if (MODE == 0) {
    seq = blockIdx.z;
    first = q_start[seq];
    last = q_start[seq + 1];
  } else {
    int z = blockIdx.z;
    for (int s = 0; s < num_seqs; ++s) {
      const int begin = q_start[s], count = q_start[s + 1] - begin;
      const int pieces = (count + segment - 1) / segment;
      if (z < pieces) {
        seq = s;
        first = begin + z * segment;
        last = min(first + segment, begin + count);
        break;
      }
      z -= pieces;
    }
  }
  if (seq < 0 || first >= last) return;
  const float c = decay[head];
  // where the block's state comes from and goes to
  float* mine = MODE == 0 ? state + (((size_t)slots[seq] * heads + head) * dim) * vdim
                          : carry + (((size_t)blockIdx.z * heads + head) * dim) * vdim;
  // A chunk's q and k (prepared rows, 2 dim floats per token and head) are copied asynchronously into `stage` while
  // the chunk before is worked on, and its values wait in registers: the products never wait for memory.
  // 16-byte pieces of a row of 2 dim floats; the launch that only builds a segment's state needs the k half alone
  const int quads_per_token = MODE == 1 ? dim >> 2 : dim >> 1;
  const int quad_offset = MODE == 1 ? dim : 0;
  auto fetch_qk = [&](float* into, int from) {
    const int count = min(WIDE, last - from);
    for (int e = tid; e < count * quads_per_token; e += 256) {
      const int t = e / quads_per_token, piece = e - t * quads_per_token;
      copy16_async(into + (size_t)t * 2 * dim + quad_offset + 4 * piece,
                   prepared + ((size_t)(from + t) * heads + head) * 2 * dim + quad_offset + 4 * piece);
    }
    copies_commit();
  };
  // The state-only launch reads k where the copy put it: it needs neither q nor the transposed tiles, so their room
  // is a second staging buffer and the chunks alternate between the two.
  float* current = stage;
  float* other = MODE == 1 ? Qt : stage;
  float ahead[16];                            // the next chunk's values for this thread's places in Vs
  auto fetch_v = [&](int from) {
    const int count = min(WIDE, last - from);
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const int e = tid + 256 * k;
      const int t = e >> 6, col = column0 + (e & 63);
      ahead[k] = (t < count && col < vdim) ? to_float<T>(rows[(size_t)(from + t) * ld + v_off + head * vdim + col]) : 0.0f;
    }
  };
  fetch_qk(current, first);
  fetch_v(first);
  if (tid <= WIDE) pw[tid] = (float)pow((double)c, (double)tid);       // each power rounded once
  for (int e = tid; e < dim * WIDE; e += 256) {
    const int i = e >> 6, col = column0 + (e & 63);
    Ss[e] = (MODE != 1 && col < vdim) ? mine[(size_t)i * vdim + col] : 0.0f;
  }
  const int ty = tid >> 4, tx = tid & 15;
  const int t0 = ty * 4, c0 = tx * 4;                    // a thread's four rows (tokens) and four columns
  for (int base = first; base < last; base += WIDE) {
    const int n = min(WIDE, last - base);
    copies_wait();
    __syncthreads();                                     // the copies, the powers and the state are there; the last chunk is done with Kt, Vd
    if (MODE != 1) {
      for (int e = tid; e < WIDE * dim; e += 256) {
        const int t = e / dim, i = e - t * dim;
        const bool live = t < n;
        Qt[i * WIDE_LD + t] = live ? stage[(size_t)t * 2 * dim + i] : 0.0f;
        Kt[i * WIDE_LD + t] = live ? stage[(size_t)t * 2 * dim + dim + i] : 0.0f;
      }
    }
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const int e = tid + 256 * k;
      const int t = e >> 6;
      const float v = activation ? silu_f(ahead[k]) : ahead[k];
      Vs[e] = t < n ? v : 0.0f;
      Vd[e] = t < n ? v * pw[n - 1 - t] : 0.0f;
    }
    __syncthreads();
    if (base + WIDE < last) {
      fetch_qk(other, base + WIDE);
      fetch_v(base + WIDE);
    }
    // scores of the chunk, decayed: tokens t0 .. t0 + 3 against keys c0 .. c0 + 3, tiles at or below the diagonal
    if (MODE != 1 && c0 <= t0) {
      float acc[4][4] = {};
#pragma unroll 4
      for (int i = 0; i < dim; ++i) {
        const float4 q4 = *reinterpret_cast<const float4*>(Qt + i * WIDE_LD + t0);
        const float4 k4 = *reinterpret_cast<const float4*>(Kt + i * WIDE_LD + c0);
        const float qa[4] = {q4.x, q4.y, q4.z, q4.w}, kb[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(qa[a], kb[b], acc[a][b]);
      }
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int j = c0 + b;
        float4 cell;
        cell.x = j <= t0 ? acc[0][b] * pw[t0 - j] : 0.0f;
        cell.y = j <= t0 + 1 ? acc[1][b] * pw[t0 + 1 - j] : 0.0f;
        cell.z = j <= t0 + 2 ? acc[2][b] * pw[t0 + 2 - j] : 0.0f;
        cell.w = j <= t0 + 3 ? acc[3][b] * pw[t0 + 3 - j] : 0.0f;
        *reinterpret_cast<float4*>(As + j * WIDE_LD + t0) = cell;
      }
    }
    __syncthreads();
    // readout: tokens t0 .. t0 + 3, columns c0 .. c0 + 3 of the block
    if (MODE != 1) {
      float acc[4][4] = {};
#pragma unroll 4
      for (int i = 0; i < dim; ++i) {
        const float4 q4 = *reinterpret_cast<const float4*>(Qt + i * WIDE_LD + t0);
        const float4 s4 = *reinterpret_cast<const float4*>(Ss + i * WIDE + c0);
        const float qa[4] = {q4.x, q4.y, q4.z, q4.w}, sb[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(qa[a], sb[b], acc[a][b]);
      }
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const float carried = pw[t0 + a + 1];
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] *= carried;
      }
      const int reach = min(t0 + 3, n - 1);
#pragma unroll 4
      for (int j = 0; j <= reach; ++j) {
        const float4 a4 = *reinterpret_cast<const float4*>(As + j * WIDE_LD + t0);
        const float4 v4 = *reinterpret_cast<const float4*>(Vs + j * WIDE + c0);
        const float aa[4] = {a4.x, a4.y, a4.z, a4.w}, vb[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(aa[a], vb[b], acc[a][b]);
      }
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        if (t0 + a < n) {
          float* dst = out + (size_t)(base + t0 + a) * heads * vdim + (size_t)head * vdim + column0 + c0;
          const int room = vdim - column0 - c0;
#pragma unroll
          for (int b = 0; b < 4; ++b)
            if (b < room) dst[b] = acc[a][b];
        }
      }
    }
    __syncthreads();
    // state: rows 8 ty .. 8 ty + 7, columns c0 .. c0 + 3 (nobody reads it after a segment's last readout)
    if (MODE != 2 || base + WIDE < last) {
      float acc[8][4] = {};
      const int i0 = ty * 8;
#pragma unroll 2
      for (int j = 0; j < n; ++j) {
        const float4 v4 = *reinterpret_cast<const float4*>(Vd + j * WIDE + c0);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          if (i0 + r < dim) {
            const float k = MODE == 1 ? current[(size_t)j * 2 * dim + dim + i0 + r] : Kt[(i0 + r) * WIDE_LD + j];
            acc[r][0] = fmaf(k, v4.x, acc[r][0]); acc[r][1] = fmaf(k, v4.y, acc[r][1]);
            acc[r][2] = fmaf(k, v4.z, acc[r][2]); acc[r][3] = fmaf(k, v4.w, acc[r][3]);
          }
        }
      }
      const float kept = pw[n];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (i0 + r < dim) {
          float4* cell = reinterpret_cast<float4*>(Ss + (i0 + r) * WIDE + c0);
          float4 s4 = *cell;
          s4.x = fmaf(kept, s4.x, acc[r][0]); s4.y = fmaf(kept, s4.y, acc[r][1]);
          s4.z = fmaf(kept, s4.z, acc[r][2]); s4.w = fmaf(kept, s4.w, acc[r][3]);
          *cell = s4;
        }
      }
    }
    if (MODE == 1) {
      float* swap = current;
      current = other;
      other = swap;
    }
  }
  __syncthreads();
  if (MODE != 2) {
    for (int e = tid; e < dim * WIDE; e += 256) {
      const int i = e >> 6, col = column0 + (e & 63);
      if (col < vdim) mine[(size_t)i * vdim + col] = Ss[e];
    }
  }
}

// Between the two segment launches: every request's segments in order.  carry[k] holds segment k's own contribution
// on the way in and the state it starts from on the way out; the request's slot gets the state after its last one.
__global__ void decay_segment_carry_kernel(float* __restrict__ carry, float* __restrict__ state, const float* __restrict__ decay,
                                           const int* __restrict__ slots, const int* __restrict__ q_start, int heads,
                                           int dim, int vdim, int segment) {
  const int seq = blockIdx.z, head = blockIdx.y;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  const int cells = dim * vdim;
  if (e >= cells) return;
  int before = 0;
  for (int s = 0; s < seq; ++s) before += (q_start[s + 1] - q_start[s] + segment - 1) / segment;
  const int count = q_start[seq + 1] - q_start[seq];
  if (count <= 0) return;
  const int pieces = (count + segment - 1) / segment;
  const double c = (double)decay[head];
  float* slot = state + ((size_t)slots[seq] * heads + head) * cells + e;
  float running = *slot;
  const float whole = (float)pow(c, (double)segment);                 // every segment but a request's last is whole
  for (int k0 = 0; k0 < pieces; k0 += 16) {
    // sixteen segments' contributions are asked for at once; the stores that follow would otherwise keep each
    // load behind the one before
    float own[16];
#pragma unroll
    for (int k = 0; k < 16; ++k)
      own[k] = k0 + k < pieces ? carry[((size_t)(before + k0 + k) * heads + head) * cells + e] : 0.0f;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      if (k0 + k < pieces) {
        carry[((size_t)(before + k0 + k) * heads + head) * cells + e] = running;
        const int length = min(segment, count - (k0 + k) * segment);
        running = fmaf(length == segment ? whole : (float)pow(c, (double)length), running, own[k]);
      }
    }
  }
  *slot = running;
}

// out[t, g*size + e] = o[t, g*size + e] / rms_g(o[t]) * weight[g*size + e] * act(gate[t, g*size + e]); one warp per
// (token, group).  weight may be null (no weight); act 0: silu, 1: sigmoid; act 2: the SiLU gate comes BEFORE the norm,
// out = y / rms_g(y) * weight with y = o * silu(gate).
template <typename T, typename TO = T>
__global__ void __launch_bounds__(128) gated_norm_kernel(const float* __restrict__ o, const T* __restrict__ gate,
                                                         long long ld_gate, const float* __restrict__ weight,
                                                         TO* __restrict__ out, long long ld_out, int tokens, int groups,
                                                         int size, float eps, int act) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (unit >= (long long)tokens * groups) return;
  const int t = (int)(unit / groups), g = (int)(unit - (long long)t * groups);
  const float* src = o + ((size_t)t * groups + g) * size;
  const T* gt = gate + (size_t)t * ld_gate + (size_t)g * size;
  TO* dst = out + (size_t)t * ld_out + (size_t)g * size;
  float sum = 0.0f;
  if (act == 2) {
    for (int e = lane; e < size; e += 32) {
      const float y = src[e] * silu_f(to_float<T>(gt[e]));
      sum = fmaf(y, y, sum);
    }
    const float scale = 1.0f / sqrtf(warp_sum(sum) / (float)size + eps);
    for (int e = lane; e < size; e += 32) {
      const float w = weight != nullptr ? weight[(size_t)g * size + e] : 1.0f;
      dst[e] = from_float<TO>(src[e] * silu_f(to_float<T>(gt[e])) * scale * w);
    }
    return;
  }
  for (int e = lane; e < size; e += 32) sum = fmaf(src[e], src[e], sum);
  sum = warp_sum(sum);
  const float scale = 1.0f / sqrtf(sum / (float)size + eps);
  for (int e = lane; e < size; e += 32) {
    const float z = to_float<T>(gt[e]);
    const float w = weight != nullptr ? weight[(size_t)g * size + e] : 1.0f;
    dst[e] = from_float<TO>(src[e] * scale * w * (act == 0 ? silu_f(z) : sigmoid_f(z)));
  }
}

// ---------------------------------------------------------------------------------------------------------
// After the q/k/v product: the short convolution over time, the per-head norm of q and k, their rotation, and the
// store.  One warp per (token, head of q, k or v).  `raw` holds the projections of this step's tokens [T, q | k | v];
// inputs from before the portion come from the request's convolution state [slots, taps-1, channels] (oldest first),
// which is zero for a request that starts.  q goes to `q_out`, k and v into their pages.
constexpr int CNR_PER_LANE = 8;    // head sizes up to 256
constexpr int MAX_TAPS = 16;

template <typename T>
__global__ void __launch_bounds__(128) conv_norm_rope_store_kernel(
    const T* __restrict__ raw, long long ld, const float* __restrict__ conv_w, int taps,
    const float* __restrict__ conv_state, const int* __restrict__ slots, const int* __restrict__ q_start,
    const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, int table_positions, int rotary,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
    int max_pages, T* __restrict__ k_pages, T* __restrict__ v_pages, int num_pages, int page_size,
    T* __restrict__ q_out, long long ld_q, int heads, int kv_heads, int dim, int vdim, int store, int* status) {
  pdl_trigger();
  pdl_wait();
  __shared__ float staged[4][32 * CNR_PER_LANE];
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int unit = blockIdx.y * 4 + warp;
  if (unit >= heads + 2 * kv_heads) return;
  const int kind = unit < heads ? 0 : (unit < heads + kv_heads ? 1 : 2);        // q, k, v
  const int head = kind == 0 ? unit : (kind == 1 ? unit - heads : unit - heads - kv_heads);
  const int size = kind == 2 ? vdim : dim;
  const int channels = (heads + kv_heads) * dim + kv_heads * vdim;
  const int channel0 = kind == 0 ? head * dim : (kind == 1 ? (heads + head) * dim : (heads + kv_heads) * dim + head * vdim);
  const int seq = seq_of_token[t];
  const int local = t - q_start[seq];                     // this token's index in its portion
  const int slot = slots[seq];
  float y[CNR_PER_LANE];
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < CNR_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    float value = 0.0f;
    if (e < size) {
      const int c = channel0 + e;
      if (taps <= 0) {
        value = to_float<T>(raw[(size_t)t * ld + c]);
      } else {
        for (int j = 0; j < taps; ++j) {
          const int back = taps - 1 - j;                  // how many tokens before this one
          float u;
          if (local - back >= 0) u = to_float<T>(raw[(size_t)(t - back) * ld + c]);
          else u = conv_state[((size_t)slot * (taps - 1) + (taps - 1 + local - back)) * channels + c];
          value = fmaf(conv_w[(size_t)c * taps + j], u, value);
        }
      }
    }
    y[i] = value;
    sum = fmaf(value, value, sum);
  }
  const float* norm_w = kind == 0 ? q_norm : (kind == 1 ? k_norm : nullptr);
  if (norm_w != nullptr) {
    sum = warp_sum(sum);
    const float scale = 1.0f / sqrtf(sum / (float)size + eps);
#pragma unroll
    for (int i = 0; i < CNR_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < size) y[i] = y[i] * scale * norm_w[e];
    }
  }
  int position = positions[t];
  if (kind != 2 && rotary > 0) {
    const int half = rotary >> 1;
    int at = position;
    if (at < 0 || at >= table_positions) {
      if (lane == 0) atomicOr(status, TGE_STATUS_BAD_ROW);
      at = 0;
    }
#pragma unroll
    for (int i = 0; i < CNR_PER_LANE; ++i) staged[warp][lane + 32 * i] = y[i];
    __syncwarp();
#pragma unroll
    for (int i = 0; i < CNR_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < rotary && e < size) {
        const int pair = e < half ? e : e - half;
        const float cs = cos_table[(size_t)at * half + pair], sn = sin_table[(size_t)at * half + pair];
        const float other = staged[warp][e < half ? e + half : e - half];
        y[i] = e < half ? y[i] * cs - other * sn : y[i] * cs + other * sn;
      }
    }
  }
  if (kind == 0) {
    T* dst = q_out + (size_t)t * ld_q + (size_t)head * dim;
#pragma unroll
    for (int i = 0; i < CNR_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < size) dst[e] = from_float<T>(y[i]);
    }
    return;
  }
  if (!store) return;
  const int page_index = position / page_size;
  const int page = (position >= 0 && page_index < max_pages) ? block_table[(size_t)seq * max_pages + page_index] : -1;
  if (page < 0 || page >= num_pages) {
    if (lane == 0) atomicOr(status, TGE_STATUS_BAD_PAGE);
    return;
  }
  T* dst = (kind == 1 ? k_pages : v_pages) + (((size_t)page * kv_heads + head) * page_size + position % page_size) * size;
#pragma unroll
  for (int i = 0; i < CNR_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    if (e < size) dst[e] = from_float<T>(y[i]);
  }
}

// The convolution state after the step: the last taps-1 projected rows of each request, oldest first.  One thread
// per (request, channel) reads what it needs before it writes, so a portion shorter than the state shifts it.
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ raw, long long ld, float* __restrict__ conv_state,
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
  float* mine = conv_state + (size_t)slots[seq] * keep * channels + c;
  float old[MAX_TAPS];
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) old[j] = j < keep ? mine[(size_t)j * channels] : 0.0f;
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) {
    if (j < keep) {
      const int at = n + j;                                // in (old state, then this step's rows)
      mine[(size_t)j * channels] = at < keep ? old[at] : to_float<T>(raw[(size_t)(first + at - keep) * ld + c]);
    }
  }
}

// The mean key and mean value of every block of `pool` positions whose last token this step brings: one block of
// threads per (token, kv head); only tokens at a block's last position do anything.  The means are taken over the
// keys and values as their pages hold them, and entry b of a request lies where position b would in the pooled pages.
template <typename T>
__global__ void __launch_bounds__(128) pool_kv_kernel(
    const T* __restrict__ k_pages, const T* __restrict__ v_pages, const int* __restrict__ block_table, int max_pages,
    int num_pages, T* __restrict__ kp_pages, T* __restrict__ vp_pages, const int* __restrict__ pool_table,
    int pool_max_pages, int pool_num_pages, int page_size, const int* __restrict__ positions,
    const int* __restrict__ seq_of_token, int kv_heads, int dim, int vdim, int pool, int* status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, head = blockIdx.y;
  const int position = positions[t];
  if (position < 0 || (position + 1) % pool != 0) return;
  const int seq = seq_of_token[t];
  const int entry = (position + 1) / pool - 1;
  const int entry_page = entry / page_size;
  const int out_page = entry_page < pool_max_pages ? pool_table[(size_t)seq * pool_max_pages + entry_page] : -1;
  if (out_page < 0 || out_page >= pool_num_pages) {
    if (threadIdx.x == 0) atomicOr(status, TGE_STATUS_BAD_PAGE);
    return;
  }
  for (int e = threadIdx.x; e < dim + vdim; e += blockDim.x) {
    const bool is_key = e < dim;
    const int size = is_key ? dim : vdim, d = is_key ? e : e - dim;
    const T* pages = is_key ? k_pages : v_pages;
    float sum = 0.0f;
    bool ok = true;
    for (int p = position - pool + 1; p <= position; ++p) {
      const int page_index = p / page_size;
      const int page = page_index < max_pages ? block_table[(size_t)seq * max_pages + page_index] : -1;
      if (page < 0 || page >= num_pages) { ok = false; break; }
      sum += to_float<T>(pages[(((size_t)page * kv_heads + head) * page_size + p % page_size) * size + d]);
    }
    if (!ok) {
      atomicOr(status, TGE_STATUS_BAD_PAGE);
      continue;
    }
    T* dst = (is_key ? kp_pages : vp_pages) + (((size_t)out_page * kv_heads + head) * page_size + entry % page_size) * size + d;
    *dst = from_float<T>(sum / (float)pool);
  }
}

template <typename T>
int launch_decay_scan(const void* rows, long long ld, int q_off, int k_off, int v_off, int heads, int dim, int vdim,
                      int activation, const float* cos_table, const float* sin_table, int table_positions, int rotary,
                      float k_scale, const float* decay, float* state, const int* slots, const int* q_start,
                      const int* positions, float* out, int num_seqs, int tokens, int max_q_len, float* prepared, float* carry, int* status,
                      cudaStream_t stream) {
  dim3 grid((vdim + 31) / 32, heads, num_seqs);
  // portions of some length go chunk by chunk; single tokens and short portions token by token
  const size_t chunked = (size_t)(2 * CHUNK * (dim + 1) + 2 * CHUNK * 32 + CHUNK * (CHUNK + 1) + dim * 32 + CHUNK + 1 + 3) * sizeof(float);
  static const bool chunks_ok = getenv("TGE_NO_CHUNKED_SCAN") == nullptr || getenv("TGE_NO_CHUNKED_SCAN")[0] == '\0';
  const size_t wide = (size_t)(2 * dim * WIDE_LD + 2 * WIDE * WIDE + WIDE * WIDE_LD + dim * WIDE + WIDE + 4 + WIDE * 2 * dim) * sizeof(float);
  if (chunks_ok && prepared != nullptr && max_q_len >= WIDE && dim <= 128 && dim % 4 == 0 && wide <= 227 * 1024) {
    static size_t configured[2] = {0, 0};
    const int which = sizeof(T) == 2 ? 1 : 0;
    if (wide > configured[which]) {
      cudaError_t err = cudaFuncSetAttribute(decay_scan_wide_kernel<T, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)wide);
      if (err == cudaSuccess)
        err = cudaFuncSetAttribute(decay_scan_wide_kernel<T, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)wide);
      if (err == cudaSuccess)
        err = cudaFuncSetAttribute(decay_scan_wide_kernel<T, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)wide);
      if (err != cudaSuccess) {
        tge_set_error("decay_scan: cannot reserve %zu bytes of shared memory: %s", wide, cudaGetErrorString(err));
        return -2;
      }
      configured[which] = wide;
    }
    dim3 wide_grid((vdim + WIDE - 1) / WIDE, heads, num_seqs);
    decay_prepare_kernel<T><<<dim3(tokens, heads), 128, 0, stream>>>((const T*)rows, ld, q_off, k_off, heads, dim, activation,
                                                                     cos_table, sin_table, table_positions, rotary, k_scale,
                                                                     positions, prepared, status);
    // few blocks and long portions: segments, so that the whole device works on one prompt
    const long long blocks = (long long)wide_grid.x * heads * num_seqs;
    if (carry != nullptr && max_q_len >= 2 * SEGMENT && blocks < 2LL * tge_sm_count() && tokens / SEGMENT + num_seqs <= 65535) {
      dim3 pieces(wide_grid.x, heads, tokens / SEGMENT + num_seqs);      // an upper bound; blocks beyond the last segment leave at once
      decay_scan_wide_kernel<T, 1><<<pieces, 256, wide, stream>>>((const T*)rows, ld, prepared, v_off, heads, dim, vdim, activation,
                                                                  decay, state, slots, q_start, out, carry, num_seqs, SEGMENT);
      decay_segment_carry_kernel<<<dim3((dim * vdim + 255) / 256, heads, num_seqs), 256, 0, stream>>>(
          carry, state, decay, slots, q_start, heads, dim, vdim, SEGMENT);
      decay_scan_wide_kernel<T, 2><<<pieces, 256, wide, stream>>>((const T*)rows, ld, prepared, v_off, heads, dim, vdim, activation,
                                                                  decay, state, slots, q_start, out, carry, num_seqs, SEGMENT);
      return tge_launched("decay_scan_segments", 4);
    }
    decay_scan_wide_kernel<T, 0><<<wide_grid, 256, wide, stream>>>((const T*)rows, ld, prepared, v_off, heads, dim, vdim,
                                                                   activation, decay, state, slots, q_start, out, nullptr, num_seqs, 0);
    return tge_launched("decay_scan_wide", 2);
  }
  if (chunks_ok && prepared != nullptr && max_q_len >= CHUNK / 2 && dim <= 256 && chunked <= 200 * 1024) {
    static size_t configured[2] = {0, 0};
    const int which = sizeof(T) == 2 ? 1 : 0;
    if (chunked > 48 * 1024 && chunked > configured[which]) {
      cudaError_t err = cudaFuncSetAttribute(decay_scan_chunked_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)chunked);
      if (err != cudaSuccess) {
        tge_set_error("decay_scan: cannot reserve %zu bytes of shared memory: %s", chunked, cudaGetErrorString(err));
        return -2;
      }
      configured[which] = chunked;
    }
    decay_prepare_kernel<T><<<dim3(tokens, heads), 128, 0, stream>>>((const T*)rows, ld, q_off, k_off, heads, dim, activation,
                                                                     cos_table, sin_table, table_positions, rotary, k_scale,
                                                                     positions, prepared, status);
    decay_scan_chunked_kernel<T><<<grid, CHUNK_THREADS, chunked, stream>>>((const T*)rows, ld, prepared, v_off, heads, dim, vdim,
                                                                          activation, decay, state, slots, q_start, out);
    return tge_launched("decay_scan_chunked", 2);
  }
  const int per_warp = (dim + SCAN_WARPS - 1) / SCAN_WARPS;
#define TGE_SCAN(ROWS, TOKENS)                                                                                    \
  tge_launch(decay_scan_kernel<T, ROWS, TOKENS>, grid, dim3(SCAN_WARPS * 32),                                     \
             (size_t)(2 * TOKENS * dim + SCAN_WARPS * TOKENS * 32) * sizeof(float), stream, (const T*)rows, ld, q_off, \
             k_off, v_off, heads, dim, vdim, activation, cos_table, sin_table, table_positions, rotary, k_scale, decay, \
             state, slots, q_start, positions, out, status)
#define TGE_SCAN_ROWS(TOKENS)                  \
  do {                                         \
    if (per_warp <= 8) TGE_SCAN(8, TOKENS);    \
    else if (per_warp <= 16) TGE_SCAN(16, TOKENS); \
    else if (per_warp <= 32) TGE_SCAN(32, TOKENS); \
    else TGE_SCAN(64, TOKENS);                 \
  } while (0)
  // a step of single tokens walks one token per request: the kernel without the eight-token round needs far
  // fewer registers, so more blocks share an SM while they wait for their state
  if (max_q_len <= 1) TGE_SCAN_ROWS(1);
  else TGE_SCAN_ROWS(SCAN_TOKENS);
#undef TGE_SCAN_ROWS
#undef TGE_SCAN
  return tge_launched("decay_scan", 1);
}

}  // namespace

TGE_API int tge_to_run_dtype(const float* x, void* out, int is_bf16, long long count, cudaStream_t stream) {
  TGE_REQUIRE(count >= 0, "to_run_dtype: negative count");
  if (count == 0) return 0;
  const unsigned blocks = (unsigned)((count + 255) / 256);
  if (is_bf16) to_run_dtype_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(x, (__nv_bfloat16*)out, (size_t)count);
  else to_run_dtype_kernel<float><<<blocks, 256, 0, stream>>>(x, (float*)out, (size_t)count);
  return tge_launched("to_run_dtype", 1);
}

TGE_API int tge_scale_add_norm(float* x, const float* y, long long ldy, const float* weight, void* copy, int copy_is_bf16,
                               int rows, int hidden, float alpha, float eps, cudaStream_t stream) {
  TGE_REQUIRE(rows >= 0 && hidden > 0 && ldy >= hidden, "scale_add_norm: bad shape (%d rows of %d)", rows, hidden);
  TGE_REQUIRE(eps > 0.0f, "scale_add_norm: eps must be positive");
  if (rows == 0) return 0;
  const bool aligned = hidden % 4 == 0 && ldy % 4 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)y % 16 == 0) &&
                       ((uintptr_t)weight % 16 == 0) && ((uintptr_t)copy % 8 == 0);
  if (aligned && hidden <= 16 * 1024) {
    int threads = ((hidden / 4 + 3) / 4 + 31) / 32 * 32;
    threads = threads < 32 ? 32 : threads;
    if (copy != nullptr && copy_is_bf16)
      tge_launch(scale_add_norm_vec_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, x, y, ldy, weight,
                 (__nv_bfloat16*)copy, hidden, alpha, eps);
    else
      tge_launch(scale_add_norm_vec_kernel<float>, dim3(rows), dim3(threads), 0, stream, x, y, ldy, weight, (float*)copy,
                 hidden, alpha, eps);
    return tge_launched("scale_add_norm", 1);
  }
  if (copy != nullptr && copy_is_bf16)
    scale_add_norm_kernel<__nv_bfloat16><<<rows, 256, 0, stream>>>(x, y, ldy, weight, (__nv_bfloat16*)copy, hidden, alpha, eps);
  else
    scale_add_norm_kernel<float><<<rows, 256, 0, stream>>>(x, y, ldy, weight, (float*)copy, hidden, alpha, eps);
  return tge_launched("scale_add_norm", 1);
}

TGE_API int tge_decay_scan(const void* rows, int is_bf16, long long ld, int q_off, int k_off, int v_off, int heads,
                           int dim, int vdim, int activation, const float* cos_table, const float* sin_table,
                           int table_positions, int rotary, float k_scale, const float* decay, float* state,
                           const int* slots, const int* q_start, const int* positions, float* out, int num_seqs,
                           int tokens, int max_q_len, float* prepared, float* carry, int* status, cudaStream_t stream) {
  TGE_REQUIRE(heads > 0 && dim > 0 && vdim > 0 && dim <= 64 * SCAN_WARPS, "decay_scan: %d heads of %d x %d (keys up to %d)",
              heads, dim, vdim, 64 * SCAN_WARPS);
  TGE_REQUIRE(rotary >= 0 && rotary % 2 == 0 && rotary <= dim, "decay_scan: %d rotated elements of %d", rotary, dim);
  TGE_REQUIRE(rotary == 0 || (cos_table != nullptr && sin_table != nullptr && table_positions > 0),
              "decay_scan: a rotation needs its tables");
  TGE_REQUIRE(num_seqs >= 0 && num_seqs <= 65535 && heads <= 65535, "decay_scan: %d requests in a step", num_seqs);
  if (num_seqs == 0 || tokens == 0) return 0;
  if (is_bf16)
    return launch_decay_scan<__nv_bfloat16>(rows, ld, q_off, k_off, v_off, heads, dim, vdim, activation, cos_table,
                                            sin_table, table_positions, rotary, k_scale, decay, state, slots, q_start,
                                            positions, out, num_seqs, tokens, max_q_len, prepared, carry, status, stream);
  return launch_decay_scan<float>(rows, ld, q_off, k_off, v_off, heads, dim, vdim, activation, cos_table, sin_table,
                                  table_positions, rotary, k_scale, decay, state, slots, q_start, positions, out, num_seqs,
                                  tokens, max_q_len, prepared, carry, status, stream);
}

TGE_API int tge_gated_norm(const float* o, const void* gate, int is_bf16, long long ld_gate, const float* weight, void* out,
                           long long ld_out, int tokens, int groups, int size, float eps, int act, int out_is_bf16,
                           cudaStream_t stream) {
  // the gate may arrive in float32 (a product that stored it so) while the rows go on in bfloat16
  TGE_REQUIRE(out_is_bf16 == is_bf16 || (!is_bf16 && out_is_bf16), "gated_norm: a bfloat16 gate goes with bfloat16 rows");
  TGE_REQUIRE(tokens >= 0 && groups > 0 && size > 0, "gated_norm: bad shape");
  TGE_REQUIRE(act >= 0 && act <= 2, "gated_norm: the gate is silu (0), sigmoid (1) or silu before the norm (2)");
  if (tokens == 0) return 0;
  const long long units = (long long)tokens * groups;
  const unsigned blocks = (unsigned)((units + 3) / 4);
  if (!is_bf16 && out_is_bf16)
    tge_launch(gated_norm_kernel<float, __nv_bfloat16>, dim3(blocks), dim3(128), 0, stream, o, (const float*)gate, ld_gate, weight,
               (__nv_bfloat16*)out, ld_out, tokens, groups, size, eps, act);
  else if (is_bf16)
    tge_launch(gated_norm_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), 0, stream, o, (const __nv_bfloat16*)gate, ld_gate,
               weight, (__nv_bfloat16*)out, ld_out, tokens, groups, size, eps, act);
  else
    tge_launch(gated_norm_kernel<float>, dim3(blocks), dim3(128), 0, stream, o, (const float*)gate, ld_gate, weight,
               (float*)out, ld_out, tokens, groups, size, eps, act);
  return tge_launched("gated_norm", 1);
}

TGE_API int tge_conv_norm_rope_store(const void* raw, int is_bf16, long long ld, const float* conv_w, int taps,
                                     float* conv_state, const int* slots, const int* q_start, const float* q_norm,
                                     const float* k_norm, float eps, const float* cos_table, const float* sin_table,
                                     int table_positions, int rotary, const int* positions, const int* seq_of_token,
                                     const int* block_table, int max_pages, void* k_pages, void* v_pages, int num_pages,
                                     int page_size, void* q_out, long long ld_q, int tokens, int num_seqs, int heads,
                                     int kv_heads, int dim, int vdim, int store, int* status, cudaStream_t stream) {
  TGE_REQUIRE(heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 && dim <= 32 * CNR_PER_LANE && vdim <= 32 * CNR_PER_LANE,
              "conv_norm_rope_store: head sizes %d and %d outside (0, %d]", dim, vdim, 32 * CNR_PER_LANE);
  TGE_REQUIRE(taps >= 0 && taps <= MAX_TAPS, "conv_norm_rope_store: %d taps (at most %d)", taps, MAX_TAPS);
  TGE_REQUIRE(taps <= 1 || conv_state != nullptr, "conv_norm_rope_store: a convolution needs its state");
  TGE_REQUIRE(taps == 0 || conv_w != nullptr, "conv_norm_rope_store: a convolution needs its weights");
  TGE_REQUIRE(rotary >= 0 && rotary % 2 == 0 && rotary <= dim, "conv_norm_rope_store: %d rotated elements of %d", rotary, dim);
  TGE_REQUIRE(rotary == 0 || (cos_table != nullptr && sin_table != nullptr && table_positions > 0),
              "conv_norm_rope_store: a rotation needs its tables");
  TGE_REQUIRE(!store || (page_size > 0 && max_pages > 0 && num_pages > 0), "conv_norm_rope_store: bad page geometry");
  if (tokens == 0) return 0;
  const int units = heads + 2 * kv_heads;
  const int channels = (heads + kv_heads) * dim + kv_heads * vdim;
  dim3 grid(tokens, (units + 3) / 4);
  int launched = 1;
  if (is_bf16) {
    tge_launch(conv_norm_rope_store_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream,
        (const __nv_bfloat16*)raw, ld, conv_w, taps, conv_state, slots, q_start, q_norm, k_norm, eps, cos_table, sin_table,
        table_positions, rotary, positions, seq_of_token, block_table, max_pages, (__nv_bfloat16*)k_pages,
        (__nv_bfloat16*)v_pages, num_pages, page_size, (__nv_bfloat16*)q_out, ld_q, heads, kv_heads, dim, vdim, store, status);
  } else {
    tge_launch(conv_norm_rope_store_kernel<float>, grid, dim3(128), 0, stream,
        (const float*)raw, ld, conv_w, taps, conv_state, slots, q_start, q_norm, k_norm, eps, cos_table, sin_table,
        table_positions, rotary, positions, seq_of_token, block_table, max_pages, (float*)k_pages, (float*)v_pages,
        num_pages, page_size, (float*)q_out, ld_q, heads, kv_heads, dim, vdim, store, status);
  }
  if (int rc = tge_check_launch("conv_norm_rope_store")) return rc;
  if (taps > 1) {
    // in stream order behind the kernel that read the old state
    dim3 update((channels + 127) / 128, num_seqs);
    if (is_bf16)
      tge_launch(conv_state_update_kernel<__nv_bfloat16>, update, dim3(128), 0, stream, (const __nv_bfloat16*)raw, ld,
                 conv_state, slots, q_start, taps, channels);
    else
      tge_launch(conv_state_update_kernel<float>, update, dim3(128), 0, stream, (const float*)raw, ld, conv_state, slots,
                 q_start, taps, channels);
    ++launched;
  }
  return tge_launched("conv_state_update", launched);
}

TGE_API int tge_pool_kv(const void* k_pages, const void* v_pages, int is_bf16, const int* block_table, int max_pages,
                        int num_pages, void* kp_pages, void* vp_pages, const int* pool_table, int pool_max_pages,
                        int pool_num_pages, int page_size, const int* positions, const int* seq_of_token, int tokens,
                        int kv_heads, int dim, int vdim, int pool, int* status, cudaStream_t stream) {
  TGE_REQUIRE(pool > 0 && kv_heads > 0 && dim > 0 && vdim > 0 && page_size > 0, "pool_kv: bad shape");
  if (tokens == 0) return 0;
  dim3 grid(tokens, kv_heads);
  if (is_bf16)
    tge_launch(pool_kv_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream,
        (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table, max_pages, num_pages,
        (__nv_bfloat16*)kp_pages, (__nv_bfloat16*)vp_pages, pool_table, pool_max_pages, pool_num_pages, page_size, positions,
        seq_of_token, kv_heads, dim, vdim, pool, status);
  else
    tge_launch(pool_kv_kernel<float>, grid, dim3(128), 0, stream, (const float*)k_pages, (const float*)v_pages, block_table, max_pages,
                                                     num_pages, (float*)kp_pages, (float*)vp_pages, pool_table,
                                                     pool_max_pages, pool_num_pages, page_size, positions, seq_of_token,
                                                     kv_heads, dim, vdim, pool, status);
  return tge_launched("pool_kv", 1);
}
