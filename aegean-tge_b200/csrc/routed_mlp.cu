// Kernels of a routed feed-forward (a mixture of small experts) and of activations that stand alone.
//
//  * router_topk      - from float32 router logits: softmax over all outputs, the choice by score + correction inside
//                       the best groups of neighbouring outputs, the chosen outputs' plain scores over their sum.
//  * activation       - relu(z)^2, or the two-parameter form z > 0: softplus(p) z^2 + z/2, else
//                       (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2, in place on rows of the run dtype.
//  * expert_up / expert_down_add - few tokens (a decode step): every (token, chosen expert) pair reads its expert's
//                       rows directly, one warp per output, and the weighted outputs are added into the float32 stream
//                       in the order of the choice; outputs beyond the experts are identity experts (the input itself).
//  * expert_dense_weigh - a step of some tokens that between them choose most experts anyway: every token goes through
//                       every expert's up matrix in ONE product, this kernel weighs the chosen experts' activated rows
//                       and zeroes the others, and ONE product with all down matrices side by side adds the sum.
//  * expert_sort / expert_gather / expert_combine_add - many tokens: the pairs are grouped by expert so that each
//                       expert's rows form one block of a buffer, which ordinary products then multiply; the last
//                       kernel adds the weighted rows back into the stream, again in the order of the choice.
//
// The router, the weights, every accumulation and the sum into the stream are float32.
#include <limits.h>

#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_f(float z) { return log1pf(expf(-fabsf(z))) + fmaxf(z, 0.0f); }

// The largest value of `values[0..n)` and its index (the lowest index among equals), found by a whole warp.
__device__ __forceinline__ void warp_argmax(const float* values, int n, int lane, float& best, int& where) {
  best = -INFINITY;
  where = INT_MAX;
  for (int i = lane; i < n; i += 32) {
    const float v = values[i];
    if (v > best || (v == best && i < where)) { best = v; where = i; }
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, best, offset);
    const int other_where = __shfl_xor_sync(0xffffffffu, where, offset);
    if (other > best || (other == best && other_where < where)) { best = other; where = other_where; }
  }
}

// One warp per token.  Shared memory per warp: 4 arrays of `outputs` floats (scores, choice values, group maxima,
// kept flags).
__global__ void __launch_bounds__(128) router_topk_kernel(const float* __restrict__ logits, long long ld,
                                                          const float* __restrict__ correction, int tokens, int outputs,
                                                          int top, int group_count, int group_keep, int* __restrict__ ids,
                                                          float* __restrict__ weights) {
  extern __shared__ float router_smem[];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= tokens) return;
  float* score = router_smem + (size_t)warp * 4 * outputs;
  float* choice = score + outputs;
  float* group_best = choice + outputs;
  float* kept = group_best + outputs;
  const float* z = logits + (size_t)t * ld;
  float m = -INFINITY;
  for (int i = lane; i < outputs; i += 32) m = fmaxf(m, z[i]);
  m = warp_max(m);
  float sum = 0.0f;
  for (int i = lane; i < outputs; i += 32) {
    const float e = expf(z[i] - m);
    score[i] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  const float inv = 1.0f / sum;
  for (int i = lane; i < outputs; i += 32) {
    const float s = score[i] * inv;
    score[i] = s;
    choice[i] = s + (correction != nullptr ? correction[i] : 0.0f);
  }
  __syncwarp();
  if (group_count > 1 && group_keep < group_count) {
    const int per = outputs / group_count;
    for (int g = 0; g < group_count; ++g) {
      float best = -INFINITY;
      for (int i = lane; i < per; i += 32) best = fmaxf(best, choice[g * per + i]);
      best = warp_max(best);
      if (lane == 0) { group_best[g] = best; kept[g] = 0.0f; }
    }
    __syncwarp();
    for (int n = 0; n < group_keep; ++n) {
      float best;
      int where;
      warp_argmax(group_best, group_count, lane, best, where);
      if (lane == 0 && where < group_count) { kept[where] = 1.0f; group_best[where] = -INFINITY; }
      __syncwarp();
    }
    for (int i = lane; i < outputs; i += 32)
      if (kept[i / per] == 0.0f) choice[i] = -INFINITY;
    __syncwarp();
  }
  float chosen_sum = 0.0f;
  for (int n = 0; n < top; ++n) {
    float best;
    int where;
    warp_argmax(choice, outputs, lane, best, where);
    if (where >= outputs) where = 0;
    if (lane == 0) {
      ids[(size_t)t * top + n] = where;
      choice[where] = -INFINITY;
    }
    chosen_sum += score[where];
    __syncwarp();
  }
  chosen_sum += 1e-20f;
  if (lane == 0)
    for (int n = 0; n < top; ++n) weights[(size_t)t * top + n] = score[ids[(size_t)t * top + n]] / chosen_sum;
}

template <typename T>
__global__ void __launch_bounds__(256) activation_kernel(T* __restrict__ rows, long long ld, int count, int width, int kind,
                                                         const float* __restrict__ params) {
  pdl_trigger();
  pdl_wait();
  float a = 0.0f, b = 0.0f;
  if (kind == 1) {
    a = softplus_f(params[0]);
    b = 0.5f + softplus_f(params[1]);
  }
  const long long total = (long long)count * width;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / width;
    const int c = (int)(idx - r * width);
    T* at = rows + r * ld + c;
    const float z = to_float<T>(*at);
    float y;
    if (kind == 0) {
      const float p = fmaxf(z, 0.0f);
      y = p * p;
    } else {
      y = z > 0.0f ? fmaf(a * z, z, 0.5f * z) : fmaf(b, expm1f(z) - z, 0.5f * z);
    }
    *at = from_float<T>(y);
  }
}

// The same on eight bfloat16 at a time: rows whose width and stride are multiples of 8 and that start on 16 bytes.
__global__ void __launch_bounds__(256) activation_vec_kernel(__nv_bfloat16* __restrict__ rows, long long ld, int count, int width,
                                                             int kind, const float* __restrict__ params) {
  pdl_trigger();
  pdl_wait();
  float a = 0.0f, b = 0.0f;
  if (kind == 1) {
    a = softplus_f(params[0]);
    b = 0.5f + softplus_f(params[1]);
  }
  const int per_row = width / 8;
  const long long total = (long long)count * per_row;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / per_row;
    const int c = (int)(idx - r * per_row);
    uint4* at = reinterpret_cast<uint4*>(rows + r * ld) + c;
    uint4 raw = *at;
    __nv_bfloat162* two = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 z = __bfloat1622float2(two[i]);
      if (kind == 0) {
        const float p = fmaxf(z.x, 0.0f), q = fmaxf(z.y, 0.0f);
        z.x = p * p;
        z.y = q * q;
      } else {
        z.x = z.x > 0.0f ? fmaf(a * z.x, z.x, 0.5f * z.x) : fmaf(b, expm1f(z.x) - z.x, 0.5f * z.x);
        z.y = z.y > 0.0f ? fmaf(a * z.y, z.y, 0.5f * z.y) : fmaf(b, expm1f(z.y) - z.y, 0.5f * z.y);
      }
      two[i] = __floats2bfloat162_rn(z.x, z.y);
    }
    *at = raw;
  }
}

// sum_k a[k] * b[k] over a warp: every lane takes the elements lane, lane + 32, ... in ascending order and the lanes'
// sums meet in a butterfly, so the order depends on nothing but n.
template <typename T>
__device__ __forceinline__ float warp_dot(const T* __restrict__ a, const T* __restrict__ b, int n, int lane) {
  float acc = 0.0f;
  for (int k = lane; k < n; k += 32) acc = fmaf(to_float<T>(a[k]), to_float<T>(b[k]), acc);
  return warp_sum(acc);
}
template <>
__device__ __forceinline__ float warp_dot<__nv_bfloat16>(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                                        int n, int lane) {
  float acc = 0.0f;
  if ((n & 7) == 0 && (((uintptr_t)a | (uintptr_t)b) & 15) == 0) {
    for (int k = lane * 8; k < n; k += 256) {
      const uint4 va = *reinterpret_cast<const uint4*>(a + k), vb = *reinterpret_cast<const uint4*>(b + k);
      const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&va);
      const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&vb);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]);
        acc = fmaf(fa.x, fb.x, acc);
        acc = fmaf(fa.y, fb.y, acc);
      }
    }
  } else {
    for (int k = lane; k < n; k += 32) acc = fmaf(__bfloat162float(a[k]), __bfloat162float(b[k]), acc);
  }
  return warp_sum(acc);
}

// inner[pair, j] = relu(w_up[expert][j, :] . h[token, :])^2 for the pairs whose choice is an expert.
template <typename T>
__global__ void __launch_bounds__(256) expert_up_kernel(const T* __restrict__ h, long long ld_h, const T* __restrict__ w_up,
                                                        const int* __restrict__ ids, T* __restrict__ inner, int top,
                                                        int experts, int width, int ff) {
  pdl_trigger();
  pdl_wait();
  const int pair = blockIdx.x;
  const int expert = ids[pair];
  if (expert < 0 || expert >= experts) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* row = h + (size_t)(pair / top) * ld_h;
  const T* w = w_up + (size_t)expert * ff * width;
  for (int j = blockIdx.y * 8 + warp; j < ff; j += gridDim.y * 8) {
    const float dot = warp_dot<T>(row, w + (size_t)j * width, width, lane);
    if (lane == 0) {
      const float p = fmaxf(dot, 0.0f);
      inner[(size_t)pair * ff + j] = from_float<T>(p * p);
    }
  }
}

// x[token, n] += sum over the token's choices, in their order, of weight * (w_down[expert][n, :] . inner[pair, :]), or
// weight * h[token, n] for an identity expert.
template <typename T>
__global__ void __launch_bounds__(256) expert_down_add_kernel(const T* __restrict__ inner, const T* __restrict__ w_down,
                                                              const T* __restrict__ h, long long ld_h,
                                                              const int* __restrict__ ids, const float* __restrict__ weights,
                                                              float* __restrict__ x, int top, int experts, int width, int ff,
                                                              long long down_expert, long long down_row) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int n = blockIdx.y * 8 + warp; n < width; n += gridDim.y * 8) {
    float acc = 0.0f;
    for (int k = 0; k < top; ++k) {
      const int pair = t * top + k;
      const int expert = ids[pair];
      const float weight = weights[pair];
      if (expert >= 0 && expert < experts)
        acc = fmaf(weight, warp_dot<T>(inner + (size_t)pair * ff, w_down + (size_t)expert * down_expert + (size_t)n * down_row, ff, lane), acc);
      else
        acc = fmaf(weight, to_float<T>(h[(size_t)t * ld_h + n]), acc);
    }
    if (lane == 0) x[(size_t)t * width + n] += acc;
  }
}

// One block.  place[pair]: the pair's row in the buffer grouped by expert (-1 for an identity expert);
// offsets[e] .. offsets[e + 1]: expert e's rows.
__global__ void __launch_bounds__(1024) expert_sort_kernel(const int* __restrict__ ids, int pairs, int experts,
                                                           int* __restrict__ place, int* __restrict__ offsets) {
  extern __shared__ int sort_smem[];
  int* count = sort_smem;
  int* cursor = sort_smem + experts;
  pdl_trigger();
  pdl_wait();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int running = 0;
    for (int e = 0; e < experts; ++e) {
      offsets[e] = running;
      cursor[e] = running;
      running += count[e];
    }
    offsets[experts] = running;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    place[p] = (e >= 0 && e < experts) ? atomicAdd(&cursor[e], 1) : -1;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) expert_gather_kernel(const T* __restrict__ h, long long ld_h, const int* __restrict__ place,
                                                            T* __restrict__ grouped, int top, int width) {
  pdl_trigger();
  pdl_wait();
  const int pair = blockIdx.x;
  const int row = place[pair];
  if (row < 0) return;
  const T* src = h + (size_t)(pair / top) * ld_h;
  for (int i = threadIdx.x; i < width; i += blockDim.x) grouped[(size_t)row * width + i] = src[i];
}

template <typename T>
__global__ void __launch_bounds__(256) expert_combine_add_kernel(const float* __restrict__ outputs, const int* __restrict__ place,
                                                                 const float* __restrict__ weights, const T* __restrict__ h,
                                                                 long long ld_h, float* __restrict__ x, int top, int width) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  for (int n = blockIdx.y * blockDim.x + threadIdx.x; n < width; n += gridDim.y * blockDim.x) {
    float acc = 0.0f;
    for (int k = 0; k < top; ++k) {
      const int pair = t * top + k;
      const int row = place[pair];
      const float v = row >= 0 ? outputs[(size_t)row * width + n] : to_float<T>(h[(size_t)t * ld_h + n]);
      acc = fmaf(weights[pair], v, acc);
    }
    x[(size_t)t * width + n] += acc;
  }
}

// The dense path, between its two products.  z [tokens, experts * ff]: every expert's up projection of every token.
// In place: a token's rows of a chosen expert become weight * relu(z)^2, all others zero, so that ONE product with
// the down matrices side by side along k adds the weighted sum of the chosen experts.  Blocks with blockIdx.y ==
// experts add the identity experts' share, weight * h, into the stream.
template <typename T>
__global__ void __launch_bounds__(256) expert_dense_weigh_kernel(T* __restrict__ z, const int* __restrict__ ids,
                                                                 const float* __restrict__ weights, const T* __restrict__ h,
                                                                 long long ld_h, float* __restrict__ x, int top, int experts,
                                                                 int width, int ff) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, e = blockIdx.y;
  if (e == experts) {
    float w = 0.0f;
    bool any = false;
    for (int k = 0; k < top; ++k) {
      const int id = ids[t * top + k];
      if (id >= experts) { w += weights[t * top + k]; any = true; }
    }
    if (!any) return;
    for (int n = threadIdx.x; n < width; n += blockDim.x) x[(size_t)t * width + n] += w * to_float<T>(h[(size_t)t * ld_h + n]);
    return;
  }
  float w = 0.0f;
  bool chosen = false;
  for (int k = 0; k < top; ++k)
    if (ids[t * top + k] == e) { w = weights[t * top + k]; chosen = true; }
  T* row = z + ((size_t)t * experts + e) * ff;
  if (!chosen) {
    for (int j = threadIdx.x; j < ff; j += blockDim.x) row[j] = from_float<T>(0.0f);
    return;
  }
  for (int j = threadIdx.x; j < ff; j += blockDim.x) {
    const float p = fmaxf(to_float<T>(row[j]), 0.0f);
    row[j] = from_float<T>(w * p * p);
  }
}

}  // namespace

// logits float32 [tokens, ld]; correction float32 [outputs] or null; ids int32 [tokens, top]; weights float32 [tokens, top].
TGE_API int tge_router_topk(const float* logits, long long ld, const float* correction, int tokens, int outputs, int top,
                            int group_count, int group_keep, int* ids, float* weights, cudaStream_t stream) {
  TGE_REQUIRE(tokens >= 0 && outputs > 0 && outputs <= 1024, "router_topk: 1 to 1024 outputs, not %d", outputs);
  TGE_REQUIRE(top > 0 && top <= outputs, "router_topk: %d choices of %d outputs", top, outputs);
  TGE_REQUIRE(group_count > 0 && outputs % group_count == 0 && group_keep > 0 && group_keep <= group_count,
              "router_topk: %d groups (%d kept) of %d outputs", group_count, group_keep, outputs);
  TGE_REQUIRE((outputs / group_count) * group_keep >= top, "router_topk: %d choices do not fit the kept groups", top);
  if (tokens == 0) return 0;
  const size_t smem = (size_t)4 * 4 * outputs * sizeof(float);
  if (smem > 48 * 1024) {
    static bool configured = false;
    if (!configured) {
      cudaFuncSetAttribute(router_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 4 * 1024 * (int)sizeof(float));
      configured = true;
    }
  }
  tge_launch(router_topk_kernel, dim3((tokens + 3) / 4), dim3(128), smem, stream, logits, ld, correction, tokens, outputs, top,
             group_count, group_keep, ids, weights);
  return tge_launched("router_topk", 1);
}

// rows: run dtype [count, width] with row stride ld, changed in place.  kind 0: relu(z)^2; 1: the two-parameter form,
// params float32 [2] on the device.
TGE_API int tge_activation(void* rows, long long ld, int count, int width, int kind, const float* params, int is_bf16,
                           cudaStream_t stream) {
  TGE_REQUIRE(count >= 0 && width > 0 && ld >= width, "activation: bad shape");
  TGE_REQUIRE(kind == 0 || (kind == 1 && params != nullptr), "activation: kind %d", kind);
  if (count == 0) return 0;
  const long long total = (long long)count * width;
  if (is_bf16 && width % 8 == 0 && ld % 8 == 0 && (uintptr_t)rows % 16 == 0) {
    const long long vectors = total / 8;
    const int vec_blocks = (int)((vectors + 255) / 256 > 148 * 32 ? 148 * 32 : (vectors + 255) / 256);
    tge_launch(activation_vec_kernel, dim3(vec_blocks), dim3(256), 0, stream, (__nv_bfloat16*)rows, ld, count, width, kind, params);
    return tge_launched("activation", 1);
  }
  const int blocks = (int)((total + 255) / 256 > 148 * 32 ? 148 * 32 : (total + 255) / 256);
  if (is_bf16) tge_launch(activation_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)rows, ld, count, width, kind, params);
  else tge_launch(activation_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)rows, ld, count, width, kind, params);
  return tge_launched("activation", 1);
}

// The direct path.  h: run dtype [tokens, >= width] with row stride ld_h; w_up [experts, ff, width]; row n of expert
// e's down matrix (ff numbers) starts at w_down + e * down_expert + n * down_row; inner: run dtype scratch
// [tokens * top, ff]; x: the float32 stream [tokens, width].
TGE_API int tge_experts_direct(const void* h, long long ld_h, const void* w_up, const void* w_down, long long down_expert,
                               long long down_row, const int* ids, const float* weights, void* inner, float* x, int tokens,
                               int top, int experts, int width, int ff, int is_bf16, cudaStream_t stream) {
  TGE_REQUIRE(tokens >= 0 && top > 0 && experts >= 0 && width > 0 && ff > 0, "experts: bad shape");
  if (tokens == 0) return 0;
  const int up_y = (ff + 7) / 8 < 64 ? (ff + 7) / 8 : 64;
  const int down_y = (width + 7) / 8 < 64 ? (width + 7) / 8 : 64;
  if (is_bf16) {
    tge_launch(expert_up_kernel<__nv_bfloat16>, dim3(tokens * top, up_y), dim3(256), 0, stream, (const __nv_bfloat16*)h, ld_h,
               (const __nv_bfloat16*)w_up, ids, (__nv_bfloat16*)inner, top, experts, width, ff);
    tge_launch(expert_down_add_kernel<__nv_bfloat16>, dim3(tokens, down_y), dim3(256), 0, stream, (const __nv_bfloat16*)inner,
               (const __nv_bfloat16*)w_down, (const __nv_bfloat16*)h, ld_h, ids, weights, x, top, experts, width, ff, down_expert,
               down_row);
  } else {
    tge_launch(expert_up_kernel<float>, dim3(tokens * top, up_y), dim3(256), 0, stream, (const float*)h, ld_h,
               (const float*)w_up, ids, (float*)inner, top, experts, width, ff);
    tge_launch(expert_down_add_kernel<float>, dim3(tokens, down_y), dim3(256), 0, stream, (const float*)inner,
               (const float*)w_down, (const float*)h, ld_h, ids, weights, x, top, experts, width, ff, down_expert, down_row);
  }
  return tge_launched("experts_direct", 2);
}

// The grouped path, first half: place int32 [tokens * top], offsets int32 [experts + 1], grouped run dtype
// [tokens * top, width] (the rows of expert e at offsets[e] .. offsets[e + 1]).
TGE_API int tge_experts_group(const void* h, long long ld_h, const int* ids, int* place, int* offsets, void* grouped,
                              int tokens, int top, int experts, int width, int is_bf16, cudaStream_t stream) {
  TGE_REQUIRE(tokens >= 0 && top > 0 && experts > 0 && experts <= 4096 && width > 0, "experts: bad shape");
  if (tokens == 0) return 0;
  tge_launch(expert_sort_kernel, dim3(1), dim3(1024), (size_t)2 * experts * sizeof(int), stream, ids, tokens * top, experts,
             place, offsets);
  if (is_bf16)
    tge_launch(expert_gather_kernel<__nv_bfloat16>, dim3(tokens * top), dim3(256), 0, stream, (const __nv_bfloat16*)h, ld_h,
               (const int*)place, (__nv_bfloat16*)grouped, top, width);
  else
    tge_launch(expert_gather_kernel<float>, dim3(tokens * top), dim3(256), 0, stream, (const float*)h, ld_h, (const int*)place,
               (float*)grouped, top, width);
  return tge_launched("experts_group", 2);
}

// The grouped path, second half: outputs float32 [tokens * top, width] in grouped order.
TGE_API int tge_experts_combine_add(const float* outputs, const int* place, const float* weights, const void* h, long long ld_h,
                                    float* x, int tokens, int top, int width, int is_bf16, cudaStream_t stream) {
  TGE_REQUIRE(tokens >= 0 && top > 0 && width > 0, "experts: bad shape");
  if (tokens == 0) return 0;
  const int chunks = (width + 1023) / 1024;
  if (is_bf16)
    tge_launch(expert_combine_add_kernel<__nv_bfloat16>, dim3(tokens, chunks), dim3(256), 0, stream, outputs, place, weights,
               (const __nv_bfloat16*)h, ld_h, x, top, width);
  else
    tge_launch(expert_combine_add_kernel<float>, dim3(tokens, chunks), dim3(256), 0, stream, outputs, place, weights,
               (const float*)h, ld_h, x, top, width);
  return tge_launched("experts_combine_add", 1);
}

// The dense path: z run dtype [tokens, experts * ff] in place (see the kernel); x float32 [tokens, width].
TGE_API int tge_experts_dense_weigh(void* z, const int* ids, const float* weights, const void* h, long long ld_h, float* x,
                                    int tokens, int top, int experts, int width, int ff, int is_bf16, cudaStream_t stream) {
  TGE_REQUIRE(tokens >= 0 && top > 0 && experts > 0 && experts < 65535 && width > 0 && ff > 0, "experts: bad shape");
  if (tokens == 0) return 0;
  if (is_bf16)
    tge_launch(expert_dense_weigh_kernel<__nv_bfloat16>, dim3(tokens, experts + 1), dim3(256), 0, stream, (__nv_bfloat16*)z, ids,
               weights, (const __nv_bfloat16*)h, ld_h, x, top, experts, width, ff);
  else
    tge_launch(expert_dense_weigh_kernel<float>, dim3(tokens, experts + 1), dim3(256), 0, stream, (float*)z, ids, weights,
               (const float*)h, ld_h, x, top, experts, width, ff);
  return tge_launched("experts_dense_weigh", 1);
}
