// Norms and token mixing that act on a token's row of the residual stream.
//
//  * group_norm         - RMS norm in groups: a row is cut into `groups` equal consecutive parts, each part is divided
//                         by its own sqrt(mean(part^2) + eps), and the whole is multiplied by a weight.  One group is
//                         the plain RMS norm.  The result is float32 (it may overwrite its input: a normalised
//                         embedding is the start of the stream) or the run dtype; rows may be gathered by index.
//  * token_shift        - every row is blended, element by element, with the row of the token before it:
//                         out_t = h_t + (h_(t-1) - h_t) * mu.  The row before a portion's first token is the one the
//                         request's state slot holds (zeros at position 0).
//  * shift_state_update - the last row of every portion goes into the request's state slot, for the next step.
//
// All statistics are float32.  The two shift kernels are separate launches because a portion's first block reads the
// slot that its last row replaces.
#include "common.cuh"

namespace {

template <typename TO>
__global__ void __launch_bounds__(256) group_norm_kernel(const float* x, const float* __restrict__ weight,
                                                         const int* __restrict__ rows, TO* out, int src_rows, int width,
                                                         int groups, float eps, int* status,
                                                         const float* __restrict__ weight2, TO* out2) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows != nullptr ? rows[r] : r;
  if (src < 0 || src >= src_rows) {
    if (threadIdx.x == 0) atomicOr(status, TGE_STATUS_BAD_ROW);
    return;
  }
  const float* row = x + (size_t)src * width;
  TO* dst = out + (size_t)r * width;
  const int size = width / groups;
  for (int g = 0; g < groups; ++g) {
    const float* part = row + (size_t)g * size;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) ss = fmaf(part[i], part[i], ss);
    ss = block_sum(ss, scratch);                     // every read of the part is done once this returns
    const float inv = 1.0f / sqrtf(ss / (float)size + eps);
    if (out2 == nullptr) {
      for (int i = threadIdx.x; i < size; i += blockDim.x)
        dst[(size_t)g * size + i] = from_float<TO>(part[i] * inv * weight[(size_t)g * size + i]);
    } else {
      // a second norm of the same rows (same groups and eps, another weight): the statistics serve both
      TO* dst2 = out2 + (size_t)r * width;
      for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float v = part[i] * inv;
        dst[(size_t)g * size + i] = from_float<TO>(v * weight[(size_t)g * size + i]);
        dst2[(size_t)g * size + i] = from_float<TO>(v * weight2[(size_t)g * size + i]);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) token_shift_kernel(const T* __restrict__ h, const float* __restrict__ mu,
                                                          const float* __restrict__ state, const int* __restrict__ slots,
                                                          int num_slots, const int* __restrict__ seq_of_token,
                                                          const int* __restrict__ q_start, const int* __restrict__ start_pos,
                                                          T* __restrict__ out, int tokens, int width, int* status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int seq = seq_of_token[t];
  const bool first = t == q_start[seq];
  const float* kept = nullptr;
  if (first && start_pos[seq] > 0) {
    const int slot = slots[seq];
    if (slot < 0 || slot >= num_slots) {
      if (threadIdx.x == 0) atomicOr(status, TGE_STATUS_BAD_ROW);
      return;
    }
    kept = state + (size_t)slot * width;
  }
  const T* row = h + (size_t)t * width;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < width; i += gridDim.y * blockDim.x) {
    const float now = to_float<T>(row[i]);
    const float before = first ? (kept != nullptr ? kept[i] : 0.0f) : to_float<T>(row[i - width]);
    out[(size_t)t * width + i] = from_float<T>(fmaf(before - now, mu[i], now));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) shift_state_update_kernel(const T* __restrict__ h, float* __restrict__ state,
                                                                 const int* __restrict__ slots, int num_slots,
                                                                 const int* __restrict__ q_start, int width, int* status) {
  pdl_trigger();
  pdl_wait();
  const int seq = blockIdx.x;
  const int last = q_start[seq + 1] - 1;
  if (last < q_start[seq]) return;
  const int slot = slots[seq];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(status, TGE_STATUS_BAD_ROW);
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    state[(size_t)slot * width + i] = to_float<T>(h[(size_t)last * width + i]);
}

}  // namespace

// x float32 [src_rows, width]; rows: null or int32 [out_rows]; out: float32 (out_kind 0; may be x itself when rows is
// null) or bfloat16 (out_kind 1), [out_rows, width].  weight2 / out2: null, or a second weight and output like the first.
TGE_API int tge_group_norm(const float* x, const float* weight, const int* rows, void* out, int out_kind, int out_rows,
                           int src_rows, int width, int groups, float eps, const float* weight2, void* out2, int* status,
                           cudaStream_t stream) {
  TGE_REQUIRE((weight2 == nullptr) == (out2 == nullptr) && (out2 == nullptr || (out2 != out && out2 != (void*)x && out != (void*)x)),
              "group_norm: a second output needs a second weight and buffers of its own");
  TGE_REQUIRE(out_rows >= 0 && src_rows >= 0 && width > 0, "group_norm: bad shape");
  TGE_REQUIRE(groups > 0 && width % groups == 0, "group_norm: %d groups do not divide a row of %d", groups, width);
  TGE_REQUIRE(eps > 0.0f, "group_norm: eps must be positive");
  TGE_REQUIRE(out_kind == 0 || out_kind == 1, "group_norm: the output is float32 (0) or bfloat16 (1)");
  if (out_rows == 0) return 0;
  if (out_kind == 0)
    tge_launch(group_norm_kernel<float>, dim3(out_rows), dim3(256), 0, stream, x, weight, rows, (float*)out, src_rows,
               width, groups, eps, status, weight2, (float*)out2);
  else
    tge_launch(group_norm_kernel<__nv_bfloat16>, dim3(out_rows), dim3(256), 0, stream, x, weight, rows,
               (__nv_bfloat16*)out, src_rows, width, groups, eps, status, weight2, (__nv_bfloat16*)out2);
  return tge_launched("group_norm", 1);
}

// h, out: [tokens, width] in the run dtype (two buffers); mu float32 [width]; state float32 [num_slots, width].
// update != 0: the portions' last rows are then written to their slots by a second launch.
TGE_API int tge_token_shift(const void* h, int is_bf16, const float* mu, float* state, const int* slots, int num_slots,
                            const int* seq_of_token, const int* q_start, const int* start_pos, void* out, int tokens,
                            int num_seqs, int width, int update, int* status, cudaStream_t stream) {
  TGE_REQUIRE(tokens >= 0 && num_seqs >= 0 && width > 0 && num_slots > 0, "token_shift: bad shape");
  TGE_REQUIRE(h != out, "token_shift: a row is read after the row behind it is written; give two buffers");
  if (tokens == 0 || num_seqs == 0) return 0;
  const int chunks = (width + 1023) / 1024;
  if (is_bf16)
    tge_launch(token_shift_kernel<__nv_bfloat16>, dim3(tokens, chunks), dim3(256), 0, stream, (const __nv_bfloat16*)h, mu,
               (const float*)state, slots, num_slots, seq_of_token, q_start, start_pos, (__nv_bfloat16*)out, tokens, width,
               status);
  else
    tge_launch(token_shift_kernel<float>, dim3(tokens, chunks), dim3(256), 0, stream, (const float*)h, mu,
               (const float*)state, slots, num_slots, seq_of_token, q_start, start_pos, (float*)out, tokens, width, status);
  int rc = tge_check_launch("token_shift");
  if (rc != 0) return rc;
  if (!update) return 1;
  if (is_bf16)
    tge_launch(shift_state_update_kernel<__nv_bfloat16>, dim3(num_seqs), dim3(256), 0, stream, (const __nv_bfloat16*)h,
               state, slots, num_slots, q_start, width, status);
  else
    tge_launch(shift_state_update_kernel<float>, dim3(num_seqs), dim3(256), 0, stream, (const float*)h, state, slots,
               num_slots, q_start, width, status);
  return tge_launched("shift_state_update", 2);
}
