// Layer norm with weight and bias over float32 rows:
//   y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w + b,
// the mean first and the variance from the deviations, both float32 sums in a fixed order. One
// CTA per row; a thread keeps its PER elements of the row in registers between the passes.
//
// lrm_layer_norm: rows of the residual stream (all, or those `rows` names) -> activations.
// lrm_layer_norm_add: a norm behind a sublayer, stream[t] += mult * y(sublayer output[t]), in
// place; with `cast_out` the updated row is also written in the activation type, which is what the
// next sublayer reads when nothing stands between it and the stream.
//
// Only the weight and the bias are `const __restrict__`: a load through such a pointer counts as
// invariant for the whole kernel and may be moved ahead of griddepcontrol.wait, next to the loads
// of w and b that stand there on purpose. What the kernel before this one writes (x, y, the stream)
// is read through plain pointers, whose loads stay behind the wait.
#include "common.cuh"

namespace {

template <int PER>
__device__ __forceinline__ void row_statistics(const float (&v)[PER], int hidden, float eps, float* scratch,
                                               float* mean_out, float* inv_out) {
  float sum = 0.f;
#pragma unroll
  for (int e = 0; e < PER; ++e) sum += v[e];  // elements beyond the row are zero
  const float mean = block_sum(sum, scratch) / static_cast<float>(hidden);
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    const int i = threadIdx.x + e * blockDim.x;
    const float dev = i < hidden ? v[e] - mean : 0.f;
    ss = fmaf(dev, dev, ss);
  }
  *mean_out = mean;
  *inv_out = 1.0f / sqrtf(block_sum(ss, scratch) / static_cast<float>(hidden) + eps);
}

// Rows of up to 8 elements per thread take weight and bias into registers ahead of the wait;
// longer rows (PER 32, up to 1024 threads) read them where they are used, which keeps the kernel
// within the registers 1024 threads can have.
template <typename O, int PER>
__global__ __launch_bounds__(1024) void layer_norm_kernel(const float* x, const float* __restrict__ w, const float* __restrict__ b, O* out,
                                  const int* rows, int hidden, float eps) {
  __shared__ float scratch[32];
  constexpr bool EARLY = PER <= 8;
  constexpr int KEPT = EARLY ? PER : 1;
  float wv[KEPT], bv[KEPT];
  if (EARLY) {
#pragma unroll
    for (int e = 0; e < KEPT; ++e) {  // weights do not depend on the kernel before this one
      const int i = threadIdx.x + e * blockDim.x;
      wv[e] = i < hidden ? w[i] : 0.f;
      bv[e] = i < hidden ? b[i] : 0.f;
    }
  }
  pdl_trigger();
  pdl_wait();
  const size_t src = static_cast<size_t>(rows != nullptr ? rows[blockIdx.x] : blockIdx.x) * hidden;
  float v[PER];
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    const int i = threadIdx.x + e * blockDim.x;
    v[e] = i < hidden ? x[src + i] : 0.f;
  }
  float mean, inv;
  row_statistics<PER>(v, hidden, eps, scratch, &mean, &inv);
  const size_t dst = static_cast<size_t>(blockIdx.x) * hidden;
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    const int i = threadIdx.x + e * blockDim.x;
    if (i < hidden)
      out[dst + i] = from_f32<O>(fmaf((v[e] - mean) * inv, EARLY ? wv[e % KEPT] : w[i], EARLY ? bv[e % KEPT] : b[i]));
  }
}

template <typename O, int PER>
__global__ __launch_bounds__(1024) void layer_norm_add_kernel(float* stream, const float* y, const float* __restrict__ w,
                                      const float* __restrict__ b, float mult, O* cast_out, int hidden, float eps) {
  __shared__ float scratch[32];
  constexpr bool EARLY = PER <= 8;
  constexpr int KEPT = EARLY ? PER : 1;
  float wv[KEPT], bv[KEPT];
  if (EARLY) {
#pragma unroll
    for (int e = 0; e < KEPT; ++e) {
      const int i = threadIdx.x + e * blockDim.x;
      wv[e] = i < hidden ? w[i] : 0.f;
      bv[e] = i < hidden ? b[i] : 0.f;
    }
  }
  pdl_trigger();
  pdl_wait();
  const size_t row = static_cast<size_t>(blockIdx.x) * hidden;
  float v[PER];
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    const int i = threadIdx.x + e * blockDim.x;
    v[e] = i < hidden ? y[row + i] : 0.f;
  }
  float mean, inv;
  row_statistics<PER>(v, hidden, eps, scratch, &mean, &inv);
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    const int i = threadIdx.x + e * blockDim.x;
    if (i < hidden) {
      const float updated = stream[row + i] + mult * fmaf((v[e] - mean) * inv, EARLY ? wv[e % KEPT] : w[i],
                                                          EARLY ? bv[e % KEPT] : b[i]);
      stream[row + i] = updated;
      if (cast_out != nullptr) cast_out[row + i] = from_f32<O>(updated);
    }
  }
}

// short rows on 32 to 256 threads, rows beyond 2048 elements on 1024
int row_threads(int hidden) { return hidden > 2048 ? 1024 : (hidden >= 1024 ? 256 : (hidden >= 256 ? 128 : 32)); }

}  // namespace

// x float32 [*, hidden]; w, b float32 [hidden]; rows int32 [n_rows] or null (row r of out is row r of x).
LRM_API int lrm_layer_norm(const float* x, const float* w, const float* b, void* out, int out_dtype, const int* rows,
                           int n_rows, int hidden, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hidden <= 0 || !(eps > 0.f) || x == nullptr || w == nullptr || b == nullptr || out == nullptr)
    return LRM_BAD_ARGUMENT;
  const int threads = row_threads(hidden), per = (hidden + threads - 1) / threads;
#define LRM_LAYER_NORM(OT, PER)                                                                                   \
  do {                                                                                                            \
    LRM_LAUNCH((layer_norm_kernel<OT, PER>), n_rows, threads, 0, stream, x, w, b, static_cast<OT*>(out), rows, hidden, \
               eps);                                                                                              \
    return 0;                                                                                                     \
  } while (0)
  if (out_dtype == LRM_F32) {
    if (per <= 4) LRM_LAYER_NORM(float, 4);
    if (per <= 8) LRM_LAYER_NORM(float, 8);
    if (per <= 32) LRM_LAYER_NORM(float, 32);
  } else if (out_dtype == LRM_BF16) {
    if (per <= 4) LRM_LAYER_NORM(__nv_bfloat16, 4);
    if (per <= 8) LRM_LAYER_NORM(__nv_bfloat16, 8);
    if (per <= 32) LRM_LAYER_NORM(__nv_bfloat16, 32);
  } else {
    return LRM_BAD_ARGUMENT;
  }
#undef LRM_LAYER_NORM
  return LRM_UNSUPPORTED;  // rows longer than 32768 elements
}

// stream, y float32 [n_rows, hidden]; cast_out [n_rows, hidden] in out_dtype, or null.
LRM_API int lrm_layer_norm_add(float* stream_rows, const float* y, const float* w, const float* b, float mult,
                               void* cast_out, int out_dtype, int n_rows, int hidden, float eps,
                               cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hidden <= 0 || !(eps > 0.f) || stream_rows == nullptr || y == nullptr || w == nullptr || b == nullptr)
    return LRM_BAD_ARGUMENT;
  const int threads = row_threads(hidden), per = (hidden + threads - 1) / threads;
#define LRM_LAYER_NORM_ADD(OT, PER)                                                                             \
  do {                                                                                                          \
    LRM_LAUNCH((layer_norm_add_kernel<OT, PER>), n_rows, threads, 0, stream, stream_rows, y, w, b, mult,        \
               static_cast<OT*>(cast_out), hidden, eps);                                                        \
    return 0;                                                                                                   \
  } while (0)
  if (out_dtype == LRM_F32) {
    if (per <= 4) LRM_LAYER_NORM_ADD(float, 4);
    if (per <= 8) LRM_LAYER_NORM_ADD(float, 8);
    if (per <= 32) LRM_LAYER_NORM_ADD(float, 32);
  } else if (out_dtype == LRM_BF16) {
    if (per <= 4) LRM_LAYER_NORM_ADD(__nv_bfloat16, 4);
    if (per <= 8) LRM_LAYER_NORM_ADD(__nv_bfloat16, 8);
    if (per <= 32) LRM_LAYER_NORM_ADD(__nv_bfloat16, 32);
  } else {
    return LRM_BAD_ARGUMENT;
  }
#undef LRM_LAYER_NORM_ADD
  return LRM_UNSUPPORTED;
}
