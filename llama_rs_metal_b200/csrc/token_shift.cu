// What a block does to the stream around its sublayers beyond norms: the mix of a sublayer's input
// with the previous token's, and the addition of a sublayer's output under a factor per channel.
#include "common.cuh"

namespace {

// out[t, c] = h[t, c] + (h[t - 1, c] - h[t, c]) * mix[c], with the previous token's row as it was
// before this replacement; for a sequence's first token of the step it comes from `last`
// [slots, width] (float32; zeros at the start of a sequence), and a sequence of padding (slot < 0)
// has zeros there. One CTA per token. The thread that read last[slot, c] for a sequence's first
// token then writes the sequence's newest h there (the row of its last token of this step), so
// `last` is up to date when the kernel ends and nobody reads an entry after it was rewritten.
template <typename A>
__global__ void token_shift_kernel(const A* h, const float* __restrict__ mix, float* last, A* __restrict__ out,
                                   const int* __restrict__ cu_seqlens, const int* __restrict__ seq_of_token,
                                   const int* __restrict__ slots, int width) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int b = seq_of_token[t], local = t - cu_seqlens[b], slot = slots[b];
  const A* row = h + static_cast<size_t>(t) * width;
  const A* before = local > 0 ? row - width : nullptr;
  float* kept = (local == 0 && slot >= 0) ? last + static_cast<size_t>(slot) * width : nullptr;
  const A* newest = h + static_cast<size_t>(cu_seqlens[b + 1] - 1) * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float x = to_f32(row[c]);
    const float p = before != nullptr ? to_f32(before[c]) : kept != nullptr ? kept[c] : 0.f;
    out[static_cast<size_t>(t) * width + c] = from_f32<A>(fmaf(p - x, mix[c], x));
    if (kept != nullptr) kept[c] = to_f32(newest[c]);
  }
}

// x[t, :] += factor * y[t, :], then out[t, :] = x[t, :] / sqrt(mean(x[t, :]^2) + eps) * w in the
// activation type: a sublayer's output enters the stream and the updated row goes through the next
// sublayer's norm in the same pass. One CTA per row; a thread reads back only what it wrote itself.
template <typename W, typename O>
__global__ void scaled_add_norm_kernel(float* x, const float* y, const float* __restrict__ factor,
                                       const W* __restrict__ w, float eps, O* __restrict__ out, int width) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  float* row = x + static_cast<size_t>(blockIdx.x) * width;
  const float* add = y + static_cast<size_t>(blockIdx.x) * width;
  O* dst = out + static_cast<size_t>(blockIdx.x) * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = fmaf(factor[c], add[c], row[c]);
    row[c] = v;
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / static_cast<float>(width) + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = from_f32<O>((row[c] * inv) * to_f32(w[c]));
}

// x[t, c] += factor[c] * y[t, c]: a sublayer's float32 output enters the float32 stream under a
// factor per channel.
__global__ void scaled_add_kernel(float* x, const float* y, const float* __restrict__ factor, int width, size_t n) {
  pdl_trigger();
  pdl_wait();
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx < n) x[idx] = fmaf(factor[idx % width], y[idx], x[idx]);
}

// y[t, :] = sigmoid(x[t, :] . w) * y[t, :] + planes[0][t, :] + planes[1][t, :] + ...: one gate per
// token from its input row (float32 sum) on a float32 output row, and `count` planes [tokens,
// out_width] of float32 sums that belong beside it, added in plane order. gridDim.y CTAs per token
// share its columns (each forms the gate itself), so that few tokens still fill the device.
template <typename A>
__global__ void row_gate_kernel(float* y, const A* x, const float* __restrict__ w, int in_width, int out_width,
                                const float* planes, int count, size_t plane) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  float acc = 0.f;
  for (int c = threadIdx.x; c < in_width; c += blockDim.x)
    acc = fmaf(to_f32(x[static_cast<size_t>(t) * in_width + c]), w[c], acc);
  const float z = block_sum(acc, scratch);
  const float gate = 1.0f / (1.0f + expf(-z));
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < out_width; c += gridDim.y * blockDim.x) {
    const size_t at = static_cast<size_t>(t) * out_width + c;
    float v = y[at] * gate;
    for (int p = 0; p < count; ++p) v += planes[p * plane + at];
    y[at] = v;
  }
}

}  // namespace

LRM_API int lrm_token_shift(const void* h, int dtype, const float* mix, float* last, void* out,
                            const int* cu_seqlens, const int* seq_of_token, const int* slots, int tokens, int width,
                            cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (width <= 0 || mix == nullptr || last == nullptr) return LRM_BAD_ARGUMENT;
  // about four columns per thread: a row's loads are under way together
  int threads = ((width / 4 + 31) / 32) * 32;
  threads = threads < 64 ? 64 : threads > 1024 ? 1024 : threads;
  if (dtype == LRM_F32)
    LRM_LAUNCH(token_shift_kernel<float>, tokens, threads, 0, stream, static_cast<const float*>(h), mix, last,
               static_cast<float*>(out), cu_seqlens, seq_of_token, slots, width);
  else if (dtype == LRM_BF16)
    LRM_LAUNCH(token_shift_kernel<__nv_bfloat16>, tokens, threads, 0, stream, static_cast<const __nv_bfloat16*>(h),
               mix, last, static_cast<__nv_bfloat16*>(out), cu_seqlens, seq_of_token, slots, width);
  else
    return LRM_BAD_ARGUMENT;
  return 0;
}

LRM_API int lrm_scaled_add(float* x, const float* y, const float* factor, long long rows, int width,
                           cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (x == nullptr || y == nullptr || factor == nullptr || width <= 0) return LRM_BAD_ARGUMENT;
  const size_t n = static_cast<size_t>(rows) * width;
  LRM_LAUNCH(scaled_add_kernel, static_cast<unsigned>((n + 255) / 256), 256, 0, stream, x, y, factor, width, n);
  return 0;
}

// w has w_dtype, out out_dtype (float32 or bfloat16 each).
LRM_API int lrm_scaled_add_norm(float* x, const float* y, const float* factor, const void* w, int w_dtype, float eps,
                                void* out, int out_dtype, long long rows, int width, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (x == nullptr || y == nullptr || factor == nullptr || w == nullptr || out == nullptr || width <= 0)
    return LRM_BAD_ARGUMENT;
  const unsigned grid = static_cast<unsigned>(rows);
  int threads = ((width / 4 + 31) / 32) * 32;  // about four columns per thread
  threads = threads < 64 ? 64 : threads > 1024 ? 1024 : threads;
#define LRM_SAN(WT, OT)                                                                                          \
  LRM_LAUNCH((scaled_add_norm_kernel<WT, OT>), grid, threads, 0, stream, x, y, factor, static_cast<const WT*>(w), eps, \
             static_cast<OT*>(out), width)
  if (w_dtype == LRM_F32 && out_dtype == LRM_F32)
    LRM_SAN(float, float);
  else if (w_dtype == LRM_BF16 && out_dtype == LRM_BF16)
    LRM_SAN(__nv_bfloat16, __nv_bfloat16);
  else if (w_dtype == LRM_F32 && out_dtype == LRM_BF16)
    LRM_SAN(float, __nv_bfloat16);
  else if (w_dtype == LRM_BF16 && out_dtype == LRM_F32)
    LRM_SAN(__nv_bfloat16, float);
  else
    return LRM_BAD_ARGUMENT;
#undef LRM_SAN
  return 0;
}

// planes: float32 [count, tokens, out_width] or null (count 0).
LRM_API int lrm_row_gate(float* y, const void* x, int x_dtype, const float* w, int tokens, int in_width, int out_width,
                         const float* planes, int count, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (y == nullptr || w == nullptr || in_width <= 0 || out_width <= 0 || count < 0 || (count > 0 && planes == nullptr))
    return LRM_BAD_ARGUMENT;
  const size_t plane = static_cast<size_t>(tokens) * out_width;
  // about four CTAs per SM in all, a CTA per 256 columns at most
  int tiles = (592 + tokens - 1) / tokens;
  if (tiles > (out_width + 255) / 256) tiles = (out_width + 255) / 256;
  if (tiles < 1) tiles = 1;
  const dim3 grid(tokens, tiles);
  if (x_dtype == LRM_F32)
    LRM_LAUNCH(row_gate_kernel<float>, grid, 256, 0, stream, y, static_cast<const float*>(x), w, in_width, out_width,
               planes, count, plane);
  else if (x_dtype == LRM_BF16)
    LRM_LAUNCH(row_gate_kernel<__nv_bfloat16>, grid, 256, 0, stream, y, static_cast<const __nv_bfloat16*>(x), w,
               in_width, out_width, planes, count, plane);
  else
    return LRM_BAD_ARGUMENT;
  return 0;
}
