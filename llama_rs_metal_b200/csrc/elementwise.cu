// Small elementwise kernels: the SiLU gate, the residual add and dtype casts.
#include "common.cuh"

// out[t, c] = silu(gate) * up where the 2I columns of `gate_up` come in
// alternating blocks of `block` gate columns and `block` up columns
// (block == I is plain [gate | up] concatenation).
// silu(g) = g / (1 + exp(-g))  (reference: elementwise.metal:8-17).
template <typename A>
__global__ void silu_mul_kernel(const A* __restrict__ gate_up, A* __restrict__ out, size_t total,
                                int inter, int block) {
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / inter;
  const int c = static_cast<int>(idx % inter);
  const size_t base = t * 2 * inter + static_cast<size_t>(c / block) * 2 * block + c % block;
  const float g = to_f32(gate_up[base]), u = to_f32(gate_up[base + block]);
  out[idx] = from_f32<A>(g / (1.0f + expf(-g)) * u);
}

// The clamped gate: g = min(gate, limit), u = clamp(up, -limit, limit),
// out = g * sigmoid(alpha * g) * (u + 1), from the same column layout. The input may be float32
// while the output has the activation type (a product that keeps its sums until the activation).
template <typename S, typename A>
__global__ void clamped_gate_mul_kernel(const S* __restrict__ gate_up, A* __restrict__ out, size_t total,
                                        int inter, int block, float limit, float alpha) {
  pdl_trigger();
  pdl_wait();
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / inter;
  const int c = static_cast<int>(idx % inter);
  const size_t base = t * 2 * inter + static_cast<size_t>(c / block) * 2 * block + c % block;
  const float g = fminf(to_f32(gate_up[base]), limit);
  const float u = fminf(fmaxf(to_f32(gate_up[base + block]), -limit), limit);
  out[idx] = from_f32<A>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
}

// The same for blocks of 8 with float32 input and bfloat16 output (a product's float32 gate and
// up columns): a thread takes one block, 64 bytes in and 16 out, with 16-byte accesses.
__global__ void clamped_gate_mul8_kernel(const float* __restrict__ gate_up, __nv_bfloat16* __restrict__ out,
                                         size_t groups, int groups_per_row, float limit, float alpha) {
  pdl_trigger();
  pdl_wait();
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx >= groups) return;
  const float4* src = reinterpret_cast<const float4*>(gate_up) + idx * 4;  // 8 gate, then 8 up
  const float4 g0 = src[0], g1 = src[1], u0 = src[2], u1 = src[3];
  const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
  const float u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
  uint32_t packed[4];
#pragma unroll
  for (int i = 0; i < 8; i += 2) {
    float y[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const float gc = fminf(g[i + j], limit), uc = fminf(fmaxf(u[i + j], -limit), limit);
      y[j] = gc / (1.0f + expf(-alpha * gc)) * (uc + 1.0f);
    }
    __nv_bfloat162 v = __floats2bfloat162_rn(y[0], y[1]);
    packed[i >> 1] = *reinterpret_cast<uint32_t*>(&v);
  }
  reinterpret_cast<uint4*>(out)[idx] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
}

// out = max(x, 0)^2, the activation of a feed-forward without a gate; the input may be float32 (a
// product that keeps its sums until the activation) while the output has the activation type.
template <typename S, typename A>
__global__ void relu_squared_kernel(const S* __restrict__ src, A* __restrict__ out, size_t n) {
  pdl_trigger();
  pdl_wait();
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx >= n) return;
  const float v = fmaxf(to_f32(src[idx]), 0.f);
  out[idx] = from_f32<A>(v * v);
}

// four elements per thread with 16-byte loads: float32 in, bfloat16 out
__global__ void relu_squared4_kernel(const float4* __restrict__ src, uint2* __restrict__ out, size_t groups) {
  pdl_trigger();
  pdl_wait();
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx >= groups) return;
  const float4 x = src[idx];
  const float a = fmaxf(x.x, 0.f), b = fmaxf(x.y, 0.f), c = fmaxf(x.z, 0.f), d = fmaxf(x.w, 0.f);
  __nv_bfloat162 lo = __floats2bfloat162_rn(a * a, b * b), hi = __floats2bfloat162_rn(c * c, d * d);
  out[idx] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
}

template <typename D>
__global__ void add_inplace_kernel(float* __restrict__ x, const D* __restrict__ delta, size_t n) {
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx < n) x[idx] += to_f32(delta[idx]);
}

// x += planes[0] + planes[1] + ... in plane order (the K slices of a product whose sum belongs
// to the residual stream), for a reader of the stream that cannot fold them itself.
__global__ void add_planes_kernel(float* __restrict__ x, const float* __restrict__ planes, int count,
                                  size_t n) {
  pdl_trigger();
  pdl_wait();
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx >= n) return;
  float v = x[idx];
  for (int p = 0; p < count; ++p) v += planes[p * n + idx];
  x[idx] = v;
}

template <typename S, typename D>
__global__ void cast_kernel(const S* __restrict__ src, D* __restrict__ dst, size_t n) {
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx < n) dst[idx] = from_f32<D>(to_f32(src[idx]));
}

static unsigned blocks_for(size_t n) { return static_cast<unsigned>((n + 255) / 256); }

LRM_API int lrm_silu_mul(const void* gate_up, void* out, int dtype, long long rows, int inter,
                         int block, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (inter <= 0 || block <= 0 || inter % block != 0) return LRM_BAD_ARGUMENT;
  const size_t total = static_cast<size_t>(rows) * inter;
  if (dtype == LRM_F32)
    silu_mul_kernel<float><<<blocks_for(total), 256, 0, stream>>>(
        static_cast<const float*>(gate_up), static_cast<float*>(out), total, inter, block);
  else if (dtype == LRM_BF16)
    silu_mul_kernel<__nv_bfloat16><<<blocks_for(total), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(out), total, inter,
        block);
  else
    return LRM_BAD_ARGUMENT;
  LRM_LAUNCH_CHECK();
  return 0;
}

LRM_API int lrm_clamped_gate_mul(const void* gate_up, int in_dtype, void* out, int out_dtype, long long rows,
                                 int inter, int block, float limit, float alpha, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (inter <= 0 || block <= 0 || inter % block != 0) return LRM_BAD_ARGUMENT;
  const size_t total = static_cast<size_t>(rows) * inter;
  if (in_dtype == LRM_F32 && out_dtype == LRM_BF16 && block == 8 &&
      reinterpret_cast<uintptr_t>(gate_up) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0) {
    LRM_LAUNCH(clamped_gate_mul8_kernel, blocks_for(total / 8), 256, 0, stream, static_cast<const float*>(gate_up),
               static_cast<__nv_bfloat16*>(out), total / 8, inter / 8, limit, alpha);
    return 0;
  }
  if (in_dtype == LRM_F32 && out_dtype == LRM_F32)
    LRM_LAUNCH((clamped_gate_mul_kernel<float, float>), blocks_for(total), 256, 0, stream,
               static_cast<const float*>(gate_up), static_cast<float*>(out), total, inter, block, limit, alpha);
  else if (in_dtype == LRM_F32 && out_dtype == LRM_BF16)
    LRM_LAUNCH((clamped_gate_mul_kernel<float, __nv_bfloat16>), blocks_for(total), 256, 0, stream,
               static_cast<const float*>(gate_up), static_cast<__nv_bfloat16*>(out), total, inter, block, limit,
               alpha);
  else if (in_dtype == LRM_BF16 && out_dtype == LRM_BF16)
    LRM_LAUNCH((clamped_gate_mul_kernel<__nv_bfloat16, __nv_bfloat16>), blocks_for(total), 256, 0, stream,
               static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(out), total, inter, block,
               limit, alpha);
  else
    return LRM_BAD_ARGUMENT;
  return 0;
}

LRM_API int lrm_relu_squared(const void* src, int in_dtype, void* out, int out_dtype, long long n,
                             cudaStream_t stream) {
  if (n <= 0) return 0;
  const size_t total = static_cast<size_t>(n);
  if (in_dtype == LRM_F32 && out_dtype == LRM_BF16 && total % 4 == 0 &&
      reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 8 == 0) {
    LRM_LAUNCH(relu_squared4_kernel, blocks_for(total / 4), 256, 0, stream, static_cast<const float4*>(src),
               static_cast<uint2*>(out), total / 4);
    return 0;
  }
  if (in_dtype == LRM_F32 && out_dtype == LRM_F32)
    LRM_LAUNCH((relu_squared_kernel<float, float>), blocks_for(total), 256, 0, stream,
               static_cast<const float*>(src), static_cast<float*>(out), total);
  else if (in_dtype == LRM_F32 && out_dtype == LRM_BF16)
    LRM_LAUNCH((relu_squared_kernel<float, __nv_bfloat16>), blocks_for(total), 256, 0, stream,
               static_cast<const float*>(src), static_cast<__nv_bfloat16*>(out), total);
  else if (in_dtype == LRM_BF16 && out_dtype == LRM_BF16)
    LRM_LAUNCH((relu_squared_kernel<__nv_bfloat16, __nv_bfloat16>), blocks_for(total), 256, 0, stream,
               static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(out), total);
  else
    return LRM_BAD_ARGUMENT;
  return 0;
}

LRM_API int lrm_add_inplace(float* x, const void* delta, int delta_dtype, long long n,
                            cudaStream_t stream) {
  if (n <= 0) return 0;
  if (delta_dtype == LRM_F32)
    add_inplace_kernel<float><<<blocks_for(n), 256, 0, stream>>>(x, static_cast<const float*>(delta), n);
  else if (delta_dtype == LRM_BF16)
    add_inplace_kernel<__nv_bfloat16><<<blocks_for(n), 256, 0, stream>>>(
        x, static_cast<const __nv_bfloat16*>(delta), n);
  else
    return LRM_BAD_ARGUMENT;
  LRM_LAUNCH_CHECK();
  return 0;
}

__global__ void scale_inplace_kernel(float* __restrict__ x, float factor, size_t n) {
  pdl_trigger();
  pdl_wait();
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx < n) x[idx] *= factor;
}

LRM_API int lrm_scale_inplace(float* x, float factor, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (x == nullptr) return LRM_BAD_ARGUMENT;
  LRM_LAUNCH(scale_inplace_kernel, blocks_for(n), 256, 0, stream, x, factor, static_cast<size_t>(n));
  return 0;
}

// x[t, :] += row[:] for every row t of x [rows, width] (a vector added to the whole residual stream).
__global__ void add_row_kernel(float* __restrict__ x, const float* __restrict__ row, int width, size_t n) {
  pdl_trigger();
  pdl_wait();
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx < n) x[idx] += row[idx % width];
}

LRM_API int lrm_add_row(float* x, const float* row, long long rows, int width, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (x == nullptr || row == nullptr || width <= 0) return LRM_BAD_ARGUMENT;
  const size_t n = static_cast<size_t>(rows) * width;
  LRM_LAUNCH(add_row_kernel, blocks_for(n), 256, 0, stream, x, row, width, n);
  return 0;
}

LRM_API int lrm_add_planes(float* x, const float* planes, int count, long long n, cudaStream_t stream) {
  if (n <= 0 || count <= 0) return 0;
  if (x == nullptr || planes == nullptr) return LRM_BAD_ARGUMENT;
  LRM_LAUNCH(add_planes_kernel, blocks_for(n), 256, 0, stream, x, planes, count, static_cast<size_t>(n));
  return 0;
}

LRM_API int lrm_cast(const void* src, int src_dtype, void* dst, int dst_dtype, long long n,
                     cudaStream_t stream) {
  if (n <= 0) return 0;
  if (src_dtype == LRM_F32 && dst_dtype == LRM_BF16)
    cast_kernel<float, __nv_bfloat16><<<blocks_for(n), 256, 0, stream>>>(
        static_cast<const float*>(src), static_cast<__nv_bfloat16*>(dst), n);
  else if (src_dtype == LRM_BF16 && dst_dtype == LRM_F32)
    cast_kernel<__nv_bfloat16, float><<<blocks_for(n), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(src), static_cast<float*>(dst), n);
  else
    return LRM_BAD_ARGUMENT;
  LRM_LAUNCH_CHECK();
  return 0;
}


// The tanh form of GELU as a gate: out = gelu(gate) * up with gelu(z) = 0.5 z (1 + tanh(sqrt(2/pi)
// (z + 0.044715 z^3))), from the gate/up column layout of silu_mul. The input may be float32 while
// the output has the activation type (a product that keeps its sums until the activation).
template <typename S, typename A>
__global__ void gelu_tanh_mul_kernel(const S* gate_up, A* __restrict__ out, size_t total, int inter, int block) {
  pdl_trigger();
  pdl_wait();
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / inter;
  const int c = static_cast<int>(idx % inter);
  const size_t base = t * 2 * inter + static_cast<size_t>(c / block) * 2 * block + c % block;
  const float g = to_f32(gate_up[base]), u = to_f32(gate_up[base + block]);
  const float inner = 0.7978845608028654f * fmaf(0.044715f * g * g, g, g);
  out[idx] = from_f32<A>(0.5f * g * (1.0f + tanhf(inner)) * u);
}

LRM_API int lrm_gelu_tanh_mul(const void* gate_up, int in_dtype, void* out, int out_dtype, long long rows, int inter,
                              int block, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (inter <= 0 || block <= 0 || inter % block != 0) return LRM_BAD_ARGUMENT;
  const size_t total = static_cast<size_t>(rows) * inter;
  if (in_dtype == LRM_F32 && out_dtype == LRM_F32)
    LRM_LAUNCH((gelu_tanh_mul_kernel<float, float>), blocks_for(total), 256, 0, stream,
               static_cast<const float*>(gate_up), static_cast<float*>(out), total, inter, block);
  else if (in_dtype == LRM_F32 && out_dtype == LRM_BF16)
    LRM_LAUNCH((gelu_tanh_mul_kernel<float, __nv_bfloat16>), blocks_for(total), 256, 0, stream,
               static_cast<const float*>(gate_up), static_cast<__nv_bfloat16*>(out), total, inter, block);
  else if (in_dtype == LRM_BF16 && out_dtype == LRM_BF16)
    LRM_LAUNCH((gelu_tanh_mul_kernel<__nv_bfloat16, __nv_bfloat16>), blocks_for(total), 256, 0, stream,
               static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(out), total, inter, block);
  else
    return LRM_BAD_ARGUMENT;
  return 0;
}

// out[t, c] = tanh(src[t * stride + c]) for c < width: some columns of a wider activation through
// tanh, rounded to the output type (the inner activation of a low-rank product).
template <typename S, typename A>
__global__ void tanh_columns_kernel(const S* src, long long stride, A* __restrict__ out, int width, size_t total) {
  pdl_trigger();
  pdl_wait();
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / width;
  out[idx] = from_f32<A>(tanhf(to_f32(src[t * stride + idx % width])));
}

LRM_API int lrm_tanh_columns(const void* src, int in_dtype, long long stride, void* out, int out_dtype, long long rows,
                             int width, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (width <= 0 || stride < width) return LRM_BAD_ARGUMENT;
  const size_t total = static_cast<size_t>(rows) * width;
  if (in_dtype == LRM_F32 && out_dtype == LRM_F32)
    LRM_LAUNCH((tanh_columns_kernel<float, float>), blocks_for(total), 256, 0, stream, static_cast<const float*>(src),
               stride, static_cast<float*>(out), width, total);
  else if (in_dtype == LRM_F32 && out_dtype == LRM_BF16)
    LRM_LAUNCH((tanh_columns_kernel<float, __nv_bfloat16>), blocks_for(total), 256, 0, stream,
               static_cast<const float*>(src), stride, static_cast<__nv_bfloat16*>(out), width, total);
  else if (in_dtype == LRM_BF16 && out_dtype == LRM_BF16)
    LRM_LAUNCH((tanh_columns_kernel<__nv_bfloat16, __nv_bfloat16>), blocks_for(total), 256, 0, stream,
               static_cast<const __nv_bfloat16*>(src), stride, static_cast<__nv_bfloat16*>(out), width, total);
  else
    return LRM_BAD_ARGUMENT;
  return 0;
}
