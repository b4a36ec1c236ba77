// Block-diagonal products and a rotation of a part of every head.
//
// blockwise_linear: the input row is cut into B blocks, and block b is multiplied by a matrix of
// its own:  out[t, b, :] = (W[b] x[t, b, :] + bias[b, :]) * row_scale[t, b]   with W [B, n, m]
// (row_scale one number per token and block, or, with scale_cols = n, one per output: [T, B, n])
// stored [out, in] per block. Rows and blocks of x and of out are addressed by strides (in
// elements), so a block may be a part of a wider head and the result may land beside other
// columns. Gates of a recurrence computed per block of channels, and the per-head matrices of
// latent attention (a query head folded into the latent space, a head's output unfolded from
// it), are such products. Sums are float32 in an order that depends on the input index only, so a
// row's result does not depend on the rows beside it.
//
// rope_heads: copies `rot` columns of every head, rotated by position (pairs i, i + rot/2,
// angle = float(position) * inv_freq[i]), from one strided layout to another.
// bfloat16 inputs whose blocks start on 16-byte boundaries (m a multiple of 8) run on the
// warp-level tensor path: a CTA computes 64 tokens x 64 outputs of one block, 32 inputs at a time
// through double-buffered shared tiles (cp.async, ldmatrix, mma.sync m16n8k16, float32 sums);
// everything else, and float32, runs the plain tiled kernel.
#include "attention_mma.cuh"

namespace {

constexpr int kMmaDepth = 32, kMmaStride = kMmaDepth + 8;

template <typename O>
__global__ __launch_bounds__(kThreads) void blockwise_linear_mma_kernel(
    const __nv_bfloat16* __restrict__ x, long long x_row, long long x_block, const __nv_bfloat16* __restrict__ w,
    const float* __restrict__ bias, const float* __restrict__ row_scale, int scale_cols, O* __restrict__ out,
    long long out_row,
    long long out_block, int T, int B, int n, int m) {
  __shared__ __align__(16) __nv_bfloat16 xs[2][kTile * kMmaStride];
  __shared__ __align__(16) __nv_bfloat16 ws[2][kTile * kMmaStride];
  const int b = blockIdx.y, t0 = blockIdx.z * kTile, n0 = blockIdx.x * kTile;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const __nv_bfloat16* xb = x + static_cast<size_t>(b) * x_block;
  const __nv_bfloat16* wb = w + static_cast<size_t>(b) * n * m;
  auto issue = [&](int k0, int stage) {
    for (int idx = threadIdx.x; idx < kTile * (kMmaDepth / 8); idx += kThreads) {
      const int r = idx / (kMmaDepth / 8), c = 8 * (idx % (kMmaDepth / 8));
      const bool in_k = k0 + c < m;
      const bool x_ok = in_k && t0 + r < T, w_ok = in_k && n0 + r < n;
      cp_async16(&xs[stage][r * kMmaStride + c], x_ok ? xb + static_cast<size_t>(t0 + r) * x_row + k0 + c : xb,
                 x_ok ? 16 : 0);
      cp_async16(&ws[stage][r * kMmaStride + c], w_ok ? wb + static_cast<size_t>(n0 + r) * m + k0 + c : wb,
                 w_ok ? 16 : 0);
    }
    cp_async_commit();
  };
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
  pdl_wait();
  const int steps = (m + kMmaDepth - 1) / kMmaDepth;
  issue(0, 0);
  for (int ki = 0; ki < steps; ++ki) {
    const int stage = ki & 1;
    if (ki + 1 < steps) {
      issue((ki + 1) * kMmaDepth, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kMmaDepth / 16; ++kk) {
      uint32_t a[4];
      ldsm_x4(a[0], a[1], a[2], a[3],
              &xs[stage][(16 * warp + (lane & 7) + 8 * ((lane >> 3) & 1)) * kMmaStride + 16 * kk + 8 * (lane >> 4)]);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(b0, b1, b2, b3,
                &ws[stage][(16 * np + (lane & 7) + 8 * (lane >> 4)) * kMmaStride + 16 * kk + 8 * ((lane >> 3) & 1)]);
        mma16816(acc[2 * np], a, b0, b1);
        mma16816(acc[2 * np + 1], a, b2, b3);
      }
    }
    __syncthreads();
  }
  pdl_trigger();
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = t0 + 16 * warp + g + 8 * half;
    if (row >= T) continue;
    const float* scales = row_scale != nullptr ? row_scale + (static_cast<size_t>(row) * B + b) * scale_cols : nullptr;
    O* dst = out + static_cast<size_t>(row) * out_row + static_cast<size_t>(b) * out_block;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int c = n0 + 8 * j + 2 * t + e;
        if (c >= n) continue;
        float v = acc[j][2 * half + e];
        if (bias != nullptr) v += bias[static_cast<size_t>(b) * n + c];
        if (scales != nullptr) v *= scales[scale_cols > 1 ? c : 0];
        dst[c] = from_f32<O>(v);
      }
    }
  }
}

constexpr int kRows = 32, kCols = 64, kDepth = 32;  // tile: 32 tokens x 64 outputs, 32 inputs at a time

template <typename X, typename WT, typename O>
__global__ __launch_bounds__(256) void blockwise_linear_kernel(
    const X* __restrict__ x, long long x_row, long long x_block, const WT* __restrict__ w,
    const float* __restrict__ bias, const float* __restrict__ row_scale, int scale_cols, O* __restrict__ out,
    long long out_row,
    long long out_block, int T, int B, int n, int m) {
  __shared__ float xs[kRows][kDepth + 1];
  __shared__ float ws[kDepth][kCols + 1];
  const int b = blockIdx.y, t0 = blockIdx.z * kRows, n0 = blockIdx.x * kCols;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // outputs 4 tx .. 4 tx + 3 of rows 2 ty, 2 ty + 1
  const WT* wb = w + static_cast<size_t>(b) * n * m;
  float acc[2][4] = {};
  pdl_wait();
  for (int k0 = 0; k0 < m; k0 += kDepth) {
    for (int i = threadIdx.x; i < kRows * kDepth; i += 256) {
      const int r = i / kDepth, k = i % kDepth;
      xs[r][k] = (t0 + r < T && k0 + k < m)
                     ? to_f32(x[static_cast<size_t>(t0 + r) * x_row + static_cast<size_t>(b) * x_block + k0 + k])
                     : 0.f;
    }
    for (int i = threadIdx.x; i < kCols * kDepth; i += 256) {
      const int c = i / kDepth, k = i % kDepth;
      ws[k][c] = (n0 + c < n && k0 + k < m) ? to_f32(wb[static_cast<size_t>(n0 + c) * m + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kDepth; ++k) {
      const float x0 = xs[2 * ty][k], x1 = xs[2 * ty + 1][k];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float wv = ws[k][4 * tx + j];
        acc[0][j] = fmaf(x0, wv, acc[0][j]);
        acc[1][j] = fmaf(x1, wv, acc[1][j]);
      }
    }
    __syncthreads();
  }
  pdl_trigger();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int t = t0 + 2 * ty + r;
    if (t >= T) continue;
    const float* scales = row_scale != nullptr ? row_scale + (static_cast<size_t>(t) * B + b) * scale_cols : nullptr;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = n0 + 4 * tx + j;
      if (c >= n) continue;
      float v = acc[r][j];
      if (bias != nullptr) v += bias[static_cast<size_t>(b) * n + c];
      if (scales != nullptr) v *= scales[scale_cols > 1 ? c : 0];
      out[static_cast<size_t>(t) * out_row + static_cast<size_t>(b) * out_block + c] = from_f32<O>(v);
    }
  }
}

template <typename A>
__global__ void rope_heads_kernel(const A* __restrict__ src, long long src_row, long long src_head,
                                  A* __restrict__ dst, long long dst_row, long long dst_head,
                                  const int* __restrict__ positions, const float* __restrict__ inv_freq, int rot,
                                  int heads, size_t total) {
  pdl_trigger();
  pdl_wait();
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx >= total) return;
  const int half = rot / 2;
  const int i = static_cast<int>(idx % half), h = static_cast<int>((idx / half) % heads);
  const size_t t = idx / half / heads;
  const float angle = __fmul_rn(static_cast<float>(positions[t]), inv_freq[i]);
  float sn, cs;
  sincosf(angle, &sn, &cs);
  const A* s = src + t * src_row + static_cast<size_t>(h) * src_head;
  A* d = dst + t * dst_row + static_cast<size_t>(h) * dst_head;
  const float u = to_f32(s[i]), v = to_f32(s[i + half]);
  d[i] = from_f32<A>(u * cs - v * sn);
  d[i + half] = from_f32<A>(v * cs + u * sn);
}

}  // namespace

// x_dtype / w_dtype / out_dtype: the activation's, the matrices' and the result's types; the
// supported combinations are all-float32, and bfloat16 x and w with a bfloat16 or float32 result.
LRM_API int lrm_blockwise_linear(const void* x, int x_dtype, long long x_row, long long x_block, const void* w,
                                 int w_dtype, const float* bias, const float* row_scale, int scale_cols, void* out,
                                 int out_dtype,
                                 long long out_row, long long out_block, int tokens, int blocks, int n, int m,
                                 cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (blocks <= 0 || n <= 0 || m <= 0 || x == nullptr || w == nullptr || out == nullptr) return LRM_BAD_ARGUMENT;
  if (row_scale != nullptr && scale_cols != 1 && scale_cols != n) return LRM_BAD_ARGUMENT;
  const int row_tiles = (tokens + kRows - 1) / kRows;
  if (blocks > 65535 || row_tiles > 65535) return LRM_UNSUPPORTED;
  auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  if (x_dtype == LRM_BF16 && w_dtype == LRM_BF16 && m % 8 == 0 && x_row % 8 == 0 && x_block % 8 == 0 && aligned(x) &&
      aligned(w)) {
    const dim3 mma_grid((n + kTile - 1) / kTile, blocks, (tokens + kTile - 1) / kTile);
    if (out_dtype == LRM_BF16) {
      LRM_LAUNCH(blockwise_linear_mma_kernel<__nv_bfloat16>, mma_grid, kThreads, 0, stream,
                 static_cast<const __nv_bfloat16*>(x), x_row, x_block, static_cast<const __nv_bfloat16*>(w), bias,
                 row_scale, scale_cols, static_cast<__nv_bfloat16*>(out), out_row, out_block, tokens, blocks, n, m);
      return 0;
    }
    if (out_dtype == LRM_F32) {
      LRM_LAUNCH(blockwise_linear_mma_kernel<float>, mma_grid, kThreads, 0, stream,
                 static_cast<const __nv_bfloat16*>(x), x_row, x_block, static_cast<const __nv_bfloat16*>(w), bias,
                 row_scale, scale_cols, static_cast<float*>(out), out_row, out_block, tokens, blocks, n, m);
      return 0;
    }
  }
  const dim3 grid((n + kCols - 1) / kCols, blocks, row_tiles);
#define LRM_BLOCKWISE(XT, WT, OT)                                                                               \
  do {                                                                                                          \
    LRM_LAUNCH((blockwise_linear_kernel<XT, WT, OT>), grid, 256, 0, stream, static_cast<const XT*>(x), x_row,  \
               x_block, static_cast<const WT*>(w), bias, row_scale, scale_cols, static_cast<OT*>(out), out_row,  \
               out_block,                                                                                       \
               tokens, blocks, n, m);                                                                           \
    return 0;                                                                                                   \
  } while (0)
  if (x_dtype == LRM_F32 && w_dtype == LRM_F32 && out_dtype == LRM_F32) LRM_BLOCKWISE(float, float, float);
  if (x_dtype == LRM_BF16 && w_dtype == LRM_BF16 && out_dtype == LRM_BF16)
    LRM_BLOCKWISE(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
  if (x_dtype == LRM_BF16 && w_dtype == LRM_BF16 && out_dtype == LRM_F32)
    LRM_BLOCKWISE(__nv_bfloat16, __nv_bfloat16, float);
#undef LRM_BLOCKWISE
  return LRM_BAD_ARGUMENT;
}

LRM_API int lrm_rope_heads(const void* src, int dtype, long long src_row, long long src_head, void* dst,
                           long long dst_row, long long dst_head, const int* positions, const float* inv_freq,
                           int rot, int tokens, int heads, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (rot <= 0 || rot % 2 || heads <= 0 || src == nullptr || dst == nullptr || positions == nullptr ||
      inv_freq == nullptr)
    return LRM_BAD_ARGUMENT;
  const size_t total = static_cast<size_t>(tokens) * heads * (rot / 2);
  const unsigned grid = static_cast<unsigned>((total + 255) / 256);
  if (dtype == LRM_F32)
    LRM_LAUNCH(rope_heads_kernel<float>, grid, 256, 0, stream, static_cast<const float*>(src), src_row, src_head,
               static_cast<float*>(dst), dst_row, dst_head, positions, inv_freq, rot, heads, total);
  else if (dtype == LRM_BF16)
    LRM_LAUNCH(rope_heads_kernel<__nv_bfloat16>, grid, 256, 0, stream, static_cast<const __nv_bfloat16*>(src),
               src_row, src_head, static_cast<__nv_bfloat16*>(dst), dst_row, dst_head, positions, inv_freq, rot,
               heads, total);
  else
    return LRM_BAD_ARGUMENT;
  return 0;
}
