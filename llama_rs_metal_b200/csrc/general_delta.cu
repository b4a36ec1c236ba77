// Inputs of the generalized delta rule (the scan itself is the state scan of recurrent_scan.cu):
// per token and head, from the fused projection row [.. r (H d) .. k (H d) .. v (H dv) .. a (H d) ..]
// and the decay's pre-activation z [T, H d] (float32):
//   g    = exp(-decay_scale * sigmoid(z + z_bias))        the decay per key channel
//   look = k / sqrt(sum k^2 + unit_eps)                   the unit key, along which the state is read
//   put  = -sigmoid(a + a_bias) * look                    what is written back along it
// and r, k, v widened to float32. Everything after the projections is float32.
#include "common.cuh"

namespace {

template <typename A>
__global__ void general_delta_prepare_kernel(const A* proj, long long stride, int r_off, int k_off, int v_off,
                                             int a_off, const float* z, const float* __restrict__ z_bias,
                                             const float* __restrict__ a_bias, float decay_scale, float unit_eps,
                                             float* __restrict__ rf, float* __restrict__ kf, float* __restrict__ vf,
                                             float* __restrict__ gf, float* __restrict__ look,
                                             float* __restrict__ put, int H, int d, int dv) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const A* row = proj + static_cast<size_t>(t) * stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float k = to_f32(row[k_off + h * d + i]);
    ss = fmaf(k, k, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) + unit_eps);
  const size_t o = (static_cast<size_t>(t) * H + h) * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const int c = h * d + i;
    const float k = to_f32(row[k_off + c]);
    const float unit = k * inv;
    const float rate = 1.0f / (1.0f + expf(-(to_f32(row[a_off + c]) + a_bias[c])));
    const float zz = z[static_cast<size_t>(t) * H * d + c] + z_bias[c];
    rf[o + i] = to_f32(row[r_off + c]);
    kf[o + i] = k;
    look[o + i] = unit;
    put[o + i] = -(rate * unit);
    gf[o + i] = expf(-decay_scale * (1.0f / (1.0f + expf(-zz))));
  }
  for (int j = threadIdx.x; j < dv; j += blockDim.x)
    vf[(static_cast<size_t>(t) * H + h) * dv + j] = to_f32(row[v_off + h * dv + j]);
}

}  // namespace

LRM_API int lrm_general_delta_prepare(const void* proj, int dtype, long long stride, int r_off, int k_off, int v_off,
                                      int a_off, const float* z, const float* z_bias, const float* a_bias,
                                      float decay_scale, float unit_eps, float* rf, float* kf, float* vf, float* gf,
                                      float* look, float* put, int tokens, int H, int d, int dv,
                                      cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (H <= 0 || H > 65535 || d <= 0 || dv <= 0 || z == nullptr || z_bias == nullptr || a_bias == nullptr)
    return LRM_BAD_ARGUMENT;
  const dim3 grid(tokens, H);
  const int widest = d > dv ? d : dv;
  const int threads = widest >= 256 ? 256 : ((widest + 31) / 32) * 32;
  if (dtype == LRM_F32)
    LRM_LAUNCH(general_delta_prepare_kernel<float>, grid, threads, 0, stream, static_cast<const float*>(proj), stride,
               r_off, k_off, v_off, a_off, z, z_bias, a_bias, decay_scale, unit_eps, rf, kf, vf, gf, look, put, H, d,
               dv);
  else if (dtype == LRM_BF16)
    LRM_LAUNCH(general_delta_prepare_kernel<__nv_bfloat16>, grid, threads, 0, stream,
               static_cast<const __nv_bfloat16*>(proj), stride, r_off, k_off, v_off, a_off, z, z_bias, a_bias,
               decay_scale, unit_eps, rf, kf, vf, gf, look, put, H, d, dv);
  else
    return LRM_BAD_ARGUMENT;
  return 0;
}
