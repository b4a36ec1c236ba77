// What latent attention does to a token's fused down-projection before any attention runs.
//
// The projection row holds, at given columns: the query latent (q_rank columns), optionally the
// key/value latent (kv_rank columns) followed by one key part of `rot` columns that all heads
// share and that is rotated by position, and `gates` gate pre-activations (one per head, or one
// per head and value dimension). One CTA per token:
//   cq   = RMSnorm(query latent) * wq                       -> [T, q_rank], activation type
//          (without wq: the q_rank columns as they are, for a design whose queries have no latent)
//   row  = [RMSnorm(key/value latent) * wc | rotate(shared key part)]
//          -> [T, kv_rank + rot] packed (a prompt attends to its own rows), and into the paged
//             cache (one key head of width kv_rank + rot; the values are its first kv_rank columns)
//   gate = sigmoid(gate pre-activation)                      -> [T, gates], float32
// Norm statistics, the rotation's angle (float(position) * inv_freq[i], pairs i, i + rot/2) and
// the gate are float32. A layer that reads another layer's latent has no key/value columns
// (c_off < 0) and writes no row. dest_rows[t] = page * page_size + row in page, < 0: not kept.
#include "common.cuh"

namespace {

template <typename S, typename A>
__global__ __launch_bounds__(256) void latent_prepare_kernel(
    const S* __restrict__ proj, long long stride, int q_off, int q_rank, const float* __restrict__ wq, int c_off,
    int kv_rank, const float* __restrict__ wc, int rot, const int* __restrict__ positions,
    const float* __restrict__ inv_freq, float eps, A* __restrict__ cq_out, A* __restrict__ row_out,
    A* __restrict__ pages, const int* __restrict__ dest_rows, int g_off, int heads, float* __restrict__ gate_out) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const S* src = proj + static_cast<size_t>(t) * stride;
  if (wq != nullptr) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
      const float v = to_f32(src[q_off + i]);
      ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / static_cast<float>(q_rank) + eps);
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
      cq_out[static_cast<size_t>(t) * q_rank + i] = from_f32<A>((to_f32(src[q_off + i]) * inv) * wq[i]);
  } else {
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
      cq_out[static_cast<size_t>(t) * q_rank + i] = from_f32<A>(to_f32(src[q_off + i]));
  }
  for (int h = threadIdx.x; h < heads; h += blockDim.x)
    gate_out[static_cast<size_t>(t) * heads + h] = 1.0f / (1.0f + expf(-to_f32(src[g_off + h])));
  if (c_off < 0) return;
  const int width = kv_rank + rot;
  const int dest = (pages != nullptr && dest_rows != nullptr) ? dest_rows[t] : -1;
  A* packed = row_out != nullptr ? row_out + static_cast<size_t>(t) * width : nullptr;
  A* cached = dest >= 0 ? pages + static_cast<size_t>(dest) * width : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
    const float v = to_f32(src[c_off + i]);
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / static_cast<float>(kv_rank) + eps);
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
    const A v = from_f32<A>((to_f32(src[c_off + i]) * inv) * wc[i]);
    if (packed != nullptr) packed[i] = v;
    if (cached != nullptr) cached[i] = v;
  }
  const int half = rot / 2;
  const float fpos = static_cast<float>(positions[t]);
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    sincosf(__fmul_rn(fpos, inv_freq[i]), &sn, &cs);
    const float u = to_f32(src[c_off + kv_rank + i]), v = to_f32(src[c_off + kv_rank + i + half]);
    const A lo = from_f32<A>(u * cs - v * sn), hi = from_f32<A>(v * cs + u * sn);
    if (packed != nullptr) packed[kv_rank + i] = lo, packed[kv_rank + i + half] = hi;
    if (cached != nullptr) cached[kv_rank + i] = lo, cached[kv_rank + i + half] = hi;
  }
}

}  // namespace

LRM_API int lrm_latent_prepare(const void* proj, int proj_dtype, long long stride, int q_off, int q_rank,
                               const float* wq, int c_off, int kv_rank, const float* wc, int rot,
                               const int* positions, const float* inv_freq, float eps, void* cq_out, void* row_out,
                               void* pages, const int* dest_rows, int g_off, int heads, float* gate_out,
                               int out_dtype, int tokens, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (proj == nullptr || q_rank < 0 || (q_rank > 0 && cq_out == nullptr) || heads <= 0 || gate_out == nullptr ||
      !(eps > 0.f))
    return LRM_BAD_ARGUMENT;
  if (c_off >= 0 && (kv_rank <= 0 || wc == nullptr || rot < 0 || rot % 2 ||
                     (rot > 0 && (positions == nullptr || inv_freq == nullptr))))
    return LRM_BAD_ARGUMENT;
#define LRM_LATENT(ST, AT)                                                                                       \
  do {                                                                                                           \
    LRM_LAUNCH((latent_prepare_kernel<ST, AT>), tokens, 256, 0, stream, static_cast<const ST*>(proj), stride,   \
               q_off, q_rank, wq, c_off, kv_rank, wc, rot, positions, inv_freq, eps, static_cast<AT*>(cq_out),   \
               static_cast<AT*>(row_out), static_cast<AT*>(pages), dest_rows, g_off, heads, gate_out);           \
    return 0;                                                                                                    \
  } while (0)
  if (proj_dtype == LRM_F32 && out_dtype == LRM_F32) LRM_LATENT(float, float);
  if (proj_dtype == LRM_F32 && out_dtype == LRM_BF16) LRM_LATENT(float, __nv_bfloat16);
  if (proj_dtype == LRM_BF16 && out_dtype == LRM_BF16) LRM_LATENT(__nv_bfloat16, __nv_bfloat16);
#undef LRM_LATENT
  return LRM_BAD_ARGUMENT;
}
