// The split of a step's fused q|k|v projection for attention layers that shape their queries and
// keys on the way: one CTA per token takes the projection row [q_heads * d | kv_heads * d |
// kv_heads * dv] through, in this order and each only if asked for,
//   1. the projections' biases (float32 [row]);
//   2. a short causal convolution over time per channel (taps [n, row], the last row the current
//      token's, no bias, zeros before the sequence's start); inputs before the step's first token
//      come from the sequence's tail [n - 1, row] of unbiased projections in the state storage,
//      the bias added here where the input's position is not before the start;
//   3. an RMS norm over the whole query part and one over the whole key part, with weights;
//   4. a rotation by position of the first `rotary` dimensions of every query and key head,
//      dimension i paired with i + rotary/2 (pairing 0) or 2i with 2i + 1 (pairing 1), angle =
//      position * inv_freq[i] formed in double precision;
//   5. the division of every query and key head by its root mean square (no weight),
// and writes q, k, v in the activation type: q packed, k and v packed (when asked for) and into
// the paged cache at dest_rows[t] (see qkv_store.cu for the layout). Everything between the
// projection and the rounding at the end is float32. Reads of the projection go through plain
// pointers: it is the output of the kernel before.
#include "common.cuh"

namespace {

template <typename S, typename A>
__global__ void shaped_qkv_kernel(const S* proj, const float* __restrict__ bias, const float* __restrict__ taps, int n,
                                  const float* tails, const int* __restrict__ cu_seqlens,
                                  const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                                  const int* __restrict__ positions, const float* __restrict__ q_norm,
                                  const float* __restrict__ k_norm, float row_eps,
                                  const double* __restrict__ inv_freq, int rotary, int pairing, int head_norm,
                                  float head_eps, A* __restrict__ q_out, A* __restrict__ k_out,
                                  A* __restrict__ v_out, A* __restrict__ k_pages, A* __restrict__ v_pages,
                                  const int* __restrict__ dest_rows, int q_heads, int kv_heads, int d, int dv,
                                  int page_size) {
  extern __shared__ float smem[];
  __shared__ float scratch[32];
  const int nq = q_heads * d, nk = kv_heads * d, nv = kv_heads * dv;
  const int width = nq + nk + nv, half = rotary / 2;
  float* row = smem;            // [width]
  float* cs = smem + width;     // [half] cosines, then [half] sines
  pdl_trigger();
  const int t = blockIdx.x;
  const int pos = positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double sn, c;
    sincos(static_cast<double>(pos) * inv_freq[i], &sn, &c);
    cs[i] = static_cast<float>(c);
    cs[half + i] = static_cast<float>(sn);
  }
  pdl_wait();
  const S* src = proj + static_cast<size_t>(t) * width;
  if (taps == nullptr || n <= 1) {
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      float x = to_f32(src[c]) + (bias != nullptr ? bias[c] : 0.f);
      if (taps != nullptr) x *= taps[c];
      row[c] = x;
    }
  } else {
    const int b = seq_of_token[t], local = t - cu_seqlens[b], slot = slots[b];
    const float* tail = slot >= 0 ? tails + static_cast<size_t>(slot) * (n - 1) * width : nullptr;
    // a thread takes kGroup columns at a time, so that the loads of one input row are all under way
    // before the first is used (one column after another, a CTA waited for n loads in turn per column)
    constexpr int kGroup = 8;
    for (int first = 0; first < width; first += kGroup * blockDim.x) {
      float acc[kGroup], add[kGroup];
#pragma unroll
      for (int e = 0; e < kGroup; ++e) {
        const int c = first + e * blockDim.x + threadIdx.x;
        acc[e] = 0.f;
        add[e] = (bias != nullptr && c < width) ? bias[c] : 0.f;
      }
      for (int back = n - 1; back >= 0; --back) {  // oldest input first
        if (pos - back < 0) continue;              // before the sequence's start: zero
        const int at = local - back;
        const S* from_step = at >= 0 ? proj + static_cast<size_t>(t - back) * width : nullptr;
        const float* from_tail = (at < 0 && tail != nullptr) ? tail + static_cast<size_t>(n - 1 + at) * width : nullptr;
        const float* tap = taps + static_cast<size_t>(n - 1 - back) * width;
#pragma unroll
        for (int e = 0; e < kGroup; ++e) {
          const int c = first + e * blockDim.x + threadIdx.x;
          if (c < width) {
            const float x = from_step != nullptr ? to_f32(from_step[c]) : from_tail != nullptr ? from_tail[c] : 0.f;
            acc[e] = fmaf(tap[c], x + add[e], acc[e]);
          }
        }
      }
#pragma unroll
      for (int e = 0; e < kGroup; ++e) {
        const int c = first + e * blockDim.x + threadIdx.x;
        if (c < width) row[c] = acc[e];
      }
    }
  }
  __syncthreads();
  if (q_norm != nullptr) {
    float sq = 0.f, sk = 0.f;
    for (int c = threadIdx.x; c < nq + nk; c += blockDim.x) {
      const float x = row[c];
      if (c < nq) sq = fmaf(x, x, sq); else sk = fmaf(x, x, sk);
    }
    const float inv_q = 1.0f / sqrtf(block_sum(sq, scratch) / static_cast<float>(nq) + row_eps);
    const float total_k = block_sum(sk, scratch);
    const float inv_k = nk > 0 ? 1.0f / sqrtf(total_k / static_cast<float>(nk) + row_eps) : 0.f;
    for (int c = threadIdx.x; c < nq + nk; c += blockDim.x)
      row[c] = c < nq ? row[c] * inv_q * q_norm[c] : row[c] * inv_k * k_norm[c - nq];
    __syncthreads();
  }
  if (half > 0) {
    const int heads = q_heads + kv_heads;  // query heads, then key heads, are contiguous rows of d
    for (int idx = threadIdx.x; idx < heads * half; idx += blockDim.x) {
      const int hd = idx / half, i = idx % half;
      float* head = row + hd * d;
      const int a = pairing == 0 ? i : 2 * i, b2 = pairing == 0 ? i + half : 2 * i + 1;
      const float u = head[a], v = head[b2], c = cs[i], sn = cs[half + i];
      head[a] = fmaf(u, c, -__fmul_rn(v, sn));
      head[b2] = fmaf(v, c, __fmul_rn(u, sn));
    }
    __syncthreads();
  }
  if (head_norm) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int hd = warp; hd < q_heads + kv_heads; hd += warps) {
      float* head = row + hd * d;
      float ss = 0.f;
      for (int i = lane; i < d; i += 32) ss = fmaf(head[i], head[i], ss);
      const float inv = 1.0f / sqrtf(warp_sum(ss) / static_cast<float>(d) + head_eps);
      for (int i = lane; i < d; i += 32) head[i] *= inv;
    }
    __syncthreads();
  }
  const int dest = k_pages != nullptr ? dest_rows[t] : -1;
  const long long page = dest >= 0 ? dest / page_size : -1;
  const int in_page = dest >= 0 ? dest % page_size : 0;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const A val = from_f32<A>(row[c]);
    if (c < nq) {
      q_out[static_cast<size_t>(t) * nq + c] = val;
    } else if (c < nq + nk) {
      const int e = c - nq, kh = e / d, j = e % d;
      if (k_out != nullptr) k_out[static_cast<size_t>(t) * nk + e] = val;
      if (page >= 0) k_pages[((static_cast<size_t>(page) * kv_heads + kh) * page_size + in_page) * d + j] = val;
    } else {
      const int e = c - nq - nk, kh = e / dv, j = e % dv;
      if (v_out != nullptr) v_out[static_cast<size_t>(t) * nv + e] = val;
      if (page >= 0) v_pages[((static_cast<size_t>(page) * kv_heads + kh) * page_size + in_page) * dv + j] = val;
    }
  }
}

}  // namespace

// proj: [tokens, q_heads * d + kv_heads * (d + dv)] float32 or bfloat16 (in_dtype); outputs of
// out_dtype. bias, taps (float32 [n, row]; + tails, cu_seqlens, seq_of_token, slots), q_norm + k_norm, inv_freq
// (double [rotary / 2]) may each be null: that step is then left out. kv_heads 0: queries only.
LRM_API int lrm_shaped_qkv_store(const void* proj, int in_dtype, const float* bias, const float* taps, int n,
                                 const float* tails, const int* cu_seqlens, const int* seq_of_token,
                                 const int* slots, const int* positions, const float* q_norm, const float* k_norm,
                                 float row_eps, const double* inv_freq, int rotary, int pairing, int head_norm,
                                 float head_eps, void* q_out, void* k_out, void* v_out, void* k_pages, void* v_pages,
                                 const int* dest_rows, int out_dtype, int tokens, int q_heads, int kv_heads, int d,
                                 int dv, int page_size, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (q_heads <= 0 || kv_heads < 0 || d <= 0 || dv < 0 || page_size <= 0 || positions == nullptr) return LRM_BAD_ARGUMENT;
  if (rotary < 0 || rotary > d || rotary % 2 || (rotary > 0 && inv_freq == nullptr) || (pairing != 0 && pairing != 1))
    return LRM_BAD_ARGUMENT;
  if (inv_freq == nullptr) rotary = 0;
  if ((q_norm != nullptr && kv_heads > 0 && k_norm == nullptr) || (q_norm == nullptr && k_norm != nullptr))
    return LRM_BAD_ARGUMENT;
  if (taps != nullptr && n > 1 && (tails == nullptr || cu_seqlens == nullptr || seq_of_token == nullptr || slots == nullptr))
    return LRM_BAD_ARGUMENT;
  if (k_pages != nullptr && dest_rows == nullptr) return LRM_BAD_ARGUMENT;
  const int width = q_heads * d + kv_heads * (d + dv);
  const size_t bytes = sizeof(float) * (static_cast<size_t>(width) + rotary);
  if (bytes > 200 * 1024) return LRM_UNSUPPORTED;
#define LRM_SHAPED(ST, AT)                                                                                      \
  do {                                                                                                          \
    static bool raised = false;                                                                                 \
    if (bytes > 48 * 1024 && !raised) {                                                                         \
      cudaError_t e = cudaFuncSetAttribute(shaped_qkv_kernel<ST, AT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           200 * 1024);                                                         \
      if (e != cudaSuccess) return static_cast<int>(e);                                                         \
      raised = true;                                                                                            \
    }                                                                                                           \
    LRM_LAUNCH((shaped_qkv_kernel<ST, AT>), tokens, width >= 2048 ? 512 : 256, bytes, stream, static_cast<const ST*>(proj), bias, taps, n, \
               tails, cu_seqlens, seq_of_token, slots, positions, q_norm, k_norm, row_eps, inv_freq, rotary,    \
               pairing, head_norm, head_eps, static_cast<AT*>(q_out), static_cast<AT*>(k_out),                  \
               static_cast<AT*>(v_out), static_cast<AT*>(k_pages), static_cast<AT*>(v_pages), dest_rows, q_heads, \
               kv_heads, d, dv, page_size);                                                                     \
  } while (0)
  if (in_dtype == LRM_F32 && out_dtype == LRM_F32)
    LRM_SHAPED(float, float);
  else if (in_dtype == LRM_F32 && out_dtype == LRM_BF16)
    LRM_SHAPED(float, __nv_bfloat16);
  else if (in_dtype == LRM_BF16 && out_dtype == LRM_BF16)
    LRM_SHAPED(__nv_bfloat16, __nv_bfloat16);
  else
    return LRM_BAD_ARGUMENT;
#undef LRM_SHAPED
  return 0;
}
