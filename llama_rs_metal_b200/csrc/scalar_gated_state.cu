// Inputs and read-outs of two mixers whose matrix state S [d, dv] per head decays by one number
// per head and token, S <- a_t S + k (b_t v)^T, o = S^T q, both run by the per-token-decay mode of
// the scan in recurrent_scan.cu. Everything here is float32 except the projection it reads (float32,
// or bfloat16 widened exactly) and the activations it hands to the next product.
//
// State-space duality (Mamba-2). The projection row holds [z (H dv) | x (H dv) | B (G N) | C (G N) |
// dt (H)]. x, B and C pass a causal convolution per channel (taps [C, n], the last tap on the
// current token, zeros before a sequence's start, a bias) and SiLU. dt = softplus(dt + dt_bias),
// without a clamp; a_t = exp(-rate_h dt) with rate_h = exp(A_log_h) made by the caller; k = B,
// q = C (head h reads group h / (H / G)), v = dt x. The read-out adds D_h x, multiplies by
// silu(z), and divides each of `parts` equal parts of the H dv channels by its own root mean
// square before the weight: the gate comes before the norm.
//
// Matrix memory (mLSTM). From pre-activations i~, f~ per head: i = cap tanh((i~ + b_i) / cap),
// f = logsigmoid(cap tanh((f~ + b_f) / cap)), a running maximum m_t = max(f + m_(t-1), i) from
// m = 0, a_t = exp(f + m_(t-1) - m_t), b_t = exp(i - m_t). The normalizer n <- a_t n + b_t k goes
// through the scan as one more value column whose value is 1 (v' = b_t [v | 1 | 0 ..], the row
// filled up to a multiple of four columns), so column dv of the scan's output is n . q; the
// read-out (head_norm_gate with a floor) divides by max(|n . q|, exp(-m_t)) + 1e-6. m is carried
// per sequence and head like S.
#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// convolution, bias and SiLU of one channel at one token
template <typename S>
__device__ __forceinline__ float conv_bias_silu(const S* __restrict__ proj, long long stride, int column, int c,
                                                int t, int local, const float* __restrict__ taps,
                                                const float* __restrict__ bias, int n,
                                                const float* __restrict__ tail, int C) {
  float acc = 0.f;
  for (int back = n - 1; back >= 0; --back) {  // oldest input first
    const int at = local - back;
    float x;
    if (at >= 0)
      x = to_f32(proj[static_cast<size_t>(t - back) * stride + column]);
    else
      x = tail != nullptr ? tail[static_cast<size_t>(n - 1 + at) * C + c] : 0.f;
    acc = fmaf(taps[static_cast<size_t>(c) * n + (n - 1 - back)], x, acc);
  }
  if (bias != nullptr) acc += bias[c];
  return acc / (1.0f + expf(-acc));
}

// One CTA per (token, segment): H value heads, then G key groups (B), G query groups (C), and one
// segment for the decays.
template <typename S>
__global__ void ssd_prepare_kernel(const S* __restrict__ proj, long long stride, int conv_off, int dt_off,
                                   const float* __restrict__ dt_bias, const float* __restrict__ rate,
                                   const float* __restrict__ taps, const float* __restrict__ conv_bias, int n,
                                   const float* __restrict__ tails, const int* __restrict__ cu_seqlens,
                                   const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                                   float* __restrict__ qf, float* __restrict__ kf, float* __restrict__ vf,
                                   float* __restrict__ xf, float* __restrict__ decay, int H, int G, int N, int dv) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, seg = blockIdx.y;
  const int C = H * dv + 2 * G * N;
  if (seg == H + 2 * G) {
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
      const float dt = softplus_f(to_f32(proj[static_cast<size_t>(t) * stride + dt_off + h]) + dt_bias[h]);
      decay[static_cast<size_t>(t) * H + h] = expf(-rate[h] * dt);
    }
    return;
  }
  const int b = seq_of_token[t], local = t - cu_seqlens[b], slot = slots[b];
  const float* tail = (slot >= 0 && n > 1) ? tails + static_cast<size_t>(slot) * (n - 1) * C : nullptr;
  if (seg < H) {
    const float dt = softplus_f(to_f32(proj[static_cast<size_t>(t) * stride + dt_off + seg]) + dt_bias[seg]);
    const int first = seg * dv;
    for (int i = threadIdx.x; i < dv; i += blockDim.x) {
      const float x = conv_bias_silu(proj, stride, conv_off + first + i, first + i, t, local, taps, conv_bias, n, tail, C);
      const size_t at = (static_cast<size_t>(t) * H + seg) * dv + i;
      xf[at] = x;
      vf[at] = dt * x;
    }
  } else {
    const int g = seg - H;  // B groups then C groups are contiguous channels behind x
    const int first = H * dv + g * N;
    float* dst = g < G ? kf + (static_cast<size_t>(t) * G + g) * N : qf + (static_cast<size_t>(t) * G + g - G) * N;
    for (int i = threadIdx.x; i < N; i += blockDim.x)
      dst[i] = conv_bias_silu(proj, stride, conv_off + first + i, first + i, t, local, taps, conv_bias, n, tail, C);
  }
}

// out[t, c] = unit_rms_over_part((o[t, c] + skip[c / dv] x[t, c]) * silu(z[t, c])) * w[c]: one CTA
// per (token, part); the part's values are formed twice rather than kept (they come from cache).
template <typename S, typename A>
__global__ void skip_gate_part_norm_kernel(const float* __restrict__ o, const float* __restrict__ x,
                                           const float* __restrict__ skip, const S* __restrict__ z,
                                           long long z_stride, const float* __restrict__ w, A* __restrict__ out,
                                           int inner, int dv, int parts, float eps) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, part = blockIdx.y, size = inner / parts, first = part * size;
  const size_t row = static_cast<size_t>(t) * inner;
  auto value = [&](int c) {
    const float zv = to_f32(z[static_cast<size_t>(t) * z_stride + c]);
    return fmaf(skip[c / dv], x[row + c], o[row + c]) * (zv / (1.0f + expf(-zv)));
  };
  float ss = 0.f;
  for (int c = first + threadIdx.x; c < first + size; c += blockDim.x) {
    const float y = value(c);
    ss = fmaf(y, y, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / static_cast<float>(size) + eps);
  for (int c = first + threadIdx.x; c < first + size; c += blockDim.x)
    out[row + c] = from_f32<A>((value(c) * inv) * w[c]);
}

// One CTA per (sequence, head). The running maximum m_t = max(f_t + m_(t-1), i_t) is the only thing
// that goes from token to token, and a run of tokens acts on it as one map m -> max(m + a, b) (a the
// sum of its f, b what the run makes of minus infinity); two such maps compose into one, and the map
// (0, -inf) changes nothing. Each thread folds a contiguous run of the step's tokens (one or two
// tokens of a long prompt) into its (a, b); the threads' maps are composed by a prefix scan over each
// warp and then over the warps' totals; each thread walks its run again from the maximum it now
// knows. The gates' logarithms rest in `decay` and `take` between the passes.
// gates: [T, >= 2H] rows with i~ at column i_off + h, f~ at f_off + h.
struct MaxMap {
  float a, reach;
};
__device__ __forceinline__ MaxMap then(MaxMap first, MaxMap second) {
  return MaxMap{first.a + second.a, fmaxf(first.reach + second.a, second.reach)};
}
// lane l ends with the composition of lanes 0 .. l, earlier lanes first
__device__ __forceinline__ MaxMap warp_prefix(MaxMap mine, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const MaxMap before{__shfl_up_sync(0xffffffffu, mine.a, o), __shfl_up_sync(0xffffffffu, mine.reach, o)};
    if (lane >= o) mine = then(before, mine);
  }
  return mine;
}

template <typename S>
__global__ void mlstm_gates_kernel(const S* __restrict__ gates, long long stride, int i_off, int f_off,
                                   const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap,
                                   float* __restrict__ top, const int* __restrict__ cu_seqlens,
                                   const int* __restrict__ slots, float* __restrict__ decay,
                                   float* __restrict__ take, float* __restrict__ floor, int H) {
  __shared__ MaxMap totals[32];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int h = blockIdx.x, b = blockIdx.y;
  const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start, slot = slots[b];
  const int per = (n + blockDim.x - 1) / blockDim.x;
  const int t0 = start + min(n, static_cast<int>(threadIdx.x) * per), t1 = start + min(n, (static_cast<int>(threadIdx.x) + 1) * per);
  const float bi = i_bias[h], bf = f_bias[h], under = 1.0f / cap;
  MaxMap mine{0.f, -INFINITY};
  for (int t = t0; t < t1; ++t) {
    const S* row = gates + static_cast<size_t>(t) * stride;
    const float ig = cap * tanhf((to_f32(row[i_off + h]) + bi) * under);
    const float fg = -softplus_f(-(cap * tanhf((to_f32(row[f_off + h]) + bf) * under)));
    const size_t at = static_cast<size_t>(t) * H + h;
    decay[at] = fg;
    take[at] = ig;
    mine = then(mine, MaxMap{fg, ig});
  }
  const MaxMap through = warp_prefix(mine, lane);  // this warp's runs up to and with this lane's
  if (lane == 31) totals[warp] = through;
  __syncthreads();
  if (warp == 0) {
    const MaxMap whole = warp_prefix(lane < warps ? totals[lane] : MaxMap{0.f, -INFINITY}, lane);
    totals[lane] = whole;  // warps 0 .. lane
  }
  __syncthreads();
  MaxMap before{__shfl_up_sync(0xffffffffu, through.a, 1), __shfl_up_sync(0xffffffffu, through.reach, 1)};
  if (lane == 0) before = MaxMap{0.f, -INFINITY};
  if (warp > 0) before = then(totals[warp - 1], before);
  const float carried = slot >= 0 ? top[static_cast<size_t>(slot) * H + h] : 0.f;
  float m = fmaxf(carried + before.a, before.reach);
  for (int t = t0; t < t1; ++t) {
    const size_t at = static_cast<size_t>(t) * H + h;
    const float fg = decay[at], ig = take[at];
    const float next = fmaxf(fg + m, ig);
    decay[at] = expf(fg + m - next);
    take[at] = expf(ig - next);
    floor[at] = expf(-next);
    m = next;
  }
  // the last thread ends on the step's last maximum (also when its own run is empty)
  if (threadIdx.x == blockDim.x - 1 && slot >= 0) top[static_cast<size_t>(slot) * H + h] = m;
}

// One CTA per (token, head): q times q_scale, k, and v' = take [v | 1 | 0 ..] of dvp columns.
template <typename S>
__global__ void mlstm_prepare_kernel(const S* __restrict__ proj, long long stride, int q_off, int k_off, int v_off,
                                     const float* __restrict__ take, float q_scale, float* __restrict__ qf,
                                     float* __restrict__ kf, float* __restrict__ vf, int H, int d, int dv, int dvp) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const S* row = proj + static_cast<size_t>(t) * stride;
  const float b = take[static_cast<size_t>(t) * H + h];
  const size_t o = (static_cast<size_t>(t) * H + h) * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    qf[o + i] = to_f32(row[q_off + h * d + i]) * q_scale;
    kf[o + i] = to_f32(row[k_off + h * d + i]);
  }
  float* dst = vf + (static_cast<size_t>(t) * H + h) * dvp;
  for (int j = threadIdx.x; j < dvp; j += blockDim.x)
    dst[j] = j < dv ? b * to_f32(row[v_off + h * dv + j]) : (j == dv ? b : 0.f);
}

int threads_for(int n) { return n >= 256 ? 256 : ((n + 31) / 32) * 32; }

}  // namespace

// proj [T, stride] (float32 or bfloat16): the convolution's C = H dv + 2 G N channels (x | B | C) at
// column conv_off, dt at dt_off. taps float32 [C, n], conv_bias [C] or null, tails float32 [slots,
// n - 1, C] (read only; update it afterwards). -> qf, kf [T, G, N], vf, xf [T, H, dv], decay [T, H].
LRM_API int lrm_ssd_prepare(const void* proj, int dtype, long long stride, int conv_off, int dt_off,
                            const float* dt_bias, const float* rate, const float* taps, const float* conv_bias, int n,
                            const float* tails, const int* cu_seqlens, const int* seq_of_token, const int* slots,
                            float* qf, float* kf, float* vf, float* xf, float* decay, int tokens, int H, int G, int N,
                            int dv, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || N <= 0 || dv <= 0 || n <= 0 || H + 2 * G + 1 > 65535 || (n > 1 && tails == nullptr))
    return LRM_BAD_ARGUMENT;
  const dim3 grid(tokens, H + 2 * G + 1);
  const int threads = threads_for(dv > N ? dv : N);
  if (dtype == LRM_F32)
    LRM_LAUNCH(ssd_prepare_kernel<float>, grid, threads, 0, stream, static_cast<const float*>(proj), stride, conv_off,
               dt_off, dt_bias, rate, taps, conv_bias, n, tails, cu_seqlens, seq_of_token, slots, qf, kf, vf, xf,
               decay, H, G, N, dv);
  else if (dtype == LRM_BF16)
    LRM_LAUNCH(ssd_prepare_kernel<__nv_bfloat16>, grid, threads, 0, stream, static_cast<const __nv_bfloat16*>(proj),
               stride, conv_off, dt_off, dt_bias, rate, taps, conv_bias, n, tails, cu_seqlens, seq_of_token, slots, qf,
               kf, vf, xf, decay, H, G, N, dv);
  else
    return LRM_BAD_ARGUMENT;
  return 0;
}

// o, x float32 [T, inner]; skip float32 [inner / dv]; z: columns of a [T, z_stride] activation
// (pointer at its first gate column); w float32 [inner]; out [T, inner] in `dtype`.
LRM_API int lrm_skip_gate_part_norm(const float* o, const float* x, const float* skip, const void* z, int z_dtype,
                                    long long z_stride, const float* w, void* out, int dtype, int tokens, int inner,
                                    int dv, int parts, float eps, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (inner <= 0 || dv <= 0 || inner % dv || parts <= 0 || inner % parts || parts > 65535 || !(eps > 0.f))
    return LRM_BAD_ARGUMENT;
  const dim3 grid(tokens, parts);
  const int threads = threads_for(inner / parts);
#define LRM_PART_NORM(ST, AT)                                                                                     \
  LRM_LAUNCH((skip_gate_part_norm_kernel<ST, AT>), grid, threads, 0, stream, o, x, skip, static_cast<const ST*>(z), \
             z_stride, w, static_cast<AT*>(out), inner, dv, parts, eps)
  if (z_dtype == LRM_F32 && dtype == LRM_F32)
    LRM_PART_NORM(float, float);
  else if (z_dtype == LRM_F32 && dtype == LRM_BF16)
    LRM_PART_NORM(float, __nv_bfloat16);
  else if (z_dtype == LRM_BF16 && dtype == LRM_BF16)
    LRM_PART_NORM(__nv_bfloat16, __nv_bfloat16);
  else
    return LRM_BAD_ARGUMENT;
#undef LRM_PART_NORM
  return 0;
}

// gates [T, stride]: i~ at column i_off + h, f~ at f_off + h. top float32 [slots, H] (the running
// maximum, carried). -> decay, take, floor float32 [T, H]. max_tokens: no sequence brings more tokens
// than this to the step (it only sizes the CTAs).
LRM_API int lrm_mlstm_gates(const void* gates, int dtype, long long stride, int i_off, int f_off,
                            const float* i_bias, const float* f_bias, float cap, float* top, const int* cu_seqlens,
                            const int* slots, float* decay, float* take, float* floor, int seqs, int H,
                            int max_tokens, cudaStream_t stream) {
  if (seqs <= 0) return 0;
  if (H <= 0 || seqs > 65535 || !(cap > 0.f) || max_tokens <= 0) return LRM_BAD_ARGUMENT;
  // as many threads as the longest sequence can have tokens, in whole warps, up to 1024
  int threads = 32;
  while (threads < max_tokens && threads < 1024) threads *= 2;
  const dim3 grid(H, seqs);
  if (dtype == LRM_F32)
    LRM_LAUNCH(mlstm_gates_kernel<float>, grid, threads, 0, stream, static_cast<const float*>(gates), stride, i_off, f_off,
               i_bias, f_bias, cap, top, cu_seqlens, slots, decay, take, floor, H);
  else if (dtype == LRM_BF16)
    LRM_LAUNCH(mlstm_gates_kernel<__nv_bfloat16>, grid, threads, 0, stream, static_cast<const __nv_bfloat16*>(gates), stride,
               i_off, f_off, i_bias, f_bias, cap, top, cu_seqlens, slots, decay, take, floor, H);
  else
    return LRM_BAD_ARGUMENT;
  return 0;
}

// proj [T, stride]: q (H d) at q_off, k at k_off, v (H dv) at v_off; take float32 [T, H].
// -> qf, kf [T, H, d], vf [T, H, dvp] with dvp > dv.
LRM_API int lrm_mlstm_prepare(const void* proj, int dtype, long long stride, int q_off, int k_off, int v_off,
                              const float* take, float q_scale, float* qf, float* kf, float* vf, int tokens, int H,
                              int d, int dv, int dvp, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (H <= 0 || H > 65535 || d <= 0 || dv <= 0 || dvp <= dv) return LRM_BAD_ARGUMENT;
  const dim3 grid(tokens, H);
  const int threads = threads_for(d > dvp ? d : dvp);
  if (dtype == LRM_F32)
    LRM_LAUNCH(mlstm_prepare_kernel<float>, grid, threads, 0, stream, static_cast<const float*>(proj), stride, q_off,
               k_off, v_off, take, q_scale, qf, kf, vf, H, d, dv, dvp);
  else if (dtype == LRM_BF16)
    LRM_LAUNCH(mlstm_prepare_kernel<__nv_bfloat16>, grid, threads, 0, stream, static_cast<const __nv_bfloat16*>(proj),
               stride, q_off, k_off, v_off, take, q_scale, qf, kf, vf, H, d, dv, dvp);
  else
    return LRM_BAD_ARGUMENT;
  return 0;
}
