// Mixture of experts: the router's choice and the chosen experts' feed-forward.
//
// Router: logits z [T, E] in float32 (the product is made by the float32 matrix kernel), plus a
// bias; the `top` largest are chosen (the lower index wins a tie) and weighted by the softmax
// over the chosen logits only.
//
// Scored router (lrm_moe_router / lrm_moe_route with `scored`): s = softmax(z) over all E outputs;
// the choice is made on s + correction (a stored vector, may be absent) and the weights are the
// chosen s themselves (divided by their sum with `renormalize`). The outputs form `groups` equal
// groups of neighbours; a group's score is its largest choice score, and only outputs of the
// `keep` best groups can be chosen (the lower index wins every tie). Outputs numbered `experts`
// and above are identity experts: they have no matrices and return their input.
//
// Activation of an expert (`act`): 0, the clamped gate below; 1, silu(gate) * up.
//
// Experts, token by token (lrm_moe_experts_rows): one CTA per (token, chosen expert, slice of
// the expert's inner width). It forms its slice of
//   y = act(W_gate x, W_up x),   clamped gate:  g = min(g, limit), u = clamp(u, -limit, limit),
//                                               y = g sigmoid(alpha g) (u + 1)
// and that slice's share of W_down y, scaled by the expert's weight, as one float32 plane
// [T, width] per (choice, slice): the planes are added to the residual stream in plane order by
// the caller (or by the next norm), so the sum has a fixed order and no atomics meet in memory.
// A row's result depends on nothing else in the batch. This is the kernel of decoding and of
// the float32 path; it reads an expert's matrices once per token that chose it.
//
// Experts, all at once (prompts in bfloat16, few experts per choice): the matrices are laid out so
// that every expert's gate and up rows form one [E * 2 ff, width] matrix and the down matrices one
// [width, E * ff] matrix. One tensor-core product gives every expert's gate and up for every
// token; lrm_moe_dense_gate turns them into y, multiplied by the expert's weight for the token
// (zero for an expert the token did not choose); a second product with the down matrix sums the
// chosen experts' outputs in its K loop. It does E / top times the arithmetic a grouped product
// would, on kernels several times faster than a grouped product on the warp-level tensor path.
//
// Layout of the matrices for both: gate_up [E][2 ff][width] (an expert's gate rows, then its up
// rows), down [width][E][ff].
#include "common.cuh"

namespace {

__device__ __forceinline__ float expert_activation(float g, float u, int act, float limit, float alpha) {
  if (act == 1) return g / (1.0f + expf(-g)) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
}

// A warp turns logits z [E] into s = softmax(z) and choice = s + correction (both [E], shared memory).
__device__ __forceinline__ void score_row(const float* __restrict__ z, const float* __restrict__ correction,
                                          float* __restrict__ s, float* __restrict__ choice, int E, int lane) {
  float top = -INFINITY;
  for (int e = lane; e < E; e += 32) top = fmaxf(top, z[e]);
  for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
  float mass = 0.f;
  for (int e = lane; e < E; e += 32) mass += expf(z[e] - top);
  mass = warp_sum(mass);
  for (int e = lane; e < E; e += 32) {
    const float v = expf(z[e] - top) / mass;
    s[e] = v;
    choice[e] = v + (correction != nullptr ? correction[e] : 0.f);
  }
}

// One thread: the `keep` best of `groups` groups by their largest choice score, then the `top` best
// allowed outputs; `open` [groups] is scratch. The weights are the chosen s, divided by (their sum +
// mass_eps) with `renormalize`, then times weight_scale.
__device__ void choose_scored(const float* __restrict__ s, const float* __restrict__ choice, unsigned char* open,
                              int E, int top, int groups, int keep, int renormalize, float mass_eps,
                              float weight_scale, int* __restrict__ ids, float* __restrict__ weights) {
  const int size = E / groups;
  if (groups > 1 && keep < groups) {
    for (int g = 0; g < groups; ++g) open[g] = 0;
    for (int c = 0; c < keep; ++c) {
      int arg = -1;
      float val = -INFINITY;
      for (int g = 0; g < groups; ++g) {
        if (open[g]) continue;
        float best = -INFINITY;
        for (int e = g * size; e < (g + 1) * size; ++e) best = fmaxf(best, choice[e]);
        if (arg < 0 || best > val) {
          arg = g;
          val = best;
        }
      }
      open[arg] = 1;
    }
  } else {
    for (int g = 0; g < groups; ++g) open[g] = 1;
  }
  float mass = 0.f;
  for (int c = 0; c < top; ++c) {
    int arg = -1;
    float val = -INFINITY;
    for (int e = 0; e < E; ++e) {
      if (!open[e / size]) continue;
      bool taken = false;
      for (int p = 0; p < c; ++p) taken |= ids[p] == e;
      if (!taken && (arg < 0 || choice[e] > val)) {
        arg = e;
        val = choice[e];
      }
    }
    ids[c] = arg;
    weights[c] = s[arg];
    mass += s[arg];
  }
  if (renormalize)
    for (int c = 0; c < top; ++c) weights[c] /= mass + mass_eps;
  if (weight_scale != 1.0f)
    for (int c = 0; c < top; ++c) weights[c] *= weight_scale;
}

// Scored routing from logits [T, E]: one warp per token; shared memory per warp: s [E], choice [E],
// and the groups' flags.
__global__ void moe_route_scored_kernel(const float* __restrict__ logits, const float* __restrict__ correction,
                                        int* __restrict__ ids, float* __restrict__ weights, int tokens, int E,
                                        int top, int groups, int keep, int renormalize, float mass_eps,
                                        float weight_scale) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int t = blockIdx.x * warps + warp;
  if (t >= tokens) return;
  const int per = 2 * E + (groups + 3) / 4;
  float* s = smem + static_cast<size_t>(warp) * per;
  float* choice = s + E;
  score_row(logits + static_cast<size_t>(t) * E, correction, s, choice, E, lane);
  __syncwarp();
  if (lane == 0)
    choose_scored(s, choice, reinterpret_cast<unsigned char*>(choice + E), E, top, groups, keep, renormalize,
                  mass_eps, weight_scale, ids + static_cast<size_t>(t) * top, weights + static_cast<size_t>(t) * top);
}

// out[t, :] += (sum of the weights of the identity experts token t chose) * x[t, :]; x is the
// float32 input itself where the caller has it, else its rounding.
template <typename A>
__global__ void moe_identity_add_kernel(float* __restrict__ out, const A* __restrict__ x, const int* __restrict__ ids,
                                        const float* __restrict__ weights, int width, int experts, int top) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  float w = 0.f;
  for (int c = 0; c < top; ++c)
    if (ids[static_cast<size_t>(t) * top + c] >= experts) w += weights[static_cast<size_t>(t) * top + c];
  if (w == 0.f) return;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const size_t at = static_cast<size_t>(t) * width + i;
    out[at] = fmaf(w, to_f32(x[at]), out[at]);
  }
}

__global__ void moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                 int* __restrict__ ids, float* __restrict__ weights, int tokens, int E,
                                 int top) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  const float* z = logits + static_cast<size_t>(t) * E;
  int* mine = ids + static_cast<size_t>(t) * top;
  float* w = weights + static_cast<size_t>(t) * top;
  float best = -INFINITY;
  for (int c = 0; c < top; ++c) {
    int arg = -1;
    float val = -INFINITY;
    for (int e = 0; e < E; ++e) {
      const float x = z[e] + (bias != nullptr ? bias[e] : 0.f);
      bool taken = false;
      for (int p = 0; p < c; ++p) taken |= mine[p] == e;
      if (!taken && (arg < 0 || x > val)) {
        arg = e;
        val = x;
      }
    }
    mine[c] = arg;
    w[c] = val;
    if (c == 0) best = val;
  }
  float mass = 0.f;
  for (int c = 0; c < top; ++c) {
    w[c] = expf(w[c] - best);
    mass += w[c];
  }
  for (int c = 0; c < top; ++c) w[c] /= mass;
}

// The router in one launch for steps of few tokens: one CTA per token forms the E float32 logits
// (a warp per expert at a time, the lanes across the row, each lane's products in ascending order
// and the lanes added by a butterfly: a fixed order whatever the batch), then thread 0 chooses.
template <typename A>
__global__ void moe_router_kernel(const A* __restrict__ x, const float* __restrict__ w,
                                  const float* __restrict__ bias, int* __restrict__ ids,
                                  float* __restrict__ weights, float* __restrict__ logits, int width, int E,
                                  int top, int scored, const float* __restrict__ correction, int groups, int keep,
                                  int renormalize, float mass_eps, float weight_scale) {
  extern __shared__ float smem[];
  float* xs = smem;          // [width]
  float* zs = smem + width;  // [E] (scored: also s [E], choice [E] and the groups' flags behind it)
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  for (int i = threadIdx.x; i < width; i += blockDim.x) xs[i] = to_f32(x[static_cast<size_t>(t) * width + i]);
  __syncthreads();
  for (int e = warp; e < E; e += warps) {
    const float* row = w + static_cast<size_t>(e) * width;
    float acc = 0.f;
    for (int i = lane; i < width; i += 32) acc = fmaf(row[i], xs[i], acc);
    acc = warp_sum(acc);
    if (lane == 0) zs[e] = acc + (bias != nullptr ? bias[e] : 0.f);
  }
  __syncthreads();
  if (logits != nullptr)
    for (int e = threadIdx.x; e < E; e += blockDim.x) logits[static_cast<size_t>(t) * E + e] = zs[e];
  int* mine = ids + static_cast<size_t>(t) * top;
  float* out = weights + static_cast<size_t>(t) * top;
  if (scored) {
    if (warp != 0) return;
    score_row(zs, correction, zs + E, zs + 2 * E, E, lane);
    __syncwarp();
    if (lane == 0)
      choose_scored(zs + E, zs + 2 * E, reinterpret_cast<unsigned char*>(zs + 3 * E), E, top, groups, keep,
                    renormalize, mass_eps, weight_scale, mine, out);
    return;
  }
  if (threadIdx.x != 0) return;
  float best = -INFINITY, mass = 0.f;
  for (int c = 0; c < top; ++c) {
    int arg = -1;
    float val = -INFINITY;
    for (int e = 0; e < E; ++e) {
      bool taken = false;
      for (int p = 0; p < c; ++p) taken |= mine[p] == e;
      if (!taken && (arg < 0 || zs[e] > val)) {
        arg = e;
        val = zs[e];
      }
    }
    mine[c] = arg;
    out[c] = val;
    if (c == 0) best = val;
  }
  for (int c = 0; c < top; ++c) {
    out[c] = expf(out[c] - best);
    mass += out[c];
  }
  for (int c = 0; c < top; ++c) out[c] /= mass;
}

template <typename T> struct Pack8;
template <> struct Pack8<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float* f) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = __bfloat1622float2(h[i]);
      f[2 * i] = v.x;
      f[2 * i + 1] = v.y;
    }
  }
};
template <> struct Pack8<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float* f) {
    const float4 raw = *reinterpret_cast<const float4*>(p);
    f[0] = raw.x, f[1] = raw.y, f[2] = raw.z, f[3] = raw.w;
  }
};

// dot of a weight row with the float32 vector `x` (shared memory), lanes of a warp across the row
template <typename W>
__device__ __forceinline__ float row_dot(const W* __restrict__ w, const float* __restrict__ x, int n,
                                         bool vector_ok, int lane) {
  float acc = 0.f;
  constexpr int N = Pack8<W>::N;
  if (vector_ok) {
    for (int i = lane * N; i < n; i += 32 * N) {
      float f[N];
      Pack8<W>::load(w + i, f);
#pragma unroll
      for (int e = 0; e < N; ++e) acc = fmaf(f[e], x[i + e], acc);
    }
  } else {
    for (int i = lane; i < n; i += 32) acc = fmaf(to_f32(w[i]), x[i], acc);
  }
  return warp_sum(acc);
}

// two rows against the same vector, their loads issued together (twice the bytes in flight)
template <typename W>
__device__ __forceinline__ void row_dot2(const W* __restrict__ a, const W* __restrict__ b,
                                         const float* __restrict__ x, int n, bool vector_ok, int lane,
                                         float* ra, float* rb) {
  constexpr int N = Pack8<W>::N;
  float acc_a = 0.f, acc_b = 0.f;
  if (vector_ok) {
    int i = lane * N;
    for (; i + 32 * N < n; i += 64 * N) {  // two chunks of each row per trip
      float fa[N], fb[N], ga[N], gb[N];
      Pack8<W>::load(a + i, fa);
      Pack8<W>::load(b + i, fb);
      Pack8<W>::load(a + i + 32 * N, ga);
      Pack8<W>::load(b + i + 32 * N, gb);
#pragma unroll
      for (int e = 0; e < N; ++e) {
        acc_a = fmaf(fa[e], x[i + e], acc_a);
        acc_b = fmaf(fb[e], x[i + e], acc_b);
      }
#pragma unroll
      for (int e = 0; e < N; ++e) {
        acc_a = fmaf(ga[e], x[i + 32 * N + e], acc_a);
        acc_b = fmaf(gb[e], x[i + 32 * N + e], acc_b);
      }
    }
    for (; i < n; i += 32 * N) {
      float fa[N], fb[N];
      Pack8<W>::load(a + i, fa);
      Pack8<W>::load(b + i, fb);
#pragma unroll
      for (int e = 0; e < N; ++e) {
        acc_a = fmaf(fa[e], x[i + e], acc_a);
        acc_b = fmaf(fb[e], x[i + e], acc_b);
      }
    }
  } else {
    for (int i = lane; i < n; i += 32) {
      acc_a = fmaf(to_f32(a[i]), x[i], acc_a);
      acc_b = fmaf(to_f32(b[i]), x[i], acc_b);
    }
  }
  *ra = warp_sum(acc_a);
  *rb = warp_sum(acc_b);
}

template <typename A, typename W>
__global__ __launch_bounds__(256) void moe_experts_rows_kernel(
    const A* __restrict__ x, const W* __restrict__ gate_up, const W* __restrict__ down,
    const int* __restrict__ ids, const float* __restrict__ weights, float* __restrict__ planes, int tokens,
    int width, int ff, int experts, int top, int slices, float limit, float alpha, int act,
    const float* __restrict__ x32) {
  extern __shared__ float smem[];
  float* xs = smem;          // [width]
  float* ys = smem + width;  // [slice length]
  const int s = blockIdx.x, c = blockIdx.y, t = blockIdx.z;
  const int per = (ff + slices - 1) / slices, f0 = s * per, f1 = min(ff, f0 + per);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  pdl_wait();
  const int e = ids[static_cast<size_t>(t) * top + c];
  const float weight = weights[static_cast<size_t>(t) * top + c];
  if (e >= experts) {  // an identity expert: its output is its input, counted once (by slice 0)
    float* dst = planes + (static_cast<size_t>(c) * slices + s) * tokens * width + static_cast<size_t>(t) * width;
    for (int r = threadIdx.x; r < width; r += blockDim.x) {
      const size_t at = static_cast<size_t>(t) * width + r;
      dst[r] = s == 0 ? weight * (x32 != nullptr ? x32[at] : to_f32(x[at])) : 0.f;
    }
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) xs[i] = to_f32(x[static_cast<size_t>(t) * width + i]);
  __syncthreads();
  const W* wg = gate_up + static_cast<size_t>(e) * 2 * ff * width;
  const W* wu = wg + static_cast<size_t>(ff) * width;
  const W* wd = down + static_cast<size_t>(e) * ff;  // row r of this expert: wd + r * experts * ff
  const bool wide_ok = width % Pack8<W>::N == 0;
  for (int f = f0 + warp; f < f1; f += warps) {
    float g, u;
    row_dot2(wg + static_cast<size_t>(f) * width, wu + static_cast<size_t>(f) * width, xs, width, wide_ok, lane, &g, &u);
    if (lane == 0) ys[f - f0] = expert_activation(g, u, act, limit, alpha);
  }
  __syncthreads();
  // the slice's share of the down projection: a thread per output, the slice's columns in order
  float* dst = planes + (static_cast<size_t>(c) * slices + s) * tokens * width + static_cast<size_t>(t) * width;
  constexpr int N = Pack8<W>::N;
  const bool slice_ok = ff % N == 0 && f0 % N == 0 && (f1 - f0) % N == 0;
  for (int r = threadIdx.x; r < width; r += blockDim.x) {
    const W* row = wd + static_cast<size_t>(r) * experts * ff;
    float acc = 0.f;
    if (slice_ok) {
      for (int f = f0; f < f1; f += N) {
        float w8[N];
        Pack8<W>::load(row + f, w8);
#pragma unroll
        for (int i = 0; i < N; ++i) acc = fmaf(w8[i], ys[f - f0 + i], acc);
      }
    } else {
      for (int f = f0; f < f1; ++f) acc = fmaf(to_f32(row[f]), ys[f - f0], acc);
    }
    dst[r] = acc * weight;
  }
}

// y[t, e, f] = weight(t, e) * act(gate, up) from gu [T, E, 2 ff] (an expert's ff gate columns, then
// its ff up columns); weight(t, e) is the router's weight if token t chose expert e, else 0.
template <typename G, typename A>
__global__ void moe_dense_gate_kernel(const G* __restrict__ gu, const int* __restrict__ ids,
                                      const float* __restrict__ weights, A* __restrict__ y, int ff,
                                      int experts, int top, float limit, float alpha, int act) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const size_t row = static_cast<size_t>(t) * experts;
  for (int item = blockIdx.y * blockDim.x + threadIdx.x; item < experts * ff; item += gridDim.y * blockDim.x) {
    const int e = item / ff, f = item % ff;
    float w = 0.f;
    for (int c = 0; c < top; ++c)
      if (ids[static_cast<size_t>(t) * top + c] == e) w = weights[static_cast<size_t>(t) * top + c];
    float out = 0.f;
    if (w != 0.f) {
      const float g = to_f32(gu[(row + e) * 2 * ff + f]), u = to_f32(gu[(row + e) * 2 * ff + ff + f]);
      out = expert_activation(g, u, act, limit, alpha) * w;
    }
    y[row * ff + item] = from_f32<A>(out);
  }
}

}  // namespace

// gu: float32 or the type of y (`gu_dtype`); y: `dtype`.
LRM_API int lrm_moe_dense_gate(const void* gu, int gu_dtype, int dtype, const int* ids, const float* weights,
                               void* y, int tokens, int ff, int experts, int top, float limit, float alpha,
                               int act, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (ff <= 0 || experts <= 0 || top <= 0 || (act != 0 && act != 1)) return LRM_BAD_ARGUMENT;
  const long long items = static_cast<long long>(experts) * ff;
  const dim3 grid(tokens, static_cast<unsigned>((items + 1023) / 1024));
  if (dtype == LRM_BF16 && gu_dtype == LRM_BF16)
    LRM_LAUNCH((moe_dense_gate_kernel<__nv_bfloat16, __nv_bfloat16>), grid, 256, 0, stream,
               static_cast<const __nv_bfloat16*>(gu), ids, weights, static_cast<__nv_bfloat16*>(y), ff, experts, top,
               limit, alpha, act);
  else if (dtype == LRM_BF16 && gu_dtype == LRM_F32)
    LRM_LAUNCH((moe_dense_gate_kernel<float, __nv_bfloat16>), grid, 256, 0, stream, static_cast<const float*>(gu),
               ids, weights, static_cast<__nv_bfloat16*>(y), ff, experts, top, limit, alpha, act);
  else if (dtype == LRM_F32 && gu_dtype == LRM_F32)
    LRM_LAUNCH((moe_dense_gate_kernel<float, float>), grid, 256, 0, stream, static_cast<const float*>(gu), ids,
               weights, static_cast<float*>(y), ff, experts, top, limit, alpha, act);
  else
    return LRM_BAD_ARGUMENT;
  return 0;
}

LRM_API int lrm_moe_route(const float* logits, const float* bias, int* ids, float* weights, int tokens, int E,
                          int top, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E) return LRM_BAD_ARGUMENT;
  LRM_LAUNCH(moe_route_kernel, (tokens + 127) / 128, 128, 0, stream, logits, bias, ids, weights, tokens, E, top);
  return 0;
}

// x [T, width] float32 or bfloat16 (widened to float32), w float32 [E, width], bias float32 [E] or
// null -> ids int32 [T, top], weights float32 [T, top]; `logits` (float32 [T, E]) may be null.
// `scored`: the scored router described at the top (correction float32 [E] or null, `groups` equal
// groups of which `keep` stay open, `renormalize` with mass_eps added to the sum, weight_scale on the weights);
// bias is then not used.
LRM_API int lrm_moe_router(const void* x, int x_dtype, const float* w, const float* bias, int* ids,
                           float* weights, float* logits, int tokens, int width, int E, int top, int scored,
                           const float* correction, int groups, int keep, int renormalize, float mass_eps,
                           float weight_scale, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (width <= 0 || E <= 0 || top <= 0 || top > E) return LRM_BAD_ARGUMENT;
  if (scored && (groups <= 0 || E % groups || keep <= 0 || keep > groups || top > keep * (E / groups)))
    return LRM_BAD_ARGUMENT;
  const size_t bytes = sizeof(float) * (static_cast<size_t>(width) + (scored ? 3 * E + (groups + 3) / 4 : E));
  if (bytes > 48 * 1024) return LRM_UNSUPPORTED;
  const int threads = E >= 8 ? 256 : 128;
  if (x_dtype == LRM_F32)
    LRM_LAUNCH(moe_router_kernel<float>, tokens, threads, bytes, stream, static_cast<const float*>(x), w, bias, ids,
               weights, logits, width, E, top, scored, correction, groups, keep, renormalize, mass_eps, weight_scale);
  else if (x_dtype == LRM_BF16)
    LRM_LAUNCH(moe_router_kernel<__nv_bfloat16>, tokens, threads, bytes, stream,
               static_cast<const __nv_bfloat16*>(x), w, bias, ids, weights, logits, width, E, top, scored, correction,
               groups, keep, renormalize, mass_eps, weight_scale);
  else
    return LRM_BAD_ARGUMENT;
  return 0;
}

// The scored router's choice from float32 logits [T, E] -> ids int32 [T, top], weights float32 [T, top].
LRM_API int lrm_moe_route_scored(const float* logits, const float* correction, int* ids, float* weights, int tokens,
                                 int E, int top, int groups, int keep, int renormalize, float mass_eps,
                                 float weight_scale, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || groups <= 0 || E % groups || keep <= 0 || keep > groups ||
      top > keep * (E / groups))
    return LRM_BAD_ARGUMENT;
  const int warps = 4;
  const size_t bytes = sizeof(float) * warps * (2 * static_cast<size_t>(E) + (groups + 3) / 4);
  if (bytes > 48 * 1024) return LRM_UNSUPPORTED;
  LRM_LAUNCH(moe_route_scored_kernel, (tokens + warps - 1) / warps, 32 * warps, bytes, stream, logits, correction, ids,
             weights, tokens, E, top, groups, keep, renormalize, mass_eps, weight_scale);
  return 0;
}

// out float32 [T, width] += (weights of the chosen ids >= experts, summed) * x [T, width].
LRM_API int lrm_moe_identity_add(float* out, const void* x, int x_dtype, const int* ids, const float* weights,
                                 int tokens, int width, int experts, int top, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (width <= 0 || top <= 0 || experts < 0) return LRM_BAD_ARGUMENT;
  const int threads = width >= 1024 ? 256 : 128;
  if (x_dtype == LRM_F32)
    LRM_LAUNCH(moe_identity_add_kernel<float>, tokens, threads, 0, stream, out, static_cast<const float*>(x), ids,
               weights, width, experts, top);
  else if (x_dtype == LRM_BF16)
    LRM_LAUNCH(moe_identity_add_kernel<__nv_bfloat16>, tokens, threads, 0, stream, out,
               static_cast<const __nv_bfloat16*>(x), ids, weights, width, experts, top);
  else
    return LRM_BAD_ARGUMENT;
  return 0;
}

// How many slices of the inner width a step of `tokens` tokens is cut into: enough CTAs to fill
// the device, no slice shorter than 32.
LRM_API int lrm_moe_rows_slices(int tokens, int top, int ff) {
  const long long items = static_cast<long long>(tokens) * top;
  long long want = (4 * 148 + items - 1) / items;
  const int most = ff / 32 > 0 ? ff / 32 : 1;
  if (want > most) want = most;
  return want < 1 ? 1 : static_cast<int>(want);
}

// x [T, width] (float32 or bfloat16); gate_up [E, 2 ff, width], down [width, E, ff] (float32 or
// bfloat16); planes float32 [top * slices, T, width]. An id >= experts is an identity expert, whose
// output is x32 [T, width] (float32, when given) or x.
LRM_API int lrm_moe_experts_rows(const void* x, int x_dtype, const void* gate_up, const void* down,
                                 int w_dtype, const int* ids, const float* weights, float* planes, int tokens,
                                 int width, int ff, int experts, int top, int slices, float limit, float alpha,
                                 int act, const float* x32, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (width <= 0 || ff <= 0 || top <= 0 || slices <= 0 || top > 65535 || tokens > 65535 || experts <= 0 ||
      (act != 0 && act != 1))
    return LRM_BAD_ARGUMENT;
  const int per = (ff + slices - 1) / slices;
  const size_t bytes = sizeof(float) * (static_cast<size_t>(width) + per);
  if (bytes > 200 * 1024) return LRM_UNSUPPORTED;
  const dim3 grid(slices, top, tokens);
#define LRM_MOE_ROWS(AT, WT)                                                                               \
  do {                                                                                                     \
    if (bytes > 48 * 1024) {                                                                               \
      cudaError_t e = cudaFuncSetAttribute(moe_experts_rows_kernel<AT, WT>,                                \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);       \
      if (e != cudaSuccess) return static_cast<int>(e);                                                    \
    }                                                                                                      \
    LRM_LAUNCH((moe_experts_rows_kernel<AT, WT>), grid, 256, bytes, stream, static_cast<const AT*>(x),     \
               static_cast<const WT*>(gate_up), static_cast<const WT*>(down), ids, weights, planes, tokens, \
               width, ff, experts, top, slices, limit, alpha, act, x32);                                   \
  } while (0)
  if (x_dtype == LRM_F32 && w_dtype == LRM_F32)
    LRM_MOE_ROWS(float, float);
  else if (x_dtype == LRM_BF16 && w_dtype == LRM_BF16)
    LRM_MOE_ROWS(__nv_bfloat16, __nv_bfloat16);
  else if (x_dtype == LRM_F32 && w_dtype == LRM_BF16)
    LRM_MOE_ROWS(float, __nv_bfloat16);
  else
    return LRM_BAD_ARGUMENT;
#undef LRM_MOE_ROWS
  return 0;
}
