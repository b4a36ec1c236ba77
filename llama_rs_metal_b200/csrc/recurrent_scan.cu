// Mixers with a fixed-size state per sequence and head: a matrix S [d, dv] in float32 that every
// token updates and reads,
//
//   plain decay (retention):   S <- a S + k v^T                      o = S^T q
//   decay per token:           S <- a_t S + k v^T                    o = S^T q
//   gated delta rule:          S <- diag(g) S;  u = b (v - S^T k);   S <- S + k u^T;   o = S^T q
//   generalized delta rule:    S <- diag(g) S + e (c^T S) + k v^T   (both terms read the old S)   o = S^T q
//
// with a one decay per head (or, per token, one per head and token: state-space and matrix-memory
// mixers, whose step size or input gate the caller has multiplied into v), g one decay per head
// and key channel and token, b one step size per head and token; in the generalized rule c is the
// direction that is read (a unit key) and e what is written back along it (minus a removal rate
// per key channel times that direction), both per head, key channel and token. Everything here is float32: the inputs are prepared in float32 by the kernels
// below (rotation, short convolutions, unit norms, decays), the state lives in float32 in the
// cache's state storage, one matrix per slot and head, and is carried from step to step.
//
// The scan: one CTA per (sequence, head, tile of value columns). Columns of S do not depend on
// one another, so a CTA keeps its columns in registers for the whole step: thread (column j,
// part p of P) holds a run of consecutive rows of column j. Per token every thread forms, over its
// rows, the three partial sums  r = sum g_i S_ij k_i,  s = sum g_i S_ij q_i,  c = sum k_i q_i,
// which are added over the P parts by shuffles, and then
//   u_j = b (v_j - r)   (or v_j without the delta rule),   o_j = s + u_j c,   S_ij <- g_i S_ij + k_i u_j,
// which is the update above with the read-out taken after the write. Tokens are staged through
// shared memory a chunk at a time by asynchronous copies, the next chunk under way while this
// one is worked on, so the inner loop has no block-wide barrier and waits for no load. A step of one
// token (decoding) and a step of a whole prompt run the same arithmetic in the same order, so
// the state after a prompt does not depend on how it was cut.
//
// A sequence of padding (slot < 0) starts from zero and stores nothing.
#include "common.cuh"

namespace {

constexpr int kScanThreads = 128;
constexpr int kChunk = 16;  // tokens per stage, halved while two stages do not fit the shared memory

__device__ __forceinline__ void scan_cp_async(float* dst, const float* src, bool valid, bool wide) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  if (wide)
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(valid ? 16 : 0));
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(d), "l"(src), "r"(valid ? 4 : 0));
}

// Thread (column j, part p) holds rows p * ROWS .. p * ROWS + ROWS - 1 of column j. A token's q, k
// and g rows lie in shared memory as [P][ROWS + 4] (the 4 floats between the parts keep the parts'
// 16-byte reads on different banks); tokens come in chunks of kChunk, two chunks in flight.
// MODE 0: one decay per head (head_decay); 1: the gated delta rule (g, beta); 2: one decay per head
// and token (in `beta`'s place, [T, H]); 3: the generalized delta rule (g, and the two more rows
// `look` = c and `put` = e per token, [T, H, d]): with t_j = sum_i c_i S_ij over the old state,
// S_ij <- g_i S_ij + e_i t_j + k_i v_j and o_j = sum_i g_i S_ij q_i + t_j (e . q) + v_j (k . q).
template <int ROWS, int MODE>
__global__ __launch_bounds__(kScanThreads) void linear_scan_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
    const float* __restrict__ g, const float* __restrict__ head_decay, const float* __restrict__ beta,
    const float* __restrict__ look, const float* __restrict__ put,
    float* __restrict__ state, float* __restrict__ out, const int* __restrict__ cu_seqlens,
    const int* __restrict__ slots, int H, int KH, int d, int dv, int P, int chunk) {
  extern __shared__ __align__(16) float smem[];
  constexpr bool DELTA = MODE == 1;
  constexpr bool GEN = MODE == 3;
  constexpr int NR = DELTA ? 3 : GEN ? 5 : 2;          // rows of d floats a token brings
  constexpr int RS = ROWS + 4;
  const int TS = P * RS, COLS = kScanThreads / P;
  const int VS = (COLS + 3) & ~3;                       // v of a token, padded to whole 16 bytes
  const int TOKEN = NR * TS + VS + 4;                   // q | k | (g) | (look | put) | v | beta
  const int STAGE = chunk * TOKEN;

  const int tid = threadIdx.x, pidx = tid % P, jl = tid / P;
  const int h = blockIdx.y, b = blockIdx.z, kh = h / (H / KH);
  const int j = blockIdx.x * COLS + jl;
  pdl_wait();
  const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start;
  const int slot = slots[b];
  float S[ROWS];
  float* mine = slot >= 0 ? state + (static_cast<size_t>(slot) * H + h) * d * dv : nullptr;
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int row = pidx * ROWS + i;
    S[i] = (mine != nullptr && row < d && j < dv) ? mine[static_cast<size_t>(row) * dv + j] : 0.f;
  }
  const float a = MODE == 0 ? head_decay[h] : 1.f;
  // 16-byte copies where every row of the inputs starts on a 16-byte boundary
  const bool wide = d % 4 == 0 && dv % 4 == 0 && COLS % 4 == 0;
  const int step = wide ? 4 : 1;

  auto issue = [&](int c0, int stage) {
    float* base = smem + stage * STAGE;
    const int cn = min(chunk, n - c0);
    const int per_token = ROWS * P / step;  // granules of a q (k, g) row, padding rows included
    for (int idx = tid; idx < cn * per_token; idx += kScanThreads) {
      const int c = idx / per_token, r = (idx % per_token) * step;
      const size_t tok = static_cast<size_t>(start + c0 + c);
      const bool in = r < d;
      float* dst = base + c * TOKEN + (r / ROWS) * RS + r % ROWS;
      scan_cp_async(dst, q + (tok * KH + kh) * d + (in ? r : 0), in, wide);
      scan_cp_async(dst + TS, k + (tok * KH + kh) * d + (in ? r : 0), in, wide);
      if (DELTA || GEN) scan_cp_async(dst + 2 * TS, g + (tok * H + h) * d + (in ? r : 0), in, wide);
      if (GEN) {
        scan_cp_async(dst + 3 * TS, look + (tok * H + h) * d + (in ? r : 0), in, wide);
        scan_cp_async(dst + 4 * TS, put + (tok * H + h) * d + (in ? r : 0), in, wide);
      }
    }
    const int v_per_token = COLS / step;
    for (int idx = tid; idx < cn * v_per_token; idx += kScanThreads) {
      const int c = idx / v_per_token, cl = (idx % v_per_token) * step, col = blockIdx.x * COLS + cl;
      const size_t tok = static_cast<size_t>(start + c0 + c);
      const bool in = col < dv;
      scan_cp_async(base + c * TOKEN + NR * TS + cl, v + (tok * H + h) * dv + (in ? col : 0), in, wide);
    }
    if (MODE == 1 || MODE == 2)
      for (int c = tid; c < cn; c += kScanThreads)
        scan_cp_async(base + c * TOKEN + NR * TS + VS, beta + static_cast<size_t>(start + c0 + c) * H + h,
                      true, false);
    asm volatile("cp.async.commit_group;\n" ::);
  };

  if (n > 0) issue(0, 0);
  for (int c0 = 0, it = 0; c0 < n; c0 += chunk, ++it) {
    const int cn = min(chunk, n - c0);
    if (c0 + chunk < n) {
      issue(c0 + chunk, (it + 1) & 1);
      asm volatile("cp.async.wait_group 1;\n" ::);
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::);
    }
    __syncthreads();
    const float* base = smem + (it & 1) * STAGE;
#pragma unroll 2
    for (int c = 0; c < cn; ++c) {
      const float* qc = base + c * TOKEN + pidx * RS;
      const float* kc = qc + TS;
      const float* gc = kc + TS;
      const float at = MODE == 2 ? base[c * TOKEN + 2 * TS + VS] : a;
      float kr[ROWS];
      float er[GEN ? ROWS : 1];
      float r0 = 0.f, r1 = 0.f, s0 = 0.f, s1 = 0.f, kq0 = 0.f, kq1 = 0.f, eq0 = 0.f, eq1 = 0.f;
#pragma unroll
      for (int i = 0; i < ROWS; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kc + i);
        const float4 q4 = *reinterpret_cast<const float4*>(qc + i);
        float4 g4 = make_float4(at, at, at, at);
        if (DELTA || GEN) g4 = *reinterpret_cast<const float4*>(gc + i);
        kr[i] = k4.x, kr[i + 1] = k4.y, kr[i + 2] = k4.z, kr[i + 3] = k4.w;
        if constexpr (GEN) {  // what the old state holds along `look`, before the decay
          const float4 c4 = *reinterpret_cast<const float4*>(gc + TS + i);
          const float4 e4 = *reinterpret_cast<const float4*>(gc + 2 * TS + i);
          r0 = fmaf(S[i], c4.x, r0), r1 = fmaf(S[i + 1], c4.y, r1);
          r0 = fmaf(S[i + 2], c4.z, r0), r1 = fmaf(S[i + 3], c4.w, r1);
          er[i] = e4.x, er[i + 1] = e4.y, er[i + 2] = e4.z, er[i + 3] = e4.w;
          eq0 = fmaf(e4.x, q4.x, eq0), eq1 = fmaf(e4.y, q4.y, eq1);
          eq0 = fmaf(e4.z, q4.z, eq0), eq1 = fmaf(e4.w, q4.w, eq1);
        }
        S[i] *= g4.x, S[i + 1] *= g4.y, S[i + 2] *= g4.z, S[i + 3] *= g4.w;
        if (DELTA) {
          r0 = fmaf(S[i], k4.x, r0), r1 = fmaf(S[i + 1], k4.y, r1);
          r0 = fmaf(S[i + 2], k4.z, r0), r1 = fmaf(S[i + 3], k4.w, r1);
        }
        s0 = fmaf(S[i], q4.x, s0), s1 = fmaf(S[i + 1], q4.y, s1);
        s0 = fmaf(S[i + 2], q4.z, s0), s1 = fmaf(S[i + 3], q4.w, s1);
        kq0 = fmaf(k4.x, q4.x, kq0), kq1 = fmaf(k4.y, q4.y, kq1);
        kq0 = fmaf(k4.z, q4.z, kq0), kq1 = fmaf(k4.w, q4.w, kq1);
      }
      float r = r0 + r1, s = s0 + s1, kq = kq0 + kq1, eq = eq0 + eq1;
      for (int o = 1; o < P; o <<= 1) {
        if (DELTA || GEN) r += __shfl_xor_sync(0xffffffffu, r, o);
        if (GEN) eq += __shfl_xor_sync(0xffffffffu, eq, o);
        s += __shfl_xor_sync(0xffffffffu, s, o);
        kq += __shfl_xor_sync(0xffffffffu, kq, o);
      }
      const float vj = base[c * TOKEN + NR * TS + jl];
      const float u = DELTA ? base[c * TOKEN + 3 * TS + VS] * (vj - r) : vj;
#pragma unroll
      for (int i = 0; i < ROWS; ++i) S[i] = fmaf(kr[i], u, S[i]);
      if constexpr (GEN) {
#pragma unroll
        for (int i = 0; i < ROWS; ++i) S[i] = fmaf(er[i], r, S[i]);
        s = fmaf(r, eq, s);
      }
      if (pidx == 0 && j < dv)
        out[(static_cast<size_t>(start + c0 + c) * H + h) * dv + j] = fmaf(u, kq, s);
    }
    __syncthreads();
  }
  if (mine != nullptr) {
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
      const int row = pidx * ROWS + i;
      if (row < d && j < dv) mine[static_cast<size_t>(row) * dv + j] = S[i];
    }
  }
}

template <int ROWS, int MODE>
int launch_scan(const float* q, const float* k, const float* v, const float* g, const float* head_decay,
                const float* beta, const float* look, const float* put, float* state, float* out, const int* cu_seqlens, const int* slots,
                int seqs, int H, int KH, int d, int dv, int P, cudaStream_t stream) {
  constexpr int NR = MODE == 1 ? 3 : MODE == 3 ? 5 : 2;
  const int COLS = kScanThreads / P, TS = P * (ROWS + 4), VS = (COLS + 3) & ~3;
  int chunk = kChunk;
  while (chunk > 1 && sizeof(float) * 2 * chunk * (static_cast<size_t>(NR) * TS + VS + 4) > 200 * 1024) chunk >>= 1;
  const size_t bytes = sizeof(float) * 2 * chunk * (static_cast<size_t>(NR) * TS + VS + 4);
  if (bytes > 200 * 1024) return LRM_UNSUPPORTED;
  static bool raised = false;  // per instantiation
  if (bytes > 48 * 1024 && !raised) {
    cudaError_t e = cudaFuncSetAttribute(linear_scan_kernel<ROWS, MODE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    raised = true;
  }
  const dim3 grid((dv + COLS - 1) / COLS, H, seqs);
  LRM_LAUNCH((linear_scan_kernel<ROWS, MODE>), grid, kScanThreads, bytes, stream, q, k, v, g, head_decay, beta,
             look, put, state, out, cu_seqlens, slots, H, KH, d, dv, P, chunk);
  return 0;
}

// How a head's key rows are cut over threads: P parts (a power of two up to 32) of ROWS rows.
// Few parts when the head is small (less to add up by shuffles), more when it is large (the
// registers a thread can keep bound ROWS to 64).
int g_scan_rows = 16;  // most rows a thread holds (tuning: lrm_linear_state_scan_rows)

void scan_shape(int d, int* rows, int* parts, int most_rows) {
  int P = 1;
  while (P < 32 && (d + P - 1) / P > most_rows) P <<= 1;
  int need = (d + P - 1) / P, R = 4;
  while (R < need) R <<= 1;
  *rows = R;
  *parts = P;
}

template <int MODE>
int dispatch_scan(const float* q, const float* k, const float* v, const float* g, const float* head_decay,
                  const float* beta, const float* look, const float* put, float* state, float* out, const int* cu_seqlens, const int* slots,
                  int seqs, int H, int KH, int d, int dv, cudaStream_t stream) {
  int R, P;
  scan_shape(d, &R, &P, g_scan_rows);
  if (MODE == 3 && g_scan_rows > 8) {
    // Few sequences (one prompt) leave most SMs without a CTA, and every CTA walks its tokens one
    // after another: with half the rows per thread a head's columns go to twice as many CTAs and a
    // token's chain of sums is shorter (one prompt of 2,048 tokens, 32 heads of 64 x 64: 643 against
    // 792 us; a quarter of the rows: 861). Steps that fill the device keep the standard shape.
    const long long ctas = static_cast<long long>((dv + kScanThreads / P - 1) / (kScanThreads / P)) * H * seqs;
    if (ctas < 148) scan_shape(d, &R, &P, g_scan_rows / 2);
  }
#define LRM_SCAN_CASE(N)                                                                             \
  case N:                                                                                            \
    return launch_scan<N, MODE>(q, k, v, g, head_decay, beta, look, put, state, out, cu_seqlens, slots, seqs, H, \
                                 KH, d, dv, P, stream)
  switch (R) {
    LRM_SCAN_CASE(4);
    LRM_SCAN_CASE(8);
    LRM_SCAN_CASE(16);
    LRM_SCAN_CASE(32);
    LRM_SCAN_CASE(64);
  }
#undef LRM_SCAN_CASE
  return LRM_UNSUPPORTED;
}

// --------------------------------------------------------------------------- read-out: norm and gate per head
// out[t, h, :] = o / sqrt(mean(o^2) + eps) * w * act(gate[t, h, :]) * out_scale; w and gate optional.
// A head's row of `o` has o_stride floats of which the first dv are read (o_stride > dv: the scan
// carried more columns). w is shared by the heads (w_stride 0) or one row per head (w_stride dv).
// With `floor` [T, H] the head is first divided by max(|o[dv]|, floor[t, h]) + den_eps: o's column dv
// then holds the read-out of a normalizer that went through the scan as one more value column.
template <typename A, typename G>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, int o_stride, const float* __restrict__ weight,
                                      int w_stride, const float* __restrict__ floor, float den_eps,
                                      const G* __restrict__ gate, long long gate_stride, int gate_act,
                                      A* __restrict__ out, int H, int dv, float eps, float out_scale) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const float* row = o + (static_cast<size_t>(t) * H + h) * o_stride;
  float under = 1.0f;
  if (floor != nullptr) under = 1.0f / (fmaxf(fabsf(row[dv]), floor[static_cast<size_t>(t) * H + h]) + den_eps);
  float ss = 0.f;
  for (int j = threadIdx.x; j < dv; j += blockDim.x) {
    const float v = row[j] * under;
    ss = fmaf(v, v, ss);
  }
  const float total = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(total / static_cast<float>(dv) + eps);
  for (int j = threadIdx.x; j < dv; j += blockDim.x) {
    float y = (row[j] * under) * inv;
    if (weight != nullptr) y *= weight[h * w_stride + j];
    if (gate != nullptr) {
      const float z = to_f32(gate[static_cast<size_t>(t) * gate_stride + h * dv + j]);
      const float sig = 1.0f / (1.0f + expf(-z));
      y *= gate_act == 1 ? z * sig : sig;
    }
    out[(static_cast<size_t>(t) * H + h) * dv + j] = from_f32<A>(y * out_scale);
  }
}

// --------------------------------------------------------------------------- retention: rotation and key scale
// From the fused projection row [.. q (H d) .. k (H d) .. v (H dv) ..]: q and k of every head are
// rotated on their first `rotary` dimensions (i paired with i + rotary/2, angle = float(position) *
// inv_freq[i], one float32 product), k is multiplied by k_scale after the rotation, v is widened.
template <typename A>
__global__ void retention_prepare_kernel(const A* __restrict__ proj, long long stride, int q_off, int k_off,
                                         int v_off, const int* __restrict__ positions,
                                         const float* __restrict__ inv_freq, int rotary, float k_scale,
                                         float* __restrict__ qf, float* __restrict__ kf,
                                         float* __restrict__ vf, int H, int d, int dv) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const A* row = proj + static_cast<size_t>(t) * stride;
  const float fpos = static_cast<float>(positions[t]);
  const int half = rotary / 2;
  const size_t o = (static_cast<size_t>(t) * H + h) * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const A* qh = row + q_off + h * d;
    const A* kh = row + k_off + h * d;
    float yq = to_f32(qh[i]), yk = to_f32(kh[i]);
    if (i < rotary) {
      const int pair = i < half ? i : i - half;
      const float angle = __fmul_rn(fpos, inv_freq[pair]);
      float sn, cs;
      sincosf(angle, &sn, &cs);
      if (i < half) {  // first of the pair: x cos - partner sin
        yq = fmaf(yq, cs, -__fmul_rn(to_f32(qh[i + half]), sn));
        yk = fmaf(yk, cs, -__fmul_rn(to_f32(kh[i + half]), sn));
      } else {         // second of the pair: x cos + partner sin
        yq = fmaf(yq, cs, __fmul_rn(to_f32(qh[i - half]), sn));
        yk = fmaf(yk, cs, __fmul_rn(to_f32(kh[i - half]), sn));
      }
    }
    qf[o + i] = yq;
    kf[o + i] = yk * k_scale;
  }
  for (int jn = threadIdx.x; jn < dv; jn += blockDim.x)
    vf[(static_cast<size_t>(t) * H + h) * dv + jn] = to_f32(row[v_off + h * dv + jn]);
}

// --------------------------------------------------------------------------- gated delta rule: inputs
// One CTA per (token, segment). Segments: G query heads, G key heads, H value heads (short causal
// convolution over time per channel, then SiLU; q and k then made unit vectors per head, q also
// times q_scale), H heads of decays g = exp(-rate_h softplus(a + dt_bias)), and one of step sizes
// b = sigmoid(.). The convolution's channels are the columns conv_off .. conv_off + C of the
// projection row in the order q | k | v; taps [C, n] with the last column the current token's;
// inputs before the step's first token come from the sequence's tail [n - 1, C] in the state
// storage (zeros at the start of a sequence).
template <typename A>
__device__ __forceinline__ float conv_silu(const A* __restrict__ proj, long long stride, int column, int c,
                                           int t, int local, const float* __restrict__ taps, int n,
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
  return acc / (1.0f + expf(-acc));
}

template <typename A>
__global__ void delta_prepare_kernel(const A* __restrict__ proj, long long stride, int conv_off, int b_off,
                                     const float* __restrict__ a, long long a_stride,
                                     const float* __restrict__ dt_bias, const float* __restrict__ rate, const float* __restrict__ taps, int n,
                                     const float* __restrict__ tails, const int* __restrict__ cu_seqlens,
                                     const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                                     float* __restrict__ qf, float* __restrict__ kf, float* __restrict__ vf,
                                     float* __restrict__ gf, float* __restrict__ bf, int H, int G, int d,
                                     int dv, float unit_eps, float q_scale) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, seg = blockIdx.y;
  const int C = 2 * G * d + H * dv;
  if (seg < 2 * G + H) {
    const int b = seq_of_token[t], local = t - cu_seqlens[b], slot = slots[b];
    const float* tail = slot >= 0 ? tails + static_cast<size_t>(slot) * (n - 1) * C : nullptr;
    if (seg < 2 * G) {  // a query or key head: convolution, SiLU, unit vector
      const int first = seg * d;  // q heads then k heads are contiguous channels
      float* dst = (seg < G ? qf + (static_cast<size_t>(t) * G + seg) * d
                            : kf + (static_cast<size_t>(t) * G + seg - G) * d);
      float ss = 0.f;
      // a thread keeps its channels' values between the two passes (d <= 8 * blockDim.x)
      float mine[8];
      int cnt = 0;
      for (int i = threadIdx.x; i < d; i += blockDim.x, ++cnt) {
        const float y = conv_silu(proj, stride, conv_off + first + i, first + i, t, local, taps, n, tail, C);
        mine[cnt] = y;
        ss = fmaf(y, y, ss);
      }
      const float total = block_sum(ss, scratch);
      const float inv = (seg < G ? q_scale : 1.0f) / sqrtf(total + unit_eps);
      cnt = 0;
      for (int i = threadIdx.x; i < d; i += blockDim.x, ++cnt) dst[i] = mine[cnt] * inv;
    } else {
      const int hv = seg - 2 * G, first = 2 * G * d + hv * dv;
      for (int i = threadIdx.x; i < dv; i += blockDim.x)
        vf[(static_cast<size_t>(t) * H + hv) * dv + i] =
            conv_silu(proj, stride, conv_off + first + i, first + i, t, local, taps, n, tail, C);
    }
  } else if (seg < 2 * G + 2 * H) {
    const int hd = seg - 2 * G - H;
    const float r = rate[hd];
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      const size_t at = (static_cast<size_t>(t) * H + hd) * d + i;
      const float z = a[static_cast<size_t>(t) * a_stride + hd * d + i] + dt_bias[hd * d + i];
      const float sp = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));
      gf[at] = expf(-r * sp);
    }
  } else {
    for (int hb = threadIdx.x; hb < H; hb += blockDim.x) {
      const float z = to_f32(proj[static_cast<size_t>(t) * stride + b_off + hb]);
      bf[static_cast<size_t>(t) * H + hb] = 1.0f / (1.0f + expf(-z));
    }
  }
}

// After a step: every sequence's tail becomes the last n - 1 convolution inputs it has seen.
// One thread per (sequence, channel), entries ascending: entry s takes input number
// m - (n - 1) + s of the step's m tokens, or, when that is before the step, the old entry s + m,
// which lies above every entry written so far.
template <typename A>
__global__ void conv_tail_update_kernel(const A* __restrict__ proj, long long stride, int conv_off, int C,
                                        int n, float* __restrict__ tails,
                                        const int* __restrict__ cu_seqlens, const int* __restrict__ slots) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  const int slot = slots[b];
  if (c >= C || slot < 0) return;
  const int start = cu_seqlens[b], m = cu_seqlens[b + 1] - start;
  float* tail = tails + static_cast<size_t>(slot) * (n - 1) * C;
  for (int s = 0; s < n - 1; ++s) {
    const int at = m - (n - 1) + s;
    tail[static_cast<size_t>(s) * C + c] =
        at >= 0 ? to_f32(proj[static_cast<size_t>(start + at) * stride + conv_off + c])
                : tail[static_cast<size_t>(s + m) * C + c];
  }
}

}  // namespace

// Tuning: the most rows of a state column one thread holds (4, 8, 16, 32 or 64; more rows mean fewer
// parts to add up by shuffles and longer chains of sums per thread). Returns the value in force.
LRM_API int lrm_linear_state_scan_rows(int rows) {
  if (rows == 4 || rows == 8 || rows == 16 || rows == 32 || rows == 64) g_scan_rows = rows;
  return g_scan_rows;
}

// q, k float32 [T, KH, d]; v float32 [T, H, dv]; out float32 [T, H, dv]; state float32
// [slots, H, d, dv]. Without `g`: plain decay per head (head_decay [H]) or, when that is null, per
// head and token (`beta` [T, H] holds the decays); with it: the gated delta rule (g [T, H, d], beta
// [T, H]).
LRM_API int lrm_linear_state_scan(const float* q, const float* k, const float* v, const float* g,
                                  const float* head_decay, const float* beta, float* state, float* out,
                                  const int* cu_seqlens, const int* slots, int seqs, int H, int KH, int d,
                                  int dv, cudaStream_t stream) {
  if (seqs <= 0) return 0;
  if (H <= 0 || KH <= 0 || H % KH || d <= 0 || dv <= 0 || seqs > 65535 || H > 65535) return LRM_BAD_ARGUMENT;
  if (d > 2048) return LRM_UNSUPPORTED;
  if (g != nullptr) {
    if (beta == nullptr) return LRM_BAD_ARGUMENT;
    return dispatch_scan<1>(q, k, v, g, nullptr, beta, nullptr, nullptr, state, out, cu_seqlens, slots, seqs, H, KH, d, dv, stream);
  }
  if (head_decay == nullptr) {  // one decay per head and token, where beta would be
    if (beta == nullptr) return LRM_BAD_ARGUMENT;
    return dispatch_scan<2>(q, k, v, nullptr, nullptr, beta, nullptr, nullptr, state, out, cu_seqlens, slots, seqs, H, KH, d, dv, stream);
  }
  return dispatch_scan<0>(q, k, v, nullptr, head_decay, nullptr, nullptr, nullptr, state, out, cu_seqlens, slots, seqs, H, KH, d,
                          dv, stream);
}

// The generalized delta rule: q, k, v, g as above (one key head per head), look and put float32
// [T, H, d]: S <- diag(g) S + put (look^T S) + k v^T with both terms reading the old S; o = S^T q.
LRM_API int lrm_general_delta_scan(const float* q, const float* k, const float* v, const float* g, const float* look,
                                   const float* put, float* state, float* out, const int* cu_seqlens,
                                   const int* slots, int seqs, int H, int d, int dv, cudaStream_t stream) {
  if (seqs <= 0) return 0;
  if (H <= 0 || d <= 0 || dv <= 0 || seqs > 65535 || H > 65535) return LRM_BAD_ARGUMENT;
  if (g == nullptr || look == nullptr || put == nullptr) return LRM_BAD_ARGUMENT;
  if (d > 2048) return LRM_UNSUPPORTED;
  return dispatch_scan<3>(q, k, v, g, nullptr, nullptr, look, put, state, out, cu_seqlens, slots, seqs, H, H, d, dv,
                          stream);
}

// `gate` (type gate_dtype, may be null) is read at gate[t * gate_stride + h * dv + j]; o at
// o[(t * H + h) * o_stride + j]; weight at weight[h * w_stride + j]; floor (may be null) at [t * H + h].
LRM_API int lrm_head_norm_gate(const float* o, int o_stride, const float* weight, int w_stride, const float* floor,
                               float den_eps, const void* gate, int gate_dtype, long long gate_stride, int gate_act,
                               void* out, int dtype, int tokens, int H, int dv, float eps, float out_scale,
                               cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (H <= 0 || H > 65535 || dv <= 0 || (gate != nullptr && gate_act != 1 && gate_act != 2)) return LRM_BAD_ARGUMENT;
  if (o_stride < dv || (floor != nullptr && o_stride <= dv) || (w_stride != 0 && w_stride != dv)) return LRM_BAD_ARGUMENT;
  const int threads = dv >= 256 ? 256 : ((dv + 31) / 32) * 32;
  const dim3 grid(tokens, H);
#define LRM_HEAD_NORM(AT, GT)                                                                              \
  LRM_LAUNCH((head_norm_gate_kernel<AT, GT>), grid, threads, 0, stream, o, o_stride, weight, w_stride, floor,    \
             den_eps, static_cast<const GT*>(gate), gate_stride, gate_act, static_cast<AT*>(out), H, dv, eps,     \
             out_scale)
  if (dtype == LRM_F32 && gate_dtype == LRM_F32)
    LRM_HEAD_NORM(float, float);
  else if (dtype == LRM_F32 && gate_dtype == LRM_BF16)
    LRM_HEAD_NORM(float, __nv_bfloat16);
  else if (dtype == LRM_BF16 && gate_dtype == LRM_F32)
    LRM_HEAD_NORM(__nv_bfloat16, float);
  else if (dtype == LRM_BF16 && gate_dtype == LRM_BF16)
    LRM_HEAD_NORM(__nv_bfloat16, __nv_bfloat16);
  else
    return LRM_BAD_ARGUMENT;
#undef LRM_HEAD_NORM
  return 0;
}

LRM_API int lrm_retention_prepare(const void* proj, int dtype, long long stride, int q_off, int k_off, int v_off,
                                  const int* positions, const float* inv_freq, int rotary, float k_scale,
                                  float* qf, float* kf, float* vf, int tokens, int H, int d, int dv,
                                  cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (H <= 0 || H > 65535 || d <= 0 || dv <= 0 || rotary < 0 || rotary > d || rotary % 2 ||
      (rotary > 0 && inv_freq == nullptr))
    return LRM_BAD_ARGUMENT;
  const dim3 grid(tokens, H);
  const int widest = d > dv ? d : dv;
  const int threads = widest >= 256 ? 256 : ((widest + 31) / 32) * 32;
  if (dtype == LRM_F32)
    LRM_LAUNCH(retention_prepare_kernel<float>, grid, threads, 0, stream, static_cast<const float*>(proj), stride,
               q_off, k_off, v_off, positions, inv_freq, rotary, k_scale, qf, kf, vf, H, d, dv);
  else if (dtype == LRM_BF16)
    LRM_LAUNCH(retention_prepare_kernel<__nv_bfloat16>, grid, threads, 0, stream,
               static_cast<const __nv_bfloat16*>(proj), stride, q_off, k_off, v_off, positions, inv_freq, rotary,
               k_scale, qf, kf, vf, H, d, dv);
  else
    return LRM_BAD_ARGUMENT;
  return 0;
}

// Every sequence's tail [slots, n - 1, C] becomes the last n - 1 inputs (columns conv_off .. conv_off
// + C of `proj`) it has seen, for a caller whose own kernel made the convolution.
LRM_API int lrm_conv_tail_update(const void* proj, int dtype, long long stride, int conv_off, int C, int n,
                                 float* tails, const int* cu_seqlens, const int* slots, int seqs,
                                 cudaStream_t stream) {
  if (seqs <= 0 || n <= 1) return 0;
  if (C <= 0 || seqs > 65535 || tails == nullptr) return LRM_BAD_ARGUMENT;
  const dim3 tail_grid((C + 255) / 256, seqs);
  if (dtype == LRM_F32)
    LRM_LAUNCH(conv_tail_update_kernel<float>, tail_grid, 256, 0, stream, static_cast<const float*>(proj), stride,
               conv_off, C, n, tails, cu_seqlens, slots);
  else if (dtype == LRM_BF16)
    LRM_LAUNCH(conv_tail_update_kernel<__nv_bfloat16>, tail_grid, 256, 0, stream,
               static_cast<const __nv_bfloat16*>(proj), stride, conv_off, C, n, tails, cu_seqlens, slots);
  else
    return LRM_BAD_ARGUMENT;
  return 0;
}

// `a` float32 is read at a[t * a_stride + h * d + i].
LRM_API int lrm_delta_prepare(const void* proj, int dtype, long long stride, int conv_off, int b_off,
                              const float* a, long long a_stride, const float* dt_bias, const float* rate, const float* taps, int n,
                              float* tails, const int* cu_seqlens, const int* seq_of_token, const int* slots,
                              float* qf, float* kf, float* vf, float* gf, float* bf, int tokens, int seqs, int H,
                              int G, int d, int dv, float unit_eps, float q_scale, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || d <= 0 || dv <= 0 || n <= 0 || seqs <= 0 || seqs > 65535) return LRM_BAD_ARGUMENT;
  const int threads = 128;
  if (d > 8 * threads || 2 * G + 2 * H + 1 > 65535) return LRM_UNSUPPORTED;
  const int C = 2 * G * d + H * dv;
  const dim3 grid(tokens, 2 * G + 2 * H + 1);
  const dim3 tail_grid((C + 255) / 256, seqs);
  if (dtype == LRM_F32) {
    const float* p = static_cast<const float*>(proj);
    LRM_LAUNCH(delta_prepare_kernel<float>, grid, threads, 0, stream, p, stride, conv_off, b_off, a, a_stride, dt_bias,
               rate, taps, n, static_cast<const float*>(tails), cu_seqlens, seq_of_token, slots, qf, kf, vf, gf, bf, H, G,
               d, dv, unit_eps, q_scale);
    if (n > 1)
      LRM_LAUNCH(conv_tail_update_kernel<float>, tail_grid, 256, 0, stream, p, stride, conv_off, C, n, tails,
                 cu_seqlens, slots);
  } else if (dtype == LRM_BF16) {
    const __nv_bfloat16* p = static_cast<const __nv_bfloat16*>(proj);
    LRM_LAUNCH(delta_prepare_kernel<__nv_bfloat16>, grid, threads, 0, stream, p, stride, conv_off, b_off, a,
               a_stride, dt_bias, rate, taps, n, static_cast<const float*>(tails), cu_seqlens, seq_of_token, slots, qf, kf,
               vf, gf, bf, H, G, d, dv, unit_eps, q_scale);
    if (n > 1)
      LRM_LAUNCH(conv_tail_update_kernel<__nv_bfloat16>, tail_grid, 256, 0, stream, p, stride, conv_off, C, n,
                 tails, cu_seqlens, slots);
  } else {
    return LRM_BAD_ARGUMENT;
  }
  return 0;
}
