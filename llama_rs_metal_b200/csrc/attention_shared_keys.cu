// bfloat16 attention over ONE key head that every query head shares and whose rows also hold
// the values (the first DV of a row's DK columns): the cache layout of latent attention, where a
// token keeps one latent vector and one rotated key part, and the per-head key/value matrices are
// folded into the queries and unfolded from the outputs. Warp-level tensor path (mma.sync
// m16n8k16, ldmatrix, cp.async), float32 softmax in the log2 domain.
//
// One CTA = 32 query rows in two groups of 16 (the heads of two tokens; more tokens when a token
// has 8 heads or fewer; 32 heads of a token at a time when it has more) against 64-key tiles,
// double buffered, which both groups read. Because all rows read the same keys, the four warps of
// a group share a tile's work by columns instead of by rows: each warp scores its 16 keys of the
// tile for the group's 16 rows; the rows' maxima meet in shared memory, the probabilities are
// written there as bfloat16, and each warp then multiplies all of them with its own 16-column
// blocks of the values (blocks w, w + 4, ...). A warp so holds DV / 4 accumulator columns, which
// is what lets DV be 256 or 512 without spilling.
//
// The same kernel serves a prompt (keys: the step's own packed rows), a portion appended to
// started sequences, and decoding (keys: the paged cache, which already holds the step's rows).
// A window w lets the query at position p see keys p - w + 1 .. p. Rows of a tile outside the
// range a CTA's queries can see are zero-filled on the way into shared memory.
// Decoding offers few CTAs (sequences x groups of 16 heads), so there the key tiles of a sequence
// may be cut into splits, a CTA each: a split leaves its rows unnormalized with their maximum and
// mass ([sequence][head][split][DV + 2] float32) and a second kernel merges the splits in order,
// out = sum acc_i 2^(m_i - M) / sum l_i 2^(m_i - M).
// Sinks (one float32 per head, or none): e^sink_h joins the softmax's denominator once, unscaled and
// without a value; it is added where a row is normalized (here, or in the merge when keys are split).
// DK a multiple of 16, DV a multiple of 16 up to 512; anything else runs the row-wise kernel.
#include "attention_mma.cuh"

namespace {

constexpr int kRowsPerCta = 32;   // two groups of 16 rows, four warps each
constexpr int kSkThreads = 256;
constexpr int kProbStride = kTile + 8;

struct SharedKeysArgs {
  const __nv_bfloat16* q;         // [queries, H, DK]
  const __nv_bfloat16* k_packed;  // [tokens, DK] (a prompt), or null
  const __nv_bfloat16* k_pages;   // [pages, 1, 64, DK], or null
  __nv_bfloat16* out;             // [queries, H * DV]
  const int* cu_seqlens;          // [B + 1] query rows of each sequence, or null: one query per sequence
  const int* kv_lens;             // [B] lengths after the step, or null: a prompt (length = its queries)
  const int* page_table;
  const int* slots;
  int table_stride, H, DK, DV, rows_per_query, queries_per_cta, window;
  float scale_log2;
  float* partials;                // with n_splits > 1 (one query per sequence): blockIdx.x is the split
  int n_splits;
  const float* sinks;             // [H], or null
};

constexpr float kLog2e = 1.4426950408889634f;

template <int PAIRS>  // 16-column blocks of the values one warp accumulates (DV <= 64 * PAIRS)
__global__ __launch_bounds__(kSkThreads) void attention_shared_keys_kernel(SharedKeysArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int STRIDE = a.DK + 8, CHUNKS = a.DK / 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [32][STRIDE]
  __nv_bfloat16* Ks = Qs + kRowsPerCta * STRIDE;                    // [2][64][STRIDE]
  __nv_bfloat16* Ps = Ks + 2 * kTile * STRIDE;                      // [32][kProbStride]
  float* wmax = reinterpret_cast<float*>(Ps + kRowsPerCta * kProbStride);  // [group][warp of the group][16]
  float* wsum = wmax + 8 * 16;

  pdl_wait();
  const int b = blockIdx.z;
  const int start = a.cu_seqlens != nullptr ? a.cu_seqlens[b] : b;
  const int n = a.cu_seqlens != nullptr ? a.cu_seqlens[b + 1] - start : 1;
  const bool split_keys = a.n_splits > 1;
  const int q0 = split_keys ? 0 : blockIdx.x * a.queries_per_cta;
  if (q0 >= n) return;
  const int len = a.kv_lens != nullptr ? a.kv_lens[b] : n;
  const int before = len - n;
  const int head0 = blockIdx.y * kRowsPerCta;  // more than 32 heads: a CTA takes 32 of one token's
  const int group = threadIdx.x >> 7, warp = (threadIdx.x >> 5) & 3;  // row group, and the warp's place in it
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  float* gmax = wmax + group * 64;
  float* gsum = wsum + group * 64;

  const int p_lo = before + q0, p_hi = before + min(q0 + a.queries_per_cta, n) - 1;
  const int first_key = a.window > 0 ? max(0, p_lo - a.window + 1) : 0;
  int kt_first = first_key / kTile, kt_last = p_hi / kTile;
  if (split_keys) {  // this CTA's share of the tiles
    const int per = (kt_last - kt_first + a.n_splits) / a.n_splits;
    kt_first += static_cast<int>(blockIdx.x) * per;
    kt_last = min(kt_last, kt_first + per - 1);
    if (kt_first > kt_last) {  // more splits than this sequence has tiles: a part that saw no key
      for (int r = threadIdx.x; r < kRowsPerCta; r += kSkThreads) {
        const int head = head0 + r % a.rows_per_query;
        if (r / a.rows_per_query == 0 && head < a.H) {
          float* part = a.partials + ((static_cast<size_t>(b) * a.H + head) * a.n_splits + blockIdx.x) * (a.DV + 2);
          part[a.DV] = -INFINITY;
          part[a.DV + 1] = 0.f;
        }
      }
      return;
    }
  }
  // row r of the CTA: query q0 + r / rows_per_query, head head0 + r % rows_per_query
  for (int idx = threadIdx.x; idx < kRowsPerCta * CHUNKS; idx += kSkThreads) {
    const int r = idx / CHUNKS, c = idx % CHUNKS;
    const int qi = q0 + r / a.rows_per_query, head = head0 + r % a.rows_per_query;
    const bool ok = qi < n && head < a.H;
    const __nv_bfloat16* src = a.q + (static_cast<size_t>(start + (ok ? qi : 0)) * a.H + (ok ? head : 0)) * a.DK + c * 8;
    cp_async16(Qs + r * STRIDE + c * 8, src, ok ? 16 : 0);
  }
  int pos[2];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = 16 * group + g + 8 * half;
    const int qi = q0 + r / a.rows_per_query, head = head0 + r % a.rows_per_query;
    pos[half] = (qi < n && head < a.H) ? before + qi : -1;  // -1: a row of padding sees no key
  }
  const int* table = a.k_pages != nullptr ? a.page_table + static_cast<size_t>(a.slots[b]) * a.table_stride : nullptr;

  auto issue = [&](int kt, int stage) {
    __nv_bfloat16* dst = Ks + stage * kTile * STRIDE;
    const __nv_bfloat16* base;
    bool held = true;
    if (table != nullptr) {
      const int page = table[kt];
      held = page >= 0;
      base = a.k_pages + static_cast<size_t>(held ? page : 0) * kTile * a.DK;
    } else {
      base = a.k_packed + static_cast<size_t>(start + kt * kTile) * a.DK;
    }
    for (int idx = threadIdx.x; idx < kTile * CHUNKS; idx += kSkThreads) {
      const int r = idx / CHUNKS, c = idx % CHUNKS;
      const int key = kt * kTile + r;
      const bool ok = held && key >= first_key && key <= p_hi;
      cp_async16(dst + r * STRIDE + c * 8, ok ? base + static_cast<size_t>(r) * a.DK + c * 8 : base, ok ? 16 : 0);
    }
    cp_async_commit();
  };
  issue(kt_first, 0);  // the group also holds the query rows

  float o[2 * PAIRS][4];
#pragma unroll
  for (int i = 0; i < 2 * PAIRS; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const int value_pairs = a.DV / 16;

  for (int kt = kt_first; kt <= kt_last; ++kt) {
    const int stage = (kt - kt_first) & 1;
    const __nv_bfloat16* Kt = Ks + stage * kTile * STRIDE;
    cp_async_wait<0>();
    __syncthreads();  // tile kt is here for every thread, and everyone is done with tile kt - 1
    if (kt < kt_last) issue(kt + 1, stage ^ 1);

    // scores of this warp's 16 keys for all 16 rows
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
    const __nv_bfloat16* q_at = Qs + (16 * group + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + 8 * (lane >> 4);
    const __nv_bfloat16* k_at = Kt + (16 * warp + (lane & 7) + 8 * (lane >> 4)) * STRIDE + 8 * ((lane >> 3) & 1);
#pragma unroll 2
    for (int ks = 0; ks < a.DK / 16; ++ks) {
      uint32_t qa[4], b0, b1, b2, b3;
      ldsm_x4(qa[0], qa[1], qa[2], qa[3], q_at + 16 * ks);
      ldsm_x4(b0, b1, b2, b3, k_at + 16 * ks);
      mma16816(s[0], qa, b0, b1);
      mma16816(s[1], qa, b2, b3);
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = kt * kTile + 16 * warp + 8 * nt + 2 * t + (e & 1);
        const int p = pos[e >> 1];
        const bool visible = key <= p && (a.window <= 0 || key > p - a.window);
        s[nt][e] = visible ? s[nt][e] * a.scale_log2 : -INFINITY;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
      }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      mx[half] = fmaxf(mx[half], __shfl_xor_sync(0xffffffffu, mx[half], 1));
      mx[half] = fmaxf(mx[half], __shfl_xor_sync(0xffffffffu, mx[half], 2));
      if (t == 0) gmax[warp * 16 + g + 8 * half] = mx[half];
    }
    __syncthreads();
    float alpha[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = g + 8 * half;
      const float tile_max = fmaxf(fmaxf(gmax[r], gmax[16 + r]), fmaxf(gmax[32 + r], gmax[48 + r]));
      const float m_new = fmaxf(m[half], tile_max);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;  // a row with no visible key yet
      alpha[half] = exp2_fast(m[half] - m_use);
      float sum = 0.f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const float p0 = exp2_fast(s[nt][2 * half] - m_use), p1 = exp2_fast(s[nt][2 * half + 1] - m_use);
        sum += p0 + p1;
        *reinterpret_cast<uint32_t*>(Ps + (16 * group + r) * kProbStride + 16 * warp + 8 * nt + 2 * t) = pack_bf16(p0, p1);
      }
      l[half] = l[half] * alpha[half] + sum;
      m[half] = m_new;
    }
#pragma unroll
    for (int i = 0; i < 2 * PAIRS; ++i) {
      o[i][0] *= alpha[0];
      o[i][1] *= alpha[0];
      o[i][2] *= alpha[1];
      o[i][3] *= alpha[1];
    }
    __syncthreads();
    // this warp's value blocks: all 64 probabilities of every row times 16 columns at a time
    const __nv_bfloat16* p_at = Ps + (16 * group + (lane & 7) + 8 * ((lane >> 3) & 1)) * kProbStride + 8 * (lane >> 4);
    const __nv_bfloat16* v_at = Kt + ((lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + 8 * (lane >> 4);
#pragma unroll
    for (int kk = 0; kk < kTile / 16; ++kk) {
      uint32_t pa[4];
      ldsm_x4(pa[0], pa[1], pa[2], pa[3], p_at + 16 * kk);
#pragma unroll
      for (int pi = 0; pi < PAIRS; ++pi) {
        const int pair = warp + 4 * pi;
        if (pair < value_pairs) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_trans(b0, b1, b2, b3, v_at + 16 * kk * STRIDE + 16 * pair);
          mma16816(o[2 * pi], pa, b0, b1);
          mma16816(o[2 * pi + 1], pa, b2, b3);
        }
      }
    }
  }
  pdl_trigger();
  // every warp holds the mass of its own 16 keys per tile: add the four shares
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    float total = l[half];
    total += __shfl_xor_sync(0xffffffffu, total, 1);
    total += __shfl_xor_sync(0xffffffffu, total, 2);
    if (t == 0) gsum[warp * 16 + g + 8 * half] = total;
  }
  __syncthreads();
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r16 = g + 8 * half, r = 16 * group + r16;
    if (pos[half] < 0) continue;
    const float mass = gsum[r16] + gsum[16 + r16] + gsum[32 + r16] + gsum[48 + r16];
    const int qi = q0 + r / a.rows_per_query, head = head0 + r % a.rows_per_query;
    if (split_keys) {
      float* part = a.partials + ((static_cast<size_t>(b) * a.H + head) * a.n_splits + blockIdx.x) * (a.DV + 2);
      if (warp == 0 && t == 0) {
        part[a.DV] = m[half];
        part[a.DV + 1] = mass;
      }
#pragma unroll
      for (int pi = 0; pi < PAIRS; ++pi) {
        const int pair = warp + 4 * pi;
        if (pair >= value_pairs) continue;
#pragma unroll
        for (int j = 0; j < 2; ++j)
          *reinterpret_cast<float2*>(part + 16 * pair + 8 * j + 2 * t) =
              make_float2(o[2 * pi + j][2 * half], o[2 * pi + j][2 * half + 1]);
      }
      continue;
    }
    const float sink = (a.sinks != nullptr && head < a.H) ? exp2f(a.sinks[head] * kLog2e - m[half]) : 0.f;
    const float inv = 1.0f / (mass + sink);
    __nv_bfloat16* dst = a.out + (static_cast<size_t>(start + qi) * a.H + head) * a.DV;
#pragma unroll
    for (int pi = 0; pi < PAIRS; ++pi) {
      const int pair = warp + 4 * pi;
      if (pair >= value_pairs) continue;
#pragma unroll
      for (int j = 0; j < 2; ++j)
        *reinterpret_cast<uint32_t*>(dst + 16 * pair + 8 * j + 2 * t) =
            pack_bf16(o[2 * pi + j][2 * half] * inv, o[2 * pi + j][2 * half + 1] * inv);
    }
  }
}

// One block per (sequence, head): the splits' parts merged in split order.
__global__ void shared_keys_merge_kernel(const float* __restrict__ partials, __nv_bfloat16* __restrict__ out,
                                         int n_parts, int DV, const float* __restrict__ sinks, int H) {
  pdl_trigger();
  pdl_wait();
  const float* src = partials + static_cast<size_t>(blockIdx.x) * n_parts * (DV + 2);
  float M = -INFINITY;
  for (int i = 0; i < n_parts; ++i) M = fmaxf(M, src[i * (DV + 2) + DV]);
  float mass = 0.f;
  for (int i = 0; i < n_parts; ++i) {
    const float mi = src[i * (DV + 2) + DV];
    if (mi != -INFINITY) mass = fmaf(src[i * (DV + 2) + DV + 1], exp2f(mi - M), mass);
  }
  if (sinks != nullptr) mass += exp2f(sinks[blockIdx.x % H] * kLog2e - M);
  for (int d = threadIdx.x; d < DV; d += blockDim.x) {
    float acc = 0.f;
    for (int i = 0; i < n_parts; ++i) {
      const float mi = src[i * (DV + 2) + DV];
      if (mi != -INFINITY) acc = fmaf(src[i * (DV + 2) + d], exp2f(mi - M), acc);
    }
    out[static_cast<size_t>(blockIdx.x) * DV + d] = __float2bfloat16_rn(acc / mass);
  }
}

size_t shared_keys_smem(int DK) {
  return static_cast<size_t>(kRowsPerCta + 2 * kTile) * (DK + 8) * 2 + kRowsPerCta * kProbStride * 2 +
         2 * 8 * 16 * sizeof(float);
}

template <int PAIRS>
int launch_shared_keys(const SharedKeysArgs& a, dim3 grid, cudaStream_t stream) {
  const size_t smem = shared_keys_smem(a.DK);
  auto kernel = attention_shared_keys_kernel<PAIRS>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  LRM_LAUNCH(kernel, grid, kSkThreads, smem, stream, a);
  if (a.n_splits > 1)
    LRM_LAUNCH(shared_keys_merge_kernel, grid.z * a.H, a.DV >= 256 ? 128 : 64, 0, stream,
               static_cast<const float*>(a.partials), a.out, a.n_splits, a.DV, a.sinks, a.H);
  return 0;
}

}  // namespace

LRM_API int lrm_attention_shared_keys_supports(int heads, int dk, int dv, int page_size) {
  return heads > 0 && dk > 0 && dk % 16 == 0 && dv > 0 && dv % 16 == 0 && dv <= dk && dv <= 512 &&
                 page_size == kTile && shared_keys_smem(dk) <= 200 * 1024
             ? 1
             : 0;
}

// CTAs of this kernel that fit on one SM at key width dk (their shared memory decides): what a caller
// that cuts a decode step's keys into splits fills the SMs with once.
LRM_API int lrm_attention_shared_keys_ctas_per_sm(int dk) {
  const size_t bytes = shared_keys_smem(dk) + 1024;  // the driver's own share of a CTA's shared memory
  const int fit = static_cast<int>((227 * 1024) / bytes);
  return fit < 1 ? 1 : (fit > 4 ? 4 : fit);
}

// q [queries, heads, dk], out [queries, heads * dv], bfloat16. A prompt: k_packed [queries, dk], cu_seqlens
// [seqs + 1], kv_lens null. Over the cache: k_pages with page_table / slots, kv_lens [seqs] the
// lengths after the step; cu_seqlens [seqs + 1] for portions of several queries (at most
// `max_queries` per sequence), or null for one query per sequence; only then may the keys be cut into
// `n_splits` > 1 splits, with `partials` holding seqs * heads * n_splits * (dv + 2) floats. `sinks`
// float32 [heads], or null.
LRM_API int lrm_attention_shared_keys(const void* q, const void* k_packed, const void* k_pages, void* out,
                                      const int* cu_seqlens, const int* kv_lens, const int* page_table,
                                      int table_stride, const int* slots, int seqs, int max_queries, int heads,
                                      int dk, int dv, float scale, int window, float* partials, int n_splits,
                                      const float* sinks, cudaStream_t stream) {
  if (seqs <= 0 || max_queries <= 0) return 0;
  if (!lrm_attention_shared_keys_supports(heads, dk, dv, kTile)) return LRM_UNSUPPORTED;
  if ((k_packed == nullptr) == (k_pages == nullptr)) return LRM_BAD_ARGUMENT;
  if (k_pages != nullptr && (kv_lens == nullptr || page_table == nullptr || slots == nullptr)) return LRM_BAD_ARGUMENT;
  if (k_packed != nullptr && (cu_seqlens == nullptr || kv_lens != nullptr)) return LRM_BAD_ARGUMENT;
  if (n_splits > 1 && (cu_seqlens != nullptr || partials == nullptr || n_splits > 65535)) return LRM_BAD_ARGUMENT;
  SharedKeysArgs a;
  a.partials = partials;
  a.n_splits = n_splits > 1 ? n_splits : 1;
  a.sinks = sinks;
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.k_packed = static_cast<const __nv_bfloat16*>(k_packed);
  a.k_pages = static_cast<const __nv_bfloat16*>(k_pages);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.cu_seqlens = cu_seqlens;
  a.kv_lens = kv_lens;
  a.page_table = page_table;
  a.slots = slots;
  a.table_stride = table_stride;
  a.H = heads;
  a.DK = dk;
  a.DV = dv;
  a.window = window;
  a.scale_log2 = scale * kLog2e;
  int head_groups = 1;
  if (heads > kRowsPerCta) {
    a.rows_per_query = kRowsPerCta;
    a.queries_per_cta = 1;
    head_groups = (heads + kRowsPerCta - 1) / kRowsPerCta;
  } else {
    int rows = 1;
    while (rows < heads) rows *= 2;
    a.rows_per_query = rows;
    a.queries_per_cta = kRowsPerCta / rows;
  }
  const int query_tiles = (max_queries + a.queries_per_cta - 1) / a.queries_per_cta;
  if (seqs > 65535 || head_groups > 65535) return LRM_UNSUPPORTED;
  const dim3 grid(a.n_splits > 1 ? a.n_splits : query_tiles, head_groups, seqs);
  const int pairs = (dv / 16 + 3) / 4;
  if (pairs <= 1) return launch_shared_keys<1>(a, grid, stream);
  if (pairs <= 2) return launch_shared_keys<2>(a, grid, stream);
  if (pairs <= 4) return launch_shared_keys<4>(a, grid, stream);
  return launch_shared_keys<8>(a, grid, stream);
}
