// Causal grouped-query attention, one warp per (query, head), keys visited one
// at a time with a streaming softmax in float32:
//   s = (q.k) * scale;  m' = max(m, s);  l = l e^(m-m') + e^(s-m');
//   acc = acc e^(m-m') + e^(s-m') v;  out = acc / l
// (reference: crates/metal-backend/src/shaders/attention.metal:28-57).
// It is the attention of the float32 path for prompts and for decoding, and
// the bfloat16 path's fallback for sizes its tiled kernels refuse (head sizes up to 1024). The two
// entry points differ only in where keys come from (the step's packed k/v, or
// the paged cache), so a prompt, its token-by-token replay and its replay in
// chunks of any size do the same arithmetic in the same order. The paged entry
// takes any number of queries per sequence (a decoded token, or a portion of
// several tokens appended to a started sequence, whose own keys are already in
// the cache). A window w lets a query at position p see keys p-w+1 .. p; a negative w stands for
// chunks of -w positions (first_visible_key).
// Values may have another width than keys (dv against d). With `slopes` (one
// float32 per query head) a key at distance n = p - j behind the query loses
// slope_h * n from its score (a linear distance penalty, no rotation needed);
// `out_scale` multiplies the result before it is rounded (a mixer whose output
// enters a weighted sum of mixers). With `sinks` (one float32 per query head) the softmax's
// denominator also holds exp(sink_h): a key that is always seen, with no value, whose score is
// not scaled. With a query temperature (`temp_every` > 0) the query at position p counts
// 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) times (the factor goes into the score's
// scale, in float32). `v_stride` is the distance between two value rows in elements: values
// that are the first dv columns of the key rows are read from the keys' storage with the keys' d.
#include "common.cuh"

constexpr int kWidest = 32;  // elements of a row one lane holds at most: head sizes up to 1024

struct PackedKeys {
  const void* k;
  const void* v;
  size_t base;  // index of the sequence's first packed token
  int kv_heads, d, vs;
  template <typename A> __device__ const A* key(int p, int kh) const {
    return static_cast<const A*>(k) + ((base + p) * kv_heads + kh) * d;
  }
  template <typename A> __device__ const A* value(int p, int kh) const {
    return static_cast<const A*>(v) + ((base + p) * kv_heads + kh) * vs;
  }
};

struct PagedKeys {
  const void* k;
  const void* v;
  const int* table;  // this slot's row of the page table
  int kv_heads, d, vs, page_size;
  template <typename A> __device__ const A* key(int p, int kh) const {
    const size_t page = table[p / page_size];
    return static_cast<const A*>(k) + ((page * kv_heads + kh) * page_size + p % page_size) * d;
  }
  template <typename A> __device__ const A* value(int p, int kh) const {
    const size_t page = table[p / page_size];
    return static_cast<const A*>(v) + ((page * kv_heads + kh) * page_size + p % page_size) * vs;
  }
};

// PER: elements of a query (and of the output) one lane keeps in registers; d, dv <= 32 * PER.
template <typename A, int PER, typename Keys>
__device__ void attend_row(const A* __restrict__ q, A* __restrict__ out, const Keys& keys, int kh,
                           int first, int last, int d, int dv, float scale, float slope,
                           float out_scale, float sink) {
  const int lane = threadIdx.x & 31;
  float qv[PER], acc[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int j = lane + 32 * i;
    qv[i] = j < d ? to_f32(q[j]) : 0.f;
    acc[i] = 0.f;
  }
  // a sink is a key met before all others: score `sink`, weight 1 at its own maximum, no value
  float m = sink, l = sink > -INFINITY ? 1.f : 0.f;
  for (int p = first; p <= last; ++p) {
    const A* kr = keys.template key<A>(p, kh);
    const A* vr = keys.template value<A>(p, kh);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int j = lane + 32 * i;
      if (j < d) dot = fmaf(qv[i], to_f32(kr[j]), dot);
    }
    float s = warp_sum(dot) * scale;
    if (slope != 0.f) s -= slope * static_cast<float>(last - p);
    const float nm = fmaxf(m, s);
    const float old = expf(m - nm), prob = expf(s - nm);
    l = fmaf(l, old, prob);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int j = lane + 32 * i;
      if (j < dv) acc[i] = fmaf(prob, to_f32(vr[j]), __fmul_rn(acc[i], old));
    }
    m = nm;
  }
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int j = lane + 32 * i;
    if (j < dv) out[j] = from_f32<A>(out_scale == 1.0f ? acc[i] / l : (acc[i] / l) * out_scale);
  }
}

__device__ __forceinline__ float query_temperature(int pos, float coef, int every) {
  return every > 0 ? 1.0f + coef * logf(static_cast<float>((pos + 1) / every + 1)) : 1.0f;
}

template <typename A, int PER>
__global__ void attention_packed_kernel(const A* __restrict__ q, const A* __restrict__ k,
                                        const A* __restrict__ v, A* __restrict__ out,
                                        const int* __restrict__ cu_seqlens,
                                        const int* __restrict__ seq_of_token, int q_heads,
                                        int kv_heads, int d, int dv, float scale, int window,
                                        const float* __restrict__ slopes, float out_scale,
                                        const float* __restrict__ sinks, float temp_coef,
                                        int temp_every, int v_stride) {
  const int t = blockIdx.x, h = blockIdx.y;
  const int start = cu_seqlens[seq_of_token[t]];
  const int pos = t - start;
  const int first = first_visible_key(pos, window);
  PackedKeys keys{k, v, static_cast<size_t>(start), kv_heads, d, v_stride};
  const size_t row = static_cast<size_t>(t) * q_heads + h;
  attend_row<A, PER>(q + row * d, out + row * dv, keys, h / (q_heads / kv_heads), first, pos, d, dv,
                scale * query_temperature(pos, temp_coef, temp_every),
                slopes != nullptr ? slopes[h] : 0.f, out_scale, sinks != nullptr ? sinks[h] : -INFINITY);
}

template <typename A, int PER>
__global__ void attention_paged_kernel(const A* __restrict__ q, const A* __restrict__ k_pages,
                                       const A* __restrict__ v_pages, A* __restrict__ out,
                                       const int* __restrict__ page_table, int table_stride,
                                       const int* __restrict__ slots,
                                       const int* __restrict__ kv_lens,
                                       const int* __restrict__ seq_of_token,
                                       const int* __restrict__ positions, int q_heads, int kv_heads,
                                       int d, int dv, int page_size, float scale, int window,
                                       const float* __restrict__ slopes, float out_scale,
                                       const float* __restrict__ sinks, float temp_coef,
                                       int temp_every, int v_stride) {
  // query t of the step belongs to sequence b and stands at position pos; without the two
  // arrays there is one query per sequence, its newest token
  const int t = blockIdx.x, h = blockIdx.y;
  const int b = seq_of_token != nullptr ? seq_of_token[t] : t;
  const int pos = positions != nullptr ? positions[t] : kv_lens[b] - 1;
  const int first = first_visible_key(pos, window);
  PagedKeys keys{k_pages, v_pages, page_table + static_cast<size_t>(slots[b]) * table_stride,
                 kv_heads, d, v_stride, page_size};
  const size_t row = static_cast<size_t>(t) * q_heads + h;
  attend_row<A, PER>(q + row * d, out + row * dv, keys, h / (q_heads / kv_heads), first, pos, d, dv,
                scale * query_temperature(pos, temp_coef, temp_every),
                slopes != nullptr ? slopes[h] : 0.f, out_scale, sinks != nullptr ? sinks[h] : -INFINITY);
}

static bool bad_geometry(int q_heads, int kv_heads, int d, int dv) {
  return q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0 || d <= 0 ||
         d > 32 * kWidest || dv <= 0 || dv > 32 * kWidest;
}

LRM_API int lrm_attention_packed_rowwise(const void* q, const void* k, const void* v, void* out,
                                         int dtype, const int* cu_seqlens, const int* seq_of_token,
                                         int tokens, int q_heads, int kv_heads, int d, int dv,
                                         float scale, int window, const float* slopes,
                                         float out_scale, const float* sinks, float temp_coef,
                                         int temp_every, int v_stride, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (v_stride <= 0) v_stride = dv;
  if (bad_geometry(q_heads, kv_heads, d, dv)) return LRM_BAD_ARGUMENT;
  if (q_heads > 65535) return LRM_UNSUPPORTED;
  const dim3 grid(tokens, q_heads);
  const int widest = d > dv ? d : dv;
#define LRM_PACKED(AT, PER)                                                                                      \
  attention_packed_kernel<AT, PER><<<grid, 32, 0, stream>>>(                                                     \
      static_cast<const AT*>(q), static_cast<const AT*>(k), static_cast<const AT*>(v), static_cast<AT*>(out),    \
      cu_seqlens, seq_of_token, q_heads, kv_heads, d, dv, scale, window, slopes, out_scale, sinks, temp_coef,    \
      temp_every, v_stride)
#define LRM_PACKED_BY_WIDTH(AT)                  \
  do {                                           \
    if (widest <= 128) LRM_PACKED(AT, 4);        \
    else if (widest <= 512) LRM_PACKED(AT, 16);  \
    else LRM_PACKED(AT, 32);                     \
  } while (0)
  if (dtype == LRM_F32)
    LRM_PACKED_BY_WIDTH(float);
  else if (dtype == LRM_BF16)
    LRM_PACKED_BY_WIDTH(__nv_bfloat16);
  else
    return LRM_BAD_ARGUMENT;
#undef LRM_PACKED_BY_WIDTH
#undef LRM_PACKED
  LRM_LAUNCH_CHECK();
  return 0;
}

// `queries` rows of q. With seq_of_token and positions (int32 [queries]) query t belongs to
// sequence seq_of_token[t] and sees keys up to positions[t]; with both null there is one query
// per sequence, at position kv_lens[b] - 1.
LRM_API int lrm_attention_paged_rowwise(const void* q, const void* k_pages, const void* v_pages,
                                        void* out, int dtype, const int* page_table,
                                        int table_stride, const int* slots, const int* kv_lens,
                                        const int* seq_of_token, const int* positions,
                                        int queries, int q_heads, int kv_heads, int d, int dv,
                                        int page_size, float scale, int window, const float* slopes,
                                        float out_scale, const float* sinks, float temp_coef,
                                        int temp_every, int v_stride, cudaStream_t stream) {
  if (queries <= 0) return 0;
  if (v_stride <= 0) v_stride = dv;
  if (bad_geometry(q_heads, kv_heads, d, dv) || page_size <= 0) return LRM_BAD_ARGUMENT;
  if ((seq_of_token == nullptr) != (positions == nullptr)) return LRM_BAD_ARGUMENT;
  if (positions == nullptr && kv_lens == nullptr) return LRM_BAD_ARGUMENT;
  if (q_heads > 65535) return LRM_UNSUPPORTED;
  const dim3 grid(queries, q_heads);
  const int widest = d > dv ? d : dv;
#define LRM_PAGED(AT, PER)                                                                                       \
  attention_paged_kernel<AT, PER><<<grid, 32, 0, stream>>>(                                                      \
      static_cast<const AT*>(q), static_cast<const AT*>(k_pages), static_cast<const AT*>(v_pages),               \
      static_cast<AT*>(out), page_table, table_stride, slots, kv_lens, seq_of_token, positions, q_heads,         \
      kv_heads, d, dv, page_size, scale, window, slopes, out_scale, sinks, temp_coef, temp_every, v_stride)
#define LRM_PAGED_BY_WIDTH(AT)                  \
  do {                                          \
    if (widest <= 128) LRM_PAGED(AT, 4);        \
    else if (widest <= 512) LRM_PAGED(AT, 16);  \
    else LRM_PAGED(AT, 32);                     \
  } while (0)
  if (dtype == LRM_F32)
    LRM_PAGED_BY_WIDTH(float);
  else if (dtype == LRM_BF16)
    LRM_PAGED_BY_WIDTH(__nv_bfloat16);
  else
    return LRM_BAD_ARGUMENT;
#undef LRM_PAGED_BY_WIDTH
#undef LRM_PAGED
  LRM_LAUNCH_CHECK();
  return 0;
}
