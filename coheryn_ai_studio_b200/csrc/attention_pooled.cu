// Sliding-window attention whose older keys are seen as block means (sm_100a; float32 arithmetic on float32 or bfloat16
// storage).  Position i sees the positions j with 0 <= i - j < window, and beside them ONE key and value for each block
// of `pool` consecutive positions that lies wholly before the window: block b (positions b*pool .. b*pool + pool - 1) is
// seen when b*pool + pool - 1 <= i - window; its key is the mean of the block's keys as the cache holds them, its value
// the mean of the values.  Positions and blocks share one softmax.  Options, each a parameter:
//   * rotation of the first `rot` channels of queries and keys (pairs (i, i + rot/2)), and of ALL channels of the values
//     (pairs (m, m + dv/2), their own frequencies); a head's output at position i is turned back by -i;
//   * score = (q . k) * scale * temp[head], then cap * tanh(score / cap);
//   * one more term exp(sink[head]) in the softmax's denominator, without key or value;
//   * the output multiplied by sigmoid(gate[t, head * dv + c]).
//
// Kernels:
//   * pooled_prepare: rotates q, k, v of every row by its position (angles from float32 frequency pairs high + low, so no
//                     table bounds the positions), writes k and v to the cache pages and q in the compute dtype;
//   * pooled_means:   for every block that the step completed, the means of its keys and values, read back from the
//                     cache in position order, into the block cache: a second set of pages under a block table of its
//                     own with ceil(page_size / pool) rows per page; block b lives in the page of its LAST position p,
//                     at row b - floor(page(p) * page_size / pool);
//   * pooled_attention: one CTA per (row, head): eight warps take the keys in turn, four neighbouring keys at a time (a
//                     key's place among the row's keys decides its warp, so a row's sums do not depend on the batch),
//                     online softmax per warp, merged in warp order.
#include "common.cuh"

namespace {

__device__ __forceinline__ void pa_sincos(float p, const float* freq, int i, float& c, float& s) {
  const float fh = freq[2 * i], fl = freq[2 * i + 1];
  const float ah = p * fh;
  const float al = fmaf(p, fh, -ah) + p * fl;      // what the rounding of p * fh lost, and the low part
  float sh, ch, sl, cl;
  sincosf(ah, &sh, &ch);
  sincosf(al, &sl, &cl);
  c = ch * cl - sh * sl;
  s = sh * cl + ch * sl;
}

// grid (T); proj float32 [T, ld]: queries from column 0, keys from q_cols, values behind them.  The cosines and sines of
// the row's position are made once (shared memory) and serve all heads.
template <typename TT>
__global__ void pooled_prepare_kernel(const float* __restrict__ proj, long ld, const int* __restrict__ positions,
                                      const float* __restrict__ freq_k, int rot, const float* __restrict__ freq_v,
                                      TT* __restrict__ q_out, long ldq, const int* __restrict__ slots, TT* __restrict__ k_cache,
                                      TT* __restrict__ v_cache, int H, int G, int dk, int dv, int page_size) {
  extern __shared__ __align__(16) float sm[];
  co_pdl_launch_dependents();
  const size_t t = blockIdx.x;
  const int hk = rot / 2, hv = freq_v ? dv / 2 : 0;
  float* cs_k = sm;               // [hk][2]
  float* cs_v = sm + 2 * hk;      // [hv][2]
  co_pdl_wait();
  const float p = (float)positions[t];
  for (int i = threadIdx.x; i < hk + hv; i += blockDim.x) {
    float c, s;
    if (i < hk) { pa_sincos(p, freq_k, i, c, s); cs_k[2 * i] = c; cs_k[2 * i + 1] = s; }
    else { pa_sincos(p, freq_v, i - hk, c, s); cs_v[2 * (i - hk)] = c; cs_v[2 * (i - hk) + 1] = s; }
  }
  __syncthreads();
  const float* row = proj + t * ld;
  size_t k_at = 0, v_at = 0;
  if (slots) {
    const int slot = slots[t];
    const size_t page = slot / page_size, off = slot % page_size;
    k_at = (page * G * page_size + off) * dk;      // + g * page_size * dk
    v_at = (page * G * page_size + off) * dv;
  }
  // queries and keys: per head dk - hk items (a pair, or a channel that does not turn)
  const int per_qk = dk - hk, units_qk = H + (slots ? G : 0);
  for (int e = threadIdx.x; e < units_qk * per_qk; e += blockDim.x) {
    const int u = e / per_qk, i = e - u * per_qk;
    const float* src = row + (size_t)u * dk;
    TT* dst = u < H ? q_out + t * ldq + (size_t)u * dk : k_cache + k_at + (size_t)(u - H) * page_size * dk;
    if (i < hk) {
      const float c = cs_k[2 * i], s = cs_k[2 * i + 1];
      const float a = src[i], b = src[i + hk];
      dst[i] = co_from_float<TT>(a * c - b * s);
      dst[i + hk] = co_from_float<TT>(b * c + a * s);
    } else {
      dst[i + hk] = co_from_float<TT>(src[i + hk]);
    }
  }
  if (!slots) return;
  const int per_v = dv - hv;
  const float* vrow = row + (size_t)(H + G) * dk;
  for (int e = threadIdx.x; e < G * per_v; e += blockDim.x) {
    const int u = e / per_v, i = e - u * per_v;
    const float* src = vrow + (size_t)u * dv;
    TT* dst = v_cache + v_at + (size_t)u * page_size * dv;
    if (i < hv) {
      const float c = cs_v[2 * i], s = cs_v[2 * i + 1];
      const float a = src[i], b = src[i + hv];
      dst[i] = co_from_float<TT>(a * c - b * s);
      dst[i + hv] = co_from_float<TT>(b * c + a * s);
    } else {
      dst[i + hv] = co_from_float<TT>(src[i + hv]);
    }
  }
}

// grid (B * per_request, G): candidate `which` of request r is block first + which, first = the first block whose last
// position the step wrote.
template <typename TT>
__global__ void pooled_means_kernel(const TT* __restrict__ k_cache, const TT* __restrict__ v_cache, TT* __restrict__ pk_cache,
                                    TT* __restrict__ pv_cache, const int* __restrict__ tables, int table_width,
                                    const int* __restrict__ pool_tables, int pool_table_width, const int* __restrict__ cu_q,
                                    const int* __restrict__ kv_lens, int per_request, int G, int dk, int dv, int page_size,
                                    int pool, int pool_rows) {
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int r = blockIdx.x / per_request, which = blockIdx.x % per_request, g = blockIdx.y;
  const int p1 = kv_lens[r], p0 = p1 - (cu_q[r + 1] - cu_q[r]);
  const int b = p0 / pool + which;                       // blocks whose last position is >= p0
  const long last = (long)b * pool + pool - 1;
  if (p1 <= p0 || last >= p1) return;
  const int* table = tables + (size_t)r * table_width;
  const int lp = (int)(last / page_size);
  const int row = b - (int)(((long)lp * page_size) / pool);
  const size_t dst_page = (size_t)pool_tables[(size_t)r * pool_table_width + lp];
  const float inv = 1.0f / (float)pool;
  for (int c = threadIdx.x; c < dk + dv; c += blockDim.x) {
    const bool is_k = c < dk;
    const int ch = is_k ? c : c - dk, width = is_k ? dk : dv;
    const TT* cache = is_k ? k_cache : v_cache;
    float sum = 0.f;
    for (int j = 0; j < pool; ++j) {
      const long pos = (long)b * pool + j;
      const size_t page = (size_t)table[pos / page_size];
      sum += co_to_float<TT>(cache[((page * G + g) * page_size + (size_t)(pos % page_size)) * width + ch]);
    }
    TT* dst = is_k ? pk_cache : pv_cache;
    dst[((dst_page * G + g) * pool_rows + row) * width + ch] = co_from_float<TT>(sum * inv);
  }
}

struct AttnArgs {
  const void* q; long ldq;
  void* out; long ldo;
  const void* k; const void* v; const void* pk; const void* pv;
  const int* tables; int table_width; const int* pool_tables; int pool_table_width;
  const int* token_req; const int* positions;
  const float* temps; const float* sinks; const float* gates; long ldgate;
  const float* freq_v;
  int H, G, dk, dv, page_size, window, pool, pool_rows;
  float scale, cap;
  int table_room;       // block-table entries that the kernel may keep in shared memory (the pages of a window)
  int splits;           // CTAs that share a row's keys (grouped kernel); their parts meet in `scratch`
  float* scratch;       // [T][G][splits][HPG * dv + 2 * HPG]: unnormalised sums, then (maximum, sum) per head
};

constexpr int PA_WARPS = 8;
constexpr int PA_KEYS = 4;          // keys a warp takes at a time
constexpr int PA_MAX_PER_LANE = 8;     // channels per lane: head sizes up to 256

template <typename TT>
__global__ void __launch_bounds__(PA_WARPS * 32) pooled_attention_kernel(AttnArgs A) {
  extern __shared__ __align__(16) float sm[];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const size_t t = blockIdx.x;
  const int h = blockIdx.y, g = h / (A.H / A.G);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int dk = A.dk, dv = A.dv;
  float* qs = sm;                                  // [dk]
  float* acc_s = qs + dk;                          // [PA_WARPS][dv]
  float* ml = acc_s + PA_WARPS * dv;               // [PA_WARPS][2]
  float* os = ml + 2 * PA_WARPS;                   // [dv]
  const TT* q = (const TT*)A.q + t * A.ldq + (size_t)h * dk;
  for (int c = threadIdx.x; c < dk; c += blockDim.x) qs[c] = co_to_float<TT>(q[c]);
  __syncthreads();
  const int i = A.positions[t];
  const int r = A.token_req[t];
  const int* table = A.tables + (size_t)r * A.table_width;
  const int lo = A.window > 0 ? max(0, i - A.window + 1) : 0;
  const int nb = (A.pool > 0 && A.window > 0 && i - A.window + 1 > 0) ? (i - A.window + 1) / A.pool : 0;
  const int total = nb + (i - lo + 1);
  const float mult = A.scale * (A.temps ? A.temps[h] : 1.f);
  float qreg[PA_MAX_PER_LANE], acc[PA_MAX_PER_LANE];
#pragma unroll
  for (int e = 0; e < PA_MAX_PER_LANE; ++e) {
    const int c = lane + 32 * e;
    qreg[e] = c < dk ? qs[c] : 0.f;
    acc[e] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  // a warp takes PA_KEYS neighbouring keys at a time (their rows are requested together), the warps in turn
  for (int n0 = warp * PA_KEYS; n0 < total; n0 += PA_WARPS * PA_KEYS) {
    const TT* kr[PA_KEYS];
    const TT* vr[PA_KEYS];
#pragma unroll
    for (int b = 0; b < PA_KEYS; ++b) {
      const int n = min(n0 + b, total - 1);
      if (n < nb) {
        const long last = (long)n * A.pool + A.pool - 1;
        const int lp = (int)(last / A.page_size);
        const int row = n - (int)(((long)lp * A.page_size) / A.pool);
        const size_t page = (size_t)A.pool_tables[(size_t)r * A.pool_table_width + lp];
        const size_t at = (page * A.G + g) * A.pool_rows + row;
        kr[b] = (const TT*)A.pk + at * dk;
        vr[b] = (const TT*)A.pv + at * dv;
      } else {
        const int pos = lo + (n - nb);
        const size_t page = (size_t)table[pos / A.page_size];
        const size_t at = (page * A.G + g) * A.page_size + (size_t)(pos % A.page_size);
        kr[b] = (const TT*)A.k + at * dk;
        vr[b] = (const TT*)A.v + at * dv;
      }
    }
    float s[PA_KEYS];
#pragma unroll
    for (int b = 0; b < PA_KEYS; ++b) {
      s[b] = 0.f;
#pragma unroll
      for (int e = 0; e < PA_MAX_PER_LANE; ++e) {
        const int c = lane + 32 * e;
        if (c < dk) s[b] = fmaf(qreg[e], co_to_float<TT>(kr[b][c]), s[b]);
      }
    }
    float vals[PA_KEYS][PA_MAX_PER_LANE];
#pragma unroll
    for (int b = 0; b < PA_KEYS; ++b) {
#pragma unroll
      for (int e = 0; e < PA_MAX_PER_LANE; ++e) {
        const int c = lane + 32 * e;
        vals[b][e] = c < dv ? co_to_float<TT>(vr[b][c]) : 0.f;
      }
    }
    float m_new = m;
#pragma unroll
    for (int b = 0; b < PA_KEYS; ++b) {
      float x = co_warp_sum(s[b]) * mult;
      if (A.cap > 0.f) x = A.cap * tanhf(x / A.cap);
      s[b] = n0 + b < total ? x : -INFINITY;
      m_new = fmaxf(m_new, s[b]);
    }
    const float f = expf(m - m_new);       // exp(-inf) = 0 before the warp's first key
    l *= f;
#pragma unroll
    for (int e = 0; e < PA_MAX_PER_LANE; ++e) acc[e] *= f;
#pragma unroll
    for (int b = 0; b < PA_KEYS; ++b) {
      const float w = expf(s[b] - m_new);
      l += w;
#pragma unroll
      for (int e = 0; e < PA_MAX_PER_LANE; ++e) acc[e] = fmaf(w, vals[b][e], acc[e]);
    }
    m = m_new;
  }
#pragma unroll
  for (int e = 0; e < PA_MAX_PER_LANE; ++e) {
    const int c = lane + 32 * e;
    if (c < dv) acc_s[warp * dv + c] = acc[e];
  }
  if (lane == 0) { ml[2 * warp] = m; ml[2 * warp + 1] = l; }
  __syncthreads();
  // merge in warp order; the sink joins the denominator once
  float top = A.sinks ? A.sinks[h] : -INFINITY;
#pragma unroll
  for (int w = 0; w < PA_WARPS; ++w) top = fmaxf(top, ml[2 * w]);
  float denom = A.sinks ? expf(A.sinks[h] - top) : 0.f;
  float fw[PA_WARPS];
#pragma unroll
  for (int w = 0; w < PA_WARPS; ++w) {
    fw[w] = ml[2 * w] == -INFINITY ? 0.f : expf(ml[2 * w] - top);
    denom += ml[2 * w + 1] * fw[w];
  }
  const float inv = 1.0f / denom;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < PA_WARPS; ++w) o = fmaf(acc_s[w * dv + c], fw[w], o);
    os[c] = o * inv;
  }
  __syncthreads();
  TT* out = (TT*)A.out + t * A.ldo + (size_t)h * dv;
  const float* gate = A.gates ? A.gates + t * A.ldgate + (size_t)h * dv : nullptr;
  if (A.freq_v) {
    const int half = dv / 2;
    const float p = (float)i;
    for (int c = threadIdx.x; c < half; c += blockDim.x) {
      float cs, sn;
      pa_sincos(p, A.freq_v, c, cs, sn);
      const float a = os[c], b = os[c + half];
      float x0 = a * cs + b * sn, x1 = b * cs - a * sn;        // turned by -p
      if (gate) {
        x0 *= 1.0f / (1.0f + expf(-gate[c]));
        x1 *= 1.0f / (1.0f + expf(-gate[c + half]));
      }
      out[c] = co_from_float<TT>(x0);
      out[c + half] = co_from_float<TT>(x1);
    }
  } else {
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
      float x = os[c];
      if (gate) x *= 1.0f / (1.0f + expf(-gate[c]));
      out[c] = co_from_float<TT>(x);
    }
  }
}

// The same attention with the query heads of a key head side by side: one CTA per (row, key head) reads every cached row
// once for all HPG heads that share it (1, 2 or 4).  NPL: channels per lane (4: head sizes up to 128).  With head sizes
// in multiples of 128 a lane holds four neighbouring channels (one 8- or 16-byte access), else channels 32 apart.
// A cached row as a lane holds it between the request and its use: the bits as they were loaded (converting them at once
// would make the warp wait for the load right there, and nothing could be requested ahead).
template <typename TT> struct Four;
template <> struct Four<float> {
  float4 d;
  __device__ __forceinline__ void load(const float* p) { d = *reinterpret_cast<const float4*>(p); }
  __device__ __forceinline__ void zero() { d = make_float4(0.f, 0.f, 0.f, 0.f); }
  __device__ __forceinline__ float get(int j) const { return j == 0 ? d.x : j == 1 ? d.y : j == 2 ? d.z : d.w; }
};
template <> struct Four<__nv_bfloat16> {
  uint2 d;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { d = *reinterpret_cast<const uint2*>(p); }
  __device__ __forceinline__ void zero() { d = make_uint2(0u, 0u); }
  __device__ __forceinline__ float get(int j) const {
    const unsigned w = j < 2 ? d.x : d.y;
    return __uint_as_float((j & 1) ? (w & 0xffff0000u) : (w << 16));
  }
};
template <typename TT, int NPL, bool VEC> struct LaneRow;
template <typename TT, int NPL> struct LaneRow<TT, NPL, true> {        // four neighbouring channels per 128
  Four<TT> d[NPL / 4];
  __device__ __forceinline__ void load(const TT* row, int n, int lane) {
#pragma unroll
    for (int e4 = 0; e4 < NPL / 4; ++e4) {
      const int c = e4 * 128 + 4 * lane;
      if (c < n) d[e4].load(row + c); else d[e4].zero();
    }
  }
  __device__ __forceinline__ float get(int e) const { return d[e >> 2].get(e & 3); }
  static __device__ __forceinline__ int channel(int e, int lane) { return (e >> 2) * 128 + 4 * lane + (e & 3); }
};
template <typename TT, int NPL> struct LaneRow<TT, NPL, false> {       // channels 32 apart
  TT d[NPL];
  __device__ __forceinline__ void load(const TT* row, int n, int lane) {
#pragma unroll
    for (int e = 0; e < NPL; ++e) {
      const int c = lane + 32 * e;
      d[e] = c < n ? row[c] : co_from_float<TT>(0.f);
    }
  }
  __device__ __forceinline__ float get(int e) const { return co_to_float<TT>(d[e]); }
  static __device__ __forceinline__ int channel(int e, int lane) { return lane + 32 * e; }
};

constexpr int PG_WARPS = 8;          // warps of the kernel that shares cached rows among the heads of a key head
template <typename TT, int HPG, int NPL, bool VEC>
__global__ void __launch_bounds__(PG_WARPS * 32) pooled_attention_group_kernel(AttnArgs A) {
  using Row = LaneRow<TT, NPL, VEC>;
  extern __shared__ __align__(16) float sm[];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const size_t t = blockIdx.x;
  const int g = blockIdx.y, h0 = g * HPG;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int dk = A.dk, dv = A.dv;
  float* acc_s = sm;                               // [PG_WARPS][HPG][dv]
  float* ml = acc_s + PG_WARPS * HPG * dv;         // [PG_WARPS][HPG][2]
  float* os = ml + 2 * PG_WARPS * HPG;             // [HPG][dv]
  int* table_s = reinterpret_cast<int*>(os + HPG * dv);     // [table_room]
  const int i = A.positions[t];
  const int r = A.token_req[t];
  const int* table = A.tables + (size_t)r * A.table_width;
  const int lo = A.window > 0 ? max(0, i - A.window + 1) : 0;
  // the pages of the window, looked up once: a warp that waits for a table entry cannot issue anything else meanwhile
  const int page_lo = lo / A.page_size;
  const bool staged = i / A.page_size - page_lo < A.table_room;
  if (staged) {
    for (int e = threadIdx.x; e <= i / A.page_size - page_lo; e += blockDim.x) table_s[e] = table[page_lo + e];
    __syncthreads();
  }
  const int nb = (A.pool > 0 && A.window > 0 && i - A.window + 1 > 0) ? (i - A.window + 1) / A.pool : 0;
  // this CTA's share of the row's keys (block means first, then positions): equal runs in multiples of PA_KEYS
  const int all_keys = nb + (i - lo + 1);
  const int per_split = ((all_keys + A.splits - 1) / A.splits + PA_KEYS - 1) / PA_KEYS * PA_KEYS;
  const int first_key = blockIdx.z * per_split;
  const int total = min(all_keys, first_key + per_split);        // one behind the share's last key
  float qreg[HPG][NPL], acc[HPG][NPL];
#pragma unroll
  for (int hh = 0; hh < HPG; ++hh) {
    Row qrow;
    qrow.load((const TT*)A.q + t * A.ldq + (size_t)(h0 + hh) * dk, dk, lane);
#pragma unroll
    for (int e = 0; e < NPL; ++e) { qreg[hh][e] = qrow.get(e); acc[hh][e] = 0.f; }
  }
  // the rows of the warp's next keys are requested before the current ones are used (two sets of registers in turn)
  auto fetch = [&](int n0, Row (&kv)[PA_KEYS], Row (&vv)[PA_KEYS]) {
#pragma unroll
    for (int b = 0; b < PA_KEYS; ++b) {
      const int n = min(n0 + b, total - 1);
      const TT* kr;
      const TT* vr;
      if (n < nb) {
        const long last = (long)n * A.pool + A.pool - 1;
        const int lp = (int)(last / A.page_size);
        const int row = n - (int)(((long)lp * A.page_size) / A.pool);
        const size_t at = ((size_t)A.pool_tables[(size_t)r * A.pool_table_width + lp] * A.G + g) * A.pool_rows + row;
        kr = (const TT*)A.pk + at * dk;
        vr = (const TT*)A.pv + at * dv;
      } else {
        const int pos = lo + (n - nb);
        const int pi = pos / A.page_size;
        const size_t page = (size_t)(staged ? table_s[pi - page_lo] : table[pi]);
        const size_t at = (page * A.G + g) * A.page_size + (size_t)(pos - pi * A.page_size);
        kr = (const TT*)A.k + at * dk;
        vr = (const TT*)A.v + at * dv;
      }
      kv[b].load(kr, dk, lane);
      vv[b].load(vr, dv, lane);
    }
  };
  // The scores of an iteration, NS = HPG x PA_KEYS of them, are summed over the lanes so that each ends up in ONE lane
  // (a pair of lanes): cap, exponentials and the running maximum are then computed once per score instead of in all 32
  // lanes, and the weights come back by shuffles.  Score (head hh, key b) has index hh * PA_KEYS + b; bit r of the index is
  // bit 4 - r of the lanes that hold it.
  constexpr int NS = HPG * PA_KEYS;
  constexpr int LOGN = NS == 4 ? 2 : NS == 8 ? 3 : 4;
  static_assert(NS == 4 || NS == 8 || NS == 16, "four, eight or sixteen scores per iteration");
  int my_idx = 0;
#pragma unroll
  for (int rr = 0; rr < LOGN; ++rr) my_idx |= ((lane >> (4 - rr)) & 1) << rr;
  const int my_h = my_idx / PA_KEYS, my_b = my_idx % PA_KEYS;
  const float my_mult = A.scale * (A.temps ? A.temps[h0 + my_h] : 1.f);
  float my_m = -INFINITY, my_l = 0.f;          // of head my_h (the lanes of a head agree)
  const float inv_cap = A.cap > 0.f ? 1.0f / A.cap : 0.f;
  auto source = [](int idx) {
    int src = 0;
#pragma unroll
    for (int rr = 0; rr < LOGN; ++rr) src |= ((idx >> rr) & 1) << (4 - rr);
    return src;
  };
  auto use = [&](int n0, const Row (&kv)[PA_KEYS], const Row (&vv)[PA_KEYS]) {
    float v[NS];
#pragma unroll
    for (int hh = 0; hh < HPG; ++hh) {
#pragma unroll
      for (int b = 0; b < PA_KEYS; ++b) {
        float x = 0.f;
#pragma unroll
        for (int e = 0; e < NPL; ++e) x = fmaf(qreg[hh][e], kv[b].get(e), x);
        v[hh * PA_KEYS + b] = x;
      }
    }
    int off = 16;
#pragma unroll
    for (int cnt = NS; cnt > 1; cnt >>= 1) {
      const bool up = (lane & off) != 0;
#pragma unroll
      for (int i = 0; i < cnt / 2; ++i) {
        const float keep = up ? v[2 * i + 1] : v[2 * i];
        const float send = up ? v[2 * i] : v[2 * i + 1];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
      }
      off >>= 1;
    }
#pragma unroll
    for (int o2 = 16 >> LOGN; o2 > 0; o2 >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], o2);
    float x = v[0] * my_mult;
    if (A.cap > 0.f) x = A.cap * tanhf(x * inv_cap);
    if (n0 + my_b >= total) x = -INFINITY;
    // the head's keys of this iteration sit in the lanes that differ in bits 4 and 3
    float top = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 16));
    top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 8));
    const float m_new = fmaxf(my_m, top);          // finite: the iteration's first key exists
    const float my_f = expf(my_m - m_new);
    const float my_w = expf(x - m_new);
    float sum = my_w + __shfl_xor_sync(0xffffffffu, my_w, 16);
    sum += __shfl_xor_sync(0xffffffffu, sum, 8);
    my_l = my_l * my_f + sum;
    my_m = m_new;
#pragma unroll
    for (int hh = 0; hh < HPG; ++hh) {
      const float f = __shfl_sync(0xffffffffu, my_f, source(hh * PA_KEYS));
#pragma unroll
      for (int e = 0; e < NPL; ++e) acc[hh][e] *= f;
#pragma unroll
      for (int b = 0; b < PA_KEYS; ++b) {
        const float w = __shfl_sync(0xffffffffu, my_w, source(hh * PA_KEYS + b));
#pragma unroll
        for (int e = 0; e < NPL; ++e) acc[hh][e] = fmaf(w, vv[b].get(e), acc[hh][e]);
      }
    }
  };
  {
    constexpr int STRIDE = PG_WARPS * PA_KEYS;
    Row ka[PA_KEYS], va[PA_KEYS], kb[PA_KEYS], vb[PA_KEYS];
    int n0 = first_key + warp * PA_KEYS;
    if (n0 < total) fetch(n0, ka, va);
    while (n0 < total) {
      const int n1 = n0 + STRIDE;
      if (n1 < total) fetch(n1, kb, vb);
      use(n0, ka, va);
      if (n1 >= total) break;
      const int n2 = n1 + STRIDE;
      if (n2 < total) fetch(n2, ka, va);
      use(n1, kb, vb);
      n0 = n2;
    }
  }
#pragma unroll
  for (int hh = 0; hh < HPG; ++hh) {
#pragma unroll
    for (int e = 0; e < NPL; ++e) {
      const int c = Row::channel(e, lane);
      if (c < dv) acc_s[(warp * HPG + hh) * dv + c] = acc[hh][e];
    }
  }
  if (lane == source(my_h * PA_KEYS)) {        // one lane per head: the one whose unused bits are zero
    ml[2 * (warp * HPG + my_h)] = my_m;
    ml[2 * (warp * HPG + my_h) + 1] = my_l;
  }
  __syncthreads();
  if (A.splits > 1) {
    // the share's sums relative to its own maximum; merge_splits_kernel adds the shares, the sink and the rest
    float* part = A.scratch + (((size_t)t * A.G + g) * A.splits + blockIdx.z) * (size_t)(HPG * dv + 2 * HPG);
    for (int e = threadIdx.x; e < HPG * dv + HPG; e += blockDim.x) {
      const int hh = e < HPG * dv ? e / dv : e - HPG * dv;
      float top = -INFINITY;
#pragma unroll
      for (int w = 0; w < PG_WARPS; ++w) top = fmaxf(top, ml[2 * (w * HPG + hh)]);
      float o = 0.f;
#pragma unroll
      for (int w = 0; w < PG_WARPS; ++w) {
        const float mw = ml[2 * (w * HPG + hh)];
        const float fw = mw == -INFINITY ? 0.f : expf(mw - top);
        o = e < HPG * dv ? fmaf(acc_s[(w * HPG + hh) * dv + (e - hh * dv)], fw, o) : fmaf(ml[2 * (w * HPG + hh) + 1], fw, o);
      }
      if (e < HPG * dv) part[e] = o;
      else { part[HPG * dv + 2 * hh] = top; part[HPG * dv + 2 * hh + 1] = o; }
    }
    return;
  }
  // merge in warp order; the sink joins the denominator once
  for (int e = threadIdx.x; e < HPG * dv; e += blockDim.x) {
    const int hh = e / dv, c = e - hh * dv;
    const float sk = A.sinks ? A.sinks[h0 + hh] : -INFINITY;
    float top = sk;
#pragma unroll
    for (int w = 0; w < PG_WARPS; ++w) top = fmaxf(top, ml[2 * (w * HPG + hh)]);
    float denom = A.sinks ? expf(sk - top) : 0.f;
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < PG_WARPS; ++w) {
      const float mw = ml[2 * (w * HPG + hh)];
      const float fw = mw == -INFINITY ? 0.f : expf(mw - top);
      denom += ml[2 * (w * HPG + hh) + 1] * fw;
      o = fmaf(acc_s[(w * HPG + hh) * dv + c], fw, o);
    }
    os[e] = o / denom;
  }
  __syncthreads();
  const int half = dv / 2;
  const float p = (float)i;
  for (int e = threadIdx.x; e < HPG * (A.freq_v ? half : dv); e += blockDim.x) {
    if (A.freq_v) {
      const int hh = e / half, c = e - hh * half;
      TT* out = (TT*)A.out + t * A.ldo + (size_t)(h0 + hh) * dv;
      const float* gate = A.gates ? A.gates + t * A.ldgate + (size_t)(h0 + hh) * dv : nullptr;
      float cs, sn;
      pa_sincos(p, A.freq_v, c, cs, sn);
      const float a = os[hh * dv + c], b = os[hh * dv + c + half];
      float x0 = a * cs + b * sn, x1 = b * cs - a * sn;        // turned by -p
      if (gate) {
        x0 *= 1.0f / (1.0f + expf(-gate[c]));
        x1 *= 1.0f / (1.0f + expf(-gate[c + half]));
      }
      out[c] = co_from_float<TT>(x0);
      out[c + half] = co_from_float<TT>(x1);
    } else {
      const int hh = e / dv, c = e - hh * dv;
      float x = os[e];
      if (A.gates) x *= 1.0f / (1.0f + expf(-A.gates[t * A.ldgate + (size_t)(h0 + hh) * dv + c]));
      ((TT*)A.out)[t * A.ldo + (size_t)(h0 + hh) * dv + c] = co_from_float<TT>(x);
    }
  }
}

// grid (T, H): adds the shares of a row's keys in order, the sink, turns the row back, applies the gate.
template <typename TT>
__global__ void merge_splits_kernel(AttnArgs A, int hpg) {
  extern __shared__ __align__(16) float sm[];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const size_t t = blockIdx.x;
  const int h = blockIdx.y, g = h / hpg, hh = h - g * hpg, dv = A.dv;
  const size_t stride = (size_t)hpg * dv + 2 * hpg;
  const float* part = A.scratch + ((size_t)t * A.G + g) * A.splits * stride;
  float* os = sm;              // [dv]
  float* mls = sm + dv;        // [splits][2]: requested by as many threads at once
  for (int e = threadIdx.x; e < 2 * A.splits; e += blockDim.x) mls[e] = part[(e >> 1) * stride + hpg * dv + 2 * hh + (e & 1)];
  __syncthreads();
  const float sk = A.sinks ? A.sinks[h] : -INFINITY;
  float top = sk;
  for (int s2 = 0; s2 < A.splits; ++s2) top = fmaxf(top, mls[2 * s2]);
  float denom = A.sinks ? expf(sk - top) : 0.f;
  for (int s2 = 0; s2 < A.splits; ++s2)
    if (mls[2 * s2] != -INFINITY) denom += mls[2 * s2 + 1] * expf(mls[2 * s2] - top);
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    float o = 0.f;
#pragma unroll 8
    for (int s2 = 0; s2 < A.splits; ++s2) {
      const float x = part[s2 * stride + hh * dv + c];
      o = fmaf(x, mls[2 * s2] == -INFINITY ? 0.f : expf(mls[2 * s2] - top), o);
    }
    os[c] = o / denom;
  }
  __syncthreads();
  TT* out = (TT*)A.out + t * A.ldo + (size_t)h * dv;
  const float* gate = A.gates ? A.gates + t * A.ldgate + (size_t)h * dv : nullptr;
  if (A.freq_v) {
    const int half = dv / 2;
    const float p = (float)A.positions[t];
    for (int c = threadIdx.x; c < half; c += blockDim.x) {
      float cs, sn;
      pa_sincos(p, A.freq_v, c, cs, sn);
      const float a = os[c], b = os[c + half];
      float x0 = a * cs + b * sn, x1 = b * cs - a * sn;        // turned by -p
      if (gate) {
        x0 *= 1.0f / (1.0f + expf(-gate[c]));
        x1 *= 1.0f / (1.0f + expf(-gate[c + half]));
      }
      out[c] = co_from_float<TT>(x0);
      out[c + half] = co_from_float<TT>(x1);
    }
  } else {
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
      float x = os[c];
      if (gate) x *= 1.0f / (1.0f + expf(-gate[c]));
      out[c] = co_from_float<TT>(x);
    }
  }
}

template <typename TT>
static bool launch_grouped(const AttnArgs& A, int T, cudaStream_t stream) {
  const int hpg = A.H / A.G, big = max(A.dk, A.dv);
  const int npl = big <= 128 ? 4 : 8;
  // wider heads or more heads per key head do not fit the registers of two sets of rows; they take the kernel per head
  if (npl != 4 || (hpg != 1 && hpg != 2 && hpg != 4)) return false;
  const size_t smem = (size_t)(PG_WARPS * hpg * A.dv + 2 * PG_WARPS * hpg + hpg * A.dv + A.table_room) * sizeof(float);
  if (smem > 96 * 1024) return false;
  // vector accesses: head sizes in multiples of 128 and query rows that start on 16-byte boundaries
  const bool vec = A.dk % 128 == 0 && A.dv % 128 == 0 && (A.ldq * sizeof(TT)) % 16 == 0 && ((uintptr_t)A.q & 15) == 0;
  dim3 grid(T, A.G, A.splits), block(PG_WARPS * 32);
#define GO1(HPG, NPL, VEC)                                                                                                       \
  do {                                                                                                                           \
    if (smem > 48 * 1024)                                                                                                        \
      cudaFuncSetAttribute(pooled_attention_group_kernel<TT, HPG, NPL, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    co_launch(pooled_attention_group_kernel<TT, HPG, NPL, VEC>, grid, block, smem, stream, A);                                   \
  } while (0)
#define GO(HPG, NPL)                      \
  do {                                    \
    if (vec) GO1(HPG, NPL, true);         \
    else GO1(HPG, NPL, false);            \
  } while (0)
  if (hpg == 1) GO(1, 4); else if (hpg == 2) GO(2, 4); else GO(4, 4);
#undef GO
#undef GO1
  if (A.splits > 1) {
    co_count_launch();
    co_launch(merge_splits_kernel<TT>, dim3(T, A.H), dim3(64), (size_t)(A.dv + 2 * A.splits) * sizeof(float), stream, A, hpg);
  }
  return true;
}

}  // namespace

CO_EXPORT int coheryn_pooled_prepare(const float* proj, long ld, const int* positions, const float* freq_k, int rot,
                                     const float* freq_v, void* q_out, long ldq, int dtype, const int* slots, void* k_cache,
                                     void* v_cache, int T, int H, int G, int dk, int dv, int page_size, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rot < 0 || rot > dk || (rot & 1)) CO_FAIL("pooled_prepare: %d rotated channels of %d", rot, dk);
  if (rot && !freq_k) CO_FAIL("pooled_prepare: a rotation needs frequencies");
  if (freq_v && (dv & 1)) CO_FAIL("pooled_prepare: rotated values need an even number of channels, not %d", dv);
  dim3 grid(T);
  const int threads = 256;
  const size_t smem = (size_t)(rot + (freq_v ? dv : 0)) * sizeof(float);
  if (dtype == CO_F32)
    co_launch(pooled_prepare_kernel<float>, grid, dim3(threads), smem, stream, proj, ld, positions, freq_k, rot, freq_v, (float*)q_out, ldq,
              slots, (float*)k_cache, (float*)v_cache, H, G, dk, dv, page_size);
  else if (dtype == CO_BF16)
    co_launch(pooled_prepare_kernel<__nv_bfloat16>, grid, dim3(threads), smem, stream, proj, ld, positions, freq_k, rot, freq_v,
              (__nv_bfloat16*)q_out, ldq, slots, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, H, G, dk, dv, page_size);
  else CO_FAIL("pooled_prepare: unknown dtype %d", dtype);
  CO_CHECK_LAUNCH("pooled_prepare");
  return 0;
}

CO_EXPORT int coheryn_pooled_means(const void* k_cache, const void* v_cache, void* pk_cache, void* pv_cache, int dtype,
                                   const int* tables, int table_width, const int* pool_tables, int pool_table_width,
                                   const int* cu_q, const int* kv_lens, int B, int max_q_len, int G, int dk, int dv, int page_size,
                                   int pool, int pool_rows, cudaStream_t stream) {
  if (B <= 0 || pool < 1) return 0;
  if (pool_rows < (page_size + pool - 1) / pool) CO_FAIL("pooled_means: %d rows per page do not hold the blocks of a page", pool_rows);
  const int per_request = max_q_len / pool + 1;
  dim3 grid(B * per_request, G);
#define GO(TT)                                                                                                               \
  co_launch(pooled_means_kernel<TT>, grid, dim3(128), 0, stream, (const TT*)k_cache, (const TT*)v_cache, (TT*)pk_cache,        \
            (TT*)pv_cache, tables, table_width, pool_tables, pool_table_width, cu_q, kv_lens, per_request, G, dk, dv, page_size, \
            pool, pool_rows)
  if (dtype == CO_F32) GO(float);
  else if (dtype == CO_BF16) GO(__nv_bfloat16);
  else CO_FAIL("pooled_means: unknown dtype %d", dtype);
#undef GO
  CO_CHECK_LAUNCH("pooled_means");
  return 0;
}

// Into how many shares the grouped kernel cuts a row's keys: so that the CTAs fill the SMs about twice, at most eight,
// one when the step has rows enough by itself or the scratch area (`scratch_floats`) is too small.  A function of the
// step's row count only.
CO_EXPORT int coheryn_pooled_attention_splits(int T, int H, int G, int dv, long scratch_floats) {
  const long ctas = (long)T * G;
  int splits = (int)(296 / (ctas > 0 ? ctas : 1));
  if (splits > 8) splits = 8;
  if (splits < 2) return 1;
  const long need = (long)T * G * splits * ((long)(H / G) * dv + 2 * (H / G));
  return scratch_floats >= need ? splits : 1;
}

CO_EXPORT int coheryn_pooled_attention(const void* q, long ldq, void* out, long ldo, const void* k, const void* v, const void* pk,
                                       const void* pv, int dtype, const int* tables, int table_width, const int* pool_tables,
                                       int pool_table_width, const int* token_req, const int* positions, const float* temps,
                                       const float* sinks, const float* gates, long ldgate, const float* freq_v, int T, int H, int G,
                                       int dk, int dv, int page_size, int window, int pool, int pool_rows, float scale, float cap,
                                       float* scratch, long scratch_floats, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H < 1 || G < 1 || H % G) CO_FAIL("pooled_attention: %d heads over %d key heads", H, G);
  if (dk < 1 || dk > 32 * PA_MAX_PER_LANE || dv < 1 || dv > 32 * PA_MAX_PER_LANE)
    CO_FAIL("pooled_attention: head sizes %d / %d (1..%d)", dk, dv, 32 * PA_MAX_PER_LANE);
  if (pool > 0 && (!pk || !pv || !pool_tables)) CO_FAIL("pooled_attention: blocks need their cache");
  AttnArgs A{q, ldq, out, ldo, k, v, pk, pv, tables, table_width, pool_tables, pool_table_width, token_req, positions, temps, sinks,
             gates, ldgate, freq_v, H, G, dk, dv, page_size, window, pool, pool_rows, scale, cap,
             window > 0 && window / page_size + 2 <= 2048 ? window / page_size + 2 : 0, 1, scratch};
  A.splits = coheryn_pooled_attention_splits(T, H, G, dv, scratch_floats);
  if (dtype != CO_F32 && dtype != CO_BF16) CO_FAIL("pooled_attention: unknown dtype %d", dtype);
  static const bool grouped = !(getenv("COHERYN_POOLED_GROUPED") && getenv("COHERYN_POOLED_GROUPED")[0] == '0');
  if (grouped && (dtype == CO_F32 ? launch_grouped<float>(A, T, stream) : launch_grouped<__nv_bfloat16>(A, T, stream))) {
    CO_CHECK_LAUNCH("pooled_attention_group");
    return 0;
  }
  const size_t smem = (size_t)(dk + (PA_WARPS + 1) * dv + 2 * PA_WARPS) * sizeof(float);
  if (dtype == CO_F32) co_launch(pooled_attention_kernel<float>, dim3(T, H), dim3(PA_WARPS * 32), smem, stream, A);
  else co_launch(pooled_attention_kernel<__nv_bfloat16>, dim3(T, H), dim3(PA_WARPS * 32), smem, stream, A);
  CO_CHECK_LAUNCH("pooled_attention");
  return 0;
}
