// Attention with options that the stock kernels do not have, over the same cache pages:
//
//   * several score MAPS per head: a query head carries `maps` queries of `dk` channels, a key/value head `maps`
//     keys (a key row in the cache is [maps][dk]) and ONE value row; every map is a softmax attention of its own
//     over the same values, and the head's output is a_0 - lambda a_1 (differential attention; maps = 1 is the
//     ordinary case);
//   * a mask by CHUNKS: position i sees j <= i with floor(i / chunk) = floor(j / chunk), chunks counted from
//     position 0 of the sequence; or a window (i - j < window); or all j <= i;
//   * a SINK: one more term exp(0) in the softmax's denominator that carries no value;
//   * the head's output divided by its root mean square over the value channels, and a constant factor;
//   * values of another head size than keys; values that are the first dv channels of the key row itself (a latent
//     attention keeps one row per position that serves as key and as value);
//   * a sink with a learned score per head instead of 0.
//
// And the kernel in front of it: queries and keys normalised per head (RMS over dk, one weight [dk] shared by the
// heads) and/or rotated by position (rotate-half pairing over the first `rot` channels of every unit of dk, the
// angle position * frequency computed here in float32 pairs, so no table bounds the positions), then keys and
// values written into their cache pages.
//
// Everything is float32 arithmetic on float32 or bfloat16 storage; scores, weights and their sums never leave
// float32.  A row's result depends on its position and the keys it sees only, in an order fixed by those.
#include "common.cuh"

namespace {

// ---------------------------------------------------------------------------------
// q_out[t, u, :] and the cache rows of token t.  A "unit" is dk consecutive channels of a projection that are
// normalised and rotated together: q has q_units of them (heads x maps), k has k_units (kv heads x maps).
// freq: [rot/2][2] float32 = (high, low) parts of each pair's frequency; angle = position * (high + low).
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
unit_norm_rope_kv_write_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, long ld,
                               const void* __restrict__ wq, const void* __restrict__ wk, int w_dtype, float eps, int normalise,
                               const int* __restrict__ positions, const float* __restrict__ freq, int rot, float rot_scale,
                               T* __restrict__ q_out, long ldq, const int* __restrict__ slots, T* __restrict__ k_cache,
                               T* __restrict__ v_cache, int q_units, int k_units, int nkv, int dk, int dv, int page_size) {
  extern __shared__ __align__(16) float sm[];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const size_t t = blockIdx.x;
  const int half = rot / 2;
  const int write = slots != nullptr;
  const int units = q_units + (write ? k_units : 0);
  float* cs = sm;                      // [half][2]
  float* scale_s = sm + 2 * half;      // [units]
  float* xs = scale_s + units;         // [units][dk]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  if (rot) {
    const float p = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float fh = freq[2 * i], fl = freq[2 * i + 1];
      const float ah = p * fh;
      const float al = fmaf(p, fh, -ah) + p * fl;      // what the rounding of p * fh lost, and the low part
      float s, c, sl, cl;
      sincosf(ah, &s, &c);
      sincosf(al, &sl, &cl);                           // |al| is at most half a unit in the last place of ah
      cs[2 * i] = (c * cl - s * sl) * rot_scale;
      cs[2 * i + 1] = (s * cl + c * sl) * rot_scale;
    }
  }
  const float* qr = q + t * ld;
  const float* kr = k + t * ld;
  for (int e = threadIdx.x; e < units * dk; e += blockDim.x) {
    const int u = e / dk;
    xs[e] = u < q_units ? qr[e] : kr[e - q_units * dk];
  }
  __syncthreads();
  for (int u = warp; u < units; u += warps) {
    float s = 1.f;
    if (normalise) {
      float ss = 0.f;
      for (int d = lane; d < dk; d += 32) ss = fmaf(xs[u * dk + d], xs[u * dk + d], ss);
      s = 1.0f / sqrtf(co_warp_sum(ss) / (float)dk + eps);
    }
    if (lane == 0) scale_s[u] = s;
  }
  __syncthreads();
  int slot = 0;
  size_t page = 0, off = 0;
  if (write) { slot = slots[t]; page = (size_t)(slot / page_size); off = (size_t)(slot % page_size); }
  const int maps = k_units / (nkv > 0 ? nkv : 1);
  for (int e = threadIdx.x; e < units * dk; e += blockDim.x) {
    const int u = e / dk, d = e % dk;
    const void* w = u < q_units ? wq : wk;
    auto val = [&](int dd) {
      const float x = xs[u * dk + dd];
      return normalise ? (x * scale_s[u]) * co_load_any(w, w_dtype, dd) : x;
    };
    float y;
    if (d < half) {
      y = val(d) * cs[2 * d] - val(d + half) * cs[2 * d + 1];
    } else if (d < rot) {
      const int i = d - half;
      y = val(d) * cs[2 * i] + val(i) * cs[2 * i + 1];
    } else {
      y = val(d);
    }
    if (u < q_units) {
      q_out[t * ldq + e] = co_from_float<T>(y);
    } else if (slot >= 0) {
      const int ku = u - q_units, g = ku / maps, m = ku % maps;
      k_cache[((page * nkv + g) * page_size + off) * ((size_t)maps * dk) + (size_t)m * dk + d] = co_from_float<T>(y);
    }
  }
  if (!write || slot < 0) return;
  const float* vr = v + t * ld;
  for (int e = threadIdx.x; e < nkv * dv; e += blockDim.x) {
    const int g = e / dv, d = e % dv;
    v_cache[((page * nkv + g) * page_size + off) * dv + d] = co_from_float<T>(vr[e]);
  }
}

// ---------------------------------------------------------------------------------
// One CTA per (token, query head); four warps each run an online softmax per map over the keys
// first + warp, first + warp + 4, ..; their (maximum, sum, accumulator) triples are merged in warp order.
// ---------------------------------------------------------------------------------
constexpr int WARPS = 4;
constexpr int MAX_MAPS = 2;
constexpr int WIDE_PER_LANE = 24; // head sizes up to 768, for a single map

struct MapsShape {
  int nh, nkv, dk, dv, maps, page_size, window, chunk, sink, head_norm;
  float scale, lambda, eps, out_scale;
  const float* sink_scores;     // [heads]: the sink's score per head (null: 0)
  long v_row;                   // channels between two value rows (dv, or the key row's size when values live in the keys)
};

template <typename T, int MAPS, int MAX_PER_LANE>
__global__ void __launch_bounds__(WARPS * 32)
attention_maps_kernel(const T* __restrict__ q, long q_stride, T* __restrict__ out, long out_stride,
                      const T* __restrict__ k_cache, const T* __restrict__ v_cache, const int* __restrict__ block_tables,
                      int max_blocks, const int* __restrict__ token_req, const int* __restrict__ positions, MapsShape S) {
  extern __shared__ __align__(16) float smem[];
  const int dk = S.dk, dv = S.dv;
  float* qs = smem;                               // [MAPS][dk]
  float* merge_acc = smem + MAPS * dk;            // [MAPS][WARPS][dv]
  __shared__ float merge_m[MAPS][WARPS], merge_l[MAPS][WARPS];
  __shared__ float scratch[33];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int req = token_req[t];
  const int pos = positions[t];
  int first = S.window > 0 ? max(0, pos - S.window + 1) : 0;
  if (S.chunk > 0) first = max(first, (pos / S.chunk) * S.chunk);
  const int kvh = h / (S.nh / S.nkv);
  const int* table = block_tables + (size_t)req * max_blocks;
  const T* qrow = q + (size_t)t * q_stride + (size_t)h * MAPS * dk;
  for (int d = threadIdx.x; d < MAPS * dk; d += blockDim.x) qs[d] = co_to_float(qrow[d]);
  __syncthreads();

  float m[MAPS], l[MAPS], acc[MAPS][MAX_PER_LANE];
#pragma unroll
  for (int a = 0; a < MAPS; ++a) {
    m[a] = -INFINITY; l[a] = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) acc[a][i] = 0.f;
  }
  for (int kp = first + warp; kp <= pos; kp += WARPS) {
    const int page = table[kp / S.page_size];
    const size_t row = ((size_t)page * S.nkv + kvh) * S.page_size + (kp % S.page_size);
    const T* kr = k_cache + row * (size_t)(MAPS * dk);
    const T* vr = v_cache + row * (size_t)S.v_row;
    float vv[MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int d = lane + 32 * i;
      vv[i] = d < dv ? co_to_float(vr[d]) : 0.f;
    }
#pragma unroll
    for (int a = 0; a < MAPS; ++a) {
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < dk) dot = fmaf(qs[a * dk + d], co_to_float(kr[a * dk + d]), dot);
      }
      const float s = co_warp_sum(dot) * S.scale;
      const float m_new = fmaxf(m[a], s);
      const float corr = expf(m[a] - m_new);    // exp(-inf) = 0 on the first key
      const float p = expf(s - m_new);
      l[a] = l[a] * corr + p;
#pragma unroll
      for (int i = 0; i < MAX_PER_LANE; ++i) acc[a][i] = acc[a][i] * corr + p * vv[i];
      m[a] = m_new;
    }
  }
#pragma unroll
  for (int a = 0; a < MAPS; ++a) {
    if (lane == 0) { merge_m[a][warp] = m[a]; merge_l[a][warp] = l[a]; }
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int d = lane + 32 * i;
      if (d < dv) merge_acc[(a * WARPS + warp) * dv + d] = acc[a][i];
    }
  }
  __syncthreads();
  float f[MAPS][WARPS], inv[MAPS];
#pragma unroll
  for (int a = 0; a < MAPS; ++a) {
    const float sink_score = S.sink_scores ? S.sink_scores[h] : 0.f;      // the sink's score: learned per head, or 0
    float M = S.sink ? sink_score : -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) M = fmaxf(M, merge_m[a][w]);
    float L = S.sink ? expf(sink_score - M) : 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      f[a][w] = merge_m[a][w] == -INFINITY ? 0.f : expf(merge_m[a][w] - M);
      L += merge_l[a][w] * f[a][w];
    }
    inv[a] = 1.0f / L;
  }
  // the head's output, one value channel per thread and round; its mean square for the norm
  float o[(MAX_PER_LANE * 32 + WARPS * 32 - 1) / (WARPS * 32)];
  float ss = 0.f;
  int n = 0;
  for (int d = threadIdx.x; d < dv; d += blockDim.x, ++n) {
    float a0 = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) a0 += merge_acc[w * dv + d] * f[0][w];
    a0 *= inv[0];
    if (MAPS == 2) {
      float a1 = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) a1 += merge_acc[(WARPS + w) * dv + d] * f[1][w];
      a0 = a0 - S.lambda * (a1 * inv[1]);
    }
    o[n] = a0;
    ss = fmaf(a0, a0, ss);
  }
  float factor = S.out_scale;
  if (S.head_norm) factor *= 1.0f / sqrtf(co_block_sum(ss, scratch) / (float)dv + S.eps);
  T* orow = out + (size_t)t * out_stride + (size_t)h * dv;
  n = 0;
  for (int d = threadIdx.x; d < dv; d += blockDim.x, ++n) orow[d] = co_from_float<T>(o[n] * factor);
}

// ---------------------------------------------------------------------------------
// Latent attention, the step in front of the scores.  A token's projections (float32, one row stride): queries head by
// head as [dim plain | rd rotated], and (for a layer with keys of its own) kv_rank latent channels followed by rd key
// channels shared by the heads.  The latent is divided by its root mean square and multiplied by a weight, the rd parts
// of queries and key turn by position over their first `rot` channels, and the cache row of the token becomes
// [latent | rotated key].  The plain query parts leave as q_plain [T, heads * dim] for the product that carries them into
// the latent space; the rotated parts go to their place in q_out [T, heads * (kv_rank + rd)], whose other columns that
// product fills.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const float* __restrict__ q, const float* __restrict__ kv, long ld, const void* __restrict__ w_norm,
                      int w_dtype, float eps, const int* __restrict__ positions, const float* __restrict__ freq, int rot,
                      float rot_scale, T* __restrict__ q_plain, T* __restrict__ q_out, const int* __restrict__ slots,
                      T* __restrict__ cache, int heads, int dim, int rd, int rank, int page_size) {
  extern __shared__ __align__(16) float sm[];
  __shared__ float scratch[33];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const size_t t = blockIdx.x;
  const int half = rot / 2;
  float* cs = sm;      // [half][2]
  if (rot) {
    const float p = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float fh = freq[2 * i], fl = freq[2 * i + 1];
      const float ah = p * fh;
      const float al = fmaf(p, fh, -ah) + p * fl;
      float s, c, sl, cl;
      sincosf(ah, &s, &c);
      sincosf(al, &sl, &cl);
      cs[2 * i] = (c * cl - s * sl) * rot_scale;
      cs[2 * i + 1] = (s * cl + c * sl) * rot_scale;
    }
  }
  __syncthreads();
  auto turned = [&](const float* x, int d) {       // channel d of a rotated part x[0 .. rd)
    if (d < half) return x[d] * cs[2 * d] - x[d + half] * cs[2 * d + 1];
    if (d < rot) return x[d] * cs[2 * (d - half)] + x[d - half] * cs[2 * (d - half) + 1];
    return x[d];
  };
  const float* qr = q + t * ld;
  const int per = dim + rd, wide = rank + rd;
  for (int e = threadIdx.x; e < heads * per; e += blockDim.x) {
    const int h = e / per, d = e % per;
    if (d < dim) q_plain[t * ((size_t)heads * dim) + (size_t)h * dim + d] = co_from_float<T>(qr[e]);
    else q_out[t * ((size_t)heads * wide) + (size_t)h * wide + rank + (d - dim)] = co_from_float<T>(turned(qr + h * per + dim, d - dim));
  }
  if (!slots) return;
  const int slot = slots[t];
  const float* kr = kv + t * ld;
  float ss = 0.f;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) ss = fmaf(kr[d], kr[d], ss);
  const float inv = 1.0f / sqrtf(co_block_sum(ss, scratch) / (float)rank + eps);
  if (slot < 0) return;
  T* row = cache + (size_t)slot * wide;          // one key/value head: row = page * page_size + offset
  for (int d = threadIdx.x; d < wide; d += blockDim.x) {
    const float y = d < rank ? (kr[d] * inv) * co_load_any(w_norm, w_dtype, d) : turned(kr + rank, d - rank);
    row[d] = co_from_float<T>(y);
  }
}

}  // namespace


// freq: float32 [rot/2][2] on the device (null when rot = 0).  wq / wk: [dk] (null when normalise = 0).  slots null: only the
// queries are made.  The key cache is [page][nkv][page_size][k_units / nkv * dk], the value cache [page][nkv][page_size][dv].
CO_EXPORT int coheryn_unit_norm_rope_kv_write(const float* q, const float* k, const float* v, long ld, const void* wq,
                                              const void* wk, int w_dtype, float eps, int normalise, const int* positions,
                                              const float* freq, int rot, float rot_scale, void* q_out, int dtype, long ldq,
                                              const int* slots, void* k_cache, void* v_cache, int T, int q_units, int k_units,
                                              int nkv, int dk, int dv, int page_size, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (q_units < 1 || dk < 1 || dv < 1 || page_size < 1 || rot < 0 || rot > dk || (rot & 1))
    CO_FAIL("unit_norm_rope_kv_write: bad sizes (units %d, channels %d, rotated %d)", q_units, dk, rot);
  if (slots && (nkv < 1 || k_units < nkv || k_units % nkv)) CO_FAIL("unit_norm_rope_kv_write: %d key units over %d kv heads", k_units, nkv);
  if (rot && (!freq || !positions)) CO_FAIL("unit_norm_rope_kv_write: a rotation needs frequencies and positions");
  const int units = q_units + (slots ? k_units : 0);
  const size_t smem = ((size_t)rot + units + (size_t)units * dk) * sizeof(float);
  if (smem > 200 * 1024) CO_FAIL("unit_norm_rope_kv_write: %d units of %d channels do not fit in shared memory", units, dk);
#define GO(TT)                                                                                                        \
  {                                                                                                                   \
    auto kern = unit_norm_rope_kv_write_kernel<TT>;                                                                   \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
    co_launch(kern, dim3(T), dim3(256), smem, stream, q, k, v, ld, wq, wk, w_dtype, eps, normalise, positions, freq, rot, \
              rot_scale, (TT*)q_out, ldq, slots, (TT*)k_cache, (TT*)v_cache, q_units, k_units, nkv, dk, dv, page_size); \
  }
  if (dtype == CO_F32) GO(float)
  else if (dtype == CO_BF16) GO(__nv_bfloat16)
  else CO_FAIL("unit_norm_rope_kv_write: unknown dtype %d", dtype);
#undef GO
  CO_CHECK_LAUNCH("unit_norm_rope_kv_write");
  return 0;
}

CO_EXPORT int coheryn_attention_maps(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                                     const void* v_cache, int dtype, const int* block_tables, int max_blocks,
                                     const int* token_req, const int* positions, int T, int nh, int nkv, int dk, int dv,
                                     int maps, int page_size, int window, int chunk, int sink, float scale, float lambda,
                                     int head_norm, float eps, float out_scale, const float* sink_scores, int values_in_keys,
                                     cudaStream_t stream) {
  if (T <= 0) return 0;
  const int widest = dk > dv ? dk : dv;
  if (widest > 32 * (maps == 1 ? WIDE_PER_LANE : 8) || dk < 1 || dv < 1)
    CO_FAIL("attention_maps: head sizes %d and %d must lie in 1..%d", dk, dv, 32 * (maps == 1 ? WIDE_PER_LANE : 8));
  if (values_in_keys && dv > maps * dk) CO_FAIL("attention_maps: %d value channels do not fit a key row of %d", dv, maps * dk);
  if (nkv <= 0 || nh % nkv != 0) CO_FAIL("attention_maps: %d heads do not group over %d kv heads", nh, nkv);
  if (maps < 1 || maps > MAX_MAPS) CO_FAIL("attention_maps: %d score maps per head (1..%d)", maps, MAX_MAPS);
  MapsShape S{nh, nkv, dk, dv, maps, page_size, window, chunk, sink, head_norm, scale, lambda, eps, out_scale, sink_scores,
              values_in_keys ? (long)maps * dk : (long)dv};
  if (values_in_keys) v_cache = k_cache;
  dim3 grid(T, nh);
  const size_t smem = ((size_t)maps * dk + (size_t)maps * WARPS * dv) * sizeof(float);
#define GO(TT, MM, PL)                                                                                                  \
  {                                                                                                                     \
    auto kern = attention_maps_kernel<TT, MM, PL>;                                                                      \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
    co_launch(kern, grid, dim3(WARPS * 32), smem, stream, (const TT*)q, q_stride, (TT*)out, out_stride,                 \
              (const TT*)k_cache, (const TT*)v_cache, block_tables, max_blocks, token_req, positions, S);               \
  }
  const bool wide = widest > 256;
  if (dtype == CO_F32) { if (maps == 2) GO(float, 2, 8) else if (wide) GO(float, 1, WIDE_PER_LANE) else GO(float, 1, 8) }
  else if (dtype == CO_BF16) { if (maps == 2) GO(__nv_bfloat16, 2, 8) else if (wide) GO(__nv_bfloat16, 1, WIDE_PER_LANE) else GO(__nv_bfloat16, 1, 8) }
  else CO_FAIL("attention_maps: unknown dtype %d", dtype);
#undef GO
  CO_CHECK_LAUNCH("attention_maps");
  return 0;
}

// q: [T, heads * (dim + rd)] and kv: [T, rank + rd], float32 rows of one stride `ld`.  slots null: a layer that reads another
// layer's cache (kv, w_norm and cache are not used).  The cache is [page][1][page_size][rank + rd].
CO_EXPORT int coheryn_latent_prepare(const float* q, const float* kv, long ld, const void* w_norm, int w_dtype, float eps,
                                     const int* positions, const float* freq, int rot, float rot_scale, void* q_plain,
                                     void* q_out, int dtype, const int* slots, void* cache, int T, int heads, int dim, int rd,
                                     int rank, int page_size, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (heads < 1 || dim < 1 || rd < 0 || rank < 1 || rot < 0 || rot > rd || (rot & 1))
    CO_FAIL("latent_prepare: bad sizes (heads %d, plain %d, rotated %d of %d, latent %d)", heads, dim, rot, rd, rank);
  if (rot && (!freq || !positions)) CO_FAIL("latent_prepare: a rotation needs frequencies and positions");
  if (slots && (!kv || !w_norm || !cache)) CO_FAIL("latent_prepare: writing the cache needs the projection, the weight and the pages");
  const size_t smem = (size_t)(rot + 2) * sizeof(float);
#define GO(TT)                                                                                                          \
  co_launch(latent_prepare_kernel<TT>, dim3(T), dim3(256), smem, stream, q, kv, ld, w_norm, w_dtype, eps, positions, freq, rot, \
            rot_scale, (TT*)q_plain, (TT*)q_out, slots, (TT*)cache, heads, dim, rd, rank, page_size)
  if (dtype == CO_F32) GO(float);
  else if (dtype == CO_BF16) GO(__nv_bfloat16);
  else CO_FAIL("latent_prepare: unknown dtype %d", dtype);
#undef GO
  CO_CHECK_LAUNCH("latent_prepare");
  return 0;
}
