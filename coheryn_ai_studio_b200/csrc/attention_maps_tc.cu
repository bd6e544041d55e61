// The attention of attention_variants.cu (score maps, chunk mask, sink, normalised output) on the tensor cores, for
// bfloat16 caches, compiled for one (channels per map, value channels, maps): CO_MAPS_DK, CO_MAPS_DV, CO_MAPS_N.
//
// The scores Q K^T are bfloat16 products accumulated in float32 (mma.sync m16n8k16); masks, maxima, exponentials,
// the sums of a row and the weights stay float32.  A weight enters the second product as the SUM OF TWO bfloat16
// numbers (w = hi + lo, lo = bf16(w - hi)): sixteen bits of mantissa instead of eight, so that weights computed in
// float32 are not cut to bfloat16 on their way into the tensor cores; the products with V accumulate in float32.
//
// Prompt portions (`maps_tiles_kernel`): a CTA owns 64 consecutive rows of one request and one query head, a warp 16
// of them.  TWO passes over the key tiles: the first finds every row's maximum and sum per map (scores only), the
// second computes the scores again (the same instructions, hence the same bits), forms
// w = e_0 / l_0 - lambda e_1 / l_1 in float32 and accumulates w V once.  No accumulator is ever rescaled, two maps
// cost one accumulator, and the difference of the maps is taken before anything is rounded.
//
// Decoding (`maps_decode_kernel` + `maps_combine_kernel`): the rows of a tile are the query heads of ONE key/value
// head for one token, the visible keys are cut into at most sixteen splits at absolute multiples of the split size,
// each of a CTA's four warps takes a quarter of a split (an online softmax over its tiles, one map after the other)
// and leaves (maximum, sum, unnormalised output) per head and map; a second kernel merges the parts in order, adds
// the sink, takes the difference of the maps, normalises and writes.
//
// Key tiles start at absolute multiples of the tile size and a masked key contributes an exact zero, so a row's
// result does not depend on what else is in its tile, its step or its batch.
#include "common.cuh"

#if !defined(CO_MAPS_DK) || !defined(CO_MAPS_DV) || !defined(CO_MAPS_N)
#error "compile with -DCO_MAPS_DK=<channels per map> -DCO_MAPS_DV=<value channels> -DCO_MAPS_N=<maps>"
#endif

namespace {

constexpr int DK = CO_MAPS_DK, DV = CO_MAPS_DV, MAPS = CO_MAPS_N;
static_assert(DK % 16 == 0 && DV % 16 == 0 && DK >= 16 && DV >= 16 && DK <= 1024 && DV <= 1024, "head sizes: multiples of 16 up to 1024");
static_assert(MAPS == 1 || MAPS == 2, "one score map or two");
constexpr int KROW = MAPS * DK;                  // channels of a key row (and of a query head)
#ifdef CO_MAPS_V_IN_K
constexpr bool V_IN_K = true;                    // the values are the first DV channels of the key row: nothing else is fetched
static_assert(DV <= KROW, "values inside the key row cannot be wider than it");
#else
constexpr bool V_IN_K = false;
#endif
constexpr int KS = KROW + 8;                     // padded row strides in shared memory: an odd number of 16-byte units
constexpr int VS = V_IN_K ? KS : DV + 8;
constexpr int VROW = V_IN_K ? 0 : VS;            // shared-memory elements of a value row (none when it is the key row)
constexpr int BM = 64, WARPS = 4;
#ifdef CO_MAPS_BN
constexpr int BN = CO_MAPS_BN;                   // a measuring switch: keys per tile
#else
constexpr int BN = 32;      // measured on a B200: tiles of 32 keys with three resident CTAs per SM beat tiles of 64 with two by 12 %
#endif
static_assert(BN == 32 || BN == 64, "key tiles of 32 or 64 positions");
// A warp's accumulator holds at most 256 value channels.  Wider values are taken in equal CHUNKS of DVC channels, one
// after the other: the pass over the keys that multiplies weights and values runs once per chunk and computes the scores
// again (the same instructions, hence the same bits), so every chunk sees the same weights.
constexpr int value_chunk(int dv) {
  if (dv <= 256) return dv;
  for (int c = 256; c > 16; c -= 16)
    if (dv % c == 0) return c;
  return 16;
}
constexpr int DVC = value_chunk(DV), NCH = DV / DVC;
constexpr int NT = BN / 8, OT = DVC / 8;
constexpr int MAX_SPLITS = 16;
typedef __nv_bfloat16 bf16;

struct MapsArgs {
  const bf16* q; long ldq; bf16* out; long ldo;
  const bf16* k_cache; const bf16* v_cache;
  const int* block_tables; int max_blocks;
  const int* cu_q; const int* kv_lens;
  int nh, nkv, page_size, window, chunk, sink, head_norm, skip_single;
  int table_cache;      // block-table entries a CTA of the prompt kernel may keep in shared memory
  float scale_log2, lambda, eps, out_scale;
  const float* sink_scores;     // [heads]: the sink's score per head (null: 0)
  const float* gates; long gates_ld;   // [tokens][heads] (row stride gates_ld): head h's output times sigmoid(gates[t, h]) (null: none)
};
__device__ __forceinline__ float gate_of(const MapsArgs& A, size_t token, int h) {
  return A.gates ? 1.0f / (1.0f + expf(-A.gates[token * A.gates_ld + h])) : 1.0f;
}
// the sink's score of head h in the log2 domain
__device__ __forceinline__ float sink_log2(const MapsArgs& A, int h) {
  return A.sink_scores ? A.sink_scores[h] * 1.4426950408889634f : 0.f;
}

__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(unsigned (&r)[4], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16 bytes from global to shared memory; `bytes` = 0 writes zeros and reads nothing.
__device__ __forceinline__ void cp_async16(void* dst, const void* src, int bytes) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(a), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ unsigned pack2(float x, float y) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
  return *reinterpret_cast<const unsigned*>(&v);
}
__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}
__device__ __forceinline__ int first_visible(int pos, int window, int chunk) {
  int f = window > 0 ? max(0, pos - window + 1) : 0;
  if (chunk > 0) f = max(f, (pos / chunk) * chunk);
  return f;
}

// 2^x by the hardware's approximation (two units in the last place; 2^-inf = 0).
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Rows `key0 .. key0 + BN - 1` of a request's keys (and values) into shared memory by THREADS threads; a position
// at or beyond `kv_len`, or on a page that is gone, becomes zeros.  A row is looked up once by the threads that share it.
template <int THREADS>
__device__ __forceinline__ void load_keys(bf16* ks, bf16* vs, const MapsArgs& A, const int* table, int kvh, int key0,
                                          int kv_len, int tid) {
  constexpr int KC = KROW / 8, VC = DV / 8;
  constexpr int TPR = THREADS >= BN ? THREADS / BN : 1;        // threads per row
  constexpr int ROWS = THREADS / TPR;                          // rows per round
  const int sub = tid % TPR;
#pragma unroll
  for (int row = tid / TPR; row < BN; row += ROWS) {
    const int j = key0 + row;
    int page = -1;
    if (j < kv_len) page = table[j / A.page_size];
    const bool ok = page >= 0;
    const int bytes = ok ? 16 : 0;
    const size_t at = ok ? ((size_t)page * A.nkv + kvh) * A.page_size + (size_t)(j % A.page_size) : 0;
    const bf16* ksrc = A.k_cache + at * KROW;
    bf16* kdst = ks + row * KS;
#pragma unroll
    for (int ch = sub; ch < KC; ch += TPR) cp_async16(kdst + ch * 8, ksrc + ch * 8, bytes);
    if (!V_IN_K && vs) {
      const bf16* vsrc = A.v_cache + at * DV;
      bf16* vdst = vs + row * VS;
#pragma unroll
      for (int ch = sub; ch < VC; ch += TPR) cp_async16(vdst + ch * 8, vsrc + ch * 8, bytes);
    }
  }
}

// s[nt][.] = the 16 x BN scores of map m: rows of qs (16 rows, stride KS) times the keys of ks (BN rows, stride KS).
__device__ __forceinline__ void scores(float (&s)[NT][4], const bf16* qs, const bf16* ks, int m, int lane) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
  for (int k0 = 0; k0 < DK; k0 += 16) {
    unsigned a[4];
    ldsm_x4(a, qs + (lane & 15) * KS + m * DK + k0 + (lane >> 4) * 8);
#pragma unroll
    for (int nt = 0; nt < NT; nt += 2) {
      unsigned b[4];
      ldsm_x4(b, ks + (nt * 8 + (lane & 7) + (lane >> 4) * 8) * KS + m * DK + k0 + ((lane >> 3) & 1) * 8);
      mma16816(s[nt], a, b[0], b[1]);
      mma16816(s[nt + 1], a, b[2], b[3]);
    }
  }
}

// o += w V for the 16 x BN weights w (float32, in the accumulator layout of `scores`) and the BN x DV values of vs:
// every weight as hi + lo in bfloat16.
__device__ __forceinline__ void weights_times_values(float (&o)[OT][4], const float (&w)[NT][4], const bf16* vs, int lane) {
#pragma unroll
  for (int kb = 0; kb < NT / 2; ++kb) {
    unsigned hi[4], lo[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float x = w[2 * kb + (i >> 1)][(i & 1) * 2], y = w[2 * kb + (i >> 1)][(i & 1) * 2 + 1];
      const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
      hi[i] = *reinterpret_cast<const unsigned*>(&h);
      lo[i] = pack2(x - __low2float(h), y - __high2float(h));
    }
#pragma unroll
    for (int nt = 0; nt < OT; nt += 2) {
      unsigned b[4];
      ldsm_x4_t(b, vs + (kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + nt * 8 + (lane >> 4) * 8);
      mma16816(o[nt], hi, b[0], b[1]);
      mma16816(o[nt], lo, b[0], b[1]);
      mma16816(o[nt + 1], hi, b[2], b[3]);
      mma16816(o[nt + 1], lo, b[2], b[3]);
    }
  }
}

// The scores of a tile in the log2 domain, masked: element (nt, e) belongs to row (e >> 1) of the thread's two rows
// and to key key0 + nt * 8 + 2 (lane & 3) + (e & 1); a key outside [first, pos] of its row becomes -infinity.
__device__ __forceinline__ void mask_scale(float (&s)[NT][4], int key0, int lane, const int (&pos)[2], const int (&first)[2], float scale_log2) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int j = key0 + nt * 8 + 2 * (lane & 3) + (e & 1), r = e >> 1;
      s[nt][e] = (j <= pos[r] && j >= first[r]) ? s[nt][e] * scale_log2 : -INFINITY;
    }
}

__device__ __forceinline__ void scale_only(float (&s)[NT][4], float scale_log2) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[nt][e] *= scale_log2;
}

// ---------------------------------------------------------------------------------
// Prompt portions.  grid: (row tiles of the longest request, requests, query heads).
// ---------------------------------------------------------------------------------
#ifndef CO_MAPS_MIN_CTAS
#define CO_MAPS_MIN_CTAS ((DV <= 128 && KROW <= 128) ? 3 : 1)      // the registers of wider heads allow one
#endif
__global__ void __launch_bounds__(WARPS * 32, CO_MAPS_MIN_CTAS) maps_tiles_kernel(MapsArgs A) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);        // [BM][KS]
  bf16* ks = qs + BM * KS;                             // [2][BN][KS]
  bf16* vs = ks + 2 * BN * KS;                         // [2][BN][VS]
  int* tbl = reinterpret_cast<int*>(vs + 2 * BN * VROW); // [table_cache]
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int r = blockIdx.y, h = blockIdx.z;
  const int q0 = A.cu_q[r], q_len = A.cu_q[r + 1] - q0, kv_len = A.kv_lens[r];
  const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;          // later rows see more keys: their CTAs start first
  if (tile * BM >= q_len || (A.skip_single && q_len == 1)) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kvh = h / (A.nh / A.nkv);
  const int* table = A.block_tables + (size_t)r * A.max_blocks;
  const int rows = min(BM, q_len - tile * BM);
  const int pos_lo = kv_len - q_len + tile * BM, pos_hi = pos_lo + rows - 1;
  for (int c = tid; c < BM * (KROW / 8); c += WARPS * 32) {       // the queries of the tile; rows beyond the portion are zeros
    const int row = c / (KROW / 8), ch = c % (KROW / 8);
    const bool ok = row < rows;
    cp_async16(qs + row * KS + ch * 8, A.q + (size_t)(q0 + tile * BM + (ok ? row : 0)) * A.ldq + (size_t)h * KROW + ch * 8, ok ? 16 : 0);
  }
  const int t_lo = first_visible(pos_lo, A.window, A.chunk) / BN, t_hi = pos_hi / BN, n_tiles = t_hi - t_lo + 1;
  {   // the pages of the CTA's keys, looked up once: the tile loads then read shared memory
    const int e0 = (t_lo * BN) / A.page_size, e1 = min(t_hi * BN + BN - 1, kv_len - 1) / A.page_size;
    if (e1 - e0 + 1 <= A.table_cache) {
      for (int i = tid; i <= e1 - e0; i += WARPS * 32) tbl[i] = table[e0 + i];
      __syncthreads();
      table = tbl - e0;
    }
  }
  int pos[2], first[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = warp * 16 + (lane >> 2) + 8 * i;
    pos[i] = row < rows ? pos_lo + row : -1;                      // -1: a row beyond the portion sees nothing
    first[i] = row < rows ? first_visible(pos[i], A.window, A.chunk) : 0;
  }
  const bf16* qw = qs + warp * 16 * KS;
  // what the warp's rows see together: a tile none of them sees is skipped, one all of them see whole needs no mask
  const bool whole_warp = warp * 16 + 15 < rows;
  const int wp_lo = pos_lo + warp * 16, wp_hi = min(pos_hi, wp_lo + 15);
  const int wf_lo = first_visible(min(wp_lo, pos_hi), A.window, A.chunk), wf_hi = first_visible(wp_hi, A.window, A.chunk);

  // pass 1: maximum and sum of every row, per map
  float mx[MAPS][2], sum[MAPS][2];
#pragma unroll
  for (int m = 0; m < MAPS; ++m) { mx[m][0] = mx[m][1] = -INFINITY; sum[m][0] = sum[m][1] = 0.f; }
  load_keys<WARPS * 32>(ks, nullptr, A, table, kvh, t_lo * BN, kv_len, tid);
  cp_commit();
  for (int i = 0; i < n_tiles; ++i) {
    if (i + 1 < n_tiles) load_keys<WARPS * 32>(ks + ((i + 1) & 1) * BN * KS, nullptr, A, table, kvh, (t_lo + i + 1) * BN, kv_len, tid);
    cp_commit();
    cp_wait<1>();
    __syncthreads();
    const bf16* kt = ks + (i & 1) * BN * KS;
    const int key0 = (t_lo + i) * BN;
    const bool unseen = warp * 16 >= rows || key0 > wp_hi || key0 + BN - 1 < wf_lo;
    const bool open = whole_warp && key0 >= wf_hi && key0 + BN - 1 <= wp_lo;
#pragma unroll
    for (int m = 0; m < MAPS; ++m) {
      if (unseen) break;
      float s[NT][4];
      scores(s, qw, kt, m, lane);
      if (open) scale_only(s, A.scale_log2);
      else mask_scale(s, key0, lane, pos, first, A.scale_log2);
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        float tm = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) tm = fmaxf(tm, fmaxf(s[nt][2 * rr], s[nt][2 * rr + 1]));
        tm = quad_max(tm);
        const float mn = fmaxf(mx[m][rr], tm);
        if (mn != -INFINITY) {
          float add = 0.f;
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) add += ex2(s[nt][2 * rr] - mn) + ex2(s[nt][2 * rr + 1] - mn);
          sum[m][rr] = sum[m][rr] * ex2(mx[m][rr] - mn) + add;     // ex2(-inf) = 0 the first time
          mx[m][rr] = mn;
        }
      }
    }
    __syncthreads();
  }
  float inv[MAPS][2];
#pragma unroll
  for (int m = 0; m < MAPS; ++m)
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      float l = quad_sum(sum[m][rr]), M = mx[m][rr];
      if (A.sink && M != -INFINITY) {               // one more term exp(sink score) that carries no value
        const float sv = sink_log2(A, h);
        const float M2 = fmaxf(M, sv);
        l = l * ex2(M - M2) + ex2(sv - M2);
        M = M2;
      }
      if (M == -INFINITY) { M = 0.f; inv[m][rr] = 0.f; }      // a row beyond the portion
      else inv[m][rr] = 1.0f / l;
      mx[m][rr] = M;
    }

  // pass 2: the weights, and their product with the values (once per chunk of value channels)
  for (int vc = 0; vc < NCH; ++vc) {
  if (vc) __syncthreads();                       // the last tile of the chunk before is read no more
  float o[OT][4];
#pragma unroll
  for (int nt = 0; nt < OT; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
  load_keys<WARPS * 32>(ks, vs, A, table, kvh, t_lo * BN, kv_len, tid);
  cp_commit();
  for (int i = 0; i < n_tiles; ++i) {
    if (i + 1 < n_tiles)
      load_keys<WARPS * 32>(ks + ((i + 1) & 1) * BN * KS, vs + ((i + 1) & 1) * BN * VS, A, table, kvh, (t_lo + i + 1) * BN, kv_len, tid);
    cp_commit();
    cp_wait<1>();
    __syncthreads();
    const bf16* kt = ks + (i & 1) * BN * KS;
    const int key0 = (t_lo + i) * BN;
    const bool unseen = warp * 16 >= rows || key0 > wp_hi || key0 + BN - 1 < wf_lo;
    const bool open = whole_warp && key0 >= wf_hi && key0 + BN - 1 <= wp_lo;
    if (!unseen) {
    float w[NT][4];
    {
      float s[NT][4];
      scores(s, qw, kt, 0, lane);
      if (open) scale_only(s, A.scale_log2);
      else mask_scale(s, key0, lane, pos, first, A.scale_log2);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) w[nt][e] = ex2(s[nt][e] - mx[0][e >> 1]) * inv[0][e >> 1];
      if (MAPS == 2) {
        scores(s, qw, kt, MAPS - 1, lane);
        if (open) scale_only(s, A.scale_log2);
        else mask_scale(s, key0, lane, pos, first, A.scale_log2);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) w[nt][e] -= A.lambda * (ex2(s[nt][e] - mx[MAPS - 1][e >> 1]) * inv[MAPS - 1][e >> 1]);
      }
    }
    weights_times_values(o, w, (V_IN_K ? kt : vs + (i & 1) * BN * VS) + vc * DVC, lane);
    }
    __syncthreads();
  }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int row = warp * 16 + (lane >> 2) + 8 * rr;
    float factor = A.out_scale;
    if (A.head_norm) {                           // (the launcher refuses it for values in several chunks)
      float ss = 0.f;
#pragma unroll
      for (int nt = 0; nt < OT; ++nt) ss += o[nt][2 * rr] * o[nt][2 * rr] + o[nt][2 * rr + 1] * o[nt][2 * rr + 1];
      factor *= 1.0f / sqrtf(quad_sum(ss) / (float)DV + A.eps);
    }
    if (row < rows) {
      factor *= gate_of(A, (size_t)(q0 + tile * BM + row), h);
      bf16* orow = A.out + (size_t)(q0 + tile * BM + row) * A.ldo + (size_t)h * DV + vc * DVC + 2 * (lane & 3);
#pragma unroll
      for (int nt = 0; nt < OT; ++nt)
        *reinterpret_cast<__nv_bfloat162*>(orow + nt * 8) = __floats2bfloat162_rn(o[nt][2 * rr] * factor, o[nt][2 * rr + 1] * factor);
    }
  }
  }
}

// ---------------------------------------------------------------------------------
// Decoding: requests that bring ONE token.  grid: (requests, kv heads, splits).  A part = (split, warp).
// scratch: [request][query head][map][splits * WARPS parts][DV + 2] = (output[DV], maximum, sum).
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(WARPS * 32) maps_decode_kernel(MapsArgs A, float* __restrict__ scratch, int split_keys, int n_splits) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);        // [16][KS]: the query heads of the kv head, then zero rows
  bf16* kall = qs + 16 * KS;                           // [WARPS][BN][KS]
  bf16* vall = kall + WARPS * BN * KS;                 // [WARPS][BN][VS]
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int r = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int q0 = A.cu_q[r], q_len = A.cu_q[r + 1] - q0;
  if (q_len != 1) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = A.nh / A.nkv;
  const int p = A.kv_lens[r] - 1, f = first_visible(p, A.window, A.chunk);
  const int key_lo = (f / split_keys + split) * split_keys;      // splits at absolute multiples of their size
  if (key_lo > p) return;                                         // the combine kernel knows which splits exist
  const int* table = A.block_tables + (size_t)r * A.max_blocks;
  for (int c = tid; c < 16 * (KROW / 8); c += WARPS * 32) {
    const int row = c / (KROW / 8), ch = c % (KROW / 8);
    const bool ok = row < group;
    cp_async16(qs + row * KS + ch * 8, A.q + (size_t)q0 * A.ldq + (size_t)(kvh * group + (ok ? row : 0)) * KROW + ch * 8, ok ? 16 : 0);
  }
  cp_commit();
  bf16* kw = kall + warp * BN * KS;
  bf16* vw = vall + warp * BN * VROW;
  const int quarter = split_keys / WARPS;                         // a multiple of BN
  const int w_lo = key_lo + warp * quarter, w_hi = min(w_lo + quarter, p + 1);
  const int pos[2] = {(lane >> 2) < group ? p : -1, (lane >> 2) + 8 < group ? p : -1};
  const int first[2] = {f, f};
  if (w_lo < w_hi) load_keys<32>(kw, vw, A, table, kvh, w_lo, p + 1, lane);     // in flight with the queries
  cp_commit();
  cp_wait<0>();
  __syncthreads();
  for (int pass = 0; pass < MAPS * NCH; ++pass) {      // a map's chunks of value channels one after the other
    const int m = pass / NCH, vc = pass % NCH;
    float mx[2] = {-INFINITY, -INFINITY}, sum[2] = {0.f, 0.f};
    float o[OT][4];
#pragma unroll
    for (int nt = 0; nt < OT; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
    for (int key0 = w_lo; key0 < w_hi; key0 += BN) {
      if (key0 != w_lo || (pass > 0 && w_lo + BN < w_hi)) {       // the first tile is there already, unless a later one took its place
        __syncwarp();
        load_keys<32>(kw, vw, A, table, kvh, key0, p + 1, lane);
        cp_commit();
        cp_wait<0>();
        __syncwarp();
      }
      float s[NT][4];
      scores(s, qs, kw, m, lane);
      mask_scale(s, key0, lane, pos, first, A.scale_log2);
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        float tm = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) tm = fmaxf(tm, fmaxf(s[nt][2 * rr], s[nt][2 * rr + 1]));
        tm = quad_max(tm);
        const float mn = fmaxf(mx[rr], tm);
        const float safe = mn == -INFINITY ? 0.f : mn;
        const float corr = ex2(mx[rr] - safe);                  // 0 the first time
        float add = 0.f;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          s[nt][2 * rr] = ex2(s[nt][2 * rr] - safe);
          s[nt][2 * rr + 1] = ex2(s[nt][2 * rr + 1] - safe);
          add += s[nt][2 * rr] + s[nt][2 * rr + 1];
          }
        sum[rr] = sum[rr] * corr + add;
        mx[rr] = mn;
#pragma unroll
        for (int nt = 0; nt < OT; ++nt) { o[nt][2 * rr] *= corr; o[nt][2 * rr + 1] *= corr; }
      }
      weights_times_values(o, s, (V_IN_K ? kw : vw) + vc * DVC, lane);
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      const int row = (lane >> 2) + 8 * rr;
      const float l = quad_sum(sum[rr]);
      if (row < group) {
        float* part = scratch + ((((size_t)r * A.nh + kvh * group + row) * MAPS + m) * (n_splits * WARPS) + split * WARPS + warp) * (DV + 2);
#pragma unroll
        for (int nt = 0; nt < OT; ++nt) {
          part[vc * DVC + nt * 8 + 2 * (lane & 3)] = o[nt][2 * rr];
          part[vc * DVC + nt * 8 + 2 * (lane & 3) + 1] = o[nt][2 * rr + 1];
        }
        if ((lane & 3) == 0) { part[DV] = mx[rr]; part[DV + 1] = l; }
      }
    }
  }
}

// grid: (requests, query heads); DV threads are enough, any block size works.  The parts' maxima and sums are fetched by
// one thread each and turned into factors in shared memory; the outputs are then added with independent loads.
__global__ void __launch_bounds__(128) maps_combine_kernel(MapsArgs A, const float* __restrict__ scratch, int split_keys, int n_splits) {
  __shared__ float red[33];
  __shared__ float factor_s[MAPS][MAX_SPLITS * WARPS];
  __shared__ float coef_s[MAPS];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y;
  const int q0 = A.cu_q[r], q_len = A.cu_q[r + 1] - q0;
  if (q_len != 1) return;
  const int p = A.kv_lens[r] - 1, f = first_visible(p, A.window, A.chunk);
  const int n_parts = (p / split_keys - f / split_keys + 1) * WARPS;
  const float* base = scratch + ((size_t)r * A.nh + h) * MAPS * (n_splits * WARPS) * (DV + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp < MAPS) {                       // a warp per map: maxima and sums of its parts, merged in a fixed tree
    const float* parts = base + (size_t)warp * (n_splits * WARPS) * (DV + 2);
    float m[(MAX_SPLITS * WARPS + 31) / 32], l[(MAX_SPLITS * WARPS + 31) / 32];
    const float sv = sink_log2(A, h);
    float M = A.sink ? sv : -INFINITY;
#pragma unroll
    for (int k = 0; k < (MAX_SPLITS * WARPS + 31) / 32; ++k) {
      const int i = lane + 32 * k;
      m[k] = i < n_parts ? parts[i * (DV + 2) + DV] : -INFINITY;
      l[k] = i < n_parts ? parts[i * (DV + 2) + DV + 1] : 0.f;
      M = fmaxf(M, m[k]);
    }
    M = co_warp_max(M);
    float L = 0.f;
#pragma unroll
    for (int k = 0; k < (MAX_SPLITS * WARPS + 31) / 32; ++k) {
      const int i = lane + 32 * k;
      const float fac = ex2(m[k] - M);                    // 0 for a part that saw no key
      if (i < n_parts) factor_s[warp][i] = fac;
      L += l[k] * fac;
    }
    L = co_warp_sum(L) + (A.sink ? ex2(sv - M) : 0.f);
    if (lane == 0) coef_s[warp] = (warp == 0 ? 1.0f : -A.lambda) / L;
  }
  __syncthreads();
  float acc[(DV + 127) / 128];
#pragma unroll
  for (int i = 0; i < (DV + 127) / 128; ++i) acc[i] = 0.f;
  for (int m = 0; m < MAPS; ++m) {
    const float* parts = base + (size_t)m * (n_splits * WARPS) * (DV + 2);
    int n = 0;
    for (int d = threadIdx.x; d < DV; d += blockDim.x, ++n) {
      float a = 0.f;
#pragma unroll 8
      for (int i = 0; i < n_parts; ++i) a = fmaf(parts[i * (DV + 2) + d], factor_s[m][i], a);
      acc[n] = fmaf(coef_s[m], a, acc[n]);
    }
  }
  float factor = A.out_scale * gate_of(A, (size_t)q0, h);
  if (A.head_norm) {
    float ss = 0.f;
    int n = 0;
    for (int d = threadIdx.x; d < DV; d += blockDim.x, ++n) ss += acc[n] * acc[n];
    factor *= 1.0f / sqrtf(co_block_sum(ss, red) / (float)DV + A.eps);
  }
  int n = 0;
  for (int d = threadIdx.x; d < DV; d += blockDim.x, ++n)
    A.out[(size_t)q0 * A.ldo + (size_t)h * DV + d] = __float2bfloat16_rn(acc[n] * factor);
}

}  // namespace

CO_EXPORT int coheryn_maps_shape(int* dk, int* dv, int* maps) { *dk = DK; *dv = DV; *maps = MAPS; return 0; }
CO_EXPORT int coheryn_maps_values_in_keys() { return V_IN_K ? 1 : 0; }

// How the keys a decoded row can see are cut: the keys per split (a multiple of what a CTA's warps take in one round, cut at
// absolute multiples of itself) and the most splits a row then has (its keys may straddle one boundary more than their
// number fills).
static void decode_plan(int max_kv_len, int window, int chunk, int* split_keys, int* n_splits) {
  int visible = max_kv_len;
  if (chunk > 0 && chunk < visible) visible = chunk;
  if (window > 0 && window < visible) visible = window;
  const int unit = WARPS * BN;
  int keys = ((visible + (MAX_SPLITS - 1) - 1) / (MAX_SPLITS - 1) + unit - 1) / unit * unit;
  if (keys < unit) keys = unit;
  *split_keys = keys;
  int n = (visible + keys - 1) / keys + 1;
  *n_splits = n > MAX_SPLITS ? MAX_SPLITS : n;
}

// Floats of scratch that the decode kernels need for `B` requests whose longest context is `max_kv_len`.
CO_EXPORT long coheryn_maps_scratch_floats(int B, int nh, int max_kv_len, int window, int chunk) {
  int keys, n;
  decode_plan(max_kv_len, window, chunk, &keys, &n);
  return (long)B * nh * MAPS * n * WARPS * (DV + 2);
}

// q [T, nh * maps * dk], out [T, nh * dv]: bfloat16.  The rows of request r are cu_q[r] .. cu_q[r+1], consecutive positions
// that end at kv_lens[r] - 1.  max_q_len, max_kv_len: host copies of the longest portion and context.  any_single /
// any_longer: whether some request brings one token / more than one.  gates (null: none): float32 [T, nh] with row stride
// gates_ld; head h's output of token t is multiplied by sigmoid(gates[t, h]).
CO_EXPORT int coheryn_attention_maps_bf16(const void* q, long ldq, void* out, long ldo, const void* k_cache, const void* v_cache,
                                          const int* block_tables, int max_blocks, const int* cu_q, const int* kv_lens, int B,
                                          int nh, int nkv, int page_size, int window, int chunk, int sink, float scale,
                                          float lambda, int head_norm, float eps, float out_scale, int max_q_len, int max_kv_len,
                                          int any_single, int any_longer, float* scratch, long scratch_floats,
                                          const float* sink_scores, const float* gates, long gates_ld, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (nkv <= 0 || nh % nkv) CO_FAIL("attention_maps_bf16: %d heads do not group over %d kv heads", nh, nkv);
  if ((ldq & 7) || (ldo & 1) || ((uintptr_t)q & 15) || ((uintptr_t)out & 3) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
    CO_FAIL("attention_maps_bf16: rows of q must start on 16-byte boundaries, rows of out on 4-byte ones");
  if (head_norm && NCH > 1) CO_FAIL("attention_maps_bf16: a normalised output needs values of at most 256 channels (%d)", DV);
  const int group = nh / nkv;
  const bool decode = any_single && group <= 16;
  MapsArgs A{(const bf16*)q, ldq, (bf16*)out, ldo, (const bf16*)k_cache, (const bf16*)v_cache, block_tables, max_blocks, cu_q,
             kv_lens, nh, nkv, page_size, window, chunk, sink, head_norm, decode ? 1 : 0, 0,
             scale * 1.4426950408889634f, lambda, eps, out_scale, sink_scores, gates, gates_ld};
  if (any_longer || !decode) {
    int visible = max_kv_len;                              // the most keys a row can see
    if (chunk > 0 && chunk < visible) visible = chunk;
    if (window > 0 && window < visible) visible = window;
    const long entries = ((long)visible + BM + 2 * BN) / page_size + 2;
    A.table_cache = entries <= 4096 ? (int)entries : 0;    // a longer table is read from global memory
    const size_t smem = ((size_t)BM * KS + (size_t)2 * BN * KS + (size_t)2 * BN * VROW) * sizeof(bf16) + (size_t)A.table_cache * sizeof(int);
    if (smem > 48 * 1024) cudaFuncSetAttribute(maps_tiles_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    co_launch(maps_tiles_kernel, dim3((max_q_len + BM - 1) / BM, B, nh), dim3(WARPS * 32), smem, stream, A);
    CO_CHECK_LAUNCH("maps_tiles");
  }
  if (decode) {
    if (scratch_floats < coheryn_maps_scratch_floats(B, nh, max_kv_len, window, chunk))
      CO_FAIL("attention_maps_bf16: scratch of %ld floats is too small", scratch_floats);
    int split_keys, n_splits;
    decode_plan(max_kv_len, window, chunk, &split_keys, &n_splits);
    const size_t smem = ((size_t)16 * KS + (size_t)WARPS * BN * (KS + VROW)) * sizeof(bf16);
    if (smem > 48 * 1024) cudaFuncSetAttribute(maps_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    co_launch(maps_decode_kernel, dim3(B, nkv, n_splits), dim3(WARPS * 32), smem, stream, A, scratch, split_keys, n_splits);
    CO_CHECK_LAUNCH("maps_decode");
    co_launch(maps_combine_kernel, dim3(B, nh), dim3(DV >= 128 ? 128 : (DV > 32 ? (DV + 31) / 32 * 32 : 64)), 0, stream, A, (const float*)scratch, split_keys, n_splits);
    CO_CHECK_LAUNCH("maps_combine");
  }
  return 0;
}
