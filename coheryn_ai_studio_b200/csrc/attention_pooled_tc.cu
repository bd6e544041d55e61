// Window attention over positions and block means on the tensor cores (sm_100a, bfloat16 storage, mma.sync m16n8k16 with
// float32 accumulation), for the rows of prompt portions.  Same arithmetic as the float32-arithmetic kernel of
// attention_pooled.cu, tile by tile:
//
//   * a CTA of four warps takes 64 consecutive rows of one request and one head; a warp 16 of them;
//   * its keys come in tiles of BN = 32 (three CTAs per SM where tiles of 64 leave room for two; 10 to 15 % faster): first the means of the blocks that its LAST row sees (rows that see fewer mask the
//     rest), then the positions from the first one its FIRST row sees, counted in absolute multiples of BN so that a row's
//     sums do not depend on where its portion was cut; rows and channels of a tile arrive by cp.async through the two
//     block tables, two stages deep;
//   * scores S = Q K^T in float32, times scale * temp[head], capped by cap * tanh(S / cap) (computed as
//     cap - 2 cap / (exp(2 S / cap) + 1), in units of log 2), masked; online softmax in float32; a weight enters the product with the values as the sum of two bfloat16 numbers (high + low part), so that it
//     carries sixteen bits of mantissa; the sink joins the denominator at the end;
//   * epilogue: the row divided by its denominator, turned back by minus its position over all value channels (the pair
//     (c, c + dv/2) sits in one thread), multiplied by sigmoid(gate), written as bfloat16.
//
// Compiled per (key channels, value channels): CO_PW_DK, CO_PW_DV, multiples of 16; dv at most 128 (the accumulators of a
// row tile stay in registers).
#include <cuda_bf16.h>

#include "common.cuh"

#ifndef CO_PW_DK
#define CO_PW_DK 128
#endif
#ifndef CO_PW_DV
#define CO_PW_DV 128
#endif

namespace {

constexpr int DK = CO_PW_DK, DV = CO_PW_DV;
#ifndef CO_PW_BN
#define CO_PW_BN 32
#endif
constexpr int BM = 64, BN = CO_PW_BN, WARPS = 4;      // rows and keys per tile
constexpr float LOG2E = 1.4426950408889634f;
constexpr int LDK = DK + 8, LDV = DV + 8;          // shared-memory row strides (elements): no bank conflicts for ldmatrix
static_assert(DK % 16 == 0 && DV % 16 == 0 && DK <= 256 && DV <= 128, "head sizes the tensor-core kernel takes");

struct TcArgs {
  const __nv_bfloat16* q; long ldq;
  __nv_bfloat16* out; long ldo;
  const __nv_bfloat16* k; const __nv_bfloat16* v; const __nv_bfloat16* pk; const __nv_bfloat16* pv;
  const int* tables; int table_width; const int* pool_tables; int pool_table_width;
  const int* cu_q; const int* kv_lens;
  const float* temps; const float* sinks; const float* gates; long ldgate;
  const float* freq_v;
  int H, G, page_size, window, pool, pool_rows;
  float scale, cap;
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;       // zero fill for rows that no key stands behind
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
// (high, low) parts of two weights as packed bfloat16 pairs
__device__ __forceinline__ void split_pack(float x, float y, unsigned& hi, unsigned& lo) {
  const __nv_bfloat16 xh = __float2bfloat16_rn(x), yh = __float2bfloat16_rn(y);
  hi = pack_bf16(__bfloat162float(xh), __bfloat162float(yh));
  lo = pack_bf16(x - __bfloat162float(xh), y - __bfloat162float(yh));
}

// 2^x and 1/x by the special-function unit (relative error about 2^-22): the scores live in units of log 2 from the cap
// on, so a weight is one subtraction and one of these.
__device__ __forceinline__ float tc_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float tc_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void tc_sincos(float p, const float* freq, int i, float& c, float& s) {
  const float fh = freq[2 * i], fl = freq[2 * i + 1];
  const float ah = p * fh;
  const float al = fmaf(p, fh, -ah) + p * fl;
  float sh, ch, sl, cl;
  sincosf(ah, &sh, &ch);
  sincosf(al, &sl, &cl);
  c = ch * cl - sh * sl;
  s = sh * cl + ch * sl;
}

// grid (row tiles of the longest request, requests, heads)
__global__ void __launch_bounds__(WARPS * 32) pooled_attention_tc_kernel(TcArgs A) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);       // [BM][LDK]
  __nv_bfloat16* Ks = Qs + BM * LDK;                                     // [2][BN][LDK]
  __nv_bfloat16* Vs = Ks + 2 * BN * LDK;                                 // [2][BN][LDV]
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int r = blockIdx.y, h = blockIdx.z, g = h / (A.H / A.G);
  const int q0 = A.cu_q[r], qn = A.cu_q[r + 1] - q0;
  const int row0 = blockIdx.x * BM;
  if (row0 >= qn) return;
  const int rows = min(BM, qn - row0);
  const int p_first = A.kv_lens[r] - qn + row0;        // position of the tile's first row
  const int p_last = p_first + rows - 1;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gi = lane >> 2, ti = lane & 3;
  const int* table = A.tables + (size_t)r * A.table_width;
  const int* ptable = A.pool ? A.pool_tables + (size_t)r * A.pool_table_width : nullptr;

  // the tile's keys: block means [0, nb_max), then positions [pos_lo, p_last]
  const int nb_max = (A.pool > 0 && p_last - A.window + 1 > 0) ? (p_last - A.window + 1) / A.pool : 0;
  const int lo_first = A.window > 0 ? max(0, p_first - A.window + 1) : 0;
  const int pos_lo = (lo_first / BN) * BN;
  const int n_pool_tiles = (nb_max + BN - 1) / BN;
  const int n_tiles = n_pool_tiles + (p_last - pos_lo) / BN + 1;

  auto load_tile = [&](int t, int stage) {
    __nv_bfloat16* ks = Ks + (size_t)stage * BN * LDK;
    __nv_bfloat16* vs = Vs + (size_t)stage * BN * LDV;
    const bool pooled = t < n_pool_tiles;
    const int first = pooled ? t * BN : pos_lo + (t - n_pool_tiles) * BN;
    // two threads per key row: one copies its key channels, the other its value channels (the row is looked up once)
    constexpr int TPR = WARPS * 32 / BN, SHARE = TPR / 2;      // threads per row; threads that share a row's keys (or values)
    static_assert(TPR * BN == WARPS * 32 && (TPR == 2 || TPR == 4), "two or four threads per cached row");
    const int row = tid / TPR, is_v = (tid % TPR) / SHARE, sub = tid % SHARE;
    const int idx = first + row;
    bool valid;
    size_t at;
    if (pooled) {
      valid = idx < nb_max;
      const int b = valid ? idx : 0;
      const long last = (long)b * A.pool + A.pool - 1;
      const int lp = (int)(last / A.page_size);
      const int prow = b - (int)(((long)lp * A.page_size) / A.pool);
      at = ((size_t)ptable[lp] * A.G + g) * A.pool_rows + prow;
    } else {
      valid = idx <= p_last;
      const int pos = valid ? idx : p_last;
      at = ((size_t)table[pos / A.page_size] * A.G + g) * A.page_size + (size_t)(pos % A.page_size);
    }
    if (is_v) {
      const __nv_bfloat16* src = (pooled ? A.pv : A.v) + at * DV;
      __nv_bfloat16* dst = vs + row * LDV;
#pragma unroll
      for (int c = sub * (DV / 8 / SHARE); c < (sub + 1) * (DV / 8 / SHARE); ++c) cp_async16(dst + c * 8, src + c * 8, valid);
    } else {
      const __nv_bfloat16* src = (pooled ? A.pk : A.k) + at * DK;
      __nv_bfloat16* dst = ks + row * LDK;
#pragma unroll
      for (int c = sub * (DK / 8 / SHARE); c < (sub + 1) * (DK / 8 / SHARE); ++c) cp_async16(dst + c * 8, src + c * 8, valid);
    }
  };

  // queries of the tile (rows beyond the request's are zero)
  {
    constexpr int QC = DK / 8;
    const __nv_bfloat16* qsrc = A.q + (size_t)(q0 + row0) * A.ldq + (size_t)h * DK;
    for (int e = tid; e < BM * QC; e += WARPS * 32) {
      const int row = e / QC, c = e % QC;
      cp_async16(Qs + row * LDK + c * 8, qsrc + (size_t)min(row, rows - 1) * A.ldq + c * 8, row < rows);
    }
  }
  load_tile(0, 0);
  cp_async_commit();

  const float mult = A.scale * (A.temps ? A.temps[h] : 1.f);
  const float inv_cap = A.cap > 0.f ? 1.0f / A.cap : 0.f;
  // this thread's two rows
  const int ia = p_first + warp * 16 + gi, ib = ia + 8;
  const int nba = (A.pool > 0 && ia - A.window + 1 > 0) ? (ia - A.window + 1) / A.pool : 0;
  const int nbb = (A.pool > 0 && ib - A.window + 1 > 0) ? (ib - A.window + 1) / A.pool : 0;
  const int loa = A.window > 0 ? ia - A.window + 1 : 0, lob = A.window > 0 ? ib - A.window + 1 : 0;

  float o[DV / 8][4];
#pragma unroll
  for (int n = 0; n < DV / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float ma = -INFINITY, mb = -INFINITY, la = 0.f, lb = 0.f;

  for (int t = 0; t < n_tiles; ++t) {
    const int stage = t & 1;
    if (t + 1 < n_tiles) load_tile(t + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const __nv_bfloat16* ks = Ks + (size_t)stage * BN * LDK;
    const __nv_bfloat16* vs = Vs + (size_t)stage * BN * LDV;
    const bool pooled = t < n_pool_tiles;
    const int first = pooled ? t * BN : pos_lo + (t - n_pool_tiles) * BN;
    // a warp whose rows see nothing of the tile skips it (its rows' windows start behind it, or it holds later positions)
    bool any;
    {
      const int wa = p_first + warp * 16, wb = wa + 15;                     // the warp's positions
      if (pooled) {
        const int nbw = (wb - A.window + 1 > 0) ? (wb - A.window + 1) / A.pool : 0;
        any = first < nbw;
      } else {
        const int low = A.window > 0 ? wa - A.window + 1 : 0;
        any = first <= wb && first + BN - 1 >= low;
      }
    }
    if (any) {
      float s[BN / 8][4];
#pragma unroll
      for (int n = 0; n < BN / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < DK / 16; ++kk) {
        unsigned a[4];
        ldmatrix_x4(a, Qs + (warp * 16 + (lane & 15)) * LDK + kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int np = 0; np < BN / 16; ++np) {
          unsigned b[4];
          ldmatrix_x4(b, ks + (np * 16 + (lane & 7) + (lane >> 4) * 8) * LDK + kk * 16 + ((lane >> 3) & 1) * 8);
          mma_bf16(s[2 * np], a, b[0], b[1]);
          mma_bf16(s[2 * np + 1], a, b[2], b[3]);
        }
      }
      // scale, cap, mask; row maxima.  A tile whose every key every row of the warp sees needs no mask.
      bool inner;
      {
        const int wa = p_first + warp * 16, wb = wa + 15;
        if (pooled) inner = first + BN <= ((wa - A.window + 1 > 0) ? (wa - A.window + 1) / A.pool : 0);
        else inner = first + BN - 1 <= wa && (A.window <= 0 || first >= wb - A.window + 1);
      }
      float ta = -INFINITY, tb = -INFINITY;
      // in units of log 2: x2 = score * scale * factor * log2(e), capped as C - 2 C / (2^(2 x2 / C) + 1) with C = cap * log2(e)
      const float cap2 = A.cap * LOG2E, to_exp = mult * 2.0f * inv_cap * LOG2E, to_log2 = mult * LOG2E;
#pragma unroll
      for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          s[n][e] = A.cap > 0.f ? fmaf(-2.0f * cap2, tc_rcp(tc_ex2(s[n][e] * to_exp) + 1.0f), cap2) : s[n][e] * to_log2;
      }
      if (!inner) {
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int idx = first + n * 8 + 2 * ti + (e & 1);
            const bool second = e >= 2;
            bool seen;
            if (pooled) seen = idx < (second ? nbb : nba);
            else seen = second ? (idx <= ib && idx >= lob) : (idx <= ia && idx >= loa);
            if (!seen) s[n][e] = -INFINITY;
          }
        }
      }
#pragma unroll
      for (int n = 0; n < BN / 8; ++n) {
        ta = fmaxf(ta, fmaxf(s[n][0], s[n][1]));
        tb = fmaxf(tb, fmaxf(s[n][2], s[n][3]));
      }
      ta = fmaxf(ta, __shfl_xor_sync(0xffffffffu, ta, 1)); ta = fmaxf(ta, __shfl_xor_sync(0xffffffffu, ta, 2));
      tb = fmaxf(tb, __shfl_xor_sync(0xffffffffu, tb, 1)); tb = fmaxf(tb, __shfl_xor_sync(0xffffffffu, tb, 2));
      const float na = fmaxf(ma, ta), nb_ = fmaxf(mb, tb);
      const float base_a = na == -INFINITY ? 0.f : na, base_b = nb_ == -INFINITY ? 0.f : nb_;
      const float fa = tc_ex2(ma - base_a), fb = tc_ex2(mb - base_b);     // 2^(-inf) = 0 while nothing was seen
      ma = na; mb = nb_;
      float sa = 0.f, sb = 0.f;
#pragma unroll
      for (int n = 0; n < BN / 8; ++n) {
        s[n][0] = tc_ex2(s[n][0] - base_a); s[n][1] = tc_ex2(s[n][1] - base_a);
        s[n][2] = tc_ex2(s[n][2] - base_b); s[n][3] = tc_ex2(s[n][3] - base_b);
        sa += s[n][0] + s[n][1];
        sb += s[n][2] + s[n][3];
      }
      la = la * fa + sa;
      lb = lb * fb + sb;
      if (__any_sync(0xffffffffu, fa != 1.f || fb != 1.f)) {        // most tiles raise no row's maximum
#pragma unroll
        for (int n = 0; n < DV / 8; ++n) { o[n][0] *= fa; o[n][1] *= fa; o[n][2] *= fb; o[n][3] *= fb; }
      }
      // O += P V, the weights as high + low parts
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk) {
        unsigned ph[4], pl[4];
        split_pack(s[2 * kk][0], s[2 * kk][1], ph[0], pl[0]);
        split_pack(s[2 * kk][2], s[2 * kk][3], ph[1], pl[1]);
        split_pack(s[2 * kk + 1][0], s[2 * kk + 1][1], ph[2], pl[2]);
        split_pack(s[2 * kk + 1][2], s[2 * kk + 1][3], ph[3], pl[3]);
#pragma unroll
        for (int np = 0; np < DV / 16; ++np) {
          unsigned b[4];
          ldmatrix_x4_trans(b, vs + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDV + np * 16 + (lane >> 4) * 8);
          mma_bf16(o[2 * np], ph, b[0], b[1]);
          mma_bf16(o[2 * np], pl, b[0], b[1]);
          mma_bf16(o[2 * np + 1], ph, b[2], b[3]);
          mma_bf16(o[2 * np + 1], pl, b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  // the rows' sums over the four lanes that share a row; the sink
  la += __shfl_xor_sync(0xffffffffu, la, 1); la += __shfl_xor_sync(0xffffffffu, la, 2);
  lb += __shfl_xor_sync(0xffffffffu, lb, 1); lb += __shfl_xor_sync(0xffffffffu, lb, 2);
  float scale_a, scale_b;
  if (A.sinks) {
    const float sk = A.sinks[h] * LOG2E;          // the maxima are in units of log 2
    const float top_a = fmaxf(ma, sk), top_b = fmaxf(mb, sk);
    const float ka = exp2f(ma - top_a), kb = exp2f(mb - top_b);
    scale_a = ka / (la * ka + exp2f(sk - top_a));
    scale_b = kb / (lb * kb + exp2f(sk - top_b));
  } else {
    scale_a = 1.0f / la;
    scale_b = 1.0f / lb;
  }
  const int ra = row0 + warp * 16 + gi, rb = ra + 8;        // rows within the request's run
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int rr = half ? rb : ra;
    if (rr >= qn) continue;
    const float sc = half ? scale_b : scale_a;
    const float p = (float)(half ? ib : ia);
    __nv_bfloat16* dst = A.out + (size_t)(q0 + rr) * A.ldo + (size_t)h * DV;
    const float* gate = A.gates ? A.gates + (size_t)(q0 + rr) * A.ldgate + (size_t)h * DV : nullptr;
    if (A.freq_v) {
#pragma unroll
      for (int n = 0; n < DV / 16; ++n) {       // columns c (tile n) and c + DV/2 (tile n + DV/16) form pairs
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int c = n * 8 + 2 * ti + e;
          float x = o[n][2 * half + e] * sc, y = o[n + DV / 16][2 * half + e] * sc;
          float cs, sn;
          tc_sincos(p, A.freq_v, c, cs, sn);
          float x0 = x * cs + y * sn, x1 = y * cs - x * sn;       // turned by -p
          if (gate) {
            x0 *= 1.0f / (1.0f + expf(-gate[c]));
            x1 *= 1.0f / (1.0f + expf(-gate[c + DV / 2]));
          }
          dst[c] = __float2bfloat16_rn(x0);
          dst[c + DV / 2] = __float2bfloat16_rn(x1);
        }
      }
    } else {
#pragma unroll
      for (int n = 0; n < DV / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int c = n * 8 + 2 * ti + e;
          float x = o[n][2 * half + e] * sc;
          if (gate) x *= 1.0f / (1.0f + expf(-gate[c]));
          dst[c] = __float2bfloat16_rn(x);
        }
      }
    }
  }
}

}  // namespace

CO_EXPORT void coheryn_pooled_tc_shape(int* dk, int* dv) { *dk = DK; *dv = DV; }

CO_EXPORT int coheryn_pooled_attention_tc(const void* q, long ldq, void* out, long ldo, const void* k, const void* v, const void* pk,
                                          const void* pv, const int* tables, int table_width, const int* pool_tables,
                                          int pool_table_width, const int* cu_q, const int* kv_lens, const float* temps,
                                          const float* sinks, const float* gates, long ldgate, const float* freq_v, int B,
                                          int max_q_len, int H, int G, int page_size, int window, int pool, int pool_rows,
                                          float scale, float cap, cudaStream_t stream) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (H < 1 || G < 1 || H % G) CO_FAIL("pooled_attention_tc: %d heads over %d key heads", H, G);
  if (pool > 0 && (!pk || !pv || !pool_tables || window <= 0)) CO_FAIL("pooled_attention_tc: blocks need their cache and a window");
  if ((ldq % 8) || ((uintptr_t)q & 15)) CO_FAIL("pooled_attention_tc: query rows must start on 16-byte boundaries");
  TcArgs A{(const __nv_bfloat16*)q, ldq, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
           (const __nv_bfloat16*)pk, (const __nv_bfloat16*)pv, tables, table_width, pool_tables, pool_table_width, cu_q, kv_lens,
           temps, sinks, gates, ldgate, freq_v, H, G, page_size, window, pool, pool_rows, scale, cap};
  const size_t smem = (size_t)(BM * LDK + 2 * BN * LDK + 2 * BN * LDV) * sizeof(__nv_bfloat16);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(pooled_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      CO_FAIL("pooled_attention_tc: %zu bytes of shared memory are not available", smem);
    configured = true;
  }
  dim3 grid((max_q_len + BM - 1) / BM, B, H);
  co_launch(pooled_attention_tc_kernel, grid, dim3(WARPS * 32), smem, stream, A);
  CO_CHECK_LAUNCH("pooled_attention_tc");
  return 0;
}
