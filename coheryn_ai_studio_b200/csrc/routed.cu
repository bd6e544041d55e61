// Routed experts and other products over GROUPS of rows that each meet a matrix of their own:
//
//   * route_select:   per token, from the router's float32 logits: softmax over all outputs, choice score = probability +
//                     correction, experts in `n_groups` equal groups of neighbours of which only the `keep` groups with the
//                     largest choice score may be chosen (the others count as minus infinity), the `top` largest choice
//                     scores, weights = the chosen probabilities / (their sum + 1e-20) * scale;
//   * route_sort:     the (token, choice) pairs that name a real expert (id < n_real) ordered by expert: row ranges per
//                     expert, each pair's row, each row's token, and the list of (expert, first row) row tiles;
//   * grouped_linear: C[rows of group g] = A[rows of group g] . W_g^T; the groups are the experts' row ranges (rows
//                     gathered through an index), or `G` equal column blocks of one matrix (the heads of an attention:
//                     every row belongs to every group, group g reads columns g * a_col .. of A and writes columns
//                     g * c_col .. of C); an optional gated epilogue (neighbouring output columns (2j, 2j+1) are gate and
//                     up) and an optional factor per (row, group), optionally through a sigmoid;
//   * route_combine:  out[t] = sum over the token's choices, in order, of weight * (the expert's output row, or the
//                     token's own input for an identity expert), in float32.
//
// float32 operands take FMA on the CUDA cores; bfloat16 operands the tensor cores (mma.sync m16n8k16, float32
// accumulation) when the sizes allow.  Either way an output element is a sum over k in an order fixed by the sizes alone,
// so a row's result depends neither on the rows it shares a tile with nor on where it sits among them.
#include "common.cuh"

namespace {

// ------------------------------------------------------------------------------------------------- router
constexpr int RS_WARPS = 4;

// smem per warp: choice[N], prob[N], gbest[n_groups]
__global__ void __launch_bounds__(RS_WARPS * 32)
route_select_kernel(const float* __restrict__ logits, long ld, const void* __restrict__ correction, int c_dtype, int T, int N,
                    int n_groups, int keep, int top, float scale, int mode, int* __restrict__ ids, float* __restrict__ weights) {
  extern __shared__ __align__(16) float sm[];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * RS_WARPS + warp;
  if (t >= T) return;
  float* choice = sm + (size_t)warp * (2 * N + n_groups);
  float* prob = choice + N;
  float* gbest = prob + N;
  const float* z = logits + (size_t)t * ld;
  if (mode == 1) {
    // the choice scores are the logits themselves (plus a bias); the weights come from the chosen ones alone
    for (int i = lane; i < N; i += 32) choice[i] = z[i] + (correction ? co_load_any(correction, c_dtype, i) : 0.f);
  } else {
    float m = -INFINITY;
    for (int i = lane; i < N; i += 32) m = fmaxf(m, z[i]);
    m = co_warp_max(m);
    float sum = 0.f;
    for (int i = lane; i < N; i += 32) {
      const float e = expf(z[i] - m);
      prob[i] = e;
      sum += e;
    }
    sum = co_warp_sum(sum);
    for (int i = lane; i < N; i += 32) {
      const float p = prob[i] / sum;
      prob[i] = p;
      choice[i] = p + (correction ? co_load_any(correction, c_dtype, i) : 0.f);
    }
  }
  __syncwarp();
  if (n_groups > 1 && keep < n_groups) {
    const int per = N / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
      float b = -INFINITY;
      for (int i = 0; i < per; ++i) b = fmaxf(b, choice[g * per + i]);
      gbest[g] = b;
    }
    __syncwarp();
    // the `keep` best groups, ties to the lower index; a kept group's best becomes NaN-free marker +inf
    for (int r = 0; r < keep; ++r) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int g = lane; g < n_groups; g += 32) {
        const float v = gbest[g];
        if (v != INFINITY && (v > bv || (v == bv && g < bi))) { bv = v; bi = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (lane == 0 && bi != 0x7fffffff) gbest[bi] = INFINITY;
      __syncwarp();
    }
    for (int i = lane; i < N; i += 32)
      if (gbest[i / per] != INFINITY) choice[i] = -INFINITY;
    __syncwarp();
  }
  // the `top` best choice scores, ties to the lower index; a chosen one is marked by NaN
  float wsum = 0.f, first = 0.f;
  for (int r = 0; r < top; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lane; i < N; i += 32) {
      const float v = choice[i];
      if (v == v && (v > bv || (v == bv && i < bi))) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    // bi is valid while fewer experts are marked than may be chosen (top <= allowed experts, checked on the host)
    if (r == 0) first = bv;
    const float p = mode == 1 ? expf(bv - first) : prob[bi];      // mode 1: softmax over the chosen logits, the largest first
    wsum += p;
    if (lane == 0) {
      ids[(size_t)t * top + r] = bi;
      weights[(size_t)t * top + r] = p;
      choice[bi] = __int_as_float(0x7fc00000);
    }
    __syncwarp();
  }
  const float f = scale / (wsum + 1e-20f);
  if (lane < top) weights[(size_t)t * top + lane] *= f;
  for (int r = 32 + lane; r < top; r += 32) weights[(size_t)t * top + r] *= f;
}

// ------------------------------------------------------------------------------------------------- sort by expert
// One CTA.  offsets[E + 1]; row_of[n] (-1 for an identity choice); token_of[row]; tiles: tile_group[], tile_row0[] and
// n_tiles[0] for row tiles of `bm` rows.
__global__ void __launch_bounds__(1024)
route_sort_kernel(const int* __restrict__ ids, int n, int top, int E, int bm, int* __restrict__ offsets, int* __restrict__ row_of,
                  int* __restrict__ token_of, int* __restrict__ tile_group, int* __restrict__ tile_row0, int* __restrict__ n_tiles) {
  extern __shared__ int ism[];
  int* count = ism;            // [E]
  int* cursor = ism + E;       // [E]
  int* tile0 = ism + 2 * E;    // [E + 1]
  co_pdl_launch_dependents();
  co_pdl_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = at;
      cursor[e] = at;
      tile0[e] = tiles;
      at += count[e];
      tiles += (count[e] + bm - 1) / bm;
    }
    offsets[E] = at;
    tile0[E] = tiles;
    n_tiles[0] = tiles;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int first = tile0[e], cnt = tile0[e + 1] - first, base = offsets[e];
    for (int i = 0; i < cnt; ++i) { tile_group[first + i] = e; tile_row0[first + i] = base + i * bm; }
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) {
      const int row = atomicAdd(&cursor[e], 1);
      row_of[i] = row;
      token_of[row] = i / top;
    } else {
      row_of[i] = -1;
    }
  }
}

// ------------------------------------------------------------------------------------------------- grouped products
struct GroupedArgs {
  const void* A; long lda; long a_col;        // A rows; group g starts at column g * a_col
  const void* W; long w_group;                // group g's matrix [N, K] at W + g * w_group elements
  void* C; long ldc; long c_col;              // C rows; group g writes from column g * c_col
  const int* gather;                          // A row of sorted row r (null: r itself)
  const int* tile_group; const int* tile_row0; const int* offsets; const int* n_tiles;   // null: uniform groups over M rows
  const float* factor; long factor_ld; int factor_sigmoid;   // C[r, g] *= (sigmoid?)(factor[r * ld + g])
  int M, N, K, G, gated, epilogue;
};

// which rows a CTA works on: returns false when the tile does not exist
template <int BM>
__device__ __forceinline__ bool tile_rows(const GroupedArgs& a, int tile, int& g, int& row0, int& row_end) {
  if (a.tile_group) {
    if (tile >= a.n_tiles[0]) return false;
    g = a.tile_group[tile];
    row0 = a.tile_row0[tile];
    row_end = a.offsets[g + 1];
  } else {
    const int per = (a.M + BM - 1) / BM;
    g = tile / per;
    row0 = (tile % per) * BM;
    row_end = a.M;
    if (g >= a.G) return false;
  }
  return row0 < row_end;
}

__device__ __forceinline__ float apply_factor(const GroupedArgs& a, int row, int g, float v) {
  if (!a.factor) return v;
  float f = a.factor[(size_t)row * a.factor_ld + g];
  if (a.factor_sigmoid) f = 1.0f / (1.0f + expf(-f));
  return v * f;
}

constexpr int SBM = 64, SBN = 64, SBK = 16, STM = 4, STN = 4;

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256) grouped_simt_kernel(GroupedArgs a) {
  __shared__ float xs[SBK][SBM + 4];
  __shared__ float ws[SBK][SBN + 4];
  __shared__ int arow_s[SBM];
  co_pdl_launch_dependents();
  co_pdl_wait();
  int g, row0, row_end;
  if (!tile_rows<SBM>(a, blockIdx.y, g, row0, row_end)) return;
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * SBN;
  for (int r = tid; r < SBM; r += 256) {
    const int row = row0 + r;
    arow_s[r] = row < row_end ? (a.gather ? a.gather[row] : row) : -1;
  }
  __syncthreads();
  const TA* A = (const TA*)a.A + (size_t)g * a.a_col;
  const TW* W = (const TW*)a.W + (size_t)g * a.w_group;
  const int tm = (tid / 16) * STM, tn = (tid % 16) * STN;
  float acc[STM][STN];
#pragma unroll
  for (int i = 0; i < STM; ++i)
#pragma unroll
    for (int j = 0; j < STN; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < a.K; k0 += SBK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = tid + e * 256;
      const int r = idx / SBK, c = idx % SBK;
      const int gk = k0 + c, gn = n0 + r;
      const int ar = arow_s[r];
      xs[c][r] = (ar >= 0 && gk < a.K) ? co_to_float(A[(size_t)ar * a.lda + gk]) : 0.f;
      ws[c][r] = (gn < a.N && gk < a.K) ? co_to_float(W[(size_t)gn * a.K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SBK; ++kk) {
      float x[STM], w[STN];
#pragma unroll
      for (int i = 0; i < STM; ++i) x[i] = xs[kk][tm + i];
#pragma unroll
      for (int j = 0; j < STN; ++j) w[j] = ws[kk][tn + j];
#pragma unroll
      for (int i = 0; i < STM; ++i)
#pragma unroll
        for (int j = 0; j < STN; ++j) acc[i][j] = fmaf(x[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
  TO* C = (TO*)a.C + (size_t)g * a.c_col;
#pragma unroll
  for (int i = 0; i < STM; ++i) {
    const int row = row0 + tm + i;
    if (row >= row_end) continue;
    if (a.gated) {
#pragma unroll
      for (int j = 0; j < STN; j += 2) {
        const int gn = n0 + tn + j;
        if (gn + 1 < a.N) C[(size_t)row * a.ldc + gn / 2] = co_from_float<TO>(apply_factor(a, row, g, co_gated(a.epilogue, acc[i][j], acc[i][j + 1])));
      }
    } else {
#pragma unroll
      for (int j = 0; j < STN; ++j) {
        const int gn = n0 + tn + j;
        if (gn < a.N) C[(size_t)row * a.ldc + gn] = co_from_float<TO>(apply_factor(a, row, g, acc[i][j]));
      }
    }
  }
}

// bfloat16 on the tensor cores: a CTA of four warps owns 64 rows x 64 columns, a warp 16 rows; K in steps of 32 through a
// ring of four stages filled by asynchronous 16-byte copies (K a multiple of 8, rows of A and W on 16-byte boundaries).
typedef __nv_bfloat16 bf16;
constexpr int TBM = 64, TBN = 64, TBK = 32, TLD = TBK + 8;
// TNS, the stages of the ring: 4 for few rows (the matrices stream from memory once, three loads in flight per CTA keep the
// memory busy), 3 for many (the tiles are reused from L2, and 30 KB instead of 40 leave room for more CTAs).

__device__ __forceinline__ void g_ldsm_x4(unsigned (&r)[4], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void g_mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void g_cp_async16(void* dst, const void* src, int bytes) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(a), "l"(src), "r"(bytes) : "memory");
}

template <typename TO, int TNS>
__global__ void __launch_bounds__(128) grouped_mma_kernel(GroupedArgs a) {
  __shared__ __align__(16) bf16 As[TNS][TBM][TLD];
  __shared__ __align__(16) bf16 Bs[TNS][TBN][TLD];
  __shared__ int arow_s[TBM];
  co_pdl_launch_dependents();
  co_pdl_wait();
  int g, row0, row_end;
  if (!tile_rows<TBM>(a, blockIdx.y, g, row0, row_end)) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n0 = blockIdx.x * TBN;
  for (int r = tid; r < TBM; r += 128) {
    const int row = row0 + r;
    arow_s[r] = row < row_end ? (a.gather ? a.gather[row] : row) : -1;
  }
  __syncthreads();
  const bf16* A = (const bf16*)a.A + (size_t)g * a.a_col;
  const bf16* W = (const bf16*)a.W + (size_t)g * a.w_group;
  const int K = a.K;
  auto load = [&](int buf, int k0) {
    // 64 rows x 4 chunks of 8 elements per operand: 256 chunks each, two per thread
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int idx = tid + e * 128;
      const int r = idx >> 2, ch = idx & 3;
      const int gk = k0 + ch * 8;
      const int ar = arow_s[r];
      const bool oka = ar >= 0 && gk < K;
      g_cp_async16(&As[buf][r][ch * 8], A + (oka ? (size_t)ar * a.lda + gk : 0), oka ? 16 : 0);
      const int gn = n0 + r;
      const bool okb = gn < a.N && gk < K;
      g_cp_async16(&Bs[buf][r][ch * 8], W + (okb ? (size_t)gn * K + gk : 0), okb ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  float acc[TBN / 8][4];
#pragma unroll
  for (int nt = 0; nt < TBN / 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
  const int steps = (K + TBK - 1) / TBK;
  // one group is committed per stage, also an empty one past the end, so that "all but the last TNS - 2 groups" always
  // means "stage s has landed"
  for (int s = 0; s < TNS - 1; ++s) {
    if (s < steps) load(s, s * TBK);
    else asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int s = 0; s < steps; ++s) {
    asm volatile("cp.async.wait_group %0;" ::"n"(TNS - 2) : "memory");
    __syncthreads();             // stage s is visible to all, and all have finished with stage s - 1, whose buffer is filled next
    if (s + TNS - 1 < steps) load((s + TNS - 1) % TNS, (s + TNS - 1) * TBK);
    else asm volatile("cp.async.commit_group;" ::: "memory");
    const int buf = s % TNS;
#pragma unroll
    for (int kk = 0; kk < TBK; kk += 16) {
      unsigned af[4];
      g_ldsm_x4(af, &As[buf][warp * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
      for (int nt = 0; nt < TBN / 8; nt += 2) {
        unsigned b[4];
        g_ldsm_x4(b, &Bs[buf][nt * 8 + (lane & 7) + (lane >> 4) * 8][kk + ((lane >> 3) & 1) * 8]);
        g_mma16816(acc[nt], af, b[0], b[1]);
        g_mma16816(acc[nt + 1], af, b[2], b[3]);
      }
    }
  }
  TO* C = (TO*)a.C + (size_t)g * a.c_col;
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int row = row0 + warp * 16 + (lane >> 2) + 8 * rr;
    if (row >= row_end) continue;
#pragma unroll
    for (int nt = 0; nt < TBN / 8; ++nt) {
      const int gn = n0 + nt * 8 + 2 * (lane & 3);
      const float v0 = acc[nt][2 * rr], v1 = acc[nt][2 * rr + 1];
      if (a.gated) {
        if (gn + 1 < a.N) C[(size_t)row * a.ldc + gn / 2] = co_from_float<TO>(apply_factor(a, row, g, co_gated(a.epilogue, v0, v1)));
      } else {
        if (gn < a.N) C[(size_t)row * a.ldc + gn] = co_from_float<TO>(apply_factor(a, row, g, v0));
        if (gn + 1 < a.N) C[(size_t)row * a.ldc + gn + 1] = co_from_float<TO>(apply_factor(a, row, g, v1));
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------- combine
template <typename TH>
__global__ void __launch_bounds__(256)
route_combine_kernel(const float* __restrict__ y, long ldy, const TH* __restrict__ h, long ldh, const int* __restrict__ ids,
                     const float* __restrict__ weights, const int* __restrict__ row_of, int top, int E, float* __restrict__ out,
                     int H, const float* __restrict__ extra, long ld_extra, const float* __restrict__ extra_gate, long ld_gate) {
  constexpr int KEEP = 64;                    // choices whose rows and weights are looked up once, into shared memory
  __shared__ int row_s[KEEP];
  __shared__ float w_s[KEEP];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const size_t t = blockIdx.x;
  // one more summand per token, added last: extra[t] times sigmoid(extra_gate[t]) (or times 1 without a gate)
  const float xw = !extra ? 0.f : extra_gate ? 1.0f / (1.0f + expf(-extra_gate[t * ld_gate])) : 1.f;
  if (top <= KEEP) {
    if ((int)threadIdx.x < top) {
      const int e = ids[t * top + threadIdx.x];
      row_s[threadIdx.x] = e < E ? row_of[t * top + threadIdx.x] : -1;      // -1: the token's own input
      w_s[threadIdx.x] = weights[t * top + threadIdx.x];
    }
    __syncthreads();
    const bool wide = (H & 3) == 0 && (ldy & 3) == 0 && ((uintptr_t)y & 15) == 0 && ((uintptr_t)out & 15) == 0 &&
                      (!extra || ((ld_extra & 3) == 0 && ((uintptr_t)extra & 15) == 0));
    if (wide) {          // four columns a thread, the rows of all choices requested before any is used
      for (int j = 4 * threadIdx.x; j < H; j += 4 * blockDim.x) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 own = make_float4(co_to_float(h[t * ldh + j]), co_to_float(h[t * ldh + j + 1]), co_to_float(h[t * ldh + j + 2]),
                                       co_to_float(h[t * ldh + j + 3]));
#pragma unroll 4
        for (int k = 0; k < top; ++k) {
          const int r = row_s[k];
          const float4 v = r >= 0 ? *reinterpret_cast<const float4*>(y + (size_t)r * ldy + j) : own;
          const float w = w_s[k];
          acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y); acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
        }
        if (extra) {
          const float4 x = *reinterpret_cast<const float4*>(extra + t * ld_extra + j);
          acc.x = fmaf(xw, x.x, acc.x); acc.y = fmaf(xw, x.y, acc.y); acc.z = fmaf(xw, x.z, acc.z); acc.w = fmaf(xw, x.w, acc.w);
        }
        *reinterpret_cast<float4*>(out + t * H + j) = acc;
      }
      return;
    }
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
      float acc = 0.f;
      for (int k = 0; k < top; ++k) {
        const int r = row_s[k];
        acc = fmaf(w_s[k], r >= 0 ? y[(size_t)r * ldy + j] : co_to_float(h[t * ldh + j]), acc);
      }
      out[t * H + j] = extra ? fmaf(xw, extra[t * ld_extra + j], acc) : acc;
    }
    return;
  }
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      const int e = ids[t * top + k];
      const float w = weights[t * top + k];
      const float v = e < E ? y[(size_t)row_of[t * top + k] * ldy + j] : co_to_float(h[t * ldh + j]);
      acc = fmaf(w, v, acc);
    }
    out[t * H + j] = extra ? fmaf(xw, extra[t * ld_extra + j], acc) : acc;
  }
}

}  // namespace

CO_EXPORT int coheryn_route_select(const float* logits, long ld, const void* correction, int c_dtype, int T, int N, int n_groups,
                                   int keep, int top, float scale, int mode, int* ids, float* weights, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (N < 1 || top < 1 || top > N) CO_FAIL("route_select: %d choices among %d outputs", top, N);
  if (mode != 0 && mode != 1) CO_FAIL("route_select: unknown mode %d", mode);
  if (n_groups < 1) n_groups = 1;
  if (N % n_groups) CO_FAIL("route_select: %d outputs do not form %d equal groups", N, n_groups);
  if (keep < 1 || keep > n_groups) keep = n_groups;
  if ((long)keep * (N / n_groups) < top) CO_FAIL("route_select: %d groups of %d cannot give %d choices", keep, N / n_groups, top);
  const size_t smem = (size_t)RS_WARPS * (2 * (size_t)N + n_groups) * sizeof(float);
  if (smem > 200 * 1024) CO_FAIL("route_select: %d outputs do not fit in shared memory", N);
  if (smem > 48 * 1024) cudaFuncSetAttribute(route_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  co_launch(route_select_kernel, dim3((T + RS_WARPS - 1) / RS_WARPS), dim3(RS_WARPS * 32), smem, stream, logits, ld, correction,
            c_dtype, T, N, n_groups, keep, top, scale, mode, ids, weights);
  CO_CHECK_LAUNCH("route_select");
  return 0;
}

// Rows per tile of the grouped products, by the kernel that will run (both use the same today).
CO_EXPORT int coheryn_grouped_tile_rows() { return TBM; }

// tile_rows: the rows per tile of the product that will read the lists (0: those of the grouped kernels of this file).
CO_EXPORT int coheryn_route_sort(const int* ids, int n, int top, int E, int* offsets, int* row_of, int* token_of, int* tile_group,
                                 int* tile_row0, int* n_tiles, int tile_rows, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (E < 1 || top < 1 || tile_rows < 0) CO_FAIL("route_sort: bad sizes");
  if (tile_rows == 0) tile_rows = TBM;
  static_assert(TBM == SBM, "both grouped kernels take the same row tiles");
  const size_t smem = (size_t)(3 * E + 1) * sizeof(int);
  if (smem > 200 * 1024) CO_FAIL("route_sort: %d experts do not fit in shared memory", E);
  if (smem > 48 * 1024) cudaFuncSetAttribute(route_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  co_launch(route_sort_kernel, dim3(1), dim3(1024), smem, stream, ids, n, top, E, tile_rows, offsets, row_of, token_of, tile_group,
            tile_row0, n_tiles);
  CO_CHECK_LAUNCH("route_sort");
  return 0;
}

// max_tiles: an upper bound of the row tiles (the grid's second dimension) when the groups come from route_sort
// (rows / tile rows + groups); ignored for uniform groups.
CO_EXPORT int coheryn_grouped_linear(const void* A, int a_dtype, long lda, long a_col, const void* W, int w_dtype, long w_group,
                                     void* C, int c_dtype, long ldc, long c_col, const int* gather, const int* tile_group,
                                     const int* tile_row0, const int* offsets, const int* n_tiles, int max_tiles,
                                     const float* factor, long factor_ld, int factor_sigmoid, int M, int N, int K, int G,
                                     int epilogue, int allow_tensor_cores, cudaStream_t stream) {
  if (N <= 0 || K <= 0 || G <= 0) CO_FAIL("grouped_linear: bad sizes N=%d K=%d G=%d", N, K, G);
  const bool routed = tile_group != nullptr;
  if (routed && (!tile_row0 || !offsets || !n_tiles || max_tiles < 1)) CO_FAIL("grouped_linear: routed groups need their tile lists");
  if (!routed && M <= 0) return 0;
  if (epilogue && !co_epilogue_known(epilogue)) CO_FAIL("grouped_linear: unknown epilogue %d", epilogue);
  if (epilogue && (N & 1)) CO_FAIL("grouped_linear: a gated epilogue needs an even number of columns");
  GroupedArgs a{A, lda, a_col, W, w_group, C, ldc, c_col, gather, tile_group, tile_row0, offsets, n_tiles,
                factor, factor_ld, factor_sigmoid, M, N, K, G, epilogue ? 1 : 0, epilogue};
  const int tiles = routed ? max_tiles : G * ((M + TBM - 1) / TBM);
  const bool tc = allow_tensor_cores && a_dtype == CO_BF16 && w_dtype == CO_BF16 && K % 8 == 0 && lda % 8 == 0 && a_col % 8 == 0 &&
                  w_group % 8 == 0 && ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0;
  if (tc) {
    dim3 grid((N + TBN - 1) / TBN, tiles);
    const bool few = M <= (routed ? 1024 : 256);        // rows in all: pairs of a routed step, tokens otherwise
    if (c_dtype != CO_BF16 && c_dtype != CO_F32) CO_FAIL("grouped_linear: unknown output dtype %d", c_dtype);
    if (c_dtype == CO_BF16) {
      if (few) co_launch(grouped_mma_kernel<bf16, 4>, grid, dim3(128), 0, stream, a);
      else co_launch(grouped_mma_kernel<bf16, 3>, grid, dim3(128), 0, stream, a);
    } else {
      if (few) co_launch(grouped_mma_kernel<float, 4>, grid, dim3(128), 0, stream, a);
      else co_launch(grouped_mma_kernel<float, 3>, grid, dim3(128), 0, stream, a);
    }
    CO_CHECK_LAUNCH("grouped_mma");
    return 0;
  }
  dim3 grid((N + SBN - 1) / SBN, tiles);
#define GO(TA, TW, TO) co_launch(grouped_simt_kernel<TA, TW, TO>, grid, dim3(256), 0, stream, a)
  if (a_dtype == CO_F32 && w_dtype == CO_F32 && c_dtype == CO_F32) GO(float, float, float);
  else if (a_dtype == CO_BF16 && w_dtype == CO_BF16 && c_dtype == CO_BF16) GO(bf16, bf16, bf16);
  else if (a_dtype == CO_BF16 && w_dtype == CO_BF16 && c_dtype == CO_F32) GO(bf16, bf16, float);
  else CO_FAIL("grouped_linear: unsupported dtypes A=%d W=%d C=%d", a_dtype, w_dtype, c_dtype);
#undef GO
  CO_CHECK_LAUNCH("grouped_simt");
  return 0;
}

// y float32 [rows, H] (row stride ldy): the experts' outputs in sorted order; h [T, H]: the tokens' inputs (identity experts).
CO_EXPORT int coheryn_route_combine(const float* y, long ldy, const void* h, int h_dtype, long ldh, const int* ids,
                                    const float* weights, const int* row_of, int top, int E, float* out, int T, int H,
                                    const float* extra, long ld_extra, const float* extra_gate, long ld_gate, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (h_dtype == CO_F32)
    co_launch(route_combine_kernel<float>, dim3(T), dim3(256), 0, stream, y, ldy, (const float*)h, ldh, ids, weights, row_of, top, E, out, H, extra, ld_extra, extra_gate, ld_gate);
  else if (h_dtype == CO_BF16)
    co_launch(route_combine_kernel<bf16>, dim3(T), dim3(256), 0, stream, y, ldy, (const bf16*)h, ldh, ids, weights, row_of, top, E, out, H, extra, ld_extra, extra_gate, ld_gate);
  else CO_FAIL("route_combine: unknown dtype %d", h_dtype);
  CO_CHECK_LAUNCH("route_combine");
  return 0;
}
