// Kernels on the float32 residual stream of blocks that normalise AFTER the residual add, and of an embedding that
// adds a row chosen by a hash of (previous token, token):
//
//   * embed_pair:         x[t] = table[id_t] * scale + pair[(prev_t * mul_prev + id_t * mul_cur) mod buckets]
//                         (row `buckets` for the first token of a sequence), optionally x <- x / rms(x) * w;
//                         prev_t is the token before t in the step, or, for the first token of a request's portion,
//                         the last token of the request's previous step, kept in a per-request state word;
//   * store_last_ids:     that state word <- the last token of every request's portion;
//   * scaled_add_norm:    mode 0: x <- (alpha x + d) / rms(alpha x + d) * w      (a norm after the sum)
//                         mode 1: x <- x + d / rms(d) * w                        (a normalised summand)
//                         d the sum of P float32 parts in order; x is written back in float32 and, when asked, as a
//                         copy in the compute dtype that the next matrix products read;
//   * gated_table_mul:    out[t, j] = gelu_tanh(z[t, j]) * table[id_t, col0 + j];
//   * copy_head_columns:  a block of columns per head from one matrix into another (or one block into every head's);
//   * head_gate:          every head's columns times the sigmoid of the head's logit.
//
// rms(v) = sqrt(mean(v^2) + eps).  Sums over a row are trees of fixed shape: a row's result does not depend on the
// other rows of the step.
#include "common.cuh"

namespace {

template <typename TW, typename TO>
__global__ void __launch_bounds__(256)
embed_pair_kernel(const TW* __restrict__ table, const TW* __restrict__ pair, const int* __restrict__ ids,
                  const int* __restrict__ positions, const int* __restrict__ token_req, const int* __restrict__ cu_q,
                  const int* __restrict__ state_slots, const int* __restrict__ last_ids, long long mul_prev,
                  long long mul_cur, long long buckets, float scale, const void* __restrict__ w, int w_dtype, float eps,
                  float* __restrict__ out, TO* __restrict__ out_cast, int H, int V, int* __restrict__ status) {
  extern __shared__ __align__(16) float row_s[];
  __shared__ float scratch[33];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    id = 0;
  }
  const TW* prow = nullptr;
  if (pair) {
    long long r = buckets;                                  // the first token of a sequence
    if (positions[t] != 0) {
      const int b = token_req[t];
      long long prev = (t == cu_q[b]) ? (long long)last_ids[state_slots[b]] : (long long)ids[t - 1];
      if (prev < 0 || prev >= V) prev = 0;
      r = ((prev % buckets) * mul_prev + ((long long)id % buckets) * mul_cur) % buckets;     // multipliers come reduced
    }
    prow = pair + (size_t)r * H;
  }
  const TW* erow = table + (size_t)id * H;
  float ss = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float v = co_to_float(erow[j]) * scale;
    if (prow) v += co_to_float(prow[j]);
    row_s[j] = v;
    ss = fmaf(v, v, ss);
  }
  float inv = 1.f;
  if (w) inv = 1.0f / sqrtf(co_block_sum(ss, scratch) / (float)H + eps);
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float v = row_s[j];
    if (w) v = v * inv * co_load_any(w, w_dtype, j);
    out[(size_t)t * H + j] = v;
    if (out_cast) out_cast[(size_t)t * H + j] = co_from_float<TO>(v);
  }
}

__global__ void store_last_ids_kernel(const int* __restrict__ ids, const int* __restrict__ cu_q,
                                      const int* __restrict__ state_slots, int* __restrict__ last_ids, int B) {
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B && cu_q[b + 1] > cu_q[b]) last_ids[state_slots[b]] = ids[cu_q[b + 1] - 1];
}

template <typename TO>
__global__ void __launch_bounds__(256)
scaled_add_norm_kernel(float* __restrict__ x, const float* __restrict__ parts, int P, long part_stride, long row_stride,
                       float alpha, int mode, const void* __restrict__ w, int w_dtype, float eps,
                       TO* __restrict__ out_cast, int H) {
  extern __shared__ __align__(16) float row_s[];
  __shared__ float scratch[33];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const size_t t = blockIdx.x;
  float* xr = x + t * H;
  float ss = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float d = 0.f;
    for (int p = 0; p < P; ++p) d += parts[(size_t)p * part_stride + t * row_stride + j];
    const float v = mode == 0 ? fmaf(alpha, xr[j], d) : d;
    row_s[j] = v;
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.0f / sqrtf(co_block_sum(ss, scratch) / (float)H + eps);
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float v = row_s[j] * inv * co_load_any(w, w_dtype, j);
    if (mode != 0) v += xr[j];
    xr[j] = v;
    if (out_cast) out_cast[t * H + j] = co_from_float<TO>(v);
  }
}

// The same with the row in registers: H a multiple of 4 and at most 256 * 4 * VPT, every pointer and stride on 16-byte
// boundaries.  Each global value is read once with 16-byte loads; the weights, which no earlier kernel writes, are
// requested before the wait for the predecessor.  d is summed part by part from 0 as above.
__device__ __forceinline__ void san_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void san_store4(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<const unsigned*>(&lo);
  u.y = *reinterpret_cast<const unsigned*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}

template <typename TO, int VPT>
__global__ void __launch_bounds__(256)
scaled_add_norm_vec_kernel(float* __restrict__ x, const float* __restrict__ parts, int P, long part_stride, long row_stride,
                           float alpha, int mode, const void* __restrict__ w, int w_dtype, float eps,
                           TO* __restrict__ out_cast, int H) {
  __shared__ float scratch[33];
  co_pdl_launch_dependents();
  const int H4 = H >> 2;
  float4 wv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int j = threadIdx.x + i * 256;
    if (j < H4) {
      if (w_dtype == CO_F32) wv[i] = reinterpret_cast<const float4*>(w)[j];
      else wv[i] = make_float4(co_load_any(w, w_dtype, 4 * j), co_load_any(w, w_dtype, 4 * j + 1), co_load_any(w, w_dtype, 4 * j + 2),
                               co_load_any(w, w_dtype, 4 * j + 3));
    }
  }
  co_pdl_wait();
  const size_t t = blockIdx.x;
  float* xr = x + t * H;
  float4 xv[VPT], v[VPT];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int j = threadIdx.x + i * 256;
    if (j < H4) {
      xv[i] = reinterpret_cast<const float4*>(xr)[j];
      float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int p = 0; p < P; ++p) {
        const float4 a = reinterpret_cast<const float4*>(parts + (size_t)p * part_stride + t * row_stride)[j];
        d.x += a.x; d.y += a.y; d.z += a.z; d.w += a.w;
      }
      v[i] = mode == 0 ? make_float4(fmaf(alpha, xv[i].x, d.x), fmaf(alpha, xv[i].y, d.y), fmaf(alpha, xv[i].z, d.z), fmaf(alpha, xv[i].w, d.w)) : d;
      ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss); ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
    }
  }
  const float inv = 1.0f / sqrtf(co_block_sum(ss, scratch) / (float)H + eps);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int j = threadIdx.x + i * 256;
    if (j < H4) {
      float4 o = make_float4(v[i].x * inv * wv[i].x, v[i].y * inv * wv[i].y, v[i].z * inv * wv[i].z, v[i].w * inv * wv[i].w);
      if (mode != 0) { o.x += xv[i].x; o.y += xv[i].y; o.z += xv[i].z; o.w += xv[i].w; }
      reinterpret_cast<float4*>(xr)[j] = o;
      if (out_cast) san_store4(out_cast + t * H + 4 * (size_t)j, o);
    }
  }
}

template <typename TZ, typename TW, typename TO>
__global__ void gated_table_mul_kernel(const TZ* __restrict__ z, long ldz, const TW* __restrict__ table, long ldt, int col0,
                                       const int* __restrict__ ids, TO* __restrict__ out, int T, int n, int V) {
  co_pdl_launch_dependents();
  co_pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long)T * n) return;
  const int t = (int)(i / n), j = (int)(i % n);
  int id = ids[t];
  if (id < 0 || id >= V) id = 0;
  out[i] = co_from_float<TO>(co_gelu_tanh(co_to_float(z[(size_t)t * ldz + j])) * co_to_float(table[(size_t)id * ldt + col0 + j]));
}

// dst[t, h * dst_head + dst_off + j] = src[t, h * src_head + src_off + j] for j < n, 16-bit elements (src_head 0: the same
// columns for every head).
__global__ void copy_head_columns_kernel(const unsigned short* __restrict__ src, long src_ld, long src_head, long src_off,
                                         unsigned short* __restrict__ dst, long dst_ld, long dst_head, long dst_off, int n, int H,
                                         long total) {
  co_pdl_launch_dependents();
  co_pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int j = (int)(i % n), h = (int)((i / n) % H);
  const long t = i / ((long)n * H);
  dst[t * dst_ld + h * dst_head + dst_off + j] = src[t * src_ld + h * src_head + src_off + j];
}

// x[t, h * n + j] *= sigmoid(g[t, h]) in place; g float32 with row stride ldg.
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ x, long ldx, const float* __restrict__ g, long ldg, int n, int H, long total) {
  co_pdl_launch_dependents();
  co_pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int j = (int)(i % n), h = (int)((i / n) % H);
  const long t = i / ((long)n * H);
  const float f = 1.0f / (1.0f + expf(-g[t * ldg + h]));
  T* p = x + t * ldx + (long)h * n + j;
  *p = co_from_float<T>(co_to_float(*p) * f);
}

}  // namespace

CO_EXPORT int coheryn_copy_head_columns(const void* src, long src_ld, long src_head, long src_off, void* dst, long dst_ld,
                                        long dst_head, long dst_off, int n, int H, int T, cudaStream_t stream) {
  const long total = (long)T * H * n;
  if (total <= 0) return 0;
  co_launch(copy_head_columns_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, (const unsigned short*)src, src_ld,
            src_head, src_off, (unsigned short*)dst, dst_ld, dst_head, dst_off, n, H, total);
  CO_CHECK_LAUNCH("copy_head_columns");
  return 0;
}

CO_EXPORT int coheryn_head_gate(void* x, int dtype, long ldx, const float* g, long ldg, int n, int H, int T, cudaStream_t stream) {
  const long total = (long)T * H * n;
  if (total <= 0) return 0;
  dim3 grid((unsigned)((total + 255) / 256));
  if (dtype == CO_BF16) co_launch(head_gate_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (__nv_bfloat16*)x, ldx, g, ldg, n, H, total);
  else if (dtype == CO_F32) co_launch(head_gate_kernel<float>, grid, dim3(256), 0, stream, (float*)x, ldx, g, ldg, n, H, total);
  else CO_FAIL("head_gate: unknown dtype %d", dtype);
  CO_CHECK_LAUNCH("head_gate");
  return 0;
}

// table [V, H], pair [buckets + 1, H] (null: no pair rows) of one dtype; out float32 [T, H]; out_cast (null or [T, H] of
// out_dtype); w (null: no norm) [H].  mul_prev and mul_cur must lie in [0, buckets).
CO_EXPORT int coheryn_embed_pair(const void* table, const void* pair, int table_dtype, const int* ids, const int* positions,
                                 const int* token_req, const int* cu_q, const int* state_slots, const int* last_ids,
                                 long long mul_prev, long long mul_cur, long long buckets, float scale, const void* w,
                                 int w_dtype, float eps, float* out, void* out_cast, int out_dtype, int T, int H, int V,
                                 int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (pair && (buckets < 1 || mul_prev < 0 || mul_cur < 0 || mul_prev >= buckets || mul_cur >= buckets || buckets > (1ll << 31)))
    CO_FAIL("embed_pair: multipliers must be reduced modulo the %lld buckets", buckets);
  if (pair && (!positions || !token_req || !cu_q || !state_slots || !last_ids)) CO_FAIL("embed_pair: the pair rows need the step's layout and the state words");
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) CO_FAIL("embed_pair: a row of %d does not fit in shared memory", H);
#define GO(TW, TO)                                                                                                     \
  {                                                                                                                    \
    auto kern = embed_pair_kernel<TW, TO>;                                                                             \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
    co_launch(kern, dim3(T), dim3(256), smem, stream, (const TW*)table, (const TW*)pair, ids, positions, token_req, cu_q, \
              state_slots, last_ids, mul_prev, mul_cur, buckets, scale, w, w_dtype, eps, out, (TO*)out_cast, H, V, status); \
  }
  const bool cast_bf16 = out_cast && out_dtype == CO_BF16;
  if (out_cast && out_dtype != CO_BF16 && out_dtype != CO_F32) CO_FAIL("embed_pair: unknown output dtype %d", out_dtype);
  if (table_dtype == CO_F32) { if (cast_bf16) GO(float, __nv_bfloat16) else GO(float, float) }
  else if (table_dtype == CO_BF16) { if (cast_bf16) GO(__nv_bfloat16, __nv_bfloat16) else GO(__nv_bfloat16, float) }
  else CO_FAIL("embed_pair: unknown table dtype %d", table_dtype);
#undef GO
  CO_CHECK_LAUNCH("embed_pair");
  return 0;
}

CO_EXPORT int coheryn_store_last_ids(const int* ids, const int* cu_q, const int* state_slots, int* last_ids, int B,
                                     cudaStream_t stream) {
  if (B <= 0) return 0;
  co_launch(store_last_ids_kernel, dim3((B + 127) / 128), dim3(128), 0, stream, ids, cu_q, state_slots, last_ids, B);
  CO_CHECK_LAUNCH("store_last_ids");
  return 0;
}

// x float32 [n, H] in place; parts float32: P summands, part p's row t at parts + p * part_stride + t * row_stride.
CO_EXPORT int coheryn_scaled_add_norm(float* x, const float* parts, int P, long part_stride, long row_stride, float alpha,
                                      int mode, const void* w, int w_dtype, float eps, void* out_cast, int out_dtype, int n,
                                      int H, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!w || P < 1 || (mode != 0 && mode != 1)) CO_FAIL("scaled_add_norm: needs a weight, a summand and mode 0 or 1");
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) CO_FAIL("scaled_add_norm: a row of %d does not fit in shared memory", H);
#define GO(TO)                                                                                                 \
  {                                                                                                            \
    auto kern = scaled_add_norm_kernel<TO>;                                                                    \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
    co_launch(kern, dim3(n), dim3(256), smem, stream, x, parts, P, part_stride, row_stride, alpha, mode, w, w_dtype, eps, \
              (TO*)out_cast, H);                                                                               \
  }
  const bool aligned = H % 4 == 0 && H <= 8192 && part_stride % 4 == 0 && row_stride % 4 == 0 && ((uintptr_t)x & 15) == 0 &&
                       ((uintptr_t)parts & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)out_cast & 15) == 0;
#define VEC(TO, VPT)                                                                                                      \
  co_launch(scaled_add_norm_vec_kernel<TO, VPT>, dim3(n), dim3(256), 0, stream, x, parts, P, part_stride, row_stride, alpha, mode, w, \
            w_dtype, eps, (TO*)out_cast, H)
#define VECS(TO)                                                                                                          \
  {                                                                                                                       \
    if (H <= 1024) VEC(TO, 1); else if (H <= 2048) VEC(TO, 2); else if (H <= 4096) VEC(TO, 4); else VEC(TO, 8);          \
  }
  if (out_cast && out_dtype != CO_BF16 && out_dtype != CO_F32) CO_FAIL("scaled_add_norm: unknown output dtype %d", out_dtype);
  if (aligned) {
    if (out_cast && out_dtype == CO_BF16) VECS(__nv_bfloat16)
    else VECS(float)
  }
  else if (out_cast && out_dtype == CO_BF16) GO(__nv_bfloat16)
  else GO(float)
#undef VECS
#undef VEC
#undef GO
  CO_CHECK_LAUNCH("scaled_add_norm");
  return 0;
}

// z [T, n] (row stride ldz) float32 or bfloat16; table [V, ldt] and out [T, n] contiguous of dtype `dtype`.
CO_EXPORT int coheryn_gated_table_mul(const void* z, int z_dtype, long ldz, const void* table, int dtype, long ldt, int col0,
                                      const int* ids, void* out, int T, int n, int V, cudaStream_t stream) {
  if (T <= 0 || n <= 0) return 0;
  const long total = (long)T * n;
  dim3 grid((unsigned)((total + 255) / 256));
#define GO(TZ, TW)                                                                                                \
  co_launch(gated_table_mul_kernel<TZ, TW, TW>, grid, dim3(256), 0, stream, (const TZ*)z, ldz, (const TW*)table, ldt, col0, \
            ids, (TW*)out, T, n, V)
  if (z_dtype == CO_F32 && dtype == CO_F32) GO(float, float);
  else if (z_dtype == CO_F32 && dtype == CO_BF16) GO(float, __nv_bfloat16);
  else if (z_dtype == CO_BF16 && dtype == CO_BF16) GO(__nv_bfloat16, __nv_bfloat16);
  else CO_FAIL("gated_table_mul: unsupported dtypes z=%d table=%d", z_dtype, dtype);
#undef GO
  CO_CHECK_LAUNCH("gated_table_mul");
  return 0;
}

// ---------------------------------------------------------------------------------
// The input of a product that mixes the stream with the embedding output: row t of `out` [T, 2 H] (compute dtype) is
// [x[t] + the pending summands | table[id[t]] * scale].  The stream itself is not changed (the product's result replaces
// it).  parts: P float32 stacks of [T, H] (part_stride apart) or null; delta16: one pending summand in bfloat16, or null.
// ---------------------------------------------------------------------------------
namespace {
template <typename TW, typename TO>
__global__ void stream_join_kernel(const float* __restrict__ x, const float* __restrict__ parts, int P, long part_stride,
                                   const __nv_bfloat16* __restrict__ delta16, const TW* __restrict__ table,
                                   const int* __restrict__ ids, float scale, TO* __restrict__ out, int H, int V) {
  co_pdl_launch_dependents();
  co_pdl_wait();
  const size_t t = blockIdx.x;
  const int id = ids[t];
  const TW* row = (id >= 0 && id < V) ? table + (size_t)id * H : nullptr;    // the embedding kernel has flagged such an id
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float v = x[t * H + j];
    for (int p = 0; p < P; ++p) v += parts[(size_t)p * part_stride + t * H + j];
    if (delta16) v += __bfloat162float(delta16[t * H + j]);
    out[t * 2 * H + j] = co_from_float<TO>(v);
    out[t * 2 * H + H + j] = co_from_float<TO>(row ? co_to_float(row[j]) * scale : 0.f);
  }
}
}  // namespace

CO_EXPORT int coheryn_stream_join(const float* x, const float* parts, int P, long part_stride, const void* delta16,
                                  const void* table, int table_dtype, const int* ids, float scale, void* out, int out_dtype,
                                  int T, int H, int V, cudaStream_t stream) {
  if (T <= 0 || H <= 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  const __nv_bfloat16* d16 = (const __nv_bfloat16*)delta16;
#define GO(TW, TO)                                                                                                     \
  co_launch(stream_join_kernel<TW, TO>, dim3(T), dim3(threads), 0, stream, x, parts, P, part_stride, d16, (const TW*)table, \
            ids, scale, (TO*)out, H, V)
  if (table_dtype == CO_F32 && out_dtype == CO_F32) GO(float, float);
  else if (table_dtype == CO_BF16 && out_dtype == CO_BF16) GO(__nv_bfloat16, __nv_bfloat16);
  else if (table_dtype == CO_F32 && out_dtype == CO_BF16) GO(float, __nv_bfloat16);
  else if (table_dtype == CO_BF16 && out_dtype == CO_F32) GO(__nv_bfloat16, float);
  else CO_FAIL("stream_join: unknown dtypes %d / %d", table_dtype, out_dtype);
#undef GO
  CO_CHECK_LAUNCH("stream_join");
  return 0;
}
