// A gated linear recurrence per channel (sm_100a), for mixers whose state is ONE number per channel and request:
//
//   * conv_bias:   u[t, c] = bias[c] + sum_j taps[c, j] * x[t - (n-1) + j, c], no activation; inputs before the step's first
//                  token of a request come from its state [n-1, C] (oldest first; zeros after admission), which then takes
//                  the request's last n-1 inputs;
//   * gated scan:  with r = sigmoid(zr + br), i = sigmoid(zi + bi) (zr, zi: the gates' pre-activations, products of u with
//                  block-diagonal matrices made elsewhere), log a = -rate * r * softplus(lam), a = exp(log a):
//                  S_t = a S_(t-1) + sqrt(1 - a^2) * i * u, out_t = S_t * gelu_tanh(y_t) (y: the other branch's pre-activation).
//
// Everything is float32.  The scan is parallel over channels AND over chunks of consecutive tokens of the step: a first
// kernel scans every chunk from zero and leaves (sum of log a, end value) per chunk and channel; the second one walks
// over the summaries of the chunks between its request's start and itself (at most tokens / chunk steps), then scans
// its chunk again from the true start value and writes the outputs.  A request's first token of the step starts from
// the request's state; the token that ends a request's run stores the state.  The order of a channel's additions is
// fixed by the token's place in its request's run, not by the other requests of the step.
//
// a is never formed: a value near 1 would be rounded to a neighbour of 1 that decays several per cent faster or slower
// (or not at all), always to the same side, and over a thousand tokens that bias shows.  With a - 1 = expm1(log a) the step
// is S <- (S + (a - 1) S) + d, whose roundings are those of S and scatter.
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 16;
constexpr int CHUNK = 32;       // tokens per chunk
constexpr int LANES = 128;      // channels per CTA

__global__ void conv_bias_kernel(const float* __restrict__ x, long ldx, float* __restrict__ y, long ldy,
                                 const void* __restrict__ taps, int taps_dtype, const void* __restrict__ bias, int bias_dtype,
                                 int n, int C, const float* __restrict__ state, long state_stride,
                                 const int* __restrict__ token_req, const int* __restrict__ cu_q,
                                 const int* __restrict__ state_slots, int T) {
  co_pdl_launch_dependents();
  co_pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)T * C) return;
  const int t = (int)(idx / C), c = (int)(idx % C);
  const int r = token_req[t];
  const int start = cu_q[r];
  const int i = t - start;
  const float* st = state + (size_t)state_slots[r] * state_stride;
  float acc = bias ? co_load_any(bias, bias_dtype, c) : 0.f;
  for (int j = 0; j < n; ++j) {
    const int p = i - (n - 1) + j;
    const float xv = p >= 0 ? x[(size_t)(start + p) * ldx + c] : st[(size_t)(n - 1 + p) * C + c];
    acc = fmaf(co_load_any(taps, taps_dtype, (size_t)c * n + j), xv, acc);
  }
  y[(size_t)t * ldy + c] = acc;
}

__global__ void conv_state_kernel(const float* __restrict__ x, long ldx, int n, int C, float* __restrict__ state,
                                  long state_stride, const int* __restrict__ cu_q, const int* __restrict__ state_slots, int B) {
  co_pdl_launch_dependents();
  co_pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)B * C) return;
  const int r = (int)(idx / C), c = (int)(idx % C);
  const int start = cu_q[r], len = cu_q[r + 1] - start;
  if (len <= 0) return;
  float* st = state + (size_t)state_slots[r] * state_stride;
  float keep[MAX_TAPS];
  for (int s = 0; s < n - 1; ++s) {
    const int p = len - (n - 1) + s;
    keep[s] = p >= 0 ? x[(size_t)(start + p) * ldx + c] : st[(size_t)(n - 1 + p) * C + c];
  }
  for (int s = 0; s < n - 1; ++s) st[(size_t)s * C + c] = keep[s];
}

struct ScanArgs {
  const float* gates; long ldg;      // [T, blocks * 2 * bs]: per block of bs channels [zr | zi]
  const void* br; const void* bi; int b_dtype;   // [C] each (null: none)
  const float* u; long ldu;          // [T, C]
  const float* y; long ldy;          // [T, C] pre-activations of the other branch
  const void* lam; int lam_dtype;    // [C]
  float rate;
  int bs;                            // channels per block of the gates
  float* state; long state_stride;   // [slots, C] (rows may be strided)
  const int* token_req; const int* cu_q; const int* state_slots;
  float* carry_a; float* carry_s;    // [chunks, C] each
  float* first;                      // [B, C]: the states the requests started from
  void* out; int out_dtype; long ldo;
  int T, C;
};

__device__ __forceinline__ float lr_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float lr_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// What a token brings for channel c: the gates' pre-activations, the input, the other branch, and whether its request's
// run begins here (then with the state to start from).
struct Tok {
  float zr, zi, u, y, start;
  int req;
  bool first;
};
constexpr int GROUP = 4;      // tokens whose inputs are requested together, ahead of the chain of multiply-adds

template <bool WITH_Y>
__device__ __forceinline__ Tok lr_load(const ScanArgs& A, int t, int c, const float* from) {
  Tok k;
  const int blk = c / A.bs, j = c - blk * A.bs;
  const float* g = A.gates + (size_t)t * A.ldg + (size_t)blk * 2 * A.bs;
  k.zr = g[j];
  k.zi = g[A.bs + j];
  k.u = A.u[(size_t)t * A.ldu + c];
  k.y = WITH_Y ? A.y[(size_t)t * A.ldy + c] : 0.f;
  k.req = A.token_req[t];
  k.first = t == A.cu_q[k.req];
  k.start = 0.f;
  if (k.first) k.start = from ? from[(size_t)k.req * A.C + c] : A.state[(size_t)A.state_slots[k.req] * A.state_stride + c];
  return k;
}

// (log a, a - 1, drive); sp = rate * softplus(lam[c]).
__device__ __forceinline__ void lr_coefficients(const Tok& k, float sp, float b_r, float b_i, float& log_a, float& am1, float& d) {
  const float r = lr_sigmoid(k.zr + b_r);
  const float i = lr_sigmoid(k.zi + b_i);
  log_a = -sp * r;
  am1 = expm1f(log_a);
  d = sqrtf(fmaxf(-expm1f(2.0f * log_a), 0.f)) * i * k.u;
}

__global__ void __launch_bounds__(LANES) scan_summaries_kernel(ScanArgs A) {
  co_pdl_launch_dependents();
  const int c = blockIdx.x * LANES + threadIdx.x;
  const int chunk = blockIdx.y;
  if (c >= A.C) return;
  const float sp = A.rate * lr_softplus(co_load_any(A.lam, A.lam_dtype, c));
  const float b_r = A.br ? co_load_any(A.br, A.b_dtype, c) : 0.f, b_i = A.bi ? co_load_any(A.bi, A.b_dtype, c) : 0.f;
  co_pdl_wait();
  const int t0 = chunk * CHUNK, t1 = min(t0 + CHUNK, A.T);
  float logs = 0.f, S = 0.f;
  for (int tg = t0; tg < t1; tg += GROUP) {
    Tok k[GROUP];
#pragma unroll
    for (int j = 0; j < GROUP; ++j)
      if (tg + j < t1) k[j] = lr_load<false>(A, tg + j, c, nullptr);
#pragma unroll
    for (int j = 0; j < GROUP; ++j) {
      if (tg + j >= t1) break;
      if (k[j].first) {        // a request's run begins: what came before does not reach beyond this token
        S = k[j].start;
        A.first[(size_t)k[j].req * A.C + c] = S;
        logs = -INFINITY;
      }
      float log_a, am1, d;
      lr_coefficients(k[j], sp, b_r, b_i, log_a, am1, d);
      S = fmaf(am1, S, S) + d;
      logs += log_a;
    }
  }
  A.carry_a[(size_t)chunk * A.C + c] = logs;
  A.carry_s[(size_t)chunk * A.C + c] = S;
}

template <typename TO>
__global__ void __launch_bounds__(LANES) scan_outputs_kernel(ScanArgs A) {
  co_pdl_launch_dependents();
  const int c = blockIdx.x * LANES + threadIdx.x;
  const int chunk = blockIdx.y;
  if (c >= A.C) return;
  const float sp = A.rate * lr_softplus(co_load_any(A.lam, A.lam_dtype, c));
  const float b_r = A.br ? co_load_any(A.br, A.b_dtype, c) : 0.f, b_i = A.bi ? co_load_any(A.bi, A.b_dtype, c) : 0.f;
  co_pdl_wait();
  const int t0 = chunk * CHUNK, t1 = min(t0 + CHUNK, A.T);
  // the value in front of the chunk's first token
  float S = 0.f;
  {
    const int r = A.token_req[t0];
    const int start = A.cu_q[r];
    if (start < t0) {
      const int c0 = start / CHUNK;     // its end value belongs to this request: the request runs on into this chunk
      S = A.carry_s[(size_t)c0 * A.C + c];
      for (int k = c0 + 1; k < chunk; ++k)
        S = fmaf(expm1f(A.carry_a[(size_t)k * A.C + c]), S, S) + A.carry_s[(size_t)k * A.C + c];
    }
  }
  TO* out = (TO*)A.out;
  for (int tg = t0; tg < t1; tg += GROUP) {
    Tok k[GROUP];
#pragma unroll
    for (int j = 0; j < GROUP; ++j)
      if (tg + j < t1) k[j] = lr_load<true>(A, tg + j, c, A.first);
#pragma unroll
    for (int j = 0; j < GROUP; ++j) {
      const int t = tg + j;
      if (t >= t1) break;
      if (k[j].first) S = k[j].start;
      float log_a, am1, d;
      lr_coefficients(k[j], sp, b_r, b_i, log_a, am1, d);
      S = fmaf(am1, S, S) + d;
      out[(size_t)t * A.ldo + c] = co_from_float<TO>(S * co_gelu_tanh(k[j].y));
      if (t + 1 == A.cu_q[k[j].req + 1]) A.state[(size_t)A.state_slots[k[j].req] * A.state_stride + c] = S;
    }
  }
}

}  // namespace

CO_EXPORT int coheryn_conv_bias(const float* x, long ldx, float* y, long ldy, const void* taps, int taps_dtype, const void* bias,
                                int bias_dtype, int n, int C, float* state, long state_stride, const int* token_req,
                                const int* cu_q, const int* state_slots, int T, int B, int update_state, cudaStream_t stream) {
  if (T <= 0 || C <= 0) return 0;
  if (n < 1 || n > MAX_TAPS) CO_FAIL("conv_bias: 1..%d taps, not %d", MAX_TAPS, n);
  const size_t total = (size_t)T * C;
  co_launch(conv_bias_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, ldx, y, ldy, taps, taps_dtype, bias,
            bias_dtype, n, C, (const float*)state, state_stride, token_req, cu_q, state_slots, T);
  CO_CHECK_LAUNCH("conv_bias");
  if (update_state && n > 1) {
    const size_t per = (size_t)B * C;
    co_launch(conv_state_kernel, dim3((unsigned)((per + 255) / 256)), dim3(256), 0, stream, x, ldx, n, C, state, state_stride, cu_q,
              state_slots, B);
    CO_CHECK_LAUNCH("conv_state");
  }
  return 0;
}

// Floats of scratch the scan needs for T tokens of B requests and C channels.
CO_EXPORT long coheryn_gated_scan_scratch(int T, int B, int C) {
  const long chunks = (T + CHUNK - 1) / CHUNK;
  return (2 * chunks + B) * (long)C;
}

CO_EXPORT int coheryn_gated_scan(const float* gates, long ldg, const void* br, const void* bi, int b_dtype, const float* u, long ldu,
                                 const float* y, long ldy, const void* lam, int lam_dtype, float rate, int bs, float* state,
                                 long state_stride, const int* token_req, const int* cu_q, const int* state_slots, float* scratch,
                                 long scratch_floats, void* out, int out_dtype, long ldo, int T, int B, int C, cudaStream_t stream) {
  if (T <= 0 || C <= 0) return 0;
  if (bs < 1 || C % bs) CO_FAIL("gated_scan: %d channels do not form blocks of %d", C, bs);
  if (scratch_floats < coheryn_gated_scan_scratch(T, B, C)) CO_FAIL("gated_scan: the scratch area is too small");
  const int chunks = (T + CHUNK - 1) / CHUNK;
  ScanArgs A{gates, ldg, br, bi, b_dtype, u, ldu, y, ldy, lam, lam_dtype, rate, bs, state, state_stride, token_req, cu_q, state_slots,
             scratch, scratch + (size_t)chunks * C, scratch + (size_t)2 * chunks * C, out, out_dtype, ldo, T, C};
  dim3 grid((C + LANES - 1) / LANES, chunks);
  co_launch(scan_summaries_kernel, grid, dim3(LANES), 0, stream, A);
  CO_CHECK_LAUNCH("scan_summaries");
  if (out_dtype == CO_F32) co_launch(scan_outputs_kernel<float>, grid, dim3(LANES), 0, stream, A);
  else if (out_dtype == CO_BF16) co_launch(scan_outputs_kernel<__nv_bfloat16>, grid, dim3(LANES), 0, stream, A);
  else CO_FAIL("gated_scan: unknown output dtype %d", out_dtype);
  CO_CHECK_LAUNCH("scan_outputs");
  return 0;
}
