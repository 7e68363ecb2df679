// Linear recurrences over time with a matrix state per head, S [dim, vdim] in float32, carried from token to token
// and from step to step (state [slots, heads, dim, vdim], zeroed when a slot opens):
//
//   decay rule   S <- d_h S + k v^T;                       o = S^T q       d_h one constant a head; q, k, v through SiLU
//   delta rule   S <- diag(g_t) S;  u = beta_t (v - S^T k);  S <- S + k u^T;  o = S^T q
//                g_t one decay a key channel and token, beta_t one scalar a token; the read-out sees the token's write
//
// One thread owns one value channel (a column of S, `dim` registers, padded to DIMP with rows that stay zero), a block
// 32 or 64 neighbouring columns of one (sequence, head); the step's tokens are walked in order, eight at a time through
// shared memory (k, q, g of the head, the same for every column).  Sums over the key channels run in ascending order in
// four interleaved partial sums, whatever the step: a token's result has the same bits whether its sequence came whole,
// in pieces or one token at a time, alone or in a batch.  Everything is float32 but the loads of q, k, v.
#include "common.cuh"

namespace {
constexpr int REC_CHUNK = 8;

__device__ __forceinline__ float rec_silu(float z) { return z / (1.0f + expf(-z)); }

template <typename TQ, typename TV, int DIMP, bool DELTA>
__global__ void __launch_bounds__(64)
k_recurrence(const TQ* __restrict__ q, int ldq, const TQ* __restrict__ k, int ldk, const TV* __restrict__ v, int ldv,
             const float* __restrict__ g, const float* __restrict__ beta, const float* __restrict__ decay,
             float* __restrict__ state, const int* __restrict__ seq_slot, const int* __restrict__ seq_first_row,
             float* __restrict__ out, int heads, int kv_heads, int dim, int vdim) {
  cima_pdl_wait();
  __shared__ __align__(16) float sk[REC_CHUNK][DIMP];
  __shared__ __align__(16) float sq[REC_CHUNK][DIMP];
  __shared__ __align__(16) float sg[DELTA ? REC_CHUNK : 1][DIMP];
  __shared__ float sb[REC_CHUNK];
  const int seq = blockIdx.z, h = blockIdx.y;
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = col < vdim;
  const int kvh = h / (heads / kv_heads);
  const int first = seq_first_row[seq], n = seq_first_row[seq + 1] - first;
  float* st = state + (((size_t)seq_slot[seq] * heads + h) * dim) * (size_t)vdim + col;
  float S[DIMP];
#pragma unroll
  for (int i = 0; i < DIMP; i++) S[i] = (live && i < dim) ? st[(size_t)i * vdim] : 0.f;
  const float dh = DELTA ? 1.f : decay[h];
  const int ldo = heads * vdim;

  for (int t0 = 0; t0 < n; t0 += REC_CHUNK) {
    const int nt = min(REC_CHUNK, n - t0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * DIMP; idx += blockDim.x) {
      const int tt = idx / DIMP, i = idx - tt * DIMP;
      const size_t row = (size_t)(first + t0 + tt);
      float kv_ = 0.f, qv = 0.f, gv = 1.f;
      if (i < dim) {
        kv_ = cima_to_f32<TQ>(k[row * ldk + (size_t)kvh * dim + i]);
        qv = cima_to_f32<TQ>(q[row * ldq + (size_t)kvh * dim + i]);
        if (!DELTA) { kv_ = rec_silu(kv_); qv = rec_silu(qv); }
        if (DELTA) gv = g[(row * heads + h) * dim + i];
      }
      sk[tt][i] = kv_;
      sq[tt][i] = qv;
      if (DELTA) sg[tt][i] = gv;
    }
    if (DELTA && threadIdx.x < nt) sb[threadIdx.x] = beta[(size_t)(first + t0 + threadIdx.x) * heads + h];
    __syncthreads();
    for (int tt = 0; tt < nt; tt++) {
      const size_t row = (size_t)(first + t0 + tt);
      float vv = live ? cima_to_f32<TV>(v[row * ldv + (size_t)h * vdim + col]) : 0.f;
      float u;
      if (DELTA) {
        float p[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < DIMP; i += 4) {
          const float4 g4 = *reinterpret_cast<const float4*>(&sg[tt][i]);
          const float4 k4 = *reinterpret_cast<const float4*>(&sk[tt][i]);
          S[i] *= g4.x; S[i + 1] *= g4.y; S[i + 2] *= g4.z; S[i + 3] *= g4.w;
          p[0] = fmaf(S[i], k4.x, p[0]); p[1] = fmaf(S[i + 1], k4.y, p[1]);
          p[2] = fmaf(S[i + 2], k4.z, p[2]); p[3] = fmaf(S[i + 3], k4.w, p[3]);
        }
        u = sb[tt] * (vv - ((p[0] + p[1]) + (p[2] + p[3])));
      } else {
        vv = rec_silu(vv);
#pragma unroll
        for (int i = 0; i < DIMP; i++) S[i] *= dh;
        u = vv;
      }
      float o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < DIMP; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(&sk[tt][i]);
        const float4 q4 = *reinterpret_cast<const float4*>(&sq[tt][i]);
        S[i] = fmaf(k4.x, u, S[i]); S[i + 1] = fmaf(k4.y, u, S[i + 1]);
        S[i + 2] = fmaf(k4.z, u, S[i + 2]); S[i + 3] = fmaf(k4.w, u, S[i + 3]);
        o[0] = fmaf(S[i], q4.x, o[0]); o[1] = fmaf(S[i + 1], q4.y, o[1]);
        o[2] = fmaf(S[i + 2], q4.z, o[2]); o[3] = fmaf(S[i + 3], q4.w, o[3]);
      }
      if (live) out[row * ldo + (size_t)h * vdim + col] = (o[0] + o[1]) + (o[2] + o[3]);
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < DIMP; i++)
      if (i < dim) st[(size_t)i * vdim] = S[i];
  }
}

template <typename TQ, typename TV, bool DELTA>
int launch_recurrence(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, const float* g, const float* beta,
                      const float* decay, float* state, const int* seq_slot, const int* seq_first_row, float* out,
                      int n_seqs, int heads, int kv_heads, int dim, int vdim, cudaStream_t stream) {
  const int threads = vdim > 32 ? 64 : 32;
  const dim3 grid((vdim + threads - 1) / threads, heads, n_seqs);
#define RUN(D) return cima_launch(k_recurrence<TQ, TV, D, DELTA>, grid, dim3(threads), (size_t)0, stream, 1, (const TQ*)q, ldq, (const TQ*)k, ldk, \
                                  (const TV*)v, ldv, g, beta, decay, state, seq_slot, seq_first_row, out, heads, kv_heads, dim, vdim)
  if (dim <= 32) RUN(32);
  if (dim <= 64) RUN(64);
  if (dim <= 128) RUN(128);
  RUN(256);
#undef RUN
}

// Everything of the delta rule that is computed per token before the recurrence, in float32:
//   qn = q / sqrt(sum q^2 + 1e-6) * dim^(-1/2),  kn = k / sqrt(sum k^2 + 1e-6)            per head of q and k
//   g  = exp(-exp(A_log[h]) * softplus(a + dt_bias)),  beta = sigmoid(b)
// One block a row; warp w takes the heads w, w + warps, ... of q and k, then the threads share g and beta.
template <typename TA>
__global__ void __launch_bounds__(128)
k_delta_prepare(const TA* __restrict__ qk, int ldqk, const TA* __restrict__ a, int lda, const TA* __restrict__ b, int ldb,
                const float* __restrict__ A_log, const float* __restrict__ dt_bias, float* __restrict__ qn, float* __restrict__ kn,
                float* __restrict__ g, float* __restrict__ beta, int heads, int kv_heads, int dim) {
  cima_pdl_wait();
  const size_t row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const float qscale = 1.0f / sqrtf((float)dim);
  for (int u = warp; u < 2 * kv_heads; u += nwarp) {           // the heads of q, then those of k
    const TA* src = qk + row * ldqk + (size_t)u * dim;
    float ss = 0.f;
    for (int i = lane; i < dim; i += 32) { const float x = cima_to_f32<TA>(src[i]); ss = fmaf(x, x, ss); }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float r = (1.0f / sqrtf(ss + 1e-6f)) * (u < kv_heads ? qscale : 1.0f);
    float* dst = u < kv_heads ? qn + (row * kv_heads + u) * dim : kn + (row * kv_heads + (u - kv_heads)) * dim;
    for (int i = lane; i < dim; i += 32) dst[i] = cima_to_f32<TA>(src[i]) * r;
  }
  for (int c = threadIdx.x; c < heads * dim; c += blockDim.x) {
    const float z = cima_to_f32<TA>(a[row * lda + c]) + dt_bias[c];
    const float sp = z > 20.f ? z : log1pf(expf(z));
    g[row * heads * dim + c] = expf(-expf(A_log[c / dim]) * sp);
  }
  for (int h = threadIdx.x; h < heads; h += blockDim.x)
    beta[row * heads + h] = 1.0f / (1.0f + expf(-cima_to_f32<TA>(b[row * ldb + h])));
}
}  // namespace

// delta != 0: q, k float32 [T, kv_heads * dim] (prepared), v (vdtype) [T, ldv], g [T, heads * dim], beta [T, heads].
// delta == 0: q, k, v of one dtype (vdtype), SiLU applied here; decay [heads].  out [T, heads * vdim] float32.
extern "C" int cima_recurrence(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, int vdtype,
                               const float* g, const float* beta, const float* decay, float* state, const int* seq_slot,
                               const int* seq_first_row, float* out, int T, int n_seqs, int heads, int kv_heads, int dim,
                               int vdim, int delta, cudaStream_t stream) {
  if (T <= 0 || n_seqs <= 0) return 0;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || heads > 65535 || n_seqs > 65535)
    return cima_fail(CIMA_E_SIZE, "recurrence: %d heads on %d key heads in %d sequences are not accepted", heads, kv_heads, n_seqs);
  if (dim <= 0 || dim > 256 || vdim <= 0) return cima_fail(CIMA_E_SIZE, "recurrence: key size %d must lie in 1..256 and value size %d be positive", dim, vdim);
  if (!state || !out || !q || !k || !v) return cima_fail(CIMA_E_ARG, "recurrence: q, k, v, the state and the output are needed");
  if (delta && (!g || !beta)) return cima_fail(CIMA_E_ARG, "recurrence: the delta rule needs the tokens' decays and step sizes");
  if (!delta && !decay) return cima_fail(CIMA_E_ARG, "recurrence: the decay rule needs the heads' decays");
  int rc;
  if (delta) {
    if (vdtype == CIMA_F32) rc = launch_recurrence<float, float, true>(q, ldq, k, ldk, v, ldv, g, beta, decay, state, seq_slot, seq_first_row, out, n_seqs, heads, kv_heads, dim, vdim, stream);
    else if (vdtype == CIMA_BF16) rc = launch_recurrence<float, __nv_bfloat16, true>(q, ldq, k, ldk, v, ldv, g, beta, decay, state, seq_slot, seq_first_row, out, n_seqs, heads, kv_heads, dim, vdim, stream);
    else return cima_fail(CIMA_E_DTYPE, "recurrence: dtype code %d is neither float32 nor bfloat16", vdtype);
  } else {
    if (vdtype == CIMA_F32) rc = launch_recurrence<float, float, false>(q, ldq, k, ldk, v, ldv, g, beta, decay, state, seq_slot, seq_first_row, out, n_seqs, heads, kv_heads, dim, vdim, stream);
    else if (vdtype == CIMA_BF16) rc = launch_recurrence<__nv_bfloat16, __nv_bfloat16, false>(q, ldq, k, ldk, v, ldv, g, beta, decay, state, seq_slot, seq_first_row, out, n_seqs, heads, kv_heads, dim, vdim, stream);
    else return cima_fail(CIMA_E_DTYPE, "recurrence: dtype code %d is neither float32 nor bfloat16", vdtype);
  }
  return rc ? rc : cima_launch_result();
}

// qk [T, ldqk]: q's heads then k's (2 * kv_heads * dim values of a row); a [T, lda]: heads * dim; b [T, ldb]: heads.
extern "C" int cima_delta_prepare(const void* qk, int ldqk, const void* a, int lda, const void* b, int ldb, int dtype,
                                  const float* A_log, const float* dt_bias, float* qn, float* kn, float* g, float* beta,
                                  int T, int heads, int kv_heads, int dim, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (heads <= 0 || kv_heads <= 0 || dim <= 0) return cima_fail(CIMA_E_SIZE, "delta_prepare: heads %d, key heads %d and key size %d must be positive", heads, kv_heads, dim);
  int rc;
  if (dtype == CIMA_F32) rc = cima_launch(k_delta_prepare<float>, dim3(T), dim3(128), (size_t)0, stream, 1, (const float*)qk, ldqk, (const float*)a, lda, (const float*)b, ldb, A_log, dt_bias, qn, kn, g, beta, heads, kv_heads, dim);
  else if (dtype == CIMA_BF16) rc = cima_launch(k_delta_prepare<__nv_bfloat16>, dim3(T), dim3(128), (size_t)0, stream, 1, (const __nv_bfloat16*)qk, ldqk, (const __nv_bfloat16*)a, lda, (const __nv_bfloat16*)b, ldb, A_log, dt_bias, qn, kn, g, beta, heads, kv_heads, dim);
  else return cima_fail(CIMA_E_DTYPE, "delta_prepare: dtype code %d is neither float32 nor bfloat16", dtype);
  return rc ? rc : cima_launch_result();
}
