// What an attention over latents needs beside the attention itself.
//
// latent_append: a row's compressed vector r (R values, a slice of a projection's output) becomes the latent
//   c = r / sqrt(mean(r^2) + eps) * g        (float32; one rounding at the store)
// and is written to the sequence's page at the row's position.  The pages hold ONE vector per position
// ([pages, 1, 1, page_size, R]): keys and values are both projected from it, so it is stored once.
//
// head_linear: the same small matrix product for every head,
//   out[t, h, n] = sum_k a[t, h, k] * w[h, n, k]        a: [T, heads, K] in rows of lda; out: [T, heads, N] in rows of ldo
// which moves a query into the latents' space (w = the key projection's head, transposed) and an attention
// result out of it (w = the value projection's head).  FFMA with one float32 accumulator per output in ascending
// k: the same bits for a row whatever comes with it.  It serves the 32-bit path at every size and the
// bfloat16 path for the few rows of a decode step; many bfloat16 rows are the caller's to give to the library's
// batched product, as it does with the other products of many rows.
#include "common.cuh"

// ------------------------------------------------------------------------------------------- latent_append
template <typename TA>
__global__ void __launch_bounds__(128)
k_latent_append(const TA* __restrict__ raw, int ld, const float* __restrict__ g, float eps, TA* __restrict__ cache,
                CimaPaged pg, const int* __restrict__ row_pos, const int* __restrict__ row_seq,
                const int* __restrict__ seq_slot, int R) {
  cima_pdl_wait();
  __shared__ float red[32];
  const int row = blockIdx.x;
  const TA* r = raw + (size_t)row * ld;
  float ss = 0.f;
  for (int i = threadIdx.x; i < R; i += blockDim.x) { const float v = cima_to_f32<TA>(r[i]); ss += v * v; }
  const float total = cima_block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)R + eps);
  TA* dst = cache + pg.offset(seq_slot[row_seq[row]], row_pos[row], 0, 0);
  for (int i = threadIdx.x; i < R; i += blockDim.x) dst[i] = cima_from_f32<TA>(cima_to_f32<TA>(r[i]) * inv * g[i]);
}

// raw: [T, ld] of `dtype`, the R values of a row starting at `raw`; cache: the layer's pages [pages, 1, 1, page_size, R].
extern "C" int cima_latent_append(const void* raw, int dtype, int ld, const float* g, float eps, void* cache,
                                  const int* table, int table_width, int ring, int page_size, const int* row_pos,
                                  const int* row_seq, const int* seq_slot, int T, int R, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (R <= 0 || ld < R) return cima_fail(CIMA_E_SIZE, "latent_append: %d values in rows of %d", R, ld);
  if (!cache || !table) return cima_fail(CIMA_E_ARG, "latent_append: the layer's pages and their block table are needed");
  CimaPaged pg{table, table_width, ring, page_size, 1, R, 1};
  int rc;
  if (dtype == CIMA_F32) rc = cima_launch(k_latent_append<float>, dim3(T), dim3(128), (size_t)0, stream, 1, (const float*)raw, ld, g, eps, (float*)cache, pg, row_pos, row_seq, seq_slot, R);
  else if (dtype == CIMA_BF16) rc = cima_launch(k_latent_append<__nv_bfloat16>, dim3(T), dim3(128), (size_t)0, stream, 1, (const __nv_bfloat16*)raw, ld, g, eps, (__nv_bfloat16*)cache, pg, row_pos, row_seq, seq_slot, R);
  else return cima_fail(CIMA_E_DTYPE, "latent_append: dtype code %d is neither float32 nor bfloat16", dtype);
  if (rc) return rc;
  return cima_launch_result();
}

// ------------------------------------------------------------------------------------------- head_linear
template <typename TA>
__global__ void __launch_bounds__(256)
k_head_linear(const TA* __restrict__ A, const TA* __restrict__ W, TA* __restrict__ out, int M, int N, int K, int lda, int ldo) {
  cima_pdl_wait();
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int head = blockIdx.z;
  A += (size_t)head * K;
  W += (size_t)head * N * K;
  out += (size_t)head * N;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int r = 0; r < 4; r++) {
      const int idx = threadIdx.x + r * 256;
      const int row = idx >> 4, kk = idx & 15;
      const int k = k0 + kk;
      float a = 0.f, w = 0.f;
      if (k < K) {
        if (m0 + row < M) a = cima_to_f32<TA>(A[(size_t)(m0 + row) * lda + k]);
        if (n0 + row < N) w = cima_to_f32<TA>(W[(size_t)(n0 + row) * K + k]);
      }
      As[kk][row] = a;
      Ws[kk][row] = w;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; kk++) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tx * 4 + j;
      if (n < N) out[(size_t)m * ldo + n] = cima_from_f32<TA>(acc[i][j]);
    }
  }
}

// Few rows (a decode step): a block takes 32 outputs n of one head; warp m of the block computes them for row m
// of A, lane l the output n0 + l: the lane walks its row of the head's matrix once (16-byte loads, a chunk of 64 k in
// registers at a time) against the row of A in shared memory (every lane reads the same value: a broadcast), one
// float32 accumulator in ascending k.  All warps of a block read the same weight rows, which the first one brings
// into the first-level cache.  The work is a few hundred KB of weights; its time is latency, so the chain of a
// thread is kept short (K fused multiply-adds) and the blocks many.
constexpr int HL_FEW_ROWS = 8;
constexpr int HL_FEW_K = 64;          // k of a row that a thread holds in registers at a time

template <typename TA> struct HlVec;
template <> struct HlVec<float> { static constexpr int N = 4; };
template <> struct HlVec<__nv_bfloat16> { static constexpr int N = 8; };

// A decode step's latents can be appended by the same launch (both read the projection that ran just before): one
// more row of blocks, of which the first does what k_latent_append does, warp m for row m.
template <typename TA>
struct LatentJob {
  const TA* raw;                // null: no job
  int ld;
  const float* g;
  float eps;
  TA* cache;
  CimaPaged pg;
  const int *row_pos, *row_seq, *seq_slot;
  int R;
};

template <typename TA>
__global__ void __launch_bounds__(32 * HL_FEW_ROWS)
k_head_linear_few(const TA* __restrict__ A, const TA* __restrict__ W, TA* __restrict__ out, int M, int N, int K, int lda, int ldo,
                  int vec, LatentJob<TA> job) {
  extern __shared__ __align__(16) float a_sh[];         // [M][Kp], Kp = K rounded up to 4
  const int Kp = (K + 3) & ~3;
  const int head = blockIdx.y;
  const int lane = threadIdx.x & 31, m = threadIdx.x >> 5;
  if (job.raw && blockIdx.y == gridDim.y - 1) {
    if (blockIdx.x != 0) return;
    cima_pdl_wait();
    const TA* r = job.raw + (size_t)m * job.ld;
    float ss = 0.f;
    for (int i = lane; i < job.R; i += 32) { const float v = cima_to_f32<TA>(r[i]); ss += v * v; }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = 1.0f / sqrtf(ss / (float)job.R + job.eps);
    TA* dst = job.cache + job.pg.offset(job.seq_slot[job.row_seq[m]], job.row_pos[m], 0, 0);
    for (int i = lane; i < job.R; i += 32) dst[i] = cima_from_f32<TA>(cima_to_f32<TA>(r[i]) * inv * job.g[i]);
    return;
  }
  const int n = blockIdx.x * 32 + lane;
  const bool live = n < N;
  const TA* wr = W + ((size_t)head * N + (live ? n : 0)) * K;
  constexpr int V = HlVec<TA>::N;
  float w[HL_FEW_K];
  // the first chunk of the weights does not depend on the kernel before this one: it is requested before the wait
  const int kn0 = min(HL_FEW_K, K);
  if (vec && kn0 == HL_FEW_K) {
#pragma unroll
    for (int q = 0; q < HL_FEW_K / V; q++) {
      const uint4 raw = *reinterpret_cast<const uint4*>(wr + q * V);
      const TA* e = reinterpret_cast<const TA*>(&raw);
#pragma unroll
      for (int i = 0; i < V; i++) w[q * V + i] = cima_to_f32<TA>(e[i]);
    }
  } else {
#pragma unroll
    for (int q = 0; q < HL_FEW_K; q++) w[q] = q < kn0 ? cima_to_f32<TA>(wr[q]) : 0.f;
  }
  cima_pdl_wait();
  A += (size_t)head * K;
  for (int e = threadIdx.x; e < M * Kp; e += blockDim.x) {
    const int r = e / Kp, k = e - r * Kp;
    a_sh[e] = k < K ? cima_to_f32<TA>(A[(size_t)r * lda + k]) : 0.f;
  }
  __syncthreads();
  const float* ar = a_sh + m * Kp;
  float acc = 0.f;
  for (int k0 = 0; k0 < K; k0 += HL_FEW_K) {
    const int kn = min(HL_FEW_K, K - k0);
    if (k0 > 0) {
      if (vec && kn == HL_FEW_K) {
#pragma unroll
        for (int q = 0; q < HL_FEW_K / V; q++) {
          const uint4 raw = *reinterpret_cast<const uint4*>(wr + k0 + q * V);
          const TA* e = reinterpret_cast<const TA*>(&raw);
#pragma unroll
          for (int i = 0; i < V; i++) w[q * V + i] = cima_to_f32<TA>(e[i]);
        }
      } else {
#pragma unroll
        for (int q = 0; q < HL_FEW_K; q++) w[q] = q < kn ? cima_to_f32<TA>(wr[k0 + q]) : 0.f;
      }
    }
    // (chunks beyond the row's end were loaded as zeros, and A's row is padded with zeros to a multiple of 4)
#pragma unroll
    for (int q = 0; q < HL_FEW_K; q += 4) {
      if (q < kn) {
        const float4 a = *reinterpret_cast<const float4*>(ar + k0 + q);
        acc = fmaf(a.x, w[q], acc);
        acc = fmaf(a.y, w[q + 1], acc);
        acc = fmaf(a.z, w[q + 2], acc);
        acc = fmaf(a.w, w[q + 3], acc);
      }
    }
  }
  if (live) out[(size_t)m * ldo + (size_t)head * N + n] = cima_from_f32<TA>(acc);
}

// a [M, heads, K] in rows of lda, w [heads, N, K] contiguous, out [M, heads, N] in rows of ldo; all of `dtype`.
// raw (may be null) ... R: the arguments of cima_latent_append for the same M rows, done by the same launch; only for
// the few rows of a decode step (M <= 8).
static int head_linear_impl(const void* a, const void* w, void* out, int dtype, int M, int heads, int N, int K, int lda,
                            int ldo, const void* raw, int ld_raw, const float* g, float eps, void* cache, const int* table,
                            int table_width, int ring, int page_size, const int* row_pos, const int* row_seq,
                            const int* seq_slot, int R, cudaStream_t stream);

extern "C" int cima_head_linear(const void* a, const void* w, void* out, int dtype, int M, int heads, int N, int K, int lda,
                                int ldo, cudaStream_t stream) {
  return head_linear_impl(a, w, out, dtype, M, heads, N, K, lda, ldo, nullptr, 0, nullptr, 0.f, nullptr, nullptr, 0, 0, 0,
                          nullptr, nullptr, nullptr, 0, stream);
}

extern "C" int cima_head_linear_append(const void* a, const void* w, void* out, int dtype, int M, int heads, int N, int K, int lda,
                                       int ldo, const void* raw, int ld_raw, const float* g, float eps, void* cache,
                                       const int* table, int table_width, int ring, int page_size, const int* row_pos,
                                       const int* row_seq, const int* seq_slot, int R, cudaStream_t stream) {
  if (M > HL_FEW_ROWS || (size_t)M * (K + 3) * 4 > 48 * 1024)
    return cima_fail(CIMA_E_SIZE, "head_linear_append: %d rows of %d values; the launch that also appends takes at most %d rows", M, K, HL_FEW_ROWS);
  if (!raw || !g || !cache || !table || R <= 0 || ld_raw < R)
    return cima_fail(CIMA_E_ARG, "head_linear_append: the compressed rows (%d values in rows of %d), the norm's weight, the pages and their table are needed", R, ld_raw);
  return head_linear_impl(a, w, out, dtype, M, heads, N, K, lda, ldo, raw, ld_raw, g, eps, cache, table, table_width, ring,
                          page_size, row_pos, row_seq, seq_slot, R, stream);
}

static int head_linear_impl(const void* a, const void* w, void* out, int dtype, int M, int heads, int N, int K, int lda,
                            int ldo, const void* raw, int ld_raw, const float* g, float eps, void* cache, const int* table,
                            int table_width, int ring, int page_size, const int* row_pos, const int* row_seq,
                            const int* seq_slot, int R, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (heads <= 0 || N <= 0 || K <= 0) return cima_fail(CIMA_E_SIZE, "head_linear: %d heads, N %d and K %d must be positive", heads, N, K);
  if (lda < heads * K || ldo < heads * N) return cima_fail(CIMA_E_SIZE, "head_linear: rows of (%d, %d) do not hold %d heads of (%d, %d)", lda, ldo, heads, K, N);
  if (heads > 65535 || (M + 63) / 64 > 65535) return cima_fail(CIMA_E_SIZE, "head_linear: %d heads / %d rows exceed one launch", heads, M);
  int rc;
  if (M <= HL_FEW_ROWS && (size_t)M * (K + 3) * 4 <= 48 * 1024) {
    const dim3 grid((N + 31) / 32, heads + (raw ? 1 : 0));
    const CimaPaged pg{table, table_width, ring, page_size, 1, R, 1};
    const size_t smem = (size_t)M * ((K + 3) & ~3) * sizeof(float);
    const int esz = dtype == CIMA_F32 ? 4 : 2;
    const int vec = (((uintptr_t)w & 15) == 0 && ((size_t)K * esz) % 16 == 0) ? 1 : 0;      // every row of w starts on 16 bytes
    if (dtype == CIMA_F32) rc = cima_launch(k_head_linear_few<float>, grid, dim3(32 * M), smem, stream, 1, (const float*)a, (const float*)w, (float*)out, M, N, K, lda, ldo, vec,
                                                LatentJob<float>{(const float*)raw, ld_raw, g, eps, (float*)cache, pg, row_pos, row_seq, seq_slot, R});
    else if (dtype == CIMA_BF16) rc = cima_launch(k_head_linear_few<__nv_bfloat16>, grid, dim3(32 * M), smem, stream, 1, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, M, N, K, lda, ldo, vec,
                                                  LatentJob<__nv_bfloat16>{(const __nv_bfloat16*)raw, ld_raw, g, eps, (__nv_bfloat16*)cache, pg, row_pos, row_seq, seq_slot, R});
    else return cima_fail(CIMA_E_DTYPE, "head_linear: dtype code %d is neither float32 nor bfloat16", dtype);
  } else if (dtype == CIMA_BF16) {
    const dim3 grid((N + 63) / 64, (M + 63) / 64, heads);
    rc = cima_launch(k_head_linear<__nv_bfloat16>, grid, dim3(256), (size_t)0, stream, 1, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, M, N, K, lda, ldo);
  } else if (dtype == CIMA_F32) {
    const dim3 grid((N + 63) / 64, (M + 63) / 64, heads);
    rc = cima_launch(k_head_linear<float>, grid, dim3(256), (size_t)0, stream, 1, (const float*)a, (const float*)w, (float*)out, M, N, K, lda, ldo);
  } else return cima_fail(CIMA_E_DTYPE, "head_linear: dtype code %d is neither float32 nor bfloat16", dtype);
  if (rc) return rc;
  return cima_launch_result();
}
