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
// bfloat16 path for the few rows of a decode step; many bfloat16 rows go to the tensor-core variant below.
#include "common.cuh"
#include <mma.h>

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

// Few rows (a decode step): one warp per (head, output n) would leave the weights' rows to single warps; instead a
// block takes one head and 32 outputs, each warp 4 of them, the lanes stride over k (coalesced reads of the weight
// rows), and the rows of A sit in shared memory.  The sum over k is a lane's partial sum in ascending k, then the
// lanes' sums in a fixed order: the same bits for a row whatever the batch.
constexpr int HL_FEW_ROWS = 8;

template <typename TA>
__global__ void __launch_bounds__(256)
k_head_linear_few(const TA* __restrict__ A, const TA* __restrict__ W, TA* __restrict__ out, int M, int N, int K, int lda, int ldo) {
  cima_pdl_wait();
  extern __shared__ float a_sh[];                       // [M][K]
  const int head = blockIdx.y;
  A += (size_t)head * K;
  W += (size_t)head * N * K;
  out += (size_t)head * N;
  for (int e = threadIdx.x; e < M * K; e += blockDim.x) a_sh[e] = cima_to_f32<TA>(A[(size_t)(e / K) * lda + (e % K)]);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int q = 0; q < 4; q++) {
    const int n = blockIdx.x * 32 + warp * 4 + q;
    if (n >= N) break;
    const TA* wr = W + (size_t)n * K;
    float acc[HL_FEW_ROWS];
#pragma unroll
    for (int m = 0; m < HL_FEW_ROWS; m++) acc[m] = 0.f;
    for (int k = lane; k < K; k += 32) {
      const float w = cima_to_f32<TA>(wr[k]);
#pragma unroll
      for (int m = 0; m < HL_FEW_ROWS; m++)
        if (m < M) acc[m] = fmaf(a_sh[m * K + k], w, acc[m]);
    }
#pragma unroll
    for (int m = 0; m < HL_FEW_ROWS; m++) {
      if (m >= M) break;
      float v = acc[m];
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) out[(size_t)m * ldo + n] = cima_from_f32<TA>(v);
    }
  }
}

// Many bfloat16 rows: warp-level tensor-core tiles (16 x 16 x 16, float32 accumulators), a block of 8 warps on
// 64 rows x 32 outputs of one head, operands staged through shared memory with zero fill at the edges.
constexpr int HT_BM = 64, HT_BN = 32, HT_BK = 32;

__global__ void __launch_bounds__(256)
k_head_linear_mma(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W, __nv_bfloat16* __restrict__ out,
                  int M, int N, int K, int lda, int ldo) {
  using namespace nvcuda;
  cima_pdl_wait();
  __shared__ __align__(32) __nv_bfloat16 As[HT_BM][HT_BK + 8];
  __shared__ __align__(32) __nv_bfloat16 Ws[HT_BN][HT_BK + 8];
  __shared__ __align__(32) float Cs[8][16][16 + 4];
  const int head = blockIdx.z;
  A += (size_t)head * K;
  W += (size_t)head * N * K;
  out += (size_t)head * N;
  const int m0 = blockIdx.y * HT_BM, n0 = blockIdx.x * HT_BN;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wm = warp >> 1, wn = warp & 1;              // 4 x 2 warps, one 16 x 16 tile each
  wmma::fragment<wmma::accumulator, 16, 16, 16, float> c;
  wmma::fill_fragment(c, 0.f);
  const __nv_bfloat16 zero = __float2bfloat16_rn(0.f);
  for (int k0 = 0; k0 < K; k0 += HT_BK) {
    for (int e = threadIdx.x; e < HT_BM * HT_BK; e += 256) {
      const int r = e / HT_BK, kk = e % HT_BK;
      As[r][kk] = (m0 + r < M && k0 + kk < K) ? A[(size_t)(m0 + r) * lda + k0 + kk] : zero;
    }
    for (int e = threadIdx.x; e < HT_BN * HT_BK; e += 256) {
      const int r = e / HT_BK, kk = e % HT_BK;
      Ws[r][kk] = (n0 + r < N && k0 + kk < K) ? W[(size_t)(n0 + r) * K + k0 + kk] : zero;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HT_BK; kk += 16) {
      wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> a;
      wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> b;
      wmma::load_matrix_sync(a, &As[wm * 16][kk], HT_BK + 8);
      wmma::load_matrix_sync(b, &Ws[wn * 16][kk], HT_BK + 8);
      wmma::mma_sync(c, a, b, c);
    }
    __syncthreads();
  }
  wmma::store_matrix_sync(&Cs[warp][0][0], c, 16 + 4, wmma::mem_row_major);
  __syncwarp();
  for (int e = lane; e < 256; e += 32) {
    const int r = e >> 4, cc = e & 15;
    const int m = m0 + wm * 16 + r, n = n0 + wn * 16 + cc;
    if (m < M && n < N) out[(size_t)m * ldo + n] = __float2bfloat16_rn(Cs[warp][r][cc]);
  }
}

// a [M, heads, K] in rows of lda, w [heads, N, K] contiguous, out [M, heads, N] in rows of ldo; all of `dtype`.
extern "C" int cima_head_linear(const void* a, const void* w, void* out, int dtype, int M, int heads, int N, int K, int lda,
                                int ldo, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (heads <= 0 || N <= 0 || K <= 0) return cima_fail(CIMA_E_SIZE, "head_linear: %d heads, N %d and K %d must be positive", heads, N, K);
  if (lda < heads * K || ldo < heads * N) return cima_fail(CIMA_E_SIZE, "head_linear: rows of (%d, %d) do not hold %d heads of (%d, %d)", lda, ldo, heads, K, N);
  if (heads > 65535 || (M + 63) / 64 > 65535) return cima_fail(CIMA_E_SIZE, "head_linear: %d heads / %d rows exceed one launch", heads, M);
  int rc;
  if (M <= HL_FEW_ROWS && (size_t)M * K * 4 <= 48 * 1024) {
    const dim3 grid((N + 31) / 32, heads);
    const size_t smem = (size_t)M * K * sizeof(float);
    if (dtype == CIMA_F32) rc = cima_launch(k_head_linear_few<float>, grid, dim3(256), smem, stream, 1, (const float*)a, (const float*)w, (float*)out, M, N, K, lda, ldo);
    else if (dtype == CIMA_BF16) rc = cima_launch(k_head_linear_few<__nv_bfloat16>, grid, dim3(256), smem, stream, 1, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, M, N, K, lda, ldo);
    else return cima_fail(CIMA_E_DTYPE, "head_linear: dtype code %d is neither float32 nor bfloat16", dtype);
  } else if (dtype == CIMA_BF16) {
    const dim3 grid((N + HT_BN - 1) / HT_BN, (M + HT_BM - 1) / HT_BM, heads);
    rc = cima_launch(k_head_linear_mma, grid, dim3(256), (size_t)0, stream, 1, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, M, N, K, lda, ldo);
  } else if (dtype == CIMA_F32) {
    const dim3 grid((N + 63) / 64, (M + 63) / 64, heads);
    rc = cima_launch(k_head_linear<float>, grid, dim3(256), (size_t)0, stream, 1, (const float*)a, (const float*)w, (float*)out, M, N, K, lda, ldo);
  } else return cima_fail(CIMA_E_DTYPE, "head_linear: dtype code %d is neither float32 nor bfloat16", dtype);
  if (rc) return rc;
  return cima_launch_result();
}
