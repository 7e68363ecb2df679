// Depth average of the residual streams, with the norm that reads the result:
//   x[t, :] = sum_{j < n} a[j] * X_j[t, :]          X_j = plane j of `stack` [planes, T, H], float32
//   y[t, :] = x[t, :] / sqrt(mean(x[t, :]^2) + eps) * w        (when w is given)
// One block per row; the sum runs in ascending j with one accumulator per element, the norm is float32 with
// 1/sqrtf, one rounding at the store of y.  x may be a plane of the stack that is not among the n summed.
//
// When every sequence brings one row (a decode step), the short convolution that reads y can run in the same
// kernel: u = y + sum_j cw[j, :] * (the sequence's last inputs, then y), each thread on its own channels, and the
// sequence's state moves on by one position: exactly what short_conv does in its one-row form, on the rounded y.
#include "common.cuh"

constexpr int DA_THREADS = 256;
constexpr int DA_MAX = 256;      // most streams of one sum (their factors go through shared memory)

template <typename TA>
__global__ void __launch_bounds__(DA_THREADS)
k_depth_average(const float* __restrict__ stack, size_t plane, const float* __restrict__ a, int n,
                float* __restrict__ x, const float* __restrict__ w, TA* __restrict__ y, int H, float eps,
                const float* __restrict__ cw, int taps, TA* __restrict__ state, const int* __restrict__ seq_slot,
                TA* __restrict__ u) {
  cima_pdl_wait();
  __shared__ float red[32];
  __shared__ float fac[DA_MAX];
  for (int j = threadIdx.x; j < n; j += DA_THREADS) fac[j] = a[j];
  __syncthreads();
  const size_t row = (size_t)blockIdx.x * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += DA_THREADS) {
    float acc = 0.f;
    for (int j = 0; j < n; j++) acc = fmaf(fac[j], stack[(size_t)j * plane + row + i], acc);
    x[row + i] = acc;
    ss += acc * acc;
  }
  if (!w) return;
  const float total = cima_block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)H + eps);
  TA* st = cw ? state + (size_t)seq_slot[blockIdx.x] * (taps - 1) * H : nullptr;
  for (int i = threadIdx.x; i < H; i += DA_THREADS) {        // each thread reads back what it wrote itself
    const TA yv = cima_from_f32<TA>(x[row + i] * inv * w[i]);
    y[row + i] = yv;
    if (cw) {
      const float cur = cima_to_f32<TA>(yv);
      float acc = cur;
      for (int j = 0; j < taps - 1; j++) {
        const TA old = st[(size_t)j * H + i];
        acc = fmaf(cw[(size_t)j * H + i], cima_to_f32<TA>(old), acc);
        if (j > 0) st[(size_t)(j - 1) * H + i] = old;
      }
      acc = fmaf(cw[(size_t)(taps - 1) * H + i], cur, acc);
      if (taps > 1) st[(size_t)(taps - 2) * H + i] = yv;
      u[row + i] = cima_from_f32<TA>(acc);
    }
  }
}

// The same for rows of at most 8192 values with at most 4 taps, which is every decode step of the usual sizes: a
// block of 256, 512 or 1024 threads by the row's width, a thread keeps its (at most 8) values of the row in registers between the sum and the norm, and reads everything
// that does not depend on the norm (the convolution's weights and the sequence's last inputs) before it waits
// for the row's sum of squares, all loads before all stores: the kernel is a chain of memory round trips, and
// this leaves three of them.  Same operations in the same order as the general kernel: the same bits.
constexpr int DA_EPT = 8, DA_PAST = 3;

template <typename TA, bool CONV, int THREADS>
__global__ void __launch_bounds__(THREADS)
k_depth_average_row(const float* __restrict__ stack, size_t plane, const float* __restrict__ a, int n,
                    float* __restrict__ x, const float* __restrict__ w, TA* __restrict__ y, int H, float eps,
                    const float* __restrict__ cw, int taps, TA* __restrict__ state, const int* __restrict__ seq_slot,
                    TA* __restrict__ u) {
  cima_pdl_wait();
  __shared__ float red[32];
  __shared__ float fac[DA_MAX];
  for (int j = threadIdx.x; j < n; j += THREADS) fac[j] = a[j];
  __syncthreads();
  const size_t row = (size_t)blockIdx.x * H;
  float xv[DA_EPT], wv[DA_EPT];
#pragma unroll
  for (int e = 0; e < DA_EPT; e++) xv[e] = 0.f;
  for (int j = 0; j < n; j++) {
    const float f = fac[j];
    const float* src = stack + (size_t)j * plane + row;
#pragma unroll
    for (int e = 0; e < DA_EPT; e++) {
      const int i = threadIdx.x + e * THREADS;
      if (i < H) xv[e] = fmaf(f, src[i], xv[e]);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < DA_EPT; e++) {
    const int i = threadIdx.x + e * THREADS;
    if (i < H) { x[row + i] = xv[e]; ss += xv[e] * xv[e]; wv[e] = w[i]; }
  }
  TA old[DA_EPT][DA_PAST];
  float cv[DA_EPT][DA_PAST + 1];
  TA* st = nullptr;
  if (CONV) {
    st = state + (size_t)seq_slot[blockIdx.x] * (taps - 1) * H;
#pragma unroll
    for (int e = 0; e < DA_EPT; e++) {
      const int i = threadIdx.x + e * THREADS;
      if (i < H) {
#pragma unroll
        for (int j = 0; j < DA_PAST; j++)
          if (j < taps - 1) { old[e][j] = st[(size_t)j * H + i]; cv[e][j] = cw[(size_t)j * H + i]; }
        cv[e][DA_PAST] = cw[(size_t)(taps - 1) * H + i];
      }
    }
  }
  const float total = cima_block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)H + eps);
#pragma unroll
  for (int e = 0; e < DA_EPT; e++) {
    const int i = threadIdx.x + e * THREADS;
    if (i < H) {
      const TA yv = cima_from_f32<TA>(xv[e] * inv * wv[e]);
      y[row + i] = yv;
      if (CONV) {
        const float cur = cima_to_f32<TA>(yv);
        float acc = cur;
#pragma unroll
        for (int j = 0; j < DA_PAST; j++) {
          if (j < taps - 1) {
            acc = fmaf(cv[e][j], cima_to_f32<TA>(old[e][j]), acc);
            if (j > 0) st[(size_t)(j - 1) * H + i] = old[e][j];
          }
        }
        acc = fmaf(cv[e][DA_PAST], cur, acc);
        if (taps > 1) st[(size_t)(taps - 2) * H + i] = yv;
        u[row + i] = cima_from_f32<TA>(acc);
      }
    }
  }
}

// stack: float32 [planes, T, H] with `plane` elements from one plane to the next; a [n] float32; x [T, H] float32;
// w [H] float32 and y [T, H] (y_dtype) or both null.  cw [taps, H] float32, state [slots, taps - 1, H], seq_slot [T], u [T, H]
// (state and u of y's dtype): the convolution of y with the state's update, for steps of one row a sequence; or all null.
extern "C" int cima_depth_average(const float* stack, long long plane, const float* a, int n, float* x, const float* w,
                                  void* y, int y_dtype, int T, int H, float eps, const float* cw, int taps, void* state,
                                  const int* seq_slot, void* u, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n < 1 || n > DA_MAX) return cima_fail(CIMA_E_SIZE, "depth_average: %d streams are outside 1..%d", n, DA_MAX);
  if (H <= 0 || plane < (long long)T * H) return cima_fail(CIMA_E_SIZE, "depth_average: planes of %lld values do not hold %d rows of %d", plane, T, H);
  if ((w == nullptr) != (y == nullptr)) return cima_fail(CIMA_E_ARG, "depth_average: the norm's weight and its output go together");
  if (cw && (!w || !u || !seq_slot || taps < 1 || taps > 16 || (taps > 1 && !state)))
    return cima_fail(CIMA_E_ARG, "depth_average: the convolution needs the norm, 1..16 taps, the sequences' slots and state, and its output");
  int rc;
  const bool row_kernel = w && H <= DA_EPT * 1024 && (!cw || taps <= DA_PAST + 1);
  const int threads = H <= DA_EPT * 256 ? 256 : (H <= DA_EPT * 512 ? 512 : 1024);
#define DA_ARGS(TA) stack, (size_t)plane, a, n, x, w, (TA*)y, H, eps, cw, taps, (TA*)state, seq_slot, (TA*)u
#define DA_ROW(TA, C) \
  (threads == 256 ? cima_launch(k_depth_average_row<TA, C, 256>, dim3(T), dim3(256), (size_t)0, stream, 1, DA_ARGS(TA)) \
   : threads == 512 ? cima_launch(k_depth_average_row<TA, C, 512>, dim3(T), dim3(512), (size_t)0, stream, 1, DA_ARGS(TA)) \
                    : cima_launch(k_depth_average_row<TA, C, 1024>, dim3(T), dim3(1024), (size_t)0, stream, 1, DA_ARGS(TA)))
#define DA_RUN(TA) \
  (row_kernel ? (cw ? DA_ROW(TA, true) : DA_ROW(TA, false)) \
              : cima_launch(k_depth_average<TA>, dim3(T), dim3(DA_THREADS), (size_t)0, stream, 1, DA_ARGS(TA)))
  if (!w || y_dtype == CIMA_F32) rc = DA_RUN(float);
  else if (y_dtype == CIMA_BF16) rc = DA_RUN(__nv_bfloat16);
  else return cima_fail(CIMA_E_DTYPE, "depth_average: dtype code %d is neither float32 nor bfloat16", y_dtype);
#undef DA_RUN
#undef DA_ROW
#undef DA_ARGS
  if (rc) return rc;
  return cima_launch_result();
}
