// Depth average of the residual streams, with the norm that reads the result:
//   x[t, :] = sum_{j < n} a[j] * X_j[t, :]          X_j = plane j of `stack` [planes, T, H], float32
//   y[t, :] = x[t, :] / sqrt(mean(x[t, :]^2) + eps) * w        (when w is given)
// One block per row; the sum runs in ascending j with one accumulator per element, the norm is float32 with
// 1/sqrtf, one rounding at the store of y.  x may be a plane of the stack that is not among the n summed.
#include "common.cuh"

constexpr int DA_THREADS = 256;
constexpr int DA_MAX = 256;      // most streams of one sum (their factors go through shared memory)

template <typename TA>
__global__ void __launch_bounds__(DA_THREADS)
k_depth_average(const float* __restrict__ stack, size_t plane, const float* __restrict__ a, int n,
                float* __restrict__ x, const float* __restrict__ w, TA* __restrict__ y, int H, float eps) {
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
  for (int i = threadIdx.x; i < H; i += DA_THREADS)          // each thread reads back what it wrote itself
    y[row + i] = cima_from_f32<TA>(x[row + i] * inv * w[i]);
}

// stack: float32 [planes, T, H] with `plane` elements from one plane to the next; a [n] float32; x [T, H] float32;
// w [H] float32 and y [T, H] (y_dtype) or both null.
extern "C" int cima_depth_average(const float* stack, long long plane, const float* a, int n, float* x, const float* w,
                                  void* y, int y_dtype, int T, int H, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n < 1 || n > DA_MAX) return cima_fail(CIMA_E_SIZE, "depth_average: %d streams are outside 1..%d", n, DA_MAX);
  if (H <= 0 || plane < (long long)T * H) return cima_fail(CIMA_E_SIZE, "depth_average: planes of %lld values do not hold %d rows of %d", plane, T, H);
  if ((w == nullptr) != (y == nullptr)) return cima_fail(CIMA_E_ARG, "depth_average: the norm's weight and its output go together");
  int rc;
  if (!w || y_dtype == CIMA_F32) rc = cima_launch(k_depth_average<float>, dim3(T), dim3(DA_THREADS), (size_t)0, stream, 1, stack, (size_t)plane, a, n, x, w, (float*)y, H, eps);
  else if (y_dtype == CIMA_BF16) rc = cima_launch(k_depth_average<__nv_bfloat16>, dim3(T), dim3(DA_THREADS), (size_t)0, stream, 1, stack, (size_t)plane, a, n, x, w, (__nv_bfloat16*)y, H, eps);
  else return cima_fail(CIMA_E_DTYPE, "depth_average: dtype code %d is neither float32 nor bfloat16", y_dtype);
  if (rc) return rc;
  return cima_launch_result();
}
