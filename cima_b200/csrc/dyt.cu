// Dynamic Tanh, a norm without row statistics:  y = tanh(alpha * x) * w + b,  alpha one scalar (read from the device,
// so a recorded step needs no host value), w and b vectors.  Everything is elementwise and float32; the result is
// rounded once, to the activations' dtype.  Two kernels:
//   dyt       y = N(x)                                         a norm in front of a sublayer
//   dyt_add   x += mult * N1(y);  optionally h = N2(x)         a norm behind a sublayer with the residual sum, and the
//                                                              norm in front of the next sublayer in the same pass
#include "common.cuh"

namespace {
constexpr int DYT_THREADS = 256;

template <typename TO>
__global__ void __launch_bounds__(DYT_THREADS)
k_dyt(const float* __restrict__ x, const float* __restrict__ alpha, const float* __restrict__ w, const float* __restrict__ b,
      TO* __restrict__ out, size_t n, int H) {
  cima_pdl_wait();
  cima_pdl_trigger();        // a short kernel: the next one may be set up while this one runs (it waits for this one's end itself)
  const float a = alpha[0];
  for (size_t i = (size_t)blockIdx.x * DYT_THREADS + threadIdx.x; i < n; i += (size_t)gridDim.x * DYT_THREADS) {
    const int c = (int)(i % (size_t)H);
    out[i] = cima_from_f32<TO>(fmaf(tanhf(a * x[i]), w[c], b[c]));
  }
}

template <typename TO>
__global__ void __launch_bounds__(DYT_THREADS)
k_dyt_add(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ alpha1, const float* __restrict__ w1,
          const float* __restrict__ b1, float mult, const float* __restrict__ alpha2, const float* __restrict__ w2,
          const float* __restrict__ b2, TO* __restrict__ h, size_t n, int H) {
  cima_pdl_wait();
  cima_pdl_trigger();        // a short kernel: the next one may be set up while this one runs (it waits for this one's end itself)
  const float a1 = alpha1[0], a2 = w2 ? alpha2[0] : 0.f;
  for (size_t i = (size_t)blockIdx.x * DYT_THREADS + threadIdx.x; i < n; i += (size_t)gridDim.x * DYT_THREADS) {
    const int c = (int)(i % (size_t)H);
    const float v = x[i] + mult * fmaf(tanhf(a1 * y[i]), w1[c], b1[c]);
    x[i] = v;
    if (w2) h[i] = cima_from_f32<TO>(fmaf(tanhf(a2 * v), w2[c], b2[c]));
  }
}

inline unsigned dyt_blocks(size_t n) {
  const size_t want = (n + DYT_THREADS - 1) / DYT_THREADS;
  return (unsigned)(want < 148 * 16 ? want : 148 * 16);
}
}  // namespace

// out [T, H] (dtype) = tanh(alpha[0] * x) * w + b, x float32.
extern "C" int cima_dyt(const float* x, const float* alpha, const float* w, const float* b, void* out, int dtype, int T, int H,
                        cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || !alpha || !w || !b) return cima_fail(CIMA_E_ARG, "dyt: the width must be positive and alpha, w, b given");
  const size_t n = (size_t)T * H;
  int rc;
  if (dtype == CIMA_F32) rc = cima_launch(k_dyt<float>, dim3(dyt_blocks(n)), dim3(DYT_THREADS), (size_t)0, stream, 1, x, alpha, w, b, (float*)out, n, H);
  else if (dtype == CIMA_BF16) rc = cima_launch(k_dyt<__nv_bfloat16>, dim3(dyt_blocks(n)), dim3(DYT_THREADS), (size_t)0, stream, 1, x, alpha, w, b, (__nv_bfloat16*)out, n, H);
  else return cima_fail(CIMA_E_DTYPE, "dyt: dtype code %d is neither float32 nor bfloat16", dtype);
  return rc ? rc : cima_launch_result();
}

// x [T, H] float32 += mult * (tanh(alpha1[0] * y) * w1 + b1), y float32; with w2 also h (dtype) = tanh(alpha2[0] * x) * w2 + b2.
extern "C" int cima_dyt_add(float* x, const float* y, const float* alpha1, const float* w1, const float* b1, float mult,
                            const float* alpha2, const float* w2, const float* b2, void* h, int dtype, int T, int H,
                            cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || !alpha1 || !w1 || !b1) return cima_fail(CIMA_E_ARG, "dyt_add: the width must be positive and alpha, w, b given");
  if (w2 && (!alpha2 || !b2 || !h)) return cima_fail(CIMA_E_ARG, "dyt_add: the second norm needs alpha, w, b and an output");
  const size_t n = (size_t)T * H;
  int rc;
  if (dtype == CIMA_F32) rc = cima_launch(k_dyt_add<float>, dim3(dyt_blocks(n)), dim3(DYT_THREADS), (size_t)0, stream, 1, x, y, alpha1, w1, b1, mult, alpha2, w2, b2, (float*)h, n, H);
  else if (dtype == CIMA_BF16) rc = cima_launch(k_dyt_add<__nv_bfloat16>, dim3(dyt_blocks(n)), dim3(DYT_THREADS), (size_t)0, stream, 1, x, y, alpha1, w1, b1, mult, alpha2, w2, b2, (__nv_bfloat16*)h, n, H);
  else return cima_fail(CIMA_E_DTYPE, "dyt_add: dtype code %d is neither float32 nor bfloat16", dtype);
  return rc ? rc : cima_launch_result();
}
