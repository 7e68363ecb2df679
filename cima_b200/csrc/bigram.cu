// Embedding with a hashed bigram table beside the token table:
//   x[t] = scale * E[tok_t] + B[(tok_(t-1) * mul_prev + tok_t * mul_cur) mod buckets],      B[buckets] at position 0.
// The token before a step's first row of a sequence is the sequence's state (one int32 per slot), which the step
// brings up to date: in the same launch when every sequence brings one row, else in a second one (a sequence's first
// row reads the old value while its last row's token becomes the new one).  Sums are float32.
#include "common.cuh"

namespace {
template <typename TW>
__global__ void __launch_bounds__(256)
k_embed_bigram(const int* __restrict__ ids, const TW* __restrict__ table, const TW* __restrict__ bigram, float* __restrict__ x,
               int H, float scale, int buckets, long long mul_prev, long long mul_cur, const int* __restrict__ row_pos,
               const int* __restrict__ row_seq, const int* __restrict__ seq_slot, const int* __restrict__ seq_first_row,
               int* __restrict__ prev_state, int one_row) {
  cima_pdl_wait();
  cima_pdl_trigger();        // a short kernel: the next one may be set up while this one runs (it waits for this one's end itself)
  const int row = blockIdx.x;
  const int tok = ids[row];
  const int seq = one_row ? row : row_seq[row];
  const int k = one_row ? 0 : row - seq_first_row[seq];
  const int slot = seq_slot[seq];
  const int prev = k > 0 ? ids[row - 1] : prev_state[slot];
  long long r = buckets;
  if (row_pos[row] > 0) {
    r = ((long long)prev * mul_prev + (long long)tok * mul_cur) % buckets;
    if (r < 0) r += buckets;
  }
  const TW* e = table + (size_t)tok * H;
  const TW* g = bigram + (size_t)r * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x)
    x[(size_t)row * H + c] = fmaf(cima_to_f32<TW>(e[c]), scale, cima_to_f32<TW>(g[c]));
  if (one_row) {
    __syncthreads();                                   // every thread has read the old token
    if (threadIdx.x == 0) prev_state[slot] = tok;
  }
}

__global__ void k_bigram_state(const int* __restrict__ ids, const int* __restrict__ seq_slot, const int* __restrict__ seq_first_row,
                               int* __restrict__ prev_state, int n_seqs) {
  cima_pdl_wait();
  cima_pdl_trigger();        // a short kernel: the next one may be set up while this one runs (it waits for this one's end itself)
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s < n_seqs) prev_state[seq_slot[s]] = ids[seq_first_row[s + 1] - 1];
}
}  // namespace

// table [V, H], bigram [buckets + 1, H] of one dtype; x [T, H] float32; prev_state [slots] int32.
extern "C" int cima_embed_bigram(const int* ids, const void* table, const void* bigram, int dtype, float* x, int T, int n_seqs,
                                 int H, float scale, int buckets, long long mul_prev, long long mul_cur, const int* row_pos,
                                 const int* row_seq, const int* seq_slot, const int* seq_first_row, int* prev_state,
                                 int one_row, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || buckets <= 0 || n_seqs <= 0) return cima_fail(CIMA_E_SIZE, "embed_bigram: width %d, %d buckets and %d sequences must be positive", H, buckets, n_seqs);
  if (one_row && T != n_seqs) return cima_fail(CIMA_E_ARG, "embed_bigram: %d rows are not one for each of %d sequences", T, n_seqs);
  const int threads = H >= 256 ? 256 : ((H + 31) / 32) * 32;
  int rc;
  if (dtype == CIMA_F32) rc = cima_launch(k_embed_bigram<float>, dim3(T), dim3(threads), (size_t)0, stream, 1, ids, (const float*)table, (const float*)bigram, x, H, scale, buckets, mul_prev, mul_cur, row_pos, row_seq, seq_slot, seq_first_row, prev_state, one_row);
  else if (dtype == CIMA_BF16) rc = cima_launch(k_embed_bigram<__nv_bfloat16>, dim3(T), dim3(threads), (size_t)0, stream, 1, ids, (const __nv_bfloat16*)table, (const __nv_bfloat16*)bigram, x, H, scale, buckets, mul_prev, mul_cur, row_pos, row_seq, seq_slot, seq_first_row, prev_state, one_row);
  else return cima_fail(CIMA_E_DTYPE, "embed_bigram: dtype code %d is neither float32 nor bfloat16", dtype);
  if (rc) return rc;
  if (!one_row) {
    rc = cima_launch(k_bigram_state, dim3((n_seqs + 127) / 128), dim3(128), (size_t)0, stream, 1, ids, seq_slot, seq_first_row, prev_state, n_seqs);
    if (rc) return rc;
  }
  return cima_launch_result();
}
