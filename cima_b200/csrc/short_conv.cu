// A short causal convolution over time on each channel, added to its input:
//   u[t, c] = h[t, c] + sum_{j < taps} w[j, c] * h[t - taps + 1 + j, c]        (zeros before a sequence's start)
// (the weight is kept tap by tap, [taps, C], so that neighbouring threads read neighbouring values)
// for the ragged rows of a step.  What lies before the step's first row of a sequence comes from the
// sequence's state [slots, taps - 1, C]: entry k holds the input of position len - (taps - 1) + k, len being the
// positions the sequence held before the step (zeros where that is negative: a slot's state is zeroed when it
// is opened).  Products and sums are float32 in ascending j, one rounding at the store, so a position's result
// does not depend on whether its neighbours came with it or from the state.
//
// Two launches: the convolution (one thread per row and channel), then the state's update (one thread per
// sequence and channel: the last taps - 1 inputs after the step).  When every sequence brings one row, a single
// launch does both, each thread owning its (sequence, channel).
#include "common.cuh"

constexpr int CONV_MAX_TAPS = 16;
constexpr int CONV_THREADS = 256;

template <typename TA, bool ONE_ROW>
__global__ void __launch_bounds__(CONV_THREADS)
k_short_conv(const TA* __restrict__ h, const float* __restrict__ w, TA* __restrict__ state,
             const int* __restrict__ row_seq, const int* __restrict__ seq_slot, const int* __restrict__ seq_first_row,
             TA* __restrict__ u, int C, int taps, int add_input, int act) {
  cima_pdl_wait();
  const int row = blockIdx.x;
  const int c = blockIdx.y * CONV_THREADS + threadIdx.x;
  if (c >= C) return;
  const int seq = ONE_ROW ? row : row_seq[row];
  const int k = ONE_ROW ? 0 : row - seq_first_row[seq];          // index of the row among the step's rows of its sequence
  const int slot = seq_slot[seq];
  TA* st = state + (size_t)slot * (taps - 1) * C + c;
  const float cur = cima_to_f32<TA>(h[(size_t)row * C + c]);
  float acc = add_input ? cur : 0.f;
  float old[CONV_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; j++) {
    if (j >= taps) break;
    const int back = taps - 1 - j;                                // positions back from this row
    float v;
    if (back == 0) v = cur;
    else if (back <= k) v = cima_to_f32<TA>(h[(size_t)(row - back) * C + c]);
    else v = cima_to_f32<TA>(st[(size_t)(taps - 1 - (back - k)) * C]);
    old[j] = v;
    acc = fmaf(w[(size_t)j * C + c], v, acc);
  }
  if (act >= 0) acc = cima_gate_act(acc, act);
  u[(size_t)row * C + c] = cima_from_f32<TA>(acc);
  if (ONE_ROW) {
    // the state moves on by one position: entries 1 .. taps - 2 go down, the row's input comes last
    // (old[j] is the input `taps - 1 - j` positions back: old[1] ... old[taps - 1] are the new entries 0 ... taps - 2)
#pragma unroll
    for (int j = 1; j < CONV_MAX_TAPS; j++) {
      if (j >= taps) break;
      st[(size_t)(j - 1) * C] = cima_from_f32<TA>(old[j]);
    }
  }
}

// Many rows: a thread takes 16 bytes of a row (8 bfloat16 or 4 float32 channels), so that a row of a few thousand
// channels is read and written in whole sectors.  Needs C a multiple of that many channels.
template <typename TA> struct ConvVec;
template <> struct ConvVec<float> { static constexpr int N = 4; };
template <> struct ConvVec<__nv_bfloat16> { static constexpr int N = 8; };

template <typename TA>
__global__ void __launch_bounds__(CONV_THREADS)
k_short_conv_wide(const TA* __restrict__ h, const float* __restrict__ w, const TA* __restrict__ state,
                  const int* __restrict__ row_seq, const int* __restrict__ seq_slot, const int* __restrict__ seq_first_row,
                  TA* __restrict__ u, int C, int taps, int add_input, int act) {
  cima_pdl_wait();
  constexpr int V = ConvVec<TA>::N;
  const int row = blockIdx.x;
  const int c = (blockIdx.y * CONV_THREADS + threadIdx.x) * V;
  if (c >= C) return;
  const int seq = row_seq[row];
  const int k = row - seq_first_row[seq];
  const TA* st = state + (size_t)seq_slot[seq] * (taps - 1) * C + c;
  float acc[V], cur[V];
  {
    const uint4 raw = *reinterpret_cast<const uint4*>(h + (size_t)row * C + c);
    const TA* e = reinterpret_cast<const TA*>(&raw);
#pragma unroll
    for (int i = 0; i < V; i++) { cur[i] = cima_to_f32<TA>(e[i]); acc[i] = add_input ? cur[i] : 0.f; }
  }
  for (int j = 0; j < taps; j++) {
    const int back = taps - 1 - j;
    float v[V];
    if (back == 0) {
#pragma unroll
      for (int i = 0; i < V; i++) v[i] = cur[i];
    } else {
      const TA* src = back <= k ? h + (size_t)(row - back) * C + c : st + (size_t)(taps - 1 - (back - k)) * C;
      const uint4 raw = *reinterpret_cast<const uint4*>(src);
      const TA* e = reinterpret_cast<const TA*>(&raw);
#pragma unroll
      for (int i = 0; i < V; i++) v[i] = cima_to_f32<TA>(e[i]);
    }
#pragma unroll
    for (int i = 0; i < V; i += 4) {
      const float4 ww = *reinterpret_cast<const float4*>(w + (size_t)j * C + c + i);
      acc[i] = fmaf(ww.x, v[i], acc[i]);
      acc[i + 1] = fmaf(ww.y, v[i + 1], acc[i + 1]);
      acc[i + 2] = fmaf(ww.z, v[i + 2], acc[i + 2]);
      acc[i + 3] = fmaf(ww.w, v[i + 3], acc[i + 3]);
    }
  }
  uint4 outv;
  TA* o = reinterpret_cast<TA*>(&outv);
#pragma unroll
  for (int i = 0; i < V; i++) o[i] = cima_from_f32<TA>(act >= 0 ? cima_gate_act(acc[i], act) : acc[i]);
  *reinterpret_cast<uint4*>(u + (size_t)row * C + c) = outv;
}

// Many rows and at most 4 taps: a thread takes 16 bytes of channels through CONV_ROWS (8, 4 or 2) consecutive rows, keeps the
// weights of its channels and the last taps - 1 inputs in registers, and so reads every input once (the block's
// first rows again, as the rows before them) instead of taps times, the chunk's eight loads all in flight at once.  Where a row is not the successor of the row
// before it in its own sequence (the chunk's first row, a sequence's first rows) its past is fetched as in the
// kernel above.  Same products in the same order: the same bits.
constexpr int CONV_FEW_TAPS = 4;

template <typename TA, int CONV_ROWS>
__global__ void __launch_bounds__(CONV_THREADS)
k_short_conv_rows(const TA* __restrict__ h, const float* __restrict__ w, const TA* __restrict__ state,
                  const int* __restrict__ row_seq, const int* __restrict__ seq_slot, const int* __restrict__ seq_first_row,
                  TA* __restrict__ u, int T, int C, int taps, int add_input, int act) {
  cima_pdl_wait();
  constexpr int V = ConvVec<TA>::N;
  const int c = (blockIdx.y * CONV_THREADS + threadIdx.x) * V;
  if (c >= C) return;
  float wv[CONV_FEW_TAPS][V], past[CONV_FEW_TAPS - 1][V];       // past[b - 1]: the input b positions back
#pragma unroll
  for (int j = 0; j < CONV_FEW_TAPS; j++)
    if (j < taps) {
#pragma unroll
      for (int i = 0; i < V; i += 4) {
        const float4 ww = *reinterpret_cast<const float4*>(w + (size_t)j * C + c + i);
        wv[j][i] = ww.x; wv[j][i + 1] = ww.y; wv[j][i + 2] = ww.z; wv[j][i + 3] = ww.w;
      }
    }
  const int r0 = blockIdx.x * CONV_ROWS, r1 = min(T, r0 + CONV_ROWS);
  // Everything the chunk needs is requested at once, before anything is waited for: its rows, the rows before it
  // (its first rows' past, if they belong to the same sequence), and the rows' places in their sequences.
  uint4 rows[CONV_ROWS], halo[CONV_FEW_TAPS - 1];
  int seqs[CONV_ROWS], ks[CONV_ROWS];
#pragma unroll
  for (int r = 0; r < CONV_ROWS; r++)
    if (r0 + r < r1) rows[r] = *reinterpret_cast<const uint4*>(h + (size_t)(r0 + r) * C + c);
#pragma unroll
  for (int b = 1; b < CONV_FEW_TAPS; b++)
    if (b < taps && r0 - b >= 0) halo[b - 1] = *reinterpret_cast<const uint4*>(h + (size_t)(r0 - b) * C + c);
#pragma unroll
  for (int r = 0; r < CONV_ROWS; r++) seqs[r] = r0 + r < r1 ? row_seq[r0 + r] : 0;
#pragma unroll
  for (int r = 0; r < CONV_ROWS; r++) ks[r] = r0 + r - seq_first_row[seqs[r]];
  int prev_seq = -1;
#pragma unroll
  for (int r = 0; r < CONV_ROWS; r++) {
    const int row = r0 + r;
    if (row >= r1) break;
    const int seq = seqs[r], k = ks[r];
    float cur[V];
    {
      const TA* e = reinterpret_cast<const TA*>(&rows[r]);
#pragma unroll
      for (int i = 0; i < V; i++) cur[i] = cima_to_f32<TA>(e[i]);
    }
    if (seq != prev_seq || k < taps - 1) {
      // the past from scratch: rows of the step where they are the sequence's (the chunk's first row has them
      // at hand), its state before that
      const TA* st = state + (size_t)seq_slot[seq] * (taps - 1) * C + c;
#pragma unroll
      for (int b = 1; b < CONV_FEW_TAPS; b++)
        if (b < taps) {
          uint4 raw;
          if (r == 0 && b <= k) raw = halo[b - 1];
          else raw = *reinterpret_cast<const uint4*>(b <= k ? h + (size_t)(row - b) * C + c : st + (size_t)(taps - 1 - (b - k)) * C);
          const TA* e = reinterpret_cast<const TA*>(&raw);
#pragma unroll
          for (int i = 0; i < V; i++) past[b - 1][i] = cima_to_f32<TA>(e[i]);
        }
      prev_seq = seq;
    }
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; i++) acc[i] = add_input ? cur[i] : 0.f;
#pragma unroll
    for (int j = 0; j < CONV_FEW_TAPS; j++)
      if (j < taps) {
        const int back = taps - 1 - j;
#pragma unroll
        for (int i = 0; i < V; i++) {
          float v = cur[i];
#pragma unroll
          for (int b = 1; b < CONV_FEW_TAPS; b++)
            if (b == back) v = past[b - 1][i];
          acc[i] = fmaf(wv[j][i], v, acc[i]);
        }
      }
    uint4 outv;
    TA* o = reinterpret_cast<TA*>(&outv);
#pragma unroll
    for (int i = 0; i < V; i++) o[i] = cima_from_f32<TA>(act >= 0 ? cima_gate_act(acc[i], act) : acc[i]);
    *reinterpret_cast<uint4*>(u + (size_t)row * C + c) = outv;
    // this row becomes the next one's nearest past
#pragma unroll
    for (int b = CONV_FEW_TAPS - 1; b >= 2; b--)
#pragma unroll
      for (int i = 0; i < V; i++) past[b - 1][i] = past[b - 2][i];
#pragma unroll
    for (int i = 0; i < V; i++) past[0][i] = cur[i];
  }
}

template <typename TA>
__global__ void __launch_bounds__(CONV_THREADS)
k_short_conv_state(const TA* __restrict__ h, TA* __restrict__ state, const int* __restrict__ seq_slot,
                   const int* __restrict__ seq_first_row, int C, int taps) {
  cima_pdl_wait();
  const int seq = blockIdx.x;
  const int c = blockIdx.y * CONV_THREADS + threadIdx.x;
  if (c >= C) return;
  const int first = seq_first_row[seq], n = seq_first_row[seq + 1] - first;
  TA* st = state + (size_t)seq_slot[seq] * (taps - 1) * C + c;
  TA v[CONV_MAX_TAPS];
#pragma unroll
  for (int k = 0; k < CONV_MAX_TAPS - 1; k++) {
    if (k >= taps - 1) break;
    const int i = n - (taps - 1) + k;                             // the step's row that becomes entry k, if it is one
    v[k] = i >= 0 ? h[(size_t)(first + i) * C + c] : st[(size_t)(k + n) * C];
  }
#pragma unroll
  for (int k = 0; k < CONV_MAX_TAPS - 1; k++) {
    if (k >= taps - 1) break;
    st[(size_t)k * C] = v[k];
  }
}

// add_input 0 leaves the input out of the sum (a plain convolution); act >= 0 applies that activation (CIMA_ACT_*) to the sum.
// h, u [T, C] and state [slots, taps - 1, C] of one dtype; w [taps, C] float32.  one_row != 0: row r is sequence r's only row.
// rows_per_thread: 0, or how many consecutive rows a thread of the many-row kernel walks (the result does not depend on it).
extern "C" int cima_short_conv(const void* h, int dtype, const float* w, void* state, const int* row_seq, const int* seq_slot,
                               const int* seq_first_row, void* u, int T, int n_seqs, int C, int taps, int one_row,
                               int rows_per_thread, int add_input, int act, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (act >= CIMA_ACT_COUNT) return cima_fail(CIMA_E_ARG, "short_conv: activation code %d is unknown", act);
  if (taps < 1 || taps > CONV_MAX_TAPS) return cima_fail(CIMA_E_SIZE, "short_conv: %d taps are outside 1..%d", taps, CONV_MAX_TAPS);
  if (C <= 0 || n_seqs <= 0) return cima_fail(CIMA_E_SIZE, "short_conv: %d channels and %d sequences must be positive", C, n_seqs);
  if (one_row && T != n_seqs) return cima_fail(CIMA_E_ARG, "short_conv: %d rows are not one for each of %d sequences", T, n_seqs);
  if (taps > 1 && !state) return cima_fail(CIMA_E_ARG, "short_conv: more than one tap needs the sequences' state");
  const dim3 block(CONV_THREADS);
  const unsigned cy = (unsigned)((C + CONV_THREADS - 1) / CONV_THREADS);
  // 16-byte accesses: the rows of h, u and the state must all start on 16 bytes
  const int per16 = dtype == CIMA_F32 ? 4 : 8;
  const bool wide = C % per16 == 0 && (((uintptr_t)h | (uintptr_t)u | (uintptr_t)state | (uintptr_t)w) & 15) == 0;
  // rows a thread walks: 8 where that still leaves the SMs a few hundred thousand threads; else one (the kernel above)
  const long long cells = (long long)T * (C / per16);
  // (measured inside a 2,048-row step at 3,584 channels: 8 rows a thread 14 to 16 us, one row 18 to 19, two rows 22; at
  // 1,536 channels all variants 8 to 10)
  int rows_each = cells >= 2ll * 148 * 2048 ? 8 : 1;
  if (rows_per_thread == 1 || rows_per_thread == 2 || rows_per_thread == 4 || rows_per_thread == 8) rows_each = rows_per_thread;
  else if (rows_per_thread != 0) return cima_fail(CIMA_E_ARG, "short_conv: %d rows a thread; 0 (chosen here), 1, 2, 4 or 8 are possible", rows_per_thread);
#define RUN(TA) { \
    int rc_; \
    if (one_row) rc_ = cima_launch(k_short_conv<TA, true>, dim3(T, cy), block, (size_t)0, stream, 1, (const TA*)h, w, (TA*)state, row_seq, seq_slot, seq_first_row, (TA*)u, C, taps, add_input, act); \
    else if (wide && taps <= CONV_FEW_TAPS && rows_each == 8) rc_ = cima_launch(k_short_conv_rows<TA, 8>, dim3((T + 7) / 8, (unsigned)((C / ConvVec<TA>::N + CONV_THREADS - 1) / CONV_THREADS)), block, (size_t)0, stream, 1, (const TA*)h, w, (const TA*)state, row_seq, seq_slot, seq_first_row, (TA*)u, T, C, taps, add_input, act); \
    else if (wide && taps <= CONV_FEW_TAPS && rows_each == 4) rc_ = cima_launch(k_short_conv_rows<TA, 4>, dim3((T + 3) / 4, (unsigned)((C / ConvVec<TA>::N + CONV_THREADS - 1) / CONV_THREADS)), block, (size_t)0, stream, 1, (const TA*)h, w, (const TA*)state, row_seq, seq_slot, seq_first_row, (TA*)u, T, C, taps, add_input, act); \
    else if (wide && taps <= CONV_FEW_TAPS && rows_each == 2) rc_ = cima_launch(k_short_conv_rows<TA, 2>, dim3((T + 1) / 2, (unsigned)((C / ConvVec<TA>::N + CONV_THREADS - 1) / CONV_THREADS)), block, (size_t)0, stream, 1, (const TA*)h, w, (const TA*)state, row_seq, seq_slot, seq_first_row, (TA*)u, T, C, taps, add_input, act); \
    else if (wide) rc_ = cima_launch(k_short_conv_wide<TA>, dim3(T, (unsigned)((C / ConvVec<TA>::N + CONV_THREADS - 1) / CONV_THREADS)), block, (size_t)0, stream, 1, (const TA*)h, w, (const TA*)state, row_seq, seq_slot, seq_first_row, (TA*)u, C, taps, add_input, act); \
    else rc_ = cima_launch(k_short_conv<TA, false>, dim3(T, cy), block, (size_t)0, stream, 1, (const TA*)h, w, (TA*)state, row_seq, seq_slot, seq_first_row, (TA*)u, C, taps, add_input, act); \
    if (rc_) return rc_; \
    if (!one_row && taps > 1) { rc_ = cima_launch(k_short_conv_state<TA>, dim3(n_seqs, cy), block, (size_t)0, stream, 1, (const TA*)h, (TA*)state, seq_slot, seq_first_row, C, taps); if (rc_) return rc_; } }
  if (dtype == CIMA_F32) RUN(float)
  else if (dtype == CIMA_BF16) RUN(__nv_bfloat16)
  else return cima_fail(CIMA_E_DTYPE, "short_conv: dtype code %d is neither float32 nor bfloat16", dtype);
#undef RUN
  return cima_launch_result();
}
