// Rows of a table of token pairs added to the embedded rows.
//
// x[t] += table[row(t)], row(t) = (token[t-1] * mul_prev + token[t] * mul_cur) mod buckets for a token
// that is not its sequence's first, and the table's extra last row (number `buckets`) for a sequence's
// first token.  The token before a step's first token comes from the sequence's state (one int32 per
// slot), which the block of the step's first token of that sequence reads and then sets to the
// sequence's last token of the step.  Sequences of slot -1 are padding and touch nothing.
#include "common.cuh"

namespace {

template <typename T>
__global__ void pair_table_add_kernel(float* __restrict__ x, const int* __restrict__ tokens, const int* __restrict__ positions,
                                      const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                                      const int* __restrict__ cu_new, const T* __restrict__ table, int* __restrict__ state,
                                      int d, long long mul_prev, long long mul_cur, int buckets, int vocab) {
  const int t = blockIdx.x;
  const int s = token_seq[t];
  const int slot = seq_slot[s];
  if (slot < 0) return;
  const int first_row = cu_new[s];
  const int tok = tokens[t];
  int row = buckets;
  if (positions[t] > 0) {
    int prev = t > first_row ? tokens[t - 1] : state[slot];
    prev = min(max(prev, 0), vocab - 1);
    long long v = ((long long)prev * mul_prev + (long long)tok * mul_cur) % buckets;
    if (v < 0) v += buckets;
    row = (int)v;
  }
  const T* src = table + (size_t)row * d;
  float* dst = x + (size_t)t * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] += to_float(src[i]);
  if (t == first_row) {
    __syncthreads();   // every thread of this block has read the state
    if (threadIdx.x == 0) state[slot] = tokens[cu_new[s + 1] - 1];
  }
}

}  // namespace

EMBER_API int ember_pair_table_add(float* x, const int* tokens, const int* positions, const int* token_seq,
                                   const int* seq_slot, const int* cu_new, const void* table, int* state, int T, int d,
                                   long long mul_prev, long long mul_cur, int buckets, int vocab, int dtype,
                                   cudaStream_t stream) {
  EMBER_CHECK(T > 0 && d > 0 && buckets > 0 && vocab > 0, "pair_table_add: bad sizes");
  if (dtype == EMBER_F32)
    pair_table_add_kernel<float><<<T, 128, 0, stream>>>(x, tokens, positions, token_seq, seq_slot, cu_new, (const float*)table,
                                                        state, d, mul_prev, mul_cur, buckets, vocab);
  else if (dtype == EMBER_BF16)
    pair_table_add_kernel<__nv_bfloat16><<<T, 128, 0, stream>>>(x, tokens, positions, token_seq, seq_slot, cu_new,
                                                                (const __nv_bfloat16*)table, state, d, mul_prev, mul_cur,
                                                                buckets, vocab);
  else
    return ember_fail("pair_table_add: element type %d", dtype);
  EMBER_LAUNCH_OK("pair_table_add");
  return 0;
}
