// Mamba-2's two sequence operations over a step's packed tokens: the short causal convolution with
// its silu, and the recurrence S_t = a_t S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t.
//
// A step holds the new tokens of several sequences back to back (cu_new gives each sequence's
// first row); what a sequence carries from earlier steps lies in per-slot state rows: the last
// taps - 1 rows that entered the convolution, and S of every head.  A sequence that starts at
// position 0 starts from zeros whatever its slot's rows hold.  Sequences of slot -1 are padding:
// their rows are set to zero and no state is touched.
//
// Step sizes, decays, the recurrence and the state are float32 in every mode; x, B and C come in
// the step's element type (the convolution's output).  A token's result depends on its sequence
// alone: every sum is made in an order that sizes fix, not the batch or the step's cut.
#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// ---------------------------------------------------------------------------- convolution
// One thread per (token, channel); grid (tokens, channel tiles).  in: `channels` columns from col0 of a matrix with row stride
// in_stride.  w [channels, taps] (the last tap is the current token's), bias [channels].
// state [slots, taps - 1, channels]: the rows before the step's first, oldest first.
template <typename T>
__global__ void conv_silu_kernel(const T* __restrict__ in, long long in_stride, int col0, int channels, int taps,
                                 const float* __restrict__ w, const float* __restrict__ bias,
                                 const float* __restrict__ state, T* __restrict__ out, const int* __restrict__ token_seq,
                                 const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                                 const int* __restrict__ cu_new) {
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int t = blockIdx.x;
  const int s = token_seq[t];
  const int slot = seq_slot[s];
  T* o = out + (size_t)t * channels + c;
  if (slot < 0) {
    *o = from_float<T>(0.f);
    return;
  }
  const int i = t - cu_new[s];  // index among the sequence's new tokens
  const bool carried = seq_start[s] > 0;
  const float* st = state + (size_t)slot * (taps - 1) * channels + c;
  float acc = bias[c];
  for (int j = 0; j < taps; ++j) {
    const int src = i - (taps - 1 - j);
    float v = 0.f;
    if (src >= 0)
      v = to_float(in[(size_t)(t - (taps - 1 - j)) * in_stride + col0 + c]);
    else if (carried)
      v = st[(size_t)(taps - 1 + src) * channels];
    acc = fmaf(w[(size_t)c * taps + j], v, acc);
  }
  *o = from_float<T>(silu_f(acc));
}

// The state after the step: its row k is the input taps - 1 - k rows before the sequence's new end.
// One thread per (sequence, channel), rows in ascending order (row k is read from a later row only).
template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ in, long long in_stride, int col0, int channels, int taps,
                                  float* __restrict__ state, const int* __restrict__ seq_slot,
                                  const int* __restrict__ seq_start, const int* __restrict__ cu_new) {
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int s = blockIdx.x;
  const int slot = seq_slot[s];
  if (slot < 0) return;
  const int t0 = cu_new[s], n = cu_new[s + 1] - t0;
  const bool carried = seq_start[s] > 0;
  float* st = state + (size_t)slot * (taps - 1) * channels + c;
  for (int k = 0; k < taps - 1; ++k) {
    const int src = n - (taps - 1) + k;
    float v = 0.f;
    if (src >= 0)
      v = to_float(in[(size_t)(t0 + src) * in_stride + col0 + c]);
    else if (carried && k + n < taps - 1)
      v = st[(size_t)(k + n) * channels];
    st[(size_t)k * channels] = v;
  }
}

// One token per sequence (token t is sequence t): the convolution and the state's shift in one launch.
template <typename T>
__global__ void conv_step_kernel(const T* __restrict__ in, long long in_stride, int col0, int channels, int taps,
                                 const float* __restrict__ w, const float* __restrict__ bias, float* __restrict__ state,
                                 T* __restrict__ out, const int* __restrict__ seq_slot, const int* __restrict__ seq_start) {
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int t = blockIdx.x;
  const int slot = seq_slot[t];
  T* o = out + (size_t)t * channels + c;
  if (slot < 0) {
    *o = from_float<T>(0.f);
    return;
  }
  const bool carried = seq_start[t] > 0;
  float* st = state + (size_t)slot * (taps - 1) * channels + c;
  const float cur = to_float(in[(size_t)t * in_stride + col0 + c]);
  float acc = bias[c];
  for (int j = 0; j < taps - 1; ++j) {
    const float v = carried ? st[(size_t)j * channels] : 0.f;
    acc = fmaf(w[(size_t)c * taps + j], v, acc);
    if (j > 0) st[(size_t)(j - 1) * channels] = v;
  }
  acc = fmaf(w[(size_t)c * taps + taps - 1], cur, acc);
  if (taps > 1) st[(size_t)(taps - 2) * channels] = cur;
  *o = from_float<T>(silu_f(acc));
}

// ---------------------------------------------------------------------------- recurrence
constexpr int kLanes = 8;      // lanes that share one value channel: each holds a run of its states
constexpr int kChannels = 16;  // value channels a block
constexpr int kScanThreads = kLanes * kChannels;
constexpr int kChunk = 16;     // tokens staged in shared memory at a time

// grid (ceil(vdim / 16), heads, sequences).  xbc [T, inner | groups*N | groups*N] (x, B, C), dt: `heads`
// columns from dt_col of a matrix with row stride dt_stride, state [slots, heads, vdim, N], y float32 [T, inner].
// Lane l of a channel holds states n = l*R .. l*R + R - 1 (R = ceil(N / 8)); B and C lie in shared
// memory with one word of padding after every R, so that the 8 lanes read 8 banks.
template <typename T, int RMAX>
__global__ void __launch_bounds__(kScanThreads)
ssd_scan_kernel(const T* __restrict__ xbc, const T* __restrict__ dt_in, long long dt_stride, int dt_col,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ skip,
                float* __restrict__ state, float* __restrict__ y, const int* __restrict__ seq_slot,
                const int* __restrict__ seq_start, const int* __restrict__ cu_new, int heads, int vdim, int groups,
                int N) {
  extern __shared__ float sm[];
  const int R = (N + kLanes - 1) / kLanes;
  const int row = kLanes * (R + 1);  // padded length of a token's B (or C)
  float* sB = sm;                    // [kChunk][row]
  float* sC = sB + kChunk * row;     // [kChunk][row]
  float* sX = sC + kChunk * row;     // [kChunk][kChannels]
  float* sDt = sX + kChunk * kChannels;
  float* sA = sDt + kChunk;

  const int s = blockIdx.z, h = blockIdx.y, p0 = blockIdx.x * kChannels;
  const int slot = seq_slot[s];
  const int t0 = cu_new[s], t1 = cu_new[s + 1];
  const int inner = heads * vdim, gn = groups * N;
  const int pl = threadIdx.x / kLanes, nl = threadIdx.x % kLanes;
  const int p = p0 + pl;
  if (slot < 0) {
    if (nl == 0 && p < vdim)
      for (int t = t0; t < t1; ++t) y[(size_t)t * inner + h * vdim + p] = 0.f;
    return;
  }
  const int g = h / (heads / groups);
  const size_t xbc_stride = (size_t)inner + 2 * gn;
  float S[RMAX];
  float* st = state + (((size_t)slot * heads + h) * vdim + min(p, vdim - 1)) * N;
  const bool carried = seq_start[s] > 0;
#pragma unroll
  for (int r = 0; r < RMAX; ++r) {
    const int n = nl * R + r;
    S[r] = (carried && r < R && n < N && p < vdim) ? st[n] : 0.f;
  }
  const float A = -expf(a_log[h]), D = skip[h], bias = dt_bias[h];

  for (int tc = t0; tc < t1; tc += kChunk) {
    const int cnt = min(kChunk, t1 - tc);
    __syncthreads();  // the chunk before has been used
    for (int e = threadIdx.x; e < cnt * kLanes * R; e += kScanThreads) {
      const int tt = e / (kLanes * R), n = e % (kLanes * R);
      const T* src = xbc + (size_t)(tc + tt) * xbc_stride + inner + (size_t)g * N + n;
      const int at = tt * row + n + n / R;
      sB[at] = n < N ? to_float(src[0]) : 0.f;
      sC[at] = n < N ? to_float(src[gn]) : 0.f;
    }
    for (int e = threadIdx.x; e < cnt * kChannels; e += kScanThreads) {
      const int tt = e / kChannels, pp = e % kChannels;
      sX[e] = p0 + pp < vdim ? to_float(xbc[(size_t)(tc + tt) * xbc_stride + h * vdim + p0 + pp]) : 0.f;
    }
    if ((int)threadIdx.x < cnt) {
      const float dt = softplus_f(to_float(dt_in[(size_t)(tc + threadIdx.x) * dt_stride + dt_col + h]) + bias);
      sDt[threadIdx.x] = dt;
      sA[threadIdx.x] = expf(A * dt);
    }
    __syncthreads();
    for (int tt = 0; tt < cnt; ++tt) {
      const float a = sA[tt], xv = sX[tt * kChannels + pl];
      const float dtx = sDt[tt] * xv;
      const float* B = sB + tt * row + nl * (R + 1);
      const float* C = sC + tt * row + nl * (R + 1);
      float acc = 0.f;
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        if (r < R) {
          S[r] = fmaf(a, S[r], dtx * B[r]);
          acc = fmaf(S[r], C[r], acc);
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (nl == 0 && p < vdim) y[(size_t)(tc + tt) * inner + h * vdim + p] = fmaf(D, xv, acc);
    }
  }
  if (p < vdim) {
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      const int n = nl * R + r;
      if (r < R && n < N) st[n] = S[r];
    }
  }
}

template <typename T>
int launch_scan(const void* xbc, const void* dt_in, long long dt_stride, int dt_col, const float* dt_bias,
                const float* a_log, const float* skip, float* state, float* y, const int* seq_slot, const int* seq_start,
                const int* cu_new, int n_seqs, int heads, int vdim, int groups, int N, cudaStream_t stream) {
  const int R = (N + kLanes - 1) / kLanes;
  const size_t smem = (size_t)(2 * kChunk * kLanes * (R + 1) + kChunk * kChannels + 2 * kChunk) * sizeof(float);
  const dim3 grid((vdim + kChannels - 1) / kChannels, heads, n_seqs);
#define EMBER_SCAN(RMAX)                                                                                               \
  ssd_scan_kernel<T, RMAX><<<grid, kScanThreads, smem, stream>>>((const T*)xbc, (const T*)dt_in, dt_stride, dt_col,   \
                                                                 dt_bias, a_log, skip, state, y, seq_slot, seq_start, \
                                                                 cu_new, heads, vdim, groups, N)
  if (R <= 1) EMBER_SCAN(1);
  else if (R <= 2) EMBER_SCAN(2);
  else if (R <= 4) EMBER_SCAN(4);
  else if (R <= 8) EMBER_SCAN(8);
  else if (R <= 16) EMBER_SCAN(16);
  else EMBER_SCAN(32);
#undef EMBER_SCAN
  EMBER_LAUNCH_OK("ssd_scan");
  return 0;
}

}  // namespace

// all_single: every sequence brings one token (token t is sequence t): one launch does the state's shift too.
EMBER_API int ember_conv_silu(const void* in, long long in_stride, int col0, int channels, int taps, const float* w,
                              const float* bias, float* state, void* out, const int* token_seq, const int* seq_slot,
                              const int* seq_start, const int* cu_new, int T, int n_seqs, int all_single, int dtype,
                              cudaStream_t stream) {
  EMBER_CHECK(T > 0 && n_seqs > 0 && channels > 0 && taps >= 1 && taps <= 16, "conv_silu: bad sizes");
  EMBER_CHECK(taps == 1 || state != nullptr, "conv_silu: a convolution of %d taps carries state", taps);
  EMBER_CHECK(dtype == EMBER_F32 || dtype == EMBER_BF16, "conv_silu: element type %d", dtype);
  const int bx = (channels + 127) / 128;
  EMBER_CHECK(bx <= 65535, "conv_silu: %d channels exceed one launch", channels);
#define EMBER_CONV(TT)                                                                                                    \
  do {                                                                                                                    \
    if (all_single && T == n_seqs) {                                                                                      \
      conv_step_kernel<TT><<<dim3(T, bx), 128, 0, stream>>>((const TT*)in, in_stride, col0, channels, taps, w, bias,      \
                                                            state, (TT*)out, seq_slot, seq_start);                        \
    } else {                                                                                                              \
      conv_silu_kernel<TT><<<dim3(T, bx), 128, 0, stream>>>((const TT*)in, in_stride, col0, channels, taps, w, bias,      \
                                                            state, (TT*)out, token_seq, seq_slot, seq_start, cu_new);     \
      if (taps > 1)                                                                                                       \
        conv_state_kernel<TT><<<dim3(n_seqs, bx), 128, 0, stream>>>((const TT*)in, in_stride, col0, channels, taps,       \
                                                                    state, seq_slot, seq_start, cu_new);                  \
    }                                                                                                                     \
  } while (0)
  if (dtype == EMBER_F32) EMBER_CONV(float); else EMBER_CONV(__nv_bfloat16);
#undef EMBER_CONV
  EMBER_LAUNCH_OK("conv_silu");
  return 0;
}

EMBER_API int ember_ssd_scan(const void* xbc, const void* dt_in, long long dt_stride, int dt_col, const float* dt_bias,
                             const float* a_log, const float* skip, float* state, float* y, const int* seq_slot,
                             const int* seq_start, const int* cu_new, int n_seqs, int heads, int vdim, int groups, int N,
                             int dtype, cudaStream_t stream) {
  EMBER_CHECK(n_seqs > 0 && heads > 0 && vdim > 0 && groups > 0 && heads % groups == 0, "ssd_scan: bad sizes");
  EMBER_CHECK(N >= 1 && N <= 256, "ssd_scan: a state of %d rows is not in [1, 256]", N);
  EMBER_CHECK(n_seqs <= 65535 && heads <= 65535, "ssd_scan: %d sequences x %d heads exceed one launch", n_seqs, heads);
  if (dtype == EMBER_F32)
    return launch_scan<float>(xbc, dt_in, dt_stride, dt_col, dt_bias, a_log, skip, state, y, seq_slot, seq_start, cu_new,
                              n_seqs, heads, vdim, groups, N, stream);
  if (dtype == EMBER_BF16)
    return launch_scan<__nv_bfloat16>(xbc, dt_in, dt_stride, dt_col, dt_bias, a_log, skip, state, y, seq_slot, seq_start,
                                      cu_new, n_seqs, heads, vdim, groups, N, stream);
  return ember_fail("ssd_scan: element type %d", dtype);
}
