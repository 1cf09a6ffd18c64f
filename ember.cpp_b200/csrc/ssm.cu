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
// A thread takes one channel through a run of 32 tokens of one sequence, the last taps - 1 inputs in registers;
// grid (sequences * runs, channel tiles).  in: `channels` columns from col0 of a matrix with row stride in_stride.
// w [channels, taps] (the last tap is the current token's), bias [channels].  state [slots, taps - 1, channels]:
// the rows before the step's first, oldest first.  The sum starts from the bias and takes the taps oldest first,
// as the one-token kernel below does.
constexpr int kConvRun = 32;

template <typename T, int TMAX>
__global__ void conv_silu_kernel(const T* __restrict__ in, long long in_stride, int col0, int channels, int taps,
                                 const float* __restrict__ w, const float* __restrict__ bias,
                                 const float* __restrict__ state, T* __restrict__ out, const int* __restrict__ seq_slot,
                                 const int* __restrict__ seq_start, const int* __restrict__ cu_new, int runs) {
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int s = blockIdx.x / runs, run = blockIdx.x % runs;
  const int t0 = cu_new[s], n = cu_new[s + 1] - t0;
  const int i0 = run * kConvRun, i1 = min(n, i0 + kConvRun);
  if (i0 >= n) return;
  const int slot = seq_slot[s];
  if (slot < 0) {
    for (int i = i0; i < i1; ++i) out[(size_t)(t0 + i) * channels + c] = from_float<T>(0.f);
    return;
  }
  const bool carried = seq_start[s] > 0;
  const float* st = state + (size_t)slot * (taps - 1) * channels + c;
  const T* src = in + (size_t)t0 * in_stride + col0 + c;
  // hist[TMAX - 1 - m]: the input m tokens back; wt: its tap, zero beyond the filter's length
  float hist[TMAX], wt[TMAX];
#pragma unroll
  for (int m = 0; m < TMAX; ++m) {
    wt[TMAX - 1 - m] = m < taps ? w[(size_t)c * taps + taps - 1 - m] : 0.f;
    float v = 0.f;
    if (m >= 1 && m < taps) {
      const int at = i0 - m;
      if (at >= 0)
        v = to_float(src[(size_t)at * in_stride]);
      else if (carried)
        v = st[(size_t)(taps - 1 + at) * channels];
    }
    hist[TMAX - 1 - m] = v;
  }
  const float b = bias[c];
  for (int i = i0; i < i1; ++i) {
    hist[TMAX - 1] = to_float(src[(size_t)i * in_stride]);
    float acc = b;
#pragma unroll
    for (int k = 0; k < TMAX; ++k) acc = fmaf(wt[k], hist[k], acc);
    out[(size_t)(t0 + i) * channels + c] = from_float<T>(silu_f(acc));
#pragma unroll
    for (int k = 0; k + 1 < TMAX; ++k) hist[k] = hist[k + 1];
  }
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
constexpr int kLanes = 8;      // lanes that share a value channel: lane l holds the states n = l, l + 8, l + 16, ...
constexpr int kPer = 2;        // value channels a thread
constexpr int kChannels = 16 * kPer;  // value channels a block
constexpr int kScanThreads = 128;
constexpr int kSplit = 128;    // tokens of a piece when a long sequence is scanned in pieces

// How many tokens a block stages in shared memory at a time (B and C of N states each, padded to 8 R).
inline int scan_stage(int R) { return max(4, min(32, 4096 / (kLanes * R))); }

// Modes of the scan.  A short sequence (and a decode step) is one pass: kWhole.  A long one is cut into pieces
// of kSplit tokens that are scanned side by side: kLocal scans every piece from a state of zeros and leaves the
// piece's end state and the product of its decays in scratch; ssd_carry_kernel walks the pieces of a sequence
// in order and turns the scratch into every piece's true starting state (and the slot's state after the step);
// kFinal scans every piece again from there and writes y.  The recurrence is linear in the state, so this is
// the same sum in another order.
enum : int { kWhole = 0, kLocal = 1, kFinal = 2 };

// grid (ceil(vdim / 32), heads, sequences * pieces).  xbc [T, inner | groups*N | groups*N] (x, B, C), dt: `heads`
// columns from dt_col of a matrix with row stride dt_stride, state [slots, heads, vdim, N], y float32 [T, inner],
// piece_state [sequences * pieces, heads, vdim, N], piece_decay [sequences * pieces, heads].
// V values of T (16 bytes) as floats
template <typename T>
__device__ __forceinline__ void load16(const T* src, float* dst);
template <>
__device__ __forceinline__ void load16<float>(const float* src, float* dst) {
  const float4 v = *reinterpret_cast<const float4*>(src);
  dst[0] = v.x, dst[1] = v.y, dst[2] = v.z, dst[3] = v.w;
}
template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* src, float* dst) {
  const uint4 raw = *reinterpret_cast<const uint4*>(src);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    dst[2 * i] = f.x, dst[2 * i + 1] = f.y;
  }
}

// VEC: the rows of x, B and C are brought in 16 bytes at a time (N a multiple of 8; inner, vdim and groups * N
// multiples of the 16-byte piece), else value by value.
template <typename T, int RMAX, bool VEC>
__global__ void __launch_bounds__(kScanThreads)
ssd_scan_kernel(const T* __restrict__ xbc, const T* __restrict__ dt_in, long long dt_stride, int dt_col,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ skip,
                float* __restrict__ state, float* __restrict__ y, const int* __restrict__ seq_slot,
                const int* __restrict__ seq_start, const int* __restrict__ cu_new, int heads, int vdim, int groups,
                int N, int stage, int mode, int pieces, float* __restrict__ piece_state, float* __restrict__ piece_decay) {
  extern __shared__ __align__(16) float sm[];
  const int R = (N + kLanes - 1) / kLanes;
  const int row = kLanes * R;          // padded length of a token's B (or C)
  float* sB = sm;                      // [stage][row]
  float* sC = sB + stage * row;        // [stage][row]
  float* sX = sC + stage * row;        // [stage][kChannels]
  float* sDt = sX + stage * kChannels;
  float* sA = sDt + stage;

  const int s = blockIdx.z / pieces, piece = blockIdx.z % pieces;
  const int h = blockIdx.y, p0 = blockIdx.x * kChannels;
  const int slot = seq_slot[s];
  int t0 = cu_new[s], t1 = cu_new[s + 1];
  const int inner = heads * vdim, gn = groups * N;
  const int pl = threadIdx.x / kLanes, nl = threadIdx.x % kLanes;
  const int p = p0 + pl * kPer;        // this thread's first value channel
  if (slot < 0) {
    if (mode != kLocal && piece == 0 && nl == 0)
      for (int t = t0; t < t1; ++t)
#pragma unroll
        for (int c = 0; c < kPer; ++c)
          if (p + c < vdim) y[(size_t)t * inner + h * vdim + p + c] = 0.f;
    return;
  }
  if (mode != kWhole) {
    t0 += piece * kSplit;
    t1 = min(t1, t0 + kSplit);
    if (t0 >= t1) return;
  }
  const int g = h / (heads / groups);
  const size_t xbc_stride = (size_t)inner + 2 * gn;
  const size_t at_piece = ((size_t)blockIdx.z * heads + h) * vdim;
  float S[kPer][RMAX];
  {
    const float* from = mode == kFinal ? piece_state + at_piece * N : state + ((size_t)slot * heads + h) * vdim * N;
    const bool have = mode == kFinal || (mode == kWhole && seq_start[s] > 0);
#pragma unroll
    for (int c = 0; c < kPer; ++c)
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        const int n = r * kLanes + nl;
        S[c][r] = (have && r < R && n < N && p + c < vdim) ? from[(size_t)(p + c) * N + n] : 0.f;
      }
  }
  const float A = -expf(a_log[h]), D = skip[h], bias = dt_bias[h];
  float decay = 1.f;

  for (int tc = t0; tc < t1; tc += stage) {
    const int cnt = min(stage, t1 - tc);
    __syncthreads();  // the tokens staged before have been used
    if constexpr (VEC) {
      constexpr int V = 16 / (int)sizeof(T);
      const int per_row = N / V;  // pieces of a token's B (and of its C); row == N here
#pragma unroll 4
      for (int e = threadIdx.x; e < cnt * 2 * per_row; e += kScanThreads) {
        const int tt = e / (2 * per_row), k = e % (2 * per_row);
        const int which = k / per_row, j = k % per_row;
        float v[V];
        load16<T>(xbc + (size_t)(tc + tt) * xbc_stride + inner + (size_t)which * gn + (size_t)g * N + j * V, v);
        float4* dst = reinterpret_cast<float4*>((which ? sC : sB) + tt * row + j * V);
#pragma unroll
        for (int i = 0; i < V / 4; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
      }
      for (int e = threadIdx.x; e < cnt * (kChannels / V); e += kScanThreads) {
        const int tt = e / (kChannels / V), j = e % (kChannels / V);
        float v[V];
#pragma unroll
        for (int i = 0; i < V; ++i) v[i] = 0.f;
        if (p0 + j * V < vdim) load16<T>(xbc + (size_t)(tc + tt) * xbc_stride + h * vdim + p0 + j * V, v);
        float4* dst = reinterpret_cast<float4*>(sX + tt * kChannels + j * V);
#pragma unroll
        for (int i = 0; i < V / 4; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
      }
    } else {
      for (int e = threadIdx.x; e < cnt * row; e += kScanThreads) {
        const int tt = e / row, n = e % row;
        const T* src = xbc + (size_t)(tc + tt) * xbc_stride + inner + (size_t)g * N + n;
        sB[e] = n < N ? to_float(src[0]) : 0.f;
        sC[e] = n < N ? to_float(src[gn]) : 0.f;
      }
      for (int e = threadIdx.x; e < cnt * kChannels; e += kScanThreads) {
        const int tt = e / kChannels, pp = e % kChannels;
        sX[e] = p0 + pp < vdim ? to_float(xbc[(size_t)(tc + tt) * xbc_stride + h * vdim + p0 + pp]) : 0.f;
      }
    }
    if ((int)threadIdx.x < cnt) {
      const float dt = softplus_f(to_float(dt_in[(size_t)(tc + threadIdx.x) * dt_stride + dt_col + h]) + bias);
      sDt[threadIdx.x] = dt;
      sA[threadIdx.x] = expf(A * dt);
    }
    __syncthreads();
    for (int tt = 0; tt < cnt; ++tt) {
      const float a = sA[tt], dt = sDt[tt];
      decay *= a;
      float xv[kPer], dtx[kPer], acc[kPer][2];
#pragma unroll
      for (int c = 0; c < kPer; ++c) {
        xv[c] = sX[tt * kChannels + pl * kPer + c];
        dtx[c] = dt * xv[c];
        acc[c][0] = acc[c][1] = 0.f;
      }
      const float* B = sB + tt * row + nl;
      const float* C = sC + tt * row + nl;
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        if (r < R) {
          const float b = B[r * kLanes], cc = C[r * kLanes];
#pragma unroll
          for (int c = 0; c < kPer; ++c) {
            S[c][r] = fmaf(a, S[c][r], dtx[c] * b);
            acc[c][r & 1] = fmaf(S[c][r], cc, acc[c][r & 1]);
          }
        }
      }
      if (mode != kLocal) {
#pragma unroll
        for (int c = 0; c < kPer; ++c) {
          float v = acc[c][0] + acc[c][1];
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          v += __shfl_xor_sync(0xffffffffu, v, 4);
          if (nl == 0 && p + c < vdim) y[(size_t)(tc + tt) * inner + h * vdim + p + c] = fmaf(D, xv[c], v);
        }
      }
    }
  }
  if (mode == kFinal) return;  // (the carry kernel has written the slot's state)
  float* to = mode == kLocal ? piece_state + at_piece * N : state + ((size_t)slot * heads + h) * vdim * N;
#pragma unroll
  for (int c = 0; c < kPer; ++c)
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      const int n = r * kLanes + nl;
      if (r < R && n < N && p + c < vdim) to[(size_t)(p + c) * N + n] = S[c][r];
    }
  if (mode == kLocal && blockIdx.x == 0 && threadIdx.x == 0) piece_decay[(size_t)blockIdx.z * heads + h] = decay;
}

// One thread per state value of a (sequence, head): the pieces in order.  piece_state[i] comes in as piece i's end
// state from zeros and leaves as its starting state; the slot's state becomes the state after the last piece.
__global__ void ssd_carry_kernel(float* __restrict__ state, float* __restrict__ piece_state,
                                 const float* __restrict__ piece_decay, const int* __restrict__ seq_slot,
                                 const int* __restrict__ seq_start, const int* __restrict__ cu_new, int heads,
                                 int per_head, int pieces) {
  const int s = blockIdx.z, h = blockIdx.y;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  const int slot = seq_slot[s];
  if (e >= per_head || slot < 0) return;
  const int n_pieces = min(pieces, (cu_new[s + 1] - cu_new[s] + kSplit - 1) / kSplit);
  float* st = state + ((size_t)slot * heads + h) * per_head + e;
  float S = seq_start[s] > 0 ? *st : 0.f;
  for (int i = 0; i < n_pieces; ++i) {
    const size_t at = (size_t)s * pieces + i;
    float* ps = piece_state + (at * heads + h) * per_head + e;
    const float local = *ps;
    *ps = S;
    S = fmaf(piece_decay[at * heads + h], S, local);
  }
  *st = S;
}

template <typename T>
int launch_scan(const void* xbc, const void* dt_in, long long dt_stride, int dt_col, const float* dt_bias,
                const float* a_log, const float* skip, float* state, float* y, const int* seq_slot, const int* seq_start,
                const int* cu_new, int n_seqs, int heads, int vdim, int groups, int N, int pieces, float* piece_state,
                float* piece_decay, cudaStream_t stream) {
  const int R = (N + kLanes - 1) / kLanes;
  const int stage = scan_stage(R);
  const size_t smem = (size_t)(2 * stage * kLanes * R + stage * kChannels + 2 * stage) * sizeof(float);
  const dim3 grid((vdim + kChannels - 1) / kChannels, heads, n_seqs * pieces);
  constexpr int V = 16 / (int)sizeof(T);
  const bool vec = N % 8 == 0 && (heads * vdim) % V == 0 && vdim % V == 0 && (groups * N) % V == 0;
#define EMBER_SCAN_ARGS                                                                                                \
  (const T*)xbc, (const T*)dt_in, dt_stride, dt_col, dt_bias, a_log, skip, state, y, seq_slot, seq_start, cu_new, heads, \
      vdim, groups, N, stage
#define EMBER_SCAN_MODE(RMAX, MODE)                                                                                    \
  do {                                                                                                                 \
    if (vec)                                                                                                           \
      ssd_scan_kernel<T, RMAX, true><<<grid, kScanThreads, smem, stream>>>(EMBER_SCAN_ARGS, MODE, pieces, piece_state, \
                                                                           piece_decay);                              \
    else                                                                                                               \
      ssd_scan_kernel<T, RMAX, false><<<grid, kScanThreads, smem, stream>>>(EMBER_SCAN_ARGS, MODE, pieces, piece_state, \
                                                                            piece_decay);                             \
  } while (0)
#define EMBER_SCAN(MODE)                 \
  do {                                   \
    if (R <= 1) EMBER_SCAN_MODE(1, MODE); \
    else if (R <= 2) EMBER_SCAN_MODE(2, MODE); \
    else if (R <= 4) EMBER_SCAN_MODE(4, MODE); \
    else if (R <= 8) EMBER_SCAN_MODE(8, MODE); \
    else if (R <= 16) EMBER_SCAN_MODE(16, MODE); \
    else EMBER_SCAN_MODE(32, MODE);       \
  } while (0)
  if (pieces <= 1) {
    EMBER_SCAN(kWhole);
  } else {
    EMBER_SCAN(kLocal);
    const int per_head = vdim * N;
    ssd_carry_kernel<<<dim3((per_head + 255) / 256, heads, n_seqs), 256, 0, stream>>>(
        state, piece_state, piece_decay, seq_slot, seq_start, cu_new, heads, per_head, pieces);
    EMBER_SCAN(kFinal);
  }
#undef EMBER_SCAN
#undef EMBER_SCAN_MODE
#undef EMBER_SCAN_ARGS
  EMBER_LAUNCH_OK("ssd_scan");
  return 0;
}

}  // namespace

// all_single: every sequence brings one token (token t is sequence t): one launch does the state's shift too.
// max_new: the most tokens one sequence brings (the launch is sized by it).
EMBER_API int ember_conv_silu(const void* in, long long in_stride, int col0, int channels, int taps, const float* w,
                              const float* bias, float* state, void* out, const int* token_seq, const int* seq_slot,
                              const int* seq_start, const int* cu_new, int T, int n_seqs, int max_new, int all_single,
                              int dtype, cudaStream_t stream) {
  EMBER_CHECK(T > 0 && n_seqs > 0 && channels > 0 && taps >= 1 && taps <= 16, "conv_silu: bad sizes");
  EMBER_CHECK(taps == 1 || state != nullptr, "conv_silu: a convolution of %d taps carries state", taps);
  EMBER_CHECK(dtype == EMBER_F32 || dtype == EMBER_BF16, "conv_silu: element type %d", dtype);
  EMBER_CHECK(max_new >= 1, "conv_silu: the longest sequence brings %d tokens", max_new);
  const int bx = (channels + 127) / 128;
  const int runs = (max_new + kConvRun - 1) / kConvRun;  // of the longest sequence
  EMBER_CHECK(bx <= 65535, "conv_silu: %d channels exceed one launch", channels);
#define EMBER_CONV(TT)                                                                                                    \
  do {                                                                                                                    \
    if (all_single && T == n_seqs) {                                                                                      \
      conv_step_kernel<TT><<<dim3(T, bx), 128, 0, stream>>>((const TT*)in, in_stride, col0, channels, taps, w, bias,      \
                                                            state, (TT*)out, seq_slot, seq_start);                        \
    } else if (taps <= 4) {                                                                                               \
      conv_silu_kernel<TT, 4><<<dim3(n_seqs * runs, bx), 128, 0, stream>>>(                                               \
          (const TT*)in, in_stride, col0, channels, taps, w, bias, state, (TT*)out, seq_slot, seq_start, cu_new, runs);   \
    } else {                                                                                                              \
      conv_silu_kernel<TT, 16><<<dim3(n_seqs * runs, bx), 128, 0, stream>>>(                                              \
          (const TT*)in, in_stride, col0, channels, taps, w, bias, state, (TT*)out, seq_slot, seq_start, cu_new, runs);   \
    }                                                                                                                     \
    if (!(all_single && T == n_seqs)) {                                                                                   \
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

// Tokens of a piece, and the floats of scratch that a call with `pieces` pieces a sequence needs (0 for one piece).
EMBER_API int ember_ssd_scan_piece(void) { return kSplit; }
EMBER_API size_t ember_ssd_scan_scratch(int n_seqs, int pieces, int heads, int vdim, int N) {
  return pieces <= 1 ? 0 : (size_t)n_seqs * pieces * heads * ((size_t)vdim * N + 1);
}

// pieces: 1, or (a step whose longest sequence brings many tokens) ceil(longest / ember_ssd_scan_piece()): every
// sequence is then scanned in that many pieces side by side, with `scratch` of ember_ssd_scan_scratch floats.
EMBER_API int ember_ssd_scan(const void* xbc, const void* dt_in, long long dt_stride, int dt_col, const float* dt_bias,
                             const float* a_log, const float* skip, float* state, float* y, const int* seq_slot,
                             const int* seq_start, const int* cu_new, int n_seqs, int heads, int vdim, int groups, int N,
                             int pieces, float* scratch, int dtype, cudaStream_t stream) {
  EMBER_CHECK(n_seqs > 0 && heads > 0 && vdim > 0 && groups > 0 && heads % groups == 0, "ssd_scan: bad sizes");
  EMBER_CHECK(N >= 1 && N <= 256, "ssd_scan: a state of %d rows is not in [1, 256]", N);
  EMBER_CHECK(pieces >= 1 && (pieces == 1 || scratch != nullptr), "ssd_scan: %d pieces need scratch", pieces);
  EMBER_CHECK((long long)n_seqs * pieces <= 65535 && heads <= 65535, "ssd_scan: %d sequences x %d pieces x %d heads exceed one launch",
              n_seqs, pieces, heads);
  float* piece_state = scratch;
  float* piece_decay = scratch ? scratch + (size_t)n_seqs * pieces * heads * vdim * N : nullptr;
  if (dtype == EMBER_F32)
    return launch_scan<float>(xbc, dt_in, dt_stride, dt_col, dt_bias, a_log, skip, state, y, seq_slot, seq_start, cu_new,
                              n_seqs, heads, vdim, groups, N, pieces, piece_state, piece_decay, stream);
  if (dtype == EMBER_BF16)
    return launch_scan<__nv_bfloat16>(xbc, dt_in, dt_stride, dt_col, dt_bias, a_log, skip, state, y, seq_slot, seq_start,
                                      cu_new, n_seqs, heads, vdim, groups, N, pieces, piece_state, piece_decay, stream);
  return ember_fail("ssd_scan: element type %d", dtype);
}
