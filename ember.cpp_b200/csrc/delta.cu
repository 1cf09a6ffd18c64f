// The gated delta rule over a step's packed tokens.
//
// Per head, with a state S of dim x vdim float32 values (S[i][j], i over the key's dimensions):
//     S <- g_t S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
// q and k are unit vectors per key head (x / sqrt(sum x^2 + unit_eps)), q times dim^(-1/2);
// beta_t = sigmoid(b_t), g_t = exp(-exp(A_log) softplus(a_t + dt_bias)).  Everything here is float32
// whatever the step's element type; q, k and v come in that type (the convolution's output).
//
// `delta_prepare` makes the unit vectors, beta and g for every token of the step (parallel over
// tokens).  `delta_scan` walks each sequence's tokens in order: a block = a run of value columns j of
// one (sequence, head), a thread a column, the column S[:, j] in registers; k, q, v, beta and g of a
// few tokens are staged in shared memory at a time.  Every column is independent of the others, so a
// token's result depends on its sequence alone, never on the batch or the step's cut.  A sequence that
// starts at position 0 starts from zeros whatever its slot's state holds; sequences of slot -1 are
// padding: their rows are zero and no state is touched.
#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// grid (T), 128 threads: a warp takes one (q or k, key head) vector at a time.
template <typename T>
__global__ void delta_prepare_kernel(const T* __restrict__ qkv, const T* __restrict__ proj, long long proj_stride, int b_col,
                                     int a_col, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                     float* __restrict__ qk, float* __restrict__ beta, float* __restrict__ decay, int heads,
                                     int kv_heads, int dim, int channels, float unit_eps) {
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const T* row = qkv + (size_t)t * channels;
  const float q_scale = rsqrtf((float)dim);
  for (int item = warp; item < 2 * kv_heads; item += warps) {   // items 0..kv-1: q heads, then the k heads
    const T* src = row + (size_t)item * dim;
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32) {
      const float v = to_float(src[d]);
      ss = fmaf(v, v, ss);
    }
    const float inv = (1.0f / sqrtf(warp_sum(ss) + unit_eps)) * (item < kv_heads ? q_scale : 1.0f);
    float* dst = qk + (size_t)t * 2 * kv_heads * dim + (size_t)item * dim;
    for (int d = lane; d < dim; d += 32) dst[d] = to_float(src[d]) * inv;
  }
  for (int h = threadIdx.x; h < heads; h += blockDim.x) {
    const float b = to_float(proj[(size_t)t * proj_stride + b_col + h]);
    const float a = to_float(proj[(size_t)t * proj_stride + a_col + h]);
    beta[(size_t)t * heads + h] = 1.0f / (1.0f + expf(-b));
    decay[(size_t)t * heads + h] = expf(-expf(a_log[h]) * softplus_f(a + dt_bias[h]));
  }
}

constexpr int kStage = 16;   // tokens staged in shared memory at a time

// grid (sequences, heads, column tiles), blockDim.x columns a block.  DMAX >= dim: the column's registers.
template <typename T, int DMAX>
__global__ void delta_scan_kernel(const float* __restrict__ qk, const T* __restrict__ qkv, const float* __restrict__ beta,
                                  const float* __restrict__ decay, float* __restrict__ state, float* __restrict__ out,
                                  const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                                  const int* __restrict__ cu_new, int heads, int kv_heads, int dim, int vdim, int channels) {
  extern __shared__ float smem[];
  float* ks = smem;                         // [kStage][DMAX]
  float* qs = ks + kStage * DMAX;           // [kStage][DMAX]
  float* vs = qs + kStage * DMAX;           // [kStage][blockDim.x]
  float* bs = vs + kStage * blockDim.x;     // [kStage] beta
  float* gs = bs + kStage;                  // [kStage] decay
  const int s = blockIdx.x, h = blockIdx.y;
  const int j = blockIdx.z * blockDim.x + threadIdx.x;
  const bool live = j < vdim;
  const int t0 = cu_new[s], n = cu_new[s + 1] - t0;
  const int slot = seq_slot[s];
  const int inner = heads * vdim;
  if (slot < 0) {
    if (live)
      for (int i = 0; i < n; ++i) out[(size_t)(t0 + i) * inner + (size_t)h * vdim + j] = 0.f;
    return;
  }
  const int kh = h / (heads / kv_heads);
  const int qk_row = 2 * kv_heads * dim;
  float* col = state + ((size_t)slot * heads + h) * dim * vdim + j;
  float S[DMAX];
  const bool carried = seq_start[s] > 0;
#pragma unroll
  for (int d = 0; d < DMAX; ++d) S[d] = (live && carried && d < dim) ? col[(size_t)d * vdim] : 0.f;

  for (int c0 = 0; c0 < n; c0 += kStage) {
    const int cn = min(kStage, n - c0);
    __syncthreads();
    for (int e = threadIdx.x; e < cn * DMAX; e += blockDim.x) {
      const int i = e / DMAX, d = e % DMAX;
      const float* src = qk + (size_t)(t0 + c0 + i) * qk_row;
      qs[e] = d < dim ? src[(size_t)kh * dim + d] : 0.f;
      ks[e] = d < dim ? src[(size_t)(kv_heads + kh) * dim + d] : 0.f;
    }
    for (int i = 0; i < cn; ++i)
      vs[i * blockDim.x + threadIdx.x] =
          live ? to_float(qkv[(size_t)(t0 + c0 + i) * channels + 2 * kv_heads * dim + (size_t)h * vdim + j]) : 0.f;
    if (threadIdx.x < cn) {
      bs[threadIdx.x] = beta[(size_t)(t0 + c0 + threadIdx.x) * heads + h];
      gs[threadIdx.x] = decay[(size_t)(t0 + c0 + threadIdx.x) * heads + h];
    }
    __syncthreads();
    for (int i = 0; i < cn; ++i) {
      const float* k = ks + i * DMAX;
      const float* q = qs + i * DMAX;
      const float g = gs[i];
      float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
#pragma unroll
      for (int d = 0; d < DMAX; d += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(k + d);
        S[d] *= g;
        S[d + 1] *= g;
        S[d + 2] *= g;
        S[d + 3] *= g;
        p0 = fmaf(S[d], kv.x, p0);
        p1 = fmaf(S[d + 1], kv.y, p1);
        p2 = fmaf(S[d + 2], kv.z, p2);
        p3 = fmaf(S[d + 3], kv.w, p3);
      }
      const float u = bs[i] * (vs[i * blockDim.x + threadIdx.x] - ((p0 + p1) + (p2 + p3)));
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int d = 0; d < DMAX; d += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(k + d);
        const float4 qv = *reinterpret_cast<const float4*>(q + d);
        S[d] = fmaf(kv.x, u, S[d]);
        S[d + 1] = fmaf(kv.y, u, S[d + 1]);
        S[d + 2] = fmaf(kv.z, u, S[d + 2]);
        S[d + 3] = fmaf(kv.w, u, S[d + 3]);
        o0 = fmaf(S[d], qv.x, o0);
        o1 = fmaf(S[d + 1], qv.y, o1);
        o2 = fmaf(S[d + 2], qv.z, o2);
        o3 = fmaf(S[d + 3], qv.w, o3);
      }
      if (live) out[(size_t)(t0 + c0 + i) * inner + (size_t)h * vdim + j] = (o0 + o1) + (o2 + o3);
    }
  }
  if (live) {
#pragma unroll
    for (int d = 0; d < DMAX; ++d)
      if (d < dim) col[(size_t)d * vdim] = S[d];
  }
}

// Any dim: the column stays in the slot's state rows (global memory) while the sequence is walked.
template <typename T>
__global__ void delta_scan_wide_kernel(const float* __restrict__ qk, const T* __restrict__ qkv, const float* __restrict__ beta,
                                       const float* __restrict__ decay, float* __restrict__ state, float* __restrict__ out,
                                       const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                                       const int* __restrict__ cu_new, int heads, int kv_heads, int dim, int vdim,
                                       int channels) {
  const int s = blockIdx.x, h = blockIdx.y;
  const int j = blockIdx.z * blockDim.x + threadIdx.x;
  if (j >= vdim) return;
  const int t0 = cu_new[s], n = cu_new[s + 1] - t0;
  const int slot = seq_slot[s];
  const int inner = heads * vdim;
  if (slot < 0) {
    for (int i = 0; i < n; ++i) out[(size_t)(t0 + i) * inner + (size_t)h * vdim + j] = 0.f;
    return;
  }
  const int kh = h / (heads / kv_heads);
  const int qk_row = 2 * kv_heads * dim;
  float* col = state + ((size_t)slot * heads + h) * dim * vdim + j;
  if (seq_start[s] == 0)
    for (int d = 0; d < dim; ++d) col[(size_t)d * vdim] = 0.f;
  for (int i = 0; i < n; ++i) {
    const float* q = qk + (size_t)(t0 + i) * qk_row + (size_t)kh * dim;
    const float* k = qk + (size_t)(t0 + i) * qk_row + (size_t)(kv_heads + kh) * dim;
    const float g = decay[(size_t)(t0 + i) * heads + h];
    float p = 0.f;
    for (int d = 0; d < dim; ++d) {
      const float sd = col[(size_t)d * vdim] * g;
      col[(size_t)d * vdim] = sd;
      p = fmaf(sd, k[d], p);
    }
    const float v = to_float(qkv[(size_t)(t0 + i) * channels + 2 * kv_heads * dim + (size_t)h * vdim + j]);
    const float u = beta[(size_t)(t0 + i) * heads + h] * (v - p);
    float o = 0.f;
    for (int d = 0; d < dim; ++d) {
      const float sd = fmaf(k[d], u, col[(size_t)d * vdim]);
      col[(size_t)d * vdim] = sd;
      o = fmaf(sd, q[d], o);
    }
    out[(size_t)(t0 + i) * inner + (size_t)h * vdim + j] = o;
  }
}

template <typename T>
int delta_rule_run(const T* qkv, const T* proj, long long proj_stride, int b_col, int a_col, const float* a_log,
                   const float* dt_bias, float* state, float* out, float* scratch, const int* seq_slot, const int* seq_start,
                   const int* cu_new, int T_tokens, int n_seq, int heads, int kv_heads, int dim, int vdim, float unit_eps,
                   cudaStream_t stream) {
  const int channels = 2 * kv_heads * dim + heads * vdim;
  float* qk = scratch;
  float* beta = qk + (size_t)T_tokens * 2 * kv_heads * dim;
  float* decay = beta + (size_t)T_tokens * heads;
  delta_prepare_kernel<T><<<T_tokens, 128, 0, stream>>>(qkv, proj, proj_stride, b_col, a_col, a_log, dt_bias, qk, beta, decay,
                                                        heads, kv_heads, dim, channels, unit_eps);
  EMBER_LAUNCH_OK("delta_prepare");
  const int cols = vdim >= 128 ? 128 : (vdim + 31) / 32 * 32;
  const dim3 grid(n_seq, heads, (vdim + cols - 1) / cols);
#define EMBER_DELTA_SCAN(DMAX)                                                                                          \
  do {                                                                                                                  \
    const size_t smem = (size_t)(2 * kStage * DMAX + kStage * cols + 2 * kStage) * sizeof(float);                       \
    delta_scan_kernel<T, DMAX><<<grid, cols, smem, stream>>>(qk, qkv, beta, decay, state, out, seq_slot, seq_start, cu_new, \
                                                             heads, kv_heads, dim, vdim, channels);                     \
  } while (0)
  if (dim <= 32)
    EMBER_DELTA_SCAN(32);
  else if (dim <= 64)
    EMBER_DELTA_SCAN(64);
  else if (dim <= 128)
    EMBER_DELTA_SCAN(128);
  else
    delta_scan_wide_kernel<T><<<grid, cols, 0, stream>>>(qk, qkv, beta, decay, state, out, seq_slot, seq_start, cu_new, heads,
                                                         kv_heads, dim, vdim, channels);
#undef EMBER_DELTA_SCAN
  EMBER_LAUNCH_OK("delta_scan");
  return 0;
}

}  // namespace

// floats of scratch for a step of T tokens: the unit vectors q | k per key head, beta and the decay per head
EMBER_API size_t ember_delta_rule_scratch(int T, int heads, int kv_heads, int dim) {
  return (size_t)T * (2 * (size_t)kv_heads * dim + 2 * (size_t)heads);
}

// qkv [T, q | k | v] (the convolution's output), b and a: `heads` columns each from b_col and a_col of `proj`;
// state float32 [slots, heads, dim, vdim] (advanced); out float32 [T, heads * vdim].
EMBER_API int ember_delta_rule(const void* qkv, const void* proj, long long proj_stride, int b_col, int a_col,
                               const float* a_log, const float* dt_bias, float* state, float* out, float* scratch,
                               const int* seq_slot, const int* seq_start, const int* cu_new, int T, int n_seq, int heads,
                               int kv_heads, int dim, int vdim, float unit_eps, int dtype, cudaStream_t stream) {
  EMBER_CHECK(T > 0 && n_seq > 0 && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0, "delta_rule: bad sizes");
  EMBER_CHECK(heads % kv_heads == 0, "delta_rule: %d heads are not a multiple of %d key heads", heads, kv_heads);
  EMBER_CHECK(heads <= 65535, "delta_rule: %d heads exceed one launch", heads);
  if (dtype == EMBER_F32)
    return delta_rule_run<float>((const float*)qkv, (const float*)proj, proj_stride, b_col, a_col, a_log, dt_bias, state, out,
                                 scratch, seq_slot, seq_start, cu_new, T, n_seq, heads, kv_heads, dim, vdim, unit_eps, stream);
  if (dtype == EMBER_BF16)
    return delta_rule_run<__nv_bfloat16>((const __nv_bfloat16*)qkv, (const __nv_bfloat16*)proj, proj_stride, b_col, a_col,
                                         a_log, dt_bias, state, out, scratch, seq_slot, seq_start, cu_new, T, n_seq, heads,
                                         kv_heads, dim, vdim, unit_eps, stream);
  return ember_fail("delta_rule: element type %d", dtype);
}
