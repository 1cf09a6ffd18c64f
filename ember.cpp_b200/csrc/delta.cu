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
                                     float* __restrict__ qk, float* __restrict__ beta, float* __restrict__ decay,
                                     float* __restrict__ log_decay, int heads, int kv_heads, int dim, int channels,
                                     float unit_eps) {
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
    const float lg = -expf(a_log[h]) * softplus_f(a + dt_bias[h]);
    decay[(size_t)t * heads + h] = expf(lg);
    log_decay[(size_t)t * heads + h] = lg;
  }
}

constexpr int kStage = 16;   // tokens staged in shared memory at a time
inline size_t align4(size_t n) { return (n + 3) & ~(size_t)3; }

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


// ---------------------------------------------------------------------------- prompts in chunks of 64 tokens
// Inside a chunk the rule has a closed form.  With L_t the sum of log g over the chunk's tokens up to t, and S0 the
// state at the chunk's start, the writes u_t of the chunk solve (I + A) U = diag(beta) V - diag(beta e^L) K S0 with
// A[t][i] = beta_t e^(L_t - L_i) (k_t . k_i) for i < t.  So with Tm = (I + A)^-1 (unit lower triangular),
//     Wv = Tm diag(beta) V,   Wk = Tm diag(beta e^L) K,   P[t][i] = e^(L_t - L_i) (q_t . k_i) for i <= t
// depend on the chunk alone (`delta_chunk_factor`, a block a (chunk, head), all chunks side by side), and then
//     U = Wv - Wk S0,   O = diag(e^L) Q S0 + P U,   S <- e^(L_end) S0 + sum_i e^(L_end - L_i) k_i u_i^T
// walk the chunks in order (`delta_chunk_scan`, a block a (sequence, head, 32 or 16 value columns): the columns of S are
// independent).  Every exponent is of a difference <= 0.  All float32 on the CUDA cores; a chunk's rows past the
// sequence's end count as beta = 0, g = 1 and zero vectors.
constexpr int kChunk = 64;

__device__ __forceinline__ void copy16(float* dst, const float* src) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(a), "l"(src));
}
__device__ __forceinline__ void copies_wait() { asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory"); }

// The chunk slot of sequence s's chunk c: chunks are numbered through the step's sequences in order.
__device__ __forceinline__ int chunk_slot(const int* cu_new, int s, int c) {
  int base = 0;
  for (int i = 0; i < s; ++i) base += (cu_new[i + 1] - cu_new[i] + kChunk - 1) / kChunk;
  return base + c;
}

template <typename T>
__global__ void __launch_bounds__(256)
delta_chunk_factor_kernel(const float* __restrict__ qk, const T* __restrict__ qkv, const float* __restrict__ beta,
                          const float* __restrict__ log_decay, float* __restrict__ wv, float* __restrict__ wk,
                          float* __restrict__ pm, float* __restrict__ lgc, const int* __restrict__ seq_slot,
                          const int* __restrict__ cu_new, int n_seq, int max_chunks, int heads, int kv_heads, int dim, int vdim,
                          int channels) {
  extern __shared__ float sm[];
  const int s = blockIdx.x / max_chunks, c = blockIdx.x % max_chunks, h = blockIdx.y;
  const int t0 = cu_new[s], n = cu_new[s + 1] - t0;
  if (seq_slot[s] < 0 || c * kChunk >= n) return;
  const int rows = min(kChunk, n - c * kChunk), first = t0 + c * kChunk;
  const int kh = h / (heads / kv_heads), qk_row = 2 * kv_heads * dim, DS = dim + 1, CS = kChunk + 4;
  float* ks = sm;                       // [64][dim + 1]
  float* qs = ks + kChunk * DS;         // [64][dim + 1]
  float* am = qs + kChunk * DS + (4 - (2 * kChunk * DS) % 4) % 4;   // [64][68]: A, then Tm scaled for Wk (on 16 bytes)
  float* tm = am + kChunk * CS;         // [64][68]: Tm
  float* lg = tm + kChunk * CS;         // [64] L_t
  float* bt = lg + kChunk;              // [64] beta_t
  float* raw = bt + kChunk;             // [64] log g_t
  const int tid = threadIdx.x;
  if (tid < kChunk) {
    raw[tid] = tid < rows ? log_decay[(size_t)(first + tid) * heads + h] : 0.f;
    bt[tid] = tid < rows ? beta[(size_t)(first + tid) * heads + h] : 0.f;
  }
  for (int e = tid; e < kChunk * dim; e += 256) {
    const int r = e / dim, d = e % dim;
    const float* src = qk + (size_t)(first + r) * qk_row;
    qs[r * DS + d] = r < rows ? src[(size_t)kh * dim + d] : 0.f;
    ks[r * DS + d] = r < rows ? src[(size_t)(kv_heads + kh) * dim + d] : 0.f;
  }
  __syncthreads();
  if (tid == 0) {
    float run = 0.f;
    for (int r = 0; r < kChunk; ++r) {
      run += raw[r];
      lg[r] = run;
    }
  }
  __syncthreads();
  const size_t slot = ((size_t)chunk_slot(cu_new, s, c) * heads + h) * kChunk;
  if (tid < kChunk) lgc[slot + tid] = lg[tid];
  // A and P in 4 x 4 tiles of (t, i), a thread a tile of the lower triangle
  {
    const int tt = (tid >> 4) * 4, ii = (tid & 15) * 4;
    if (ii <= tt) {
      float kk[4][4], qd[4][4];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) kk[a][b] = qd[a][b] = 0.f;
      for (int d = 0; d < dim; ++d) {
        float kt[4], qt[4], ki[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          kt[a] = ks[(tt + a) * DS + d];
          qt[a] = qs[(tt + a) * DS + d];
          ki[a] = ks[(ii + a) * DS + d];
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            kk[a][b] = fmaf(kt[a], ki[b], kk[a][b]);
            qd[a][b] = fmaf(qt[a], ki[b], qd[a][b]);
          }
      }
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int t = tt + a, i = ii + b;
          const float w = i <= t ? expf(lg[t] - lg[i]) : 0.f;
          am[t * CS + i] = i < t ? bt[t] * w * kk[a][b] : 0.f;
          pm[(slot + t) * kChunk + i] = w * qd[a][b];
        }
    } else {
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          am[(tt + a) * CS + ii + b] = 0.f;
          pm[(slot + tt + a) * kChunk + ii + b] = 0.f;
        }
    }
  }
  __syncthreads();
  // Tm = (I + A)^-1 by forward substitution, a thread a column (a column needs only itself)
  if (tid < kChunk) {
    const int col = tid;
    for (int t = 0; t < kChunk; ++t) {
      float v = t == col ? 1.f : 0.f;
      for (int i = col; i < t; ++i) v = fmaf(-am[t * CS + i], tm[i * CS + col], v);   // (rows above `col` are zero)
      tm[t * CS + col] = t >= col ? v : 0.f;
    }
  }
  __syncthreads();
  // columns scaled: tm <- Tm diag(beta), am <- Tm diag(beta e^L)
  for (int e = tid; e < kChunk * kChunk; e += 256) {
    const int r = e >> 6, i = e & 63;
    const float v = tm[r * CS + i] * bt[i];
    tm[r * CS + i] = v;
    am[r * CS + i] = v * expf(lg[i]);
  }
  __syncthreads();
  const int rg = tid >> 5, lane = tid & 31;
  const int quads = (rows + 3) / 4;         // (rows past the sequence's end have beta = 0: their columns of Tm are zero)
  for (int c0 = 0; c0 < vdim; c0 += 32) {   // Wv: rows rg + 8 j, column c0 + lane
    const int col = c0 + lane;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const T* vsrc = qkv + (size_t)first * channels + 2 * kv_heads * dim + (size_t)h * vdim + col;
    for (int iq = 0; iq < quads; ++iq) {
      float v[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) v[b] = (col < vdim && 4 * iq + b < rows) ? to_float(vsrc[(size_t)(4 * iq + b) * channels]) : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 tv = *reinterpret_cast<const float4*>(tm + (rg + 8 * j) * CS + 4 * iq);
        acc[j] = fmaf(tv.x, v[0], fmaf(tv.y, v[1], fmaf(tv.z, v[2], fmaf(tv.w, v[3], acc[j]))));
      }
    }
    if (col < vdim)
#pragma unroll
      for (int j = 0; j < 8; ++j) wv[(slot + rg + 8 * j) * vdim + col] = acc[j];
  }
  for (int c0 = 0; c0 < dim; c0 += 32) {    // Wk
    const int col = c0 + lane;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int iq = 0; iq < quads; ++iq) {
      float v[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) v[b] = col < dim ? ks[(4 * iq + b) * DS + col] : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 tv = *reinterpret_cast<const float4*>(am + (rg + 8 * j) * CS + 4 * iq);
        acc[j] = fmaf(tv.x, v[0], fmaf(tv.y, v[1], fmaf(tv.z, v[2], fmaf(tv.w, v[3], acc[j]))));
      }
    }
    if (col < dim)
#pragma unroll
      for (int j = 0; j < 8; ++j) wk[(slot + rg + 8 * j) * dim + col] = acc[j];
  }
}

// TILE value columns a block (32, or 16 where that is what fills the chip); 256 threads = 256 / TILE groups of rows.
// Rows of the tiles are padded by four values so that two neighbouring rows, read by the two halves of a warp at
// TILE = 16, lie in different banks.
template <int TILE>
__global__ void __launch_bounds__(256)
delta_chunk_scan_kernel(const float* __restrict__ qk, const float* __restrict__ wv, const float* __restrict__ wk,
                        const float* __restrict__ pm, const float* __restrict__ lgc, float* __restrict__ state,
                        float* __restrict__ out, const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                        const int* __restrict__ cu_new, int n_seq, int heads, int kv_heads, int dim, int vdim) {
  constexpr int NRG = 256 / TILE;          // groups of rows
  constexpr int RPT = kChunk / NRG;        // rows of a chunk a thread
  constexpr int PS = kChunk + 4;           // row stride of P
  extern __shared__ __align__(16) float sm[];
  const int DP = dim + 4;                   // row stride of the tiles Wk, Q, K
  float* wks = sm;                          // [64][dim + 4]
  float* qs = wks + kChunk * DP;            // [64][dim + 4]
  float* ks = qs + kChunk * DP;             // [64][dim + 4]
  float* ps = ks + kChunk * DP;             // [64][68]
  float* us = ps + kChunk * PS;             // [64][TILE]: Wv's columns, then U
  float* ss = us + kChunk * TILE;           // [dim][TILE]: the state's columns
  float* lg = ss + dim * TILE;              // [64] L_t
  float* wj = lg + kChunk;                  // [64] e^(L_end - L_t)
  const int s = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * TILE;
  const int tid = threadIdx.x, cl = tid % TILE, rg = tid / TILE;
  const int col = c0 + cl;
  const bool live = col < vdim;
  const int t0 = cu_new[s], n = cu_new[s + 1] - t0;
  const int slot = seq_slot[s];
  const int inner = heads * vdim;
  if (slot < 0) {
    if (live)
      for (int i = rg; i < n; i += NRG) out[(size_t)(t0 + i) * inner + (size_t)h * vdim + col] = 0.f;
    return;
  }
  const int kh = h / (heads / kv_heads), qk_row = 2 * kv_heads * dim;
  float* st = state + ((size_t)slot * heads + h) * dim * vdim;
  const bool carried = seq_start[s] > 0;
  for (int d = rg; d < dim; d += NRG) ss[d * TILE + cl] = (live && carried) ? st[(size_t)d * vdim + col] : 0.f;
  const int base = chunk_slot(cu_new, s, 0);
  const int n_chunks = (n + kChunk - 1) / kChunk;
  const int per = (dim + 4 * NRG - 1) / (4 * NRG) * 4;   // rows of the state a thread updates: NRG runs cover dim
  const int vecs = dim / 4;
  for (int c = 0; c < n_chunks; ++c) {
    const int rows = min(kChunk, n - c * kChunk), first = t0 + c * kChunk;
    const size_t cs = ((size_t)(base + c) * heads + h) * kChunk;
    __syncthreads();   // the chunk before is done with the tiles
    // the chunk's tiles by 16-byte asynchronous copies, all in flight together
    for (int e = tid; e < kChunk * vecs; e += 256) {
      const int r = e / vecs, d = (e % vecs) * 4;
      copy16(wks + r * DP + d, wk + (cs + r) * dim + d);
      const float* src = qk + (size_t)(first + r) * qk_row;
      if (r < rows) {
        copy16(qs + r * DP + d, src + (size_t)kh * dim + d);
        copy16(ks + r * DP + d, src + (size_t)(kv_heads + kh) * dim + d);
      } else {
        *reinterpret_cast<float4*>(qs + r * DP + d) = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4*>(ks + r * DP + d) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    for (int e = tid; e < kChunk * (kChunk / 4); e += 256) {
      const int r = e / (kChunk / 4), i = (e % (kChunk / 4)) * 4;
      copy16(ps + r * PS + i, pm + (cs + r) * kChunk + i);
    }
    if (vdim % 4 == 0 && c0 + TILE <= vdim) {
      for (int e = tid * 4; e < kChunk * TILE; e += 1024) copy16(us + e, wv + (cs + e / TILE) * vdim + c0 + e % TILE);
    } else {
      for (int r = rg; r < kChunk; r += NRG) us[r * TILE + cl] = live ? wv[(cs + r) * vdim + col] : 0.f;
    }
    copies_wait();
    if (tid < kChunk) lg[tid] = lgc[cs + tid];
    __syncthreads();
    if (tid < kChunk) wj[tid] = tid < rows ? expf(lg[kChunk - 1] - lg[tid]) : 0.f;
    // U = Wv - Wk S0 and Q S0 for rows rg + NRG j
    float au[RPT], aq[RPT];
#pragma unroll
    for (int j = 0; j < RPT; ++j) au[j] = aq[j] = 0.f;
    for (int d = 0; d < dim; d += 4) {
      const float s0 = ss[d * TILE + cl], s1 = ss[(d + 1) * TILE + cl], s2 = ss[(d + 2) * TILE + cl], s3 = ss[(d + 3) * TILE + cl];
#pragma unroll
      for (int j = 0; j < RPT; ++j) {
        const float4 w = *reinterpret_cast<const float4*>(wks + (rg + NRG * j) * DP + d);
        const float4 qv = *reinterpret_cast<const float4*>(qs + (rg + NRG * j) * DP + d);
        au[j] = fmaf(w.x, s0, fmaf(w.y, s1, fmaf(w.z, s2, fmaf(w.w, s3, au[j]))));
        aq[j] = fmaf(qv.x, s0, fmaf(qv.y, s1, fmaf(qv.z, s2, fmaf(qv.w, s3, aq[j]))));
      }
    }
#pragma unroll
    for (int j = 0; j < RPT; ++j) us[(rg + NRG * j) * TILE + cl] -= au[j];
    __syncthreads();
    // O = e^L (Q S0) + P U (P is zero above its diagonal)
    float o[RPT];
#pragma unroll
    for (int j = 0; j < RPT; ++j) o[j] = expf(lg[rg + NRG * j]) * aq[j];
    for (int i = 0; i < kChunk; i += 4) {
      const float u0 = us[i * TILE + cl], u1 = us[(i + 1) * TILE + cl], u2 = us[(i + 2) * TILE + cl], u3 = us[(i + 3) * TILE + cl];
#pragma unroll
      for (int j = 0; j < RPT; ++j) {
        const float4 pv = *reinterpret_cast<const float4*>(ps + (rg + NRG * j) * PS + i);
        o[j] = fmaf(pv.x, u0, fmaf(pv.y, u1, fmaf(pv.z, u2, fmaf(pv.w, u3, o[j]))));
      }
    }
#pragma unroll
    for (int j = 0; j < RPT; ++j) {
      const int r = rg + NRG * j;
      if (live && r < rows) out[(size_t)(first + r) * inner + (size_t)h * vdim + col] = o[j];
    }
    // S <- e^(L_end) S0 + sum_i e^(L_end - L_i) k_i u_i^T: a thread keeps a run of the state's rows of its column
    // (every thread read the state's old columns before the barrier above; a thread writes only what it owns)
    {
      const float tail = expf(lg[kChunk - 1]);
      const int d0 = rg * per;
      float acc[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] = (j < per && d0 + j < dim) ? tail * ss[(d0 + j) * TILE + cl] : 0.f;
      for (int i = 0; i < rows; ++i) {
        const float u = wj[i] * us[i * TILE + cl];
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
          if (4 * j4 < per && d0 + 4 * j4 < dim) {
            const float4 kv = *reinterpret_cast<const float4*>(ks + i * DP + d0 + 4 * j4);
            acc[4 * j4] = fmaf(kv.x, u, acc[4 * j4]);
            acc[4 * j4 + 1] = fmaf(kv.y, u, acc[4 * j4 + 1]);
            acc[4 * j4 + 2] = fmaf(kv.z, u, acc[4 * j4 + 2]);
            acc[4 * j4 + 3] = fmaf(kv.w, u, acc[4 * j4 + 3]);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (j < per && d0 + j < dim) ss[(d0 + j) * TILE + cl] = acc[j];
    }
  }
  __syncthreads();
  if (live)
    for (int d = rg; d < dim; d += NRG) st[(size_t)d * vdim + col] = ss[d * TILE + cl];
}

template <typename T>
int delta_rule_run(const T* qkv, const T* proj, long long proj_stride, int b_col, int a_col, const float* a_log,
                   const float* dt_bias, float* state, float* out, float* scratch, const int* seq_slot, const int* seq_start,
                   const int* cu_new, int T_tokens, int n_seq, int heads, int kv_heads, int dim, int vdim, float unit_eps,
                   int max_new, int chunk_slots, cudaStream_t stream) {
  const int channels = 2 * kv_heads * dim + heads * vdim;
  float* qk = scratch;                                                       // (every part starts on 16 bytes)
  float* beta = qk + align4((size_t)T_tokens * 2 * kv_heads * dim);
  float* decay = beta + align4((size_t)T_tokens * heads);
  float* log_decay = decay + align4((size_t)T_tokens * heads);
  delta_prepare_kernel<T><<<T_tokens, 128, 0, stream>>>(qkv, proj, proj_stride, b_col, a_col, a_log, dt_bias, qk, beta, decay,
                                                        log_decay, heads, kv_heads, dim, channels, unit_eps);
  EMBER_LAUNCH_OK("delta_prepare");
  if (chunk_slots > 0) {
    const int max_chunks = (max_new + kChunk - 1) / kChunk;
    float* wv = log_decay + align4((size_t)T_tokens * heads);               // [chunk slots][heads][64][vdim]
    float* wk = wv + (size_t)chunk_slots * heads * kChunk * vdim;           // [chunk slots][heads][64][dim]
    float* pm = wk + (size_t)chunk_slots * heads * kChunk * dim;            // [chunk slots][heads][64][64]
    float* lgc = pm + (size_t)chunk_slots * heads * kChunk * kChunk;        // [chunk slots][heads][64]: the sums of logarithms
    const size_t smem1 = (size_t)(2 * kChunk * (dim + 1) + 4 + 2 * kChunk * (kChunk + 4) + 3 * kChunk) * sizeof(float);
    // 16 value columns a block where blocks of 32 would leave SMs without one
    const int tile = (long long)n_seq * heads * ((vdim + 31) / 32) < sm_count() ? 16 : 32;
    const size_t smem2 = (size_t)(3 * kChunk * (dim + 4) + kChunk * (kChunk + 4) + kChunk * tile + dim * tile + 2 * kChunk) * sizeof(float);
    static bool raised[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!raised[dev & 63]) {
      if (cudaFuncSetAttribute(delta_chunk_factor_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess ||
          cudaFuncSetAttribute(delta_chunk_scan_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
          cudaFuncSetAttribute(delta_chunk_scan_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
        return ember_fail("delta_rule: the chunk kernels' shared memory could not be raised");
      raised[dev & 63] = true;
    }
    delta_chunk_factor_kernel<T><<<dim3(n_seq * max_chunks, heads), 256, smem1, stream>>>(
        qk, qkv, beta, log_decay, wv, wk, pm, lgc, seq_slot, cu_new, n_seq, max_chunks, heads, kv_heads, dim, vdim, channels);
    EMBER_LAUNCH_OK("delta_chunk_factor");
    if (tile == 16)
      delta_chunk_scan_kernel<16><<<dim3(n_seq, heads, (vdim + 15) / 16), 256, smem2, stream>>>(
          qk, wv, wk, pm, lgc, state, out, seq_slot, seq_start, cu_new, n_seq, heads, kv_heads, dim, vdim);
    else
      delta_chunk_scan_kernel<32><<<dim3(n_seq, heads, (vdim + 31) / 32), 256, smem2, stream>>>(
          qk, wv, wk, pm, lgc, state, out, seq_slot, seq_start, cu_new, n_seq, heads, kv_heads, dim, vdim);
    EMBER_LAUNCH_OK("delta_chunk_scan");
    return 0;
  }
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
// chunk_slots > 0 (the chunked form): room for that many chunks of 64 tokens more (see delta_rule_run)
EMBER_API size_t ember_delta_rule_scratch(int T, int heads, int kv_heads, int dim, int vdim, int chunk_slots) {
  return align4((size_t)T * 2 * kv_heads * dim) + 3 * align4((size_t)T * heads) +
         (size_t)chunk_slots * heads * kChunk * ((size_t)vdim + dim + kChunk + 1);
}

// qkv [T, q | k | v] (the convolution's output), b and a: `heads` columns each from b_col and a_col of `proj`;
// state float32 [slots, heads, dim, vdim] (advanced); out float32 [T, heads * vdim].
EMBER_API int ember_delta_rule(const void* qkv, const void* proj, long long proj_stride, int b_col, int a_col,
                               const float* a_log, const float* dt_bias, float* state, float* out, float* scratch,
                               const int* seq_slot, const int* seq_start, const int* cu_new, int T, int n_seq, int heads,
                               int kv_heads, int dim, int vdim, float unit_eps, int max_new, int chunk_slots, int dtype,
                               cudaStream_t stream) {
  EMBER_CHECK(chunk_slots == 0 || (dim % 4 == 0 && dim <= 128 && max_new > 0), "delta_rule: the chunked form takes key sizes "
              "that are multiples of 4 up to 128 (here %d)", dim);
  EMBER_CHECK(T > 0 && n_seq > 0 && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0, "delta_rule: bad sizes");
  EMBER_CHECK(heads % kv_heads == 0, "delta_rule: %d heads are not a multiple of %d key heads", heads, kv_heads);
  EMBER_CHECK(heads <= 65535, "delta_rule: %d heads exceed one launch", heads);
  if (dtype == EMBER_F32)
    return delta_rule_run<float>((const float*)qkv, (const float*)proj, proj_stride, b_col, a_col, a_log, dt_bias, state, out,
                                 scratch, seq_slot, seq_start, cu_new, T, n_seq, heads, kv_heads, dim, vdim, unit_eps, max_new, chunk_slots, stream);
  if (dtype == EMBER_BF16)
    return delta_rule_run<__nv_bfloat16>((const __nv_bfloat16*)qkv, (const __nv_bfloat16*)proj, proj_stride, b_col, a_col,
                                         a_log, dt_bias, state, out, scratch, seq_slot, seq_start, cu_new, T, n_seq, heads,
                                         kv_heads, dim, vdim, unit_eps, max_new, chunk_slots, stream);
  return ember_fail("delta_rule: element type %d", dtype);
}
