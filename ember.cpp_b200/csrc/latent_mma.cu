// Attention over cached low-rank rows on the tensor cores (bfloat16, mma.sync m16n8k16).
//
// All heads of a token share the cached rows, so the rows of the product are (token, head) pairs: a
// sequence's new tokens times its heads, token-major, 16 to 64 of them a block.  A block walks the
// pages of 64 positions that its rows can see; a page's rows c | k_r (rank + rot values a key) come into
// shared memory once for all the block's rows, the block's query rows stay there from the start.
// Two warps share a group of 16 rows: each makes the group's scores S = Q K^T for half of the page's
// keys; they tell each other their rows' maxima and hand each other their probabilities (bfloat16)
// through shared memory, meeting at a barrier of their own, and each adds P C for all 64 keys to its own
// half of the output's `rank` columns, which stays in registers (up to 128 float32 values a thread).
// Keys past a row's own position are masked by selection; float32 softmax in base 2.
//
// One token a sequence (a decode step): the pages are cut into chunks, a block a chunk (grid z); blocks
// leave unnormalised sums with their maximum and total, and `latent_merge` combines them.  Otherwise
// (prompts, portions) a block sees all its pages and writes the output itself.
//
// Sizes: rank a multiple of 32 up to 512, rot a multiple of 16; others take the plain kernel.
#include "common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void ldsm_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(a), "l"(src));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory"); }
__device__ __forceinline__ unsigned pack2(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const unsigned*>(&v);
}

constexpr int kKeys = 64;   // keys a tile: one page
constexpr int kPS = kKeys + 8;   // row stride of the probabilities in shared memory (rows 16 bytes apart in banks)

// The two warps of a group of rows meet (barrier 1 + group; barrier 0 is the block's).
__device__ __forceinline__ void pair_sync(int g) { asm volatile("bar.sync %0, 64;\n" ::"r"(1 + g) : "memory"); }

// grid (row tiles, sequences, chunks); blockDim.x = 64 * G for G groups of 16 rows.
template <int RMAX>
__global__ void __launch_bounds__(256, 1)
latent_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc, const bf16* __restrict__ vc, bf16* __restrict__ out,
                  float* __restrict__ part_o, float* __restrict__ part_ml, const int* __restrict__ seq_slot,
                  const int* __restrict__ seq_start, const int* __restrict__ cu_new, const int* __restrict__ pages,
                  int max_blocks, int heads, int rank, int rot, float scale_log2, int ppc, int n_chunks) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int W = rank + rot, WS = W + 8, vecs = W / 8;
  const int G = blockDim.x >> 6;
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);   // [16 G][WS]
  bf16* ks = qs + (size_t)16 * G * WS;            // [64][WS]
  bf16* pb = ks + (size_t)kKeys * WS;             // [G][16][kPS]: a group's probabilities of the page
  float* xb = reinterpret_cast<float*>(pb + (size_t)G * 16 * kPS);   // [G][2][16]: what the two warps of a group tell each other
  const int s = blockIdx.y, chunk = blockIdx.z;
  const int t0 = cu_new[s], n_new = cu_new[s + 1] - t0;
  const int R = n_new * heads, r0 = blockIdx.x * 16 * G;
  if (r0 >= R) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = warp >> 1, half = warp & 1;
  const size_t row_base = (size_t)t0 * heads;
  const int ra = r0 + g * 16 + (lane >> 2), rb = ra + 8;   // this thread's two rows
  const int NP = rank / 16;                                // pairs of 8-column tiles of the output
  const int np_begin = half ? (NP + 1) / 2 : 0, np_count = half ? NP / 2 : (NP + 1) / 2;
  const int slot = seq_slot[s];
  const int start = seq_start[s];
  const int p_max = start + (min(R, r0 + 16 * G) - 1) / heads;
  const int pg0 = chunk * ppc, pg1 = min(pg0 + ppc, p_max / kPage + 1);
  if (slot < 0 || pg0 >= pg1) {   // padding, or a chunk past this block's rows: nothing to add
    if (n_chunks == 1) {
      for (int i = threadIdx.x; i < 16 * G * rank; i += blockDim.x) {
        const int r = r0 + i / rank;
        if (r < R) out[(row_base + r) * rank + i % rank] = __float2bfloat16_rn(0.f);
      }
    } else if (half == 0 && (lane & 3) == 0) {
      if (ra < R) { part_ml[((row_base + ra) * n_chunks + chunk) * 2] = -INFINITY; part_ml[((row_base + ra) * n_chunks + chunk) * 2 + 1] = 0.f; }
      if (rb < R) { part_ml[((row_base + rb) * n_chunks + chunk) * 2] = -INFINITY; part_ml[((row_base + rb) * n_chunks + chunk) * 2 + 1] = 0.f; }
    }
    return;
  }
  // the block's query rows
  for (int i = threadIdx.x; i < 16 * G * vecs; i += blockDim.x) {
    const int row = i / vecs, v = i % vecs, r = r0 + row;
    if (r < R)
      cp_async16(qs + (size_t)row * WS + v * 8, q + (row_base + r) * W + v * 8);
    else
      *reinterpret_cast<uint4*>(qs + (size_t)row * WS + v * 8) = make_uint4(0, 0, 0, 0);
  }
  const int pa_row = start + ra / heads, pb_row = start + rb / heads;   // the rows' own positions
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  float o_acc[RMAX / 16][4];
#pragma unroll
  for (int i = 0; i < RMAX / 16; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;

  for (int pg = pg0; pg < pg1; ++pg) {
    const int page = pages[(size_t)s * max_blocks + pg];
    for (int i = threadIdx.x; i < kKeys * vecs; i += blockDim.x) {
      const int key = i / vecs, col = (i % vecs) * 8;
      bf16* dst = ks + (size_t)key * WS + col;
      if (page >= 0)
        cp_async16(dst, col < rank ? kc + ((size_t)page * kPage + key) * rank + col
                                   : vc + ((size_t)page * kPage + key) * rot + (col - rank));
      else
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    cp_async_wait_all();
    __syncthreads();

    float sa[4][4];   // this warp's half of the page's keys: 32 keys from 32 * half
#pragma unroll
    for (int i = 0; i < 4; ++i) sa[i][0] = sa[i][1] = sa[i][2] = sa[i][3] = 0.f;
    for (int k0 = 0; k0 < W; k0 += 16) {
      unsigned a[4];
      ldsm_x4(a[0], a[1], a[2], a[3], qs + (size_t)(g * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * WS + k0 + 8 * (lane >> 4));
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        unsigned b0, b1, b2, b3;
        ldsm_x4(b0, b1, b2, b3, ks + (size_t)(half * 32 + np * 16 + (lane & 7) + 8 * (lane >> 4)) * WS + k0 + 8 * ((lane >> 3) & 1));
        mma_bf16(sa[2 * np], a, b0, b1);
        mma_bf16(sa[2 * np + 1], a, b2, b3);
      }
    }
    // scores in base 2, keys past a row's own position masked by selection
    float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = pg * kPage + half * 32 + nt * 8 + 2 * (lane & 3) + (e & 1);
        const bool top = e < 2;
        const bool seen = page >= 0 && (top ? (ra < R && j <= pa_row) : (rb < R && j <= pb_row));
        const float v = seen ? sa[nt][e] * scale_log2 : -INFINITY;
        sa[nt][e] = v;
        if (top) mx_a = fmaxf(mx_a, v); else mx_b = fmaxf(mx_b, v);
      }
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    float* mine = xb + (size_t)(g * 2 + half) * 16;
    const float* theirs = xb + (size_t)(g * 2 + (half ^ 1)) * 16;
    if ((lane & 3) == 0) {
      mine[lane >> 2] = mx_a;
      mine[(lane >> 2) + 8] = mx_b;
    }
    pair_sync(g);
    const float mn_a = fmaxf(m_a, fmaxf(mx_a, theirs[lane >> 2])), mn_b = fmaxf(m_b, fmaxf(mx_b, theirs[(lane >> 2) + 8]));
    const float corr_a = mn_a == -INFINITY ? 1.f : exp2f(m_a - mn_a), corr_b = mn_b == -INFINITY ? 1.f : exp2f(m_b - mn_b);
    float sum_a = 0.f, sum_b = 0.f;
    bf16* prow_a = pb + (size_t)(g * 16 + (lane >> 2)) * kPS + half * 32 + 2 * (lane & 3);
    bf16* prow_b = prow_a + 8 * kPS;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const float p0 = mn_a == -INFINITY ? 0.f : exp2f(sa[nt][0] - mn_a), p1 = mn_a == -INFINITY ? 0.f : exp2f(sa[nt][1] - mn_a);
      const float p2 = mn_b == -INFINITY ? 0.f : exp2f(sa[nt][2] - mn_b), p3 = mn_b == -INFINITY ? 0.f : exp2f(sa[nt][3] - mn_b);
      sum_a += p0 + p1;
      sum_b += p2 + p3;
      *reinterpret_cast<unsigned*>(prow_a + nt * 8) = pack2(p0, p1);
      *reinterpret_cast<unsigned*>(prow_b + nt * 8) = pack2(p2, p3);
    }
    l_a = l_a * corr_a + sum_a;   // (this warp's keys; the two warps' totals are added at the end)
    l_b = l_b * corr_b + sum_b;
    m_a = mn_a;
    m_b = mn_b;
    pair_sync(g);                 // the group's probabilities of all 64 keys are in place
    unsigned pf[4][4];   // the probabilities as the left operand of P C, 16 keys a step
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      ldsm_x4(pf[kk][0], pf[kk][1], pf[kk][2], pf[kk][3],
              pb + (size_t)(g * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * kPS + kk * 16 + 8 * (lane >> 4));
#pragma unroll
    for (int i = 0; i < RMAX / 32; ++i) {
      if (i < np_count) {
        o_acc[2 * i][0] *= corr_a; o_acc[2 * i][1] *= corr_a; o_acc[2 * i][2] *= corr_b; o_acc[2 * i][3] *= corr_b;
        o_acc[2 * i + 1][0] *= corr_a; o_acc[2 * i + 1][1] *= corr_a; o_acc[2 * i + 1][2] *= corr_b; o_acc[2 * i + 1][3] *= corr_b;
        const int dim0 = (np_begin + i) * 16;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          unsigned b0, b1, b2, b3;
          ldsm_x4_t(b0, b1, b2, b3, ks + (size_t)(kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * WS + dim0 + 8 * (lane >> 4));
          mma_bf16(o_acc[2 * i], pf[kk], b0, b1);
          mma_bf16(o_acc[2 * i + 1], pf[kk], b2, b3);
        }
      }
    }
    __syncthreads();   // the tile is free for the next page
  }
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  {   // the row's total is the two warps' together (both have scaled theirs by the same corrections)
    float* mine = xb + (size_t)(g * 2 + half) * 16;
    const float* theirs = xb + (size_t)(g * 2 + (half ^ 1)) * 16;
    if ((lane & 3) == 0) {
      mine[lane >> 2] = l_a;
      mine[(lane >> 2) + 8] = l_b;
    }
    pair_sync(g);
    l_a += theirs[lane >> 2];
    l_b += theirs[(lane >> 2) + 8];
  }
  if (n_chunks == 1) {
    const float inv_a = l_a > 0.f ? 1.0f / l_a : 0.f, inv_b = l_b > 0.f ? 1.0f / l_b : 0.f;
#pragma unroll
    for (int i = 0; i < RMAX / 32; ++i) {
      if (i < np_count) {
#pragma unroll
        for (int tt = 0; tt < 2; ++tt) {
          const int col = (np_begin + i) * 16 + tt * 8 + 2 * (lane & 3);
          if (ra < R)
            *reinterpret_cast<__nv_bfloat162*>(out + (row_base + ra) * rank + col) =
                __floats2bfloat162_rn(o_acc[2 * i + tt][0] * inv_a, o_acc[2 * i + tt][1] * inv_a);
          if (rb < R)
            *reinterpret_cast<__nv_bfloat162*>(out + (row_base + rb) * rank + col) =
                __floats2bfloat162_rn(o_acc[2 * i + tt][2] * inv_b, o_acc[2 * i + tt][3] * inv_b);
        }
      }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < RMAX / 32; ++i) {
    if (i < np_count) {
#pragma unroll
      for (int tt = 0; tt < 2; ++tt) {
        const int col = (np_begin + i) * 16 + tt * 8 + 2 * (lane & 3);
        if (ra < R)
          *reinterpret_cast<float2*>(part_o + ((row_base + ra) * n_chunks + chunk) * rank + col) =
              make_float2(o_acc[2 * i + tt][0], o_acc[2 * i + tt][1]);
        if (rb < R)
          *reinterpret_cast<float2*>(part_o + ((row_base + rb) * n_chunks + chunk) * rank + col) =
              make_float2(o_acc[2 * i + tt][2], o_acc[2 * i + tt][3]);
      }
    }
  }
  if (half == 0 && (lane & 3) == 0) {
    if (ra < R) { part_ml[((row_base + ra) * n_chunks + chunk) * 2] = m_a; part_ml[((row_base + ra) * n_chunks + chunk) * 2 + 1] = l_a; }
    if (rb < R) { part_ml[((row_base + rb) * n_chunks + chunk) * 2] = m_b; part_ml[((row_base + rb) * n_chunks + chunk) * 2 + 1] = l_b; }
  }
}

// grid (rows): the chunks' sums of one (token, head) row, in chunk order.
__global__ void latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                                    int rank, int n_chunks) {
  const size_t row = blockIdx.x;
  const float* ml = part_ml + row * n_chunks * 2;
  float M = -INFINITY;
  for (int c = 0; c < n_chunks; ++c)
    if (ml[2 * c + 1] > 0.f) M = fmaxf(M, ml[2 * c]);
  float L = 0.f;
  for (int c = 0; c < n_chunks; ++c)
    if (ml[2 * c + 1] > 0.f) L += ml[2 * c + 1] * exp2f(ml[2 * c] - M);
  const float inv = L > 0.f ? 1.0f / L : 0.f;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    float acc = 0.f;
    for (int c = 0; c < n_chunks; ++c)
      if (ml[2 * c + 1] > 0.f) acc = fmaf(part_o[(row * n_chunks + c) * rank + d], exp2f(ml[2 * c] - M), acc);
    out[row * rank + d] = __float2bfloat16_rn(acc * inv);
  }
}

}  // namespace

// floats of scratch for `rows` (token, head) rows cut into n_chunks: the partial sums, then (maximum, total) pairs
EMBER_API size_t ember_latent_attention_mma_scratch(int rows, int rank, int n_chunks) {
  return n_chunks <= 1 ? 0 : (size_t)rows * n_chunks * ((size_t)rank + 2);
}

// Returns 2 (and launches nothing) for sizes that this kernel has no form for.  q bfloat16 [T, heads * (rank + rot)],
// out bfloat16 [T, heads * rank]; n_chunks > 1 only with one token a sequence; scratch as the function above says.
EMBER_API int ember_latent_attention_mma(const void* q, const void* kc, const void* vc, void* out, float* scratch,
                                         const int* seq_slot, const int* seq_start, const int* cu_new, const int* pages,
                                         int max_blocks, int n_seq, int max_new, int T, int heads, int rank, int rot, float scale,
                                         int n_chunks, int pages_per_chunk, cudaStream_t stream) {
  EMBER_CHECK(n_seq > 0 && max_new > 0 && heads > 0 && max_blocks > 0 && n_chunks >= 1 && pages_per_chunk >= 1,
              "latent_attention_mma: bad sizes");
  if (rank % 32 != 0 || rank > 512 || rot % 16 != 0 || rot <= 0 || !(scale > 0.f)) return 2;
  EMBER_CHECK(n_chunks == 1 || max_new == 1, "latent_attention_mma: chunks are for steps of one token a sequence");
  const long long rows = (long long)max_new * heads;
  const int G = rows >= 64 ? 4 : (int)((rows + 15) / 16);
  const dim3 grid((unsigned)((rows + 16 * G - 1) / (16 * G)), n_seq, n_chunks);
  EMBER_CHECK(n_seq <= 65535 && n_chunks <= 65535, "latent_attention_mma: %d sequences in %d chunks exceed one launch", n_seq, n_chunks);
  const size_t smem = (size_t)(16 * G + kKeys) * (rank + rot + 8) * sizeof(bf16) + (size_t)G * 16 * kPS * sizeof(bf16) +
                      (size_t)G * 2 * 16 * sizeof(float);
  float* part_o = scratch;
  float* part_ml = scratch ? scratch + (size_t)T * heads * n_chunks * rank : nullptr;
  EMBER_CHECK(n_chunks == 1 || scratch != nullptr, "latent_attention_mma: chunks need scratch");
  const float scale_log2 = scale * 1.4426950408889634f;
#define EMBER_LATENT_MMA(RMAX)                                                                                            \
  do {                                                                                                                    \
    static bool raised[64] = {false};                                                                                     \
    int dev = 0;                                                                                                          \
    cudaGetDevice(&dev);                                                                                                  \
    if (smem > 48 * 1024 && !raised[dev & 63]) {                                                                          \
      if (cudaFuncSetAttribute(latent_mma_kernel<RMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) \
        return ember_fail("latent_attention_mma: the kernel's shared memory could not be raised");                       \
      raised[dev & 63] = true;                                                                                            \
    }                                                                                                                     \
    latent_mma_kernel<RMAX><<<grid, 64 * G, smem, stream>>>((const bf16*)q, (const bf16*)kc, (const bf16*)vc, (bf16*)out, part_o, \
                                                            part_ml, seq_slot, seq_start, cu_new, pages, max_blocks, heads, rank, \
                                                            rot, scale_log2, pages_per_chunk, n_chunks);                  \
  } while (0)
  if (smem > 200 * 1024) return 2;
  if (rank <= 128)
    EMBER_LATENT_MMA(128);
  else if (rank <= 256)
    EMBER_LATENT_MMA(256);
  else
    EMBER_LATENT_MMA(512);
#undef EMBER_LATENT_MMA
  EMBER_LAUNCH_OK("latent_attention_mma");
  if (n_chunks > 1) {
    latent_merge_kernel<<<(unsigned)((long long)T * heads), 128, 0, stream>>>(part_o, part_ml, (bf16*)out, rank, n_chunks);
    EMBER_LAUNCH_OK("latent_merge");
  }
  return 0;
}
