// RMS norm, the norm of a weighted sum added to the stream, and the gates of the gated layers.
//
// Everything here is float32 arithmetic on rows: statistics, sums and products are float32 whatever
// the element type of the rows that go in or come out.  A row is summed by one block in an order
// that depends on its length alone, so a row's result does not depend on the batch it is in.  The kernels are
// launched the ordinary way.  Programmatic dependent launch was tried for all the small kernels of this file, of
// ssm.cu, moe.cu and attention_decode_kept.cu and lost: a one-token step of four layers took 0.757 ms with ordinary
// launches, 0.865 ms with every kernel waiting for the one in front and releasing its follower at once, and 0.903 ms
// with the wait alone.  Several of these kernels run in more than one wave of blocks, and blocks that sit on the SMs
// waiting take the room of the waves that should run.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxBranches = 16;

// Sum over the block; every thread gets it, added in warp order.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float total = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) total += red[i];
  return total;
}

__device__ __forceinline__ float sigmoidf(float v) { return 1.0f / (1.0f + expf(-v)); }

// out = x / sqrt(mean(x^2) + eps) * (offset + w)
template <typename TOUT>
__global__ void __launch_bounds__(kThreads)
rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, TOUT* __restrict__ out, int d, float eps,
               float offset) {
  __shared__ float red[kThreads / 32];
  const float* row = x + (size_t)blockIdx.x * d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += kThreads) {
    const float v = row[i];
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
  TOUT* o = out + (size_t)blockIdx.x * d;
  for (int i = threadIdx.x; i < d; i += kThreads) o[i] = from_float<TOUT>(row[i] * inv * (offset + w[i]));
}

struct Branches {
  const float* rows[kMaxBranches];
  long long stride[kMaxBranches];  // elements between two rows
  float factor[kMaxBranches];
  int n;
};

__device__ __forceinline__ float weighted(const Branches& b, size_t row, int i) {
  float s = 0.f;
  for (int k = 0; k < b.n; ++k) s = fmaf(b.factor[k], b.rows[k][row * (size_t)b.stride[k] + i], s);
  return s;
}

// x += norm(sum_k factor_k * rows_k): the sum is made twice (once for the statistics, once for the
// result) in the same order, so nothing is kept between the passes.
__global__ void __launch_bounds__(kThreads)
add_normed_kernel(float* __restrict__ x, const Branches b, const float* __restrict__ w, int d, float eps, float offset) {
  __shared__ float red[kThreads / 32];
  const size_t row = blockIdx.x;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += kThreads) {
    const float v = weighted(b, row, i);
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
  float* o = x + row * d;
  for (int i = threadIdx.x; i < d; i += kThreads) o[i] += weighted(b, row, i) * inv * (offset + w[i]);
}

// rows of [gate | up] (n each) -> act(gate) * up
//   kind 0: g * sigmoid(g) * u
//   kind 1: g = min(g, limit), u = clamp(u, -limit, limit): g * sigmoid(alpha * g) * (u + shift)
template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gu, T* __restrict__ out, size_t total, int n, int kind,
                                 float limit, float alpha, float shift) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / n;
    const int c = (int)(i % n);
    float g = to_float(gu[row * 2 * n + c]), u = to_float(gu[row * 2 * n + n + c]);
    float y;
    if (kind == 0) {
      y = g * sigmoidf(g) * u;
    } else {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
      y = g * sigmoidf(alpha * g) * (u + shift);
    }
    out[i] = from_float<T>(y);
  }
}

// out = unit(y * silu(z)) * w, the root mean square taken over each of `parts` equal pieces of a row.
// y float32 [T, n]; z: n columns of a wider matrix (row stride z_stride).  grid (T, parts).
template <typename T>
__global__ void __launch_bounds__(kThreads)
gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ z, long long z_stride,
                        const float* __restrict__ w, T* __restrict__ out, int n, int part, float eps) {
  __shared__ float red[kThreads / 32];
  const size_t t = blockIdx.x;
  const int c0 = blockIdx.y * part;
  const float* yr = y + t * n + c0;
  const T* zr = z + t * (size_t)z_stride + c0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < part; i += kThreads) {
    const float zv = to_float(zr[i]);
    const float v = yr[i] * (zv * sigmoidf(zv));
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)part + eps);
  T* o = out + t * n + c0;
  for (int i = threadIdx.x; i < part; i += kThreads) {
    const float zv = to_float(zr[i]);
    o[i] = from_float<T>(yr[i] * (zv * sigmoidf(zv)) * inv * w[c0 + i]);
  }
}

}  // namespace

EMBER_API int ember_rmsnorm(const float* x, const float* w, void* out, int rows, int d, float eps, float offset,
                            int out_dtype, cudaStream_t stream) {
  EMBER_CHECK(rows > 0 && d > 0, "rmsnorm: %d rows of %d", rows, d);
  cudaError_t e;
  if (out_dtype == EMBER_F32)
    e = launch_plain(rmsnorm_kernel<float>, dim3(rows), dim3(kThreads), 0, stream, x, w, (float*)out, d, eps, offset);
  else if (out_dtype == EMBER_BF16)
    e = launch_plain(rmsnorm_kernel<__nv_bfloat16>, dim3(rows), dim3(kThreads), 0, stream, x, w, (__nv_bfloat16*)out, d, eps, offset);
  else
    return ember_fail("rmsnorm: element type %d", out_dtype);
  if (e != cudaSuccess) return ember_fail("rmsnorm: %s", cudaGetErrorString(e));
  return 0;
}

// rows[k], strides[k] (elements), factors[k] for k < n_branches (host arrays)
EMBER_API int ember_add_normed(float* x, const void* const* rows, const long long* strides, const float* factors,
                               int n_branches, const float* w, int n_rows, int d, float eps, float offset,
                               cudaStream_t stream) {
  EMBER_CHECK(n_rows > 0 && d > 0, "add_normed: %d rows of %d", n_rows, d);
  EMBER_CHECK(n_branches >= 1 && n_branches <= kMaxBranches, "add_normed: %d branches (1 to %d)", n_branches, kMaxBranches);
  Branches b;
  b.n = n_branches;
  for (int k = 0; k < n_branches; ++k) {
    b.rows[k] = (const float*)rows[k];
    b.stride[k] = strides[k];
    b.factor[k] = factors[k];
  }
  const cudaError_t e = launch_plain(add_normed_kernel, dim3(n_rows), dim3(kThreads), 0, stream, x, b, w, d, eps, offset);
  if (e != cudaSuccess) return ember_fail("add_normed: %s", cudaGetErrorString(e));
  return 0;
}

EMBER_API int ember_gated_act(const void* gu, void* out, int rows, int n, int kind, float limit, float alpha, float shift,
                              int dtype, cudaStream_t stream) {
  EMBER_CHECK(rows > 0 && n > 0 && (kind == 0 || kind == 1), "gated_act: %d rows of %d, kind %d", rows, n, kind);
  const size_t total = (size_t)rows * n;
  const int grid = (int)((total + 255) / 256 < 65535 * 16 ? (total + 255) / 256 : 65535 * 16);
  cudaError_t e;
  if (dtype == EMBER_F32)
    e = launch_plain(gated_act_kernel<float>, dim3(grid), dim3(256), 0, stream, (const float*)gu, (float*)out, total, n, kind,
                   limit, alpha, shift);
  else if (dtype == EMBER_BF16)
    e = launch_plain(gated_act_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, (const __nv_bfloat16*)gu,
                   (__nv_bfloat16*)out, total, n, kind, limit, alpha, shift);
  else
    return ember_fail("gated_act: element type %d", dtype);
  if (e != cudaSuccess) return ember_fail("gated_act: %s", cudaGetErrorString(e));
  return 0;
}

EMBER_API int ember_gated_group_norm(const float* y, const void* z, long long z_stride, const float* w, void* out, int rows,
                                     int n, int parts, float eps, int dtype, cudaStream_t stream) {
  EMBER_CHECK(rows > 0 && n > 0 && parts > 0 && n % parts == 0, "gated_group_norm: %d rows of %d in %d parts", rows, n, parts);
  EMBER_CHECK(parts <= 65535, "gated_group_norm: %d parts exceed one launch", parts);
  const dim3 grid(rows, parts);
  cudaError_t e;
  if (dtype == EMBER_F32)
    e = launch_plain(gated_group_norm_kernel<float>, grid, dim3(kThreads), 0, stream, y, (const float*)z, z_stride, w,
                   (float*)out, n, n / parts, eps);
  else if (dtype == EMBER_BF16)
    e = launch_plain(gated_group_norm_kernel<__nv_bfloat16>, grid, dim3(kThreads), 0, stream, y, (const __nv_bfloat16*)z,
                   z_stride, w, (__nv_bfloat16*)out, n, n / parts, eps);
  else
    return ember_fail("gated_group_norm: element type %d", dtype);
  if (e != cudaSuccess) return ember_fail("gated_group_norm: %s", cudaGetErrorString(e));
  return 0;
}
