// Layer normalisation (weight, no bias) around the float32 residual stream, for layers that norm a sublayer's
// output before it is added ("sandwich" layers), and the re-entry of a looped span of layers.
// Each kernel has a float32 and a bfloat16 instantiation; all arithmetic is float32, sums in an order that
// depends on the row size and the block size only.
#include "common.cuh"

using namespace dli;

namespace {

// mean and 1 / sqrt(variance + eps) of row[0..H), the variance taken as the mean of the squared deviations
__device__ __forceinline__ void row_stats(const float* row, int H, float eps, float* red, float& mean, float& rstd) {
  float s = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) s += row[i];
  mean = block_sum(s, red) / (float)H;
  float q = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float d = row[i] - mean;
    q = fmaf(d, d, q);
  }
  rstd = 1.f / sqrtf(block_sum(q, red) / (float)H + eps);
}

// For output row r (source row s = rows ? rows[r] : r):
//   v = h[s] + (a ? LN(a[s]) * w_post : 0)     written back to h[s] when rows == nullptr
//   y[r] = LN(v) * w_pre                        when y != nullptr
// One block per row; the row lives in shared memory (H floats) between the passes.
template <typename T>
__global__ void post_add_layernorm_kernel(T* __restrict__ y, float* __restrict__ h, const T* __restrict__ a,
                                          const float* __restrict__ w_post, const float* __restrict__ w_pre,
                                          const int* __restrict__ rows, int H, float eps_post, float eps_pre) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row[];
  __shared__ float red[33];
  const int r = blockIdx.x;
  const int s = rows ? rows[r] : r;
  float* hrow = h + (size_t)s * H;
  if (a) {
    const T* arow = a + (size_t)s * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = to_float(arow[i]);
    float mean, rstd;
    row_stats(row, H, eps_post, red, mean, rstd);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float v = hrow[i] + (row[i] - mean) * rstd * w_post[i];
      row[i] = v;
      if (!rows) hrow[i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = hrow[i];
  }
  if (!y) return;
  float mean, rstd;
  row_stats(row, H, eps_pre, red, mean, rstd);
  T* yrow = y + (size_t)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) yrow[i] = from_float<T>((row[i] - mean) * rstd * w_pre[i]);
}

// The same for H % 8 == 0 and H <= 8 * THREADS * CHUNKS: each thread owns CHUNKS runs of 8 columns, read and
// written 16 or 32 bytes at a time, and keeps them in registers through both norms.
template <int CHUNKS>
__device__ __forceinline__ void reg_stats(const float (&v)[CHUNKS][8], const bool (&on)[CHUNKS], int H, float eps, float* red, float& mean,
                                          float& rstd) {
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c)
    if (on[c]) {
#pragma unroll
      for (int k = 0; k < 8; ++k) s += v[c][k];
    }
  mean = block_sum(s, red) / (float)H;
  float q = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c)
    if (on[c]) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float d = v[c][k] - mean;
        q = fmaf(d, d, q);
      }
    }
  rstd = 1.f / sqrtf(block_sum(q, red) / (float)H + eps);
}

template <typename T, int THREADS, int CHUNKS>
__global__ void __launch_bounds__(THREADS) post_add_layernorm_vec_kernel(T* __restrict__ y, float* __restrict__ h, const T* __restrict__ a,
                                                                         const float* __restrict__ w_post, const float* __restrict__ w_pre,
                                                                         const int* __restrict__ rows, int H, float eps_post, float eps_pre) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int r = blockIdx.x;
  const int s = rows ? rows[r] : r;
  float* hrow = h + (size_t)s * H;
  float v[CHUNKS][8];
  bool on[CHUNKS];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) on[c] = (threadIdx.x + c * THREADS) * 8 < H;
  if (a) {
    const T* arow = a + (size_t)s * H;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
      if (on[c]) load8(arow + (threadIdx.x + c * THREADS) * 8, v[c]);
    float mean, rstd;
    reg_stats<CHUNKS>(v, on, H, eps_post, red, mean, rstd);
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
      if (on[c]) {
        const int col = (threadIdx.x + c * THREADS) * 8;
        float hv[8], wv[8];
        load8(hrow + col, hv);
        load8(w_post + col, wv);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[c][k] = hv[k] + (v[c][k] - mean) * rstd * wv[k];
        if (!rows) store8(hrow + col, v[c]);
      }
  } else {
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
      if (on[c]) load8(hrow + (threadIdx.x + c * THREADS) * 8, v[c]);
  }
  if (!y) return;
  float mean, rstd;
  reg_stats<CHUNKS>(v, on, H, eps_pre, red, mean, rstd);
  T* yrow = y + (size_t)r * H;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c)
    if (on[c]) {
      const int col = (threadIdx.x + c * THREADS) * 8;
      float wv[8], o[8];
      load8(w_pre + col, wv);
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = (v[c][k] - mean) * rstd * wv[k];
      store8(yrow + col, o);
    }
}

// h[t] += table[ids[t]] (if table) + vec: what a looped span of layers adds to the stream before a pass.
template <typename T>
__global__ void stream_reinject_kernel(float* __restrict__ h, const T* __restrict__ table, const int* __restrict__ ids,
                                       const float* __restrict__ vec, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  float* hrow = h + (size_t)t * H;
  const T* src = table ? table + (size_t)ids[t] * H : nullptr;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = hrow[i];
    if (src) v += to_float(src[i]);
    if (vec) v += vec[i];
    hrow[i] = v;
  }
}

}  // namespace

DLI_EXPORT int dli_post_add_layernorm(void* y, float* h, const void* a, const float* w_post, const float* w_pre, const int* rows,
                                      int n_rows, int H, float eps_post, float eps_pre, int dtype, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  if (H < 1 || (size_t)H * sizeof(float) > 200 * 1024 || (a && !w_post) || (y && !w_pre)) return DLI_ERR_UNSUPPORTED;
  const bool aligned = (H % 8) == 0 && (((uintptr_t)y | (uintptr_t)h | (uintptr_t)a | (uintptr_t)w_post | (uintptr_t)w_pre) & 15) == 0;
  if (aligned && H <= 8192) {
#define DLI_LN_VEC(T, THREADS, CHUNKS)                                                                                              \
  return (int)launch_pdl((post_add_layernorm_vec_kernel<T, THREADS, CHUNKS>), dim3(n_rows), dim3(THREADS), 0, stream, 1, (T*)y, h, \
                         (const T*)a, w_post, w_pre, rows, H, eps_post, eps_pre)
#define DLI_LN_SIZES(T)                        \
  if (H <= 512) DLI_LN_VEC(T, 64, 1);          \
  if (H <= 1024) DLI_LN_VEC(T, 128, 1);        \
  if (H <= 2048) DLI_LN_VEC(T, 256, 1);        \
  if (H <= 4096) DLI_LN_VEC(T, 256, 2);        \
  DLI_LN_VEC(T, 256, 4)
    if (dtype == DLI_F32) {
      DLI_LN_SIZES(float);
    } else {
      DLI_LN_SIZES(__nv_bfloat16);
    }
#undef DLI_LN_SIZES
#undef DLI_LN_VEC
  }
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  const size_t smem = (size_t)H * sizeof(float);
  cudaError_t e;
  if (dtype == DLI_F32) {
    static MaxPerDevice set;
    if ((int)smem > 48 * 1024 && set.here() < (int)smem) {
      e = cudaFuncSetAttribute(post_add_layernorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      set.here() = (int)smem;
    }
    e = launch_pdl((post_add_layernorm_kernel<float>), dim3(n_rows), dim3(threads), smem, stream, 1, (float*)y, h, (const float*)a, w_post,
                   w_pre, rows, H, eps_post, eps_pre);
  } else {
    static MaxPerDevice set;
    if ((int)smem > 48 * 1024 && set.here() < (int)smem) {
      e = cudaFuncSetAttribute(post_add_layernorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      set.here() = (int)smem;
    }
    e = launch_pdl((post_add_layernorm_kernel<__nv_bfloat16>), dim3(n_rows), dim3(threads), smem, stream, 1, (__nv_bfloat16*)y, h,
                   (const __nv_bfloat16*)a, w_post, w_pre, rows, H, eps_post, eps_pre);
  }
  return (int)e;
}

DLI_EXPORT int dli_stream_reinject(float* h, const void* table, const int* ids, const float* vec, int n, int H, int dtype,
                                   cudaStream_t stream) {
  if (n == 0) return 0;
  if (table && !ids) return DLI_ERR_UNSUPPORTED;
  const int threads = H >= 1024 ? 256 : 128;
  cudaError_t e;
  if (dtype == DLI_F32)
    e = launch_pdl((stream_reinject_kernel<float>), dim3(n), dim3(threads), 0, stream, 1, h, (const float*)table, ids, vec, H);
  else
    e = launch_pdl((stream_reinject_kernel<__nv_bfloat16>), dim3(n), dim3(threads), 0, stream, 1, h, (const __nv_bfloat16*)table, ids, vec, H);
  return (int)e;
}
