// What lies between an attention mixer's projections and its attention kernel when queries and keys are
// normed over their whole projection, and what lies behind the attention kernel when its output is gated.
// float32 and bfloat16 instantiations; all arithmetic is float32.
#include "common.cuh"

using namespace dli;

namespace {

// One block per token.  proj row: q (nh * d columns) | k (nkv * d columns), then whatever else the product made.
//   q <- q / rms(q over all nh * d) * wq,  k <- k / rms(k over all nkv * d) * wk      (normed != 0)
//   rotary (rotate-half pairing, first `rot` dimensions of each head, angle float32(position) * inv_freq[i])
//   q -> q_out [n, nh * d];  k -> k_pool at the token's slot;
//   v_pool gets the keys as projected (values_from_keys != 0) or the nkv * d columns behind k.
template <typename T>
__global__ void qk_norm_rotary_store_kernel(T* __restrict__ q_out, const T* __restrict__ proj, long long proj_stride,
                                            const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                                            const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                            const int* __restrict__ slots, T* __restrict__ k_pool, T* __restrict__ v_pool, int nh,
                                            int nkv, int d, int rot, int page_size, int write_kv, int normed, int values_from_keys) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row[];  // (nh + nkv) * d
  __shared__ float red[33];
  const int t = blockIdx.x;
  const int nq = nh * d, nk = nkv * d;
  const T* src = proj + (size_t)t * proj_stride;
  float sq = 0.f, sk = 0.f;
  for (int e = threadIdx.x; e < nq + nk; e += blockDim.x) {
    const float x = to_float(src[e]);
    row[e] = x;
    if (e < nq) sq = fmaf(x, x, sq); else sk = fmaf(x, x, sk);
  }
  float rq = 1.f, rk = 1.f;
  if (normed) {
    rq = 1.f / sqrtf(block_sum(sq, red) / (float)nq + eps);
    rk = 1.f / sqrtf(block_sum(sk, red) / (float)nk + eps);
  } else {
    __syncthreads();
  }
  const float pos = (float)positions[t];
  const int half = rot >> 1;
  long long kv_base = 0;
  if (write_kv) {
    const int slot = slots[t];
    kv_base = ((long long)(slot / page_size) * nkv * page_size + slot % page_size) * d;  // + kvh * page_size * d + i
  }
  for (int e = threadIdx.x; e < nq + nk; e += blockDim.x) {
    const bool is_q = e < nq;
    if (!is_q && !write_kv) continue;
    const int c = is_q ? e : e - nq;          // column inside q or k
    const int head = c / d, i = c - head * d;
    const float r = is_q ? rq : rk;
    const float* w = is_q ? wq : wk;
    float x = row[e] * r * (normed ? w[c] : 1.f);
    if (i < rot) {
      const int j = i < half ? i : i - half;
      const int pe = i < half ? e + half : e - half, pc = i < half ? c + half : c - half;
      const float xp = row[pe] * r * (normed ? w[pc] : 1.f);
      float sn, cs;
      sincosf(pos * inv_freq[j], &sn, &cs);
      x = i < half ? x * cs - xp * sn : x * cs + xp * sn;
    }
    if (is_q) {
      q_out[(size_t)t * nq + c] = from_float<T>(x);
    } else {
      const long long at = kv_base + (long long)head * page_size * d + i;
      k_pool[at] = from_float<T>(x);
      v_pool[at] = values_from_keys ? src[e] : src[e + nk];
    }
  }
}

// out[t, c] *= sigmoid(gate[t * gate_stride + c])
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ out, const T* __restrict__ gate, long long gate_stride, int n, int cols) {
  pdl_launch_dependents();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n * cols) return;
  const int t = (int)(idx / cols), c = (int)(idx - (long long)t * cols);
  const float g = to_float(gate[(size_t)t * gate_stride + c]);
  out[idx] = from_float<T>(to_float(out[idx]) / (1.f + expf(-g)));
}

}  // namespace

DLI_EXPORT int dli_qk_norm_rotary_store(void* q_out, const void* proj, long long proj_stride, const float* wq, const float* wk,
                                        float eps, const int* positions, const float* inv_freq, const int* slots, void* k_pool,
                                        void* v_pool, int n, int nh, int nkv, int d, int rot, int page_size, int write_kv,
                                        int normed, int values_from_keys, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  const size_t smem = (size_t)(nh + nkv) * d * sizeof(float);
  if (nh < 1 || nkv < 1 || d < 1 || rot < 0 || rot > d || (rot & 1) || smem > 200 * 1024 || (rot && !inv_freq) ||
      (normed && (!wq || !wk)) || (write_kv && (!slots || !k_pool || !v_pool)))
    return DLI_ERR_UNSUPPORTED;
  const int threads = (nh + nkv) * d >= 2048 ? 512 : 256;
  cudaError_t e;
  if (dtype == DLI_F32) {
    static MaxPerDevice set;
    if ((int)smem > 48 * 1024 && set.here() < (int)smem) {
      e = cudaFuncSetAttribute(qk_norm_rotary_store_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      set.here() = (int)smem;
    }
    e = launch_pdl((qk_norm_rotary_store_kernel<float>), dim3(n), dim3(threads), smem, stream, 1, (float*)q_out, (const float*)proj,
                   proj_stride, wq, wk, eps, positions, inv_freq, slots, (float*)k_pool, (float*)v_pool, nh, nkv, d, rot, page_size,
                   write_kv, normed, values_from_keys);
  } else {
    static MaxPerDevice set;
    if ((int)smem > 48 * 1024 && set.here() < (int)smem) {
      e = cudaFuncSetAttribute(qk_norm_rotary_store_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      set.here() = (int)smem;
    }
    e = launch_pdl((qk_norm_rotary_store_kernel<__nv_bfloat16>), dim3(n), dim3(threads), smem, stream, 1, (__nv_bfloat16*)q_out,
                   (const __nv_bfloat16*)proj, proj_stride, wq, wk, eps, positions, inv_freq, slots, (__nv_bfloat16*)k_pool,
                   (__nv_bfloat16*)v_pool, nh, nkv, d, rot, page_size, write_kv, normed, values_from_keys);
  }
  return (int)e;
}

DLI_EXPORT int dli_sigmoid_gate(void* out, const void* gate, long long gate_stride, int n, int cols, int dtype, cudaStream_t stream) {
  if (n == 0 || cols == 0) return 0;
  const long long total = (long long)n * cols;
  const int blocks = (int)((total + 255) / 256);
  cudaError_t e;
  if (dtype == DLI_F32)
    e = launch_pdl((sigmoid_gate_kernel<float>), dim3(blocks), dim3(256), 0, stream, 1, (float*)out, (const float*)gate, gate_stride, n, cols);
  else
    e = launch_pdl((sigmoid_gate_kernel<__nv_bfloat16>), dim3(blocks), dim3(256), 0, stream, 1, (__nv_bfloat16*)out,
                   (const __nv_bfloat16*)gate, gate_stride, n, cols);
  return (int)e;
}
