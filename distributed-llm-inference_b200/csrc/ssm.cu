// A state-space mixer's steps between its two projections: the short causal convolution with its carried
// inputs, the selective scan with its carried state, and the gated norm in groups.  A step's tokens are any
// mix of prompt portions and single decoded tokens; each sequence continues from its own state slot.
// Everything that enters the recurrence is float32: step sizes, decays, the state and the sums.
#include "common.cuh"

using namespace dli;

namespace {

__device__ __forceinline__ float silu(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// out[t, c] = silu(bias[c] + sum_j w[c, j] * in(t - (taps - 1) + j, c)); in() of a place before the step's
// first token of the sequence is the sequence's carried input (state [slots, taps - 1, C], oldest first;
// zeros when the sequence begins).  The input's channel c is column col0 + c of u.
template <typename T>
__global__ void causal_conv_silu_kernel(T* __restrict__ out, const T* __restrict__ u, long long u_stride, int col0,
                                        const float* __restrict__ w, const float* __restrict__ bias, const T* __restrict__ state,
                                        const int* __restrict__ seq_of_token, const int* __restrict__ q_start,
                                        const int* __restrict__ state_slot, int C, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int t = blockIdx.x;
  const int s = seq_of_token[t];
  const int first = q_start[s];
  const int r0 = t - first;
  const T* carried = state + (size_t)state_slot[s] * (taps - 1) * C;
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int r = r0 - (taps - 1) + j;
    const float x = r >= 0 ? to_float(u[(size_t)(first + r) * u_stride + col0 + c]) : to_float(carried[(size_t)(taps - 1 + r) * C + c]);
    acc = fmaf(w[(size_t)c * taps + j], x, acc);
  }
  out[(size_t)t * C + c] = from_float<T>(silu(acc));
}

// The same, eight channels a thread with 16-byte accesses (C, col0 and the row strides multiples of 8, at most 8 taps).
template <typename T>
__global__ void causal_conv_silu_vec_kernel(T* __restrict__ out, const T* __restrict__ u, long long u_stride, int col0,
                                            const float* __restrict__ w, const float* __restrict__ bias, const T* __restrict__ state,
                                            const int* __restrict__ seq_of_token, const int* __restrict__ q_start,
                                            const int* __restrict__ state_slot, int C, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c >= C) return;
  const int t = blockIdx.x;
  const int s = seq_of_token[t];
  const int first = q_start[s];
  const int r0 = t - first;
  const T* carried = state + (size_t)state_slot[s] * (taps - 1) * C;
  float acc[8];
  if (bias) load8(bias + c, acc);
  else {
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  }
  for (int j = 0; j < taps; ++j) {
    const int r = r0 - (taps - 1) + j;
    float x[8];
    if (r >= 0) load8(u + (size_t)(first + r) * u_stride + col0 + c, x);
    else load8(carried + (size_t)(taps - 1 + r) * C + c, x);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = fmaf(w[(size_t)(c + k) * taps + j], x[k], acc[k]);
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = silu(acc[k]);
  store8(out + (size_t)t * C + c, acc);
}

// After the convolution: each sequence's carried inputs become its last taps - 1 inputs (older carried
// inputs move up when the step brought fewer).  In place: slot i is written from slot i + q_len or from u.
template <typename T>
__global__ void conv_state_update_kernel(T* __restrict__ state, const T* __restrict__ u, long long u_stride, int col0,
                                         const int* __restrict__ q_start, const int* __restrict__ state_slot, int C, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int s = blockIdx.y;
  const int first = q_start[s], len = q_start[s + 1] - first;
  T* carried = state + (size_t)state_slot[s] * (taps - 1) * C;
  for (int i = 0; i < taps - 1; ++i) {
    const int r = len - (taps - 1) + i;
    carried[(size_t)i * C + c] = r >= 0 ? u[(size_t)(first + r) * u_stride + col0 + c] : carried[(size_t)(i + len) * C + c];
  }
}

// The scan.  Per (sequence, head): S <- exp(-exp(A_log) dt) S + dt B x^T (S is N x P), y = S^T C + D x, with
// dt = softplus(dt_raw + dt_bias), over the sequence's tokens of this step in order; S starts from and returns
// to the sequence's slot of state [slots, heads, P, N] (N fastest: a thread's share of a column is contiguous).
// A CTA owns PB columns p of one head; eight threads share a column, thread nl holding n = (k * 8 + nl) * 4 + j
// (k < NPT / 4, j < 4), and add their shares of y by shuffles, always in the same order.  The step's tokens
// come through shared memory in tiles of TB tokens (x of the CTA's columns, B and C of the head's group, the
// step sizes and decays, which one thread per token computes), so the walk over a tile touches no global memory;
// the tile's y leaves through shared memory too.
//   xbc [n, inner + 2 G N]: x | B | C after convolution and activation; dt_raw: column dt_col + head of u.
constexpr int SCAN_TB = 32;
constexpr int SCAN_NS = 8;

template <typename T, int NPT>
__global__ void __launch_bounds__(256) ssm_scan_kernel(float* __restrict__ y, const T* __restrict__ xbc, const T* __restrict__ u,
                                                       long long u_stride, int dt_col, const float* __restrict__ dt_bias,
                                                       const float* __restrict__ A_log, const float* __restrict__ D,
                                                       float* __restrict__ state, const int* __restrict__ q_start,
                                                       const int* __restrict__ state_slot, int heads, int P, int N, int groups, int PB) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int NP = NPT * SCAN_NS;  // N rounded up: rows beyond N hold zeros and stay zero
  extern __shared__ __align__(16) float smem[];
  float* Bs = smem;                     // [TB][NP]
  float* Cs = Bs + SCAN_TB * NP;        // [TB][NP]
  float* xs = Cs + SCAN_TB * NP;        // [TB][PB]
  float* ys = xs + SCAN_TB * PB;        // [TB][PB]
  float* dts = ys + SCAN_TB * PB;       // [TB]
  float* decs = dts + SCAN_TB;          // [TB]
  const int head = blockIdx.x, s = blockIdx.y;
  const int tid = threadIdx.x, nl = tid & (SCAN_NS - 1), pl = tid / SCAN_NS;
  const int p0 = blockIdx.z * PB, p = p0 + pl;
  const bool live = p < P;
  const int inner = heads * P, C = inner + 2 * groups * N;
  const int g = head / (heads / groups);
  const int first = q_start[s], last = q_start[s + 1];
  float* S0 = state + (((size_t)state_slot[s] * heads + head) * P + (live ? p : 0)) * N;
  const bool vec = (N & 3) == 0;
  float S[NPT];
#pragma unroll
  for (int k = 0; k < NPT / 4; ++k) {
    const int n0 = (k * SCAN_NS + nl) * 4;
    if (live && vec && n0 < N) {
      const float4 v = *reinterpret_cast<const float4*>(S0 + n0);
      S[4 * k] = v.x; S[4 * k + 1] = v.y; S[4 * k + 2] = v.z; S[4 * k + 3] = v.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) S[4 * k + j] = (live && n0 + j < N) ? S0[n0 + j] : 0.f;
    }
  }
  const float A = expf(A_log[head]), bias = dt_bias[head], Dh = D[head];
  const int xcol = head * P + p0, bcol = inner + g * N, ccol = inner + groups * N + g * N;
  const int width = PB + 2 * NP;
  for (int tile = first; tile < last; tile += SCAN_TB) {
    const int cnt = min(SCAN_TB, last - tile);
    for (int e = tid; e < cnt * width; e += blockDim.x) {
      const int tok = e / width, off = e - tok * width;
      const T* row = xbc + (size_t)(tile + tok) * C;
      if (off < PB) {
        xs[tok * PB + off] = (p0 + off < P) ? to_float(row[xcol + off]) : 0.f;
      } else if (off < PB + NP) {
        const int n = off - PB;
        Bs[tok * NP + n] = n < N ? to_float(row[bcol + n]) : 0.f;
      } else {
        const int n = off - PB - NP;
        Cs[tok * NP + n] = n < N ? to_float(row[ccol + n]) : 0.f;
      }
    }
    if (tid < cnt) {
      const float dt = softplus(to_float(u[(size_t)(tile + tid) * u_stride + dt_col + head]) + bias);
      dts[tid] = dt;
      decs[tid] = expf(-A * dt);
    }
    __syncthreads();
    for (int t = 0; t < cnt; ++t) {
      const float x = xs[t * PB + pl];
      const float dtx = dts[t] * x, decay = decs[t];
      const float4* b4 = reinterpret_cast<const float4*>(Bs + t * NP);
      const float4* c4 = reinterpret_cast<const float4*>(Cs + t * NP);
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < NPT / 4; ++k) {
        const float4 b = b4[k * SCAN_NS + nl], c = c4[k * SCAN_NS + nl];
        S[4 * k] = fmaf(decay, S[4 * k], b.x * dtx);
        S[4 * k + 1] = fmaf(decay, S[4 * k + 1], b.y * dtx);
        S[4 * k + 2] = fmaf(decay, S[4 * k + 2], b.z * dtx);
        S[4 * k + 3] = fmaf(decay, S[4 * k + 3], b.w * dtx);
        acc = fmaf(S[4 * k], c.x, acc);
        acc = fmaf(S[4 * k + 1], c.y, acc);
        acc = fmaf(S[4 * k + 2], c.z, acc);
        acc = fmaf(S[4 * k + 3], c.w, acc);
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (nl == 0) ys[t * PB + pl] = fmaf(Dh, x, acc);
    }
    __syncthreads();
    for (int e = tid; e < cnt * PB; e += blockDim.x) {
      const int tok = e / PB, off = e - tok * PB;
      if (p0 + off < P) y[(size_t)(tile + tok) * inner + xcol + off] = ys[e];
    }
    // the next tile's staging writes xs, Bs, Cs (read before the barrier above) and its walk writes ys after
    // the barrier behind the staging, which every thread reaches only after these stores
  }
  if (!live) return;
#pragma unroll
  for (int k = 0; k < NPT / 4; ++k) {
    const int n0 = (k * SCAN_NS + nl) * 4;
    if (vec && n0 < N) {
      *reinterpret_cast<float4*>(S0 + n0) = make_float4(S[4 * k], S[4 * k + 1], S[4 * k + 2], S[4 * k + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (n0 + j < N) S0[n0 + j] = S[4 * k + j];
    }
  }
}

// out[t, part] = g / sqrt(mean(g^2 over the part) + eps) * w, g = y * silu(z); the row is cut into `parts`
// equal runs.  z is column z_col + c of u.  One block per (token, part).
template <typename T>
__global__ void gated_group_rmsnorm_kernel(T* __restrict__ out, const float* __restrict__ y, const T* __restrict__ u, long long u_stride,
                                           int z_col, const float* __restrict__ w, int inner, int parts, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int part = blockIdx.y, t = blockIdx.x;
  const int size = inner / parts, c0 = part * size;
  const float* yrow = y + (size_t)t * inner + c0;
  const T* zrow = u + (size_t)t * u_stride + z_col + c0;
  float q = 0.f;
  for (int i = threadIdx.x; i < size; i += blockDim.x) {
    const float gv = yrow[i] * silu(to_float(zrow[i]));
    q = fmaf(gv, gv, q);
  }
  const float r = 1.f / sqrtf(block_sum(q, red) / (float)size + eps);
  for (int i = threadIdx.x; i < size; i += blockDim.x) {
    const float gv = yrow[i] * silu(to_float(zrow[i]));
    out[(size_t)t * inner + c0 + i] = from_float<T>(gv * r * w[c0 + i]);
  }
}

// The same with the part's values in registers between the two passes and 16- and 32-byte accesses: a thread owns
// CHUNKS runs of eight columns (size % 8 == 0, size <= 8 * THREADS * CHUNKS, aligned rows).
template <typename T, int THREADS, int CHUNKS>
__global__ void __launch_bounds__(THREADS) gated_group_rmsnorm_vec_kernel(T* __restrict__ out, const float* __restrict__ y,
                                                                          const T* __restrict__ u, long long u_stride, int z_col,
                                                                          const float* __restrict__ w, int inner, int parts, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int part = blockIdx.y, t = blockIdx.x;
  const int size = inner / parts, c0 = part * size;
  const float* yrow = y + (size_t)t * inner + c0;
  const T* zrow = u + (size_t)t * u_stride + z_col + c0;
  float gv[CHUNKS][8];
  float q = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = (threadIdx.x + c * THREADS) * 8;
    if (col < size) {
      float z[8];
      load8(yrow + col, gv[c]);
      load8(zrow + col, z);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        gv[c][k] *= silu(z[k]);
        q = fmaf(gv[c][k], gv[c][k], q);
      }
    }
  }
  const float r = 1.f / sqrtf(block_sum(q, red) / (float)size + eps);
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = (threadIdx.x + c * THREADS) * 8;
    if (col < size) {
      float wv[8], o[8];
      load8(w + c0 + col, wv);
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = gv[c][k] * r * wv[k];
      store8(out + (size_t)t * inner + c0 + col, o);
    }
  }
}

template <typename T, int NPT>
int launch_scan_npt(float* y, const T* xbc, const T* u, long long u_stride, int dt_col, const float* dt_bias, const float* A_log,
                    const float* D, float* state, const int* q_start, const int* state_slot, int num_seqs, int heads, int P, int N, int groups,
                    cudaStream_t stream) {
  // columns per CTA: 32 (256 threads), fewer for narrow heads; 16 where that is what it takes to give every SM a CTA
  int PB = P >= 32 ? 32 : ((P + 3) / 4) * 4;
  if (PB == 32 && (long long)heads * num_seqs * ((P + 31) / 32) < sm_count()) PB = 16;
  const dim3 grid(heads, num_seqs, (P + PB - 1) / PB), block(PB * SCAN_NS);
  const size_t smem = (size_t)(2 * SCAN_TB * NPT * SCAN_NS + 2 * SCAN_TB * PB + 2 * SCAN_TB) * sizeof(float);
  static MaxPerDevice set;
  if ((int)smem > 48 * 1024 && set.here() < (int)smem) {
    cudaError_t e = cudaFuncSetAttribute(ssm_scan_kernel<T, NPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    set.here() = (int)smem;
  }
  return (int)launch_pdl((ssm_scan_kernel<T, NPT>), grid, block, smem, stream, 1, y, xbc, u, u_stride, dt_col, dt_bias, A_log, D, state,
                         q_start, state_slot, heads, P, N, groups, PB);
}

template <typename T>
int launch_scan(float* y, const T* xbc, const T* u, long long u_stride, int dt_col, const float* dt_bias, const float* A_log,
                const float* D, float* state, const int* q_start, const int* state_slot, int num_seqs, int heads, int P, int N, int groups,
                cudaStream_t stream) {
#define DLI_SCAN(NPT) \
  return launch_scan_npt<T, NPT>(y, xbc, u, u_stride, dt_col, dt_bias, A_log, D, state, q_start, state_slot, num_seqs, heads, P, N, groups, stream)
  if (N <= 32) DLI_SCAN(4);
  if (N <= 64) DLI_SCAN(8);
  if (N <= 128) DLI_SCAN(16);
  if (N <= 256) DLI_SCAN(32);
#undef DLI_SCAN
  return DLI_ERR_UNSUPPORTED;
}

}  // namespace

DLI_EXPORT int dli_causal_conv_silu(void* out, const void* u, long long u_stride, int col0, const float* w, const float* bias,
                                    const void* state, const int* seq_of_token, const int* q_start, const int* state_slot, int n, int C,
                                    int taps, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (C < 1 || taps < 1 || (C + 127) / 128 > 65535) return DLI_ERR_UNSUPPORTED;
  cudaError_t e;
  if ((C % 8) == 0 && (col0 % 8) == 0 && (u_stride % 8) == 0 && (((uintptr_t)out | (uintptr_t)u | (uintptr_t)state | (uintptr_t)bias) & 15) == 0) {
    const int items = C / 8, vt = items >= 256 ? 256 : (items >= 128 ? 128 : 64);
    const dim3 vgrid(n, (items + vt - 1) / vt);
    if (dtype == DLI_F32)
      e = launch_pdl((causal_conv_silu_vec_kernel<float>), vgrid, dim3(vt), 0, stream, 1, (float*)out, (const float*)u, u_stride, col0, w, bias,
                     (const float*)state, seq_of_token, q_start, state_slot, C, taps);
    else
      e = launch_pdl((causal_conv_silu_vec_kernel<__nv_bfloat16>), vgrid, dim3(vt), 0, stream, 1, (__nv_bfloat16*)out, (const __nv_bfloat16*)u,
                     u_stride, col0, w, bias, (const __nv_bfloat16*)state, seq_of_token, q_start, state_slot, C, taps);
    return (int)e;
  }
  const dim3 grid(n, (C + 127) / 128), block(128);
  if (dtype == DLI_F32)
    e = launch_pdl((causal_conv_silu_kernel<float>), grid, block, 0, stream, 1, (float*)out, (const float*)u, u_stride, col0, w, bias,
                   (const float*)state, seq_of_token, q_start, state_slot, C, taps);
  else
    e = launch_pdl((causal_conv_silu_kernel<__nv_bfloat16>), grid, block, 0, stream, 1, (__nv_bfloat16*)out, (const __nv_bfloat16*)u, u_stride,
                   col0, w, bias, (const __nv_bfloat16*)state, seq_of_token, q_start, state_slot, C, taps);
  return (int)e;
}

DLI_EXPORT int dli_conv_state_update(void* state, const void* u, long long u_stride, int col0, const int* q_start, const int* state_slot,
                                     int num_seqs, int C, int taps, int dtype, cudaStream_t stream) {
  if (num_seqs == 0 || taps <= 1) return 0;
  if (num_seqs > 65535) return DLI_ERR_UNSUPPORTED;
  const dim3 grid((C + 127) / 128, num_seqs), block(128);
  cudaError_t e;
  if (dtype == DLI_F32)
    e = launch_pdl((conv_state_update_kernel<float>), grid, block, 0, stream, 1, (float*)state, (const float*)u, u_stride, col0, q_start,
                   state_slot, C, taps);
  else
    e = launch_pdl((conv_state_update_kernel<__nv_bfloat16>), grid, block, 0, stream, 1, (__nv_bfloat16*)state, (const __nv_bfloat16*)u,
                   u_stride, col0, q_start, state_slot, C, taps);
  return (int)e;
}

DLI_EXPORT int dli_ssm_scan(float* y, const void* xbc, const void* u, long long u_stride, int dt_col, const float* dt_bias,
                            const float* A_log, const float* D, float* state, const int* q_start, const int* state_slot, int num_seqs,
                            int heads, int P, int N, int groups, int dtype, cudaStream_t stream) {
  if (num_seqs == 0) return 0;
  if (heads < 1 || groups < 1 || heads % groups || P < 1 || N < 1 || num_seqs > 65535) return DLI_ERR_UNSUPPORTED;
  if (dtype == DLI_F32)
    return launch_scan<float>(y, (const float*)xbc, (const float*)u, u_stride, dt_col, dt_bias, A_log, D, state, q_start, state_slot,
                              num_seqs, heads, P, N, groups, stream);
  return launch_scan<__nv_bfloat16>(y, (const __nv_bfloat16*)xbc, (const __nv_bfloat16*)u, u_stride, dt_col, dt_bias, A_log, D, state,
                                    q_start, state_slot, num_seqs, heads, P, N, groups, stream);
}

DLI_EXPORT int dli_gated_group_rmsnorm(void* out, const float* y, const void* u, long long u_stride, int z_col, const float* w, int n,
                                       int inner, int parts, float eps, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (parts < 1 || parts > 65535 || inner % parts) return DLI_ERR_UNSUPPORTED;
  const int size = inner / parts;
  const dim3 grid(n, parts);
  cudaError_t e;
  if ((size % 8) == 0 && size <= 8192 && (z_col % 8) == 0 && (u_stride % 8) == 0 &&
      (((uintptr_t)out | (uintptr_t)y | (uintptr_t)u | (uintptr_t)w) & 15) == 0) {
#define DLI_GN_VEC(T, THREADS, CHUNKS)                                                                                               \
  return (int)launch_pdl((gated_group_rmsnorm_vec_kernel<T, THREADS, CHUNKS>), grid, dim3(THREADS), 0, stream, 1, (T*)out, y, (const T*)u, \
                         u_stride, z_col, w, inner, parts, eps)
#define DLI_GN_SIZES(T)                       \
  if (size <= 256) DLI_GN_VEC(T, 32, 1);      \
  if (size <= 512) DLI_GN_VEC(T, 64, 1);      \
  if (size <= 1024) DLI_GN_VEC(T, 128, 1);    \
  if (size <= 2048) DLI_GN_VEC(T, 256, 1);    \
  if (size <= 4096) DLI_GN_VEC(T, 256, 2);    \
  DLI_GN_VEC(T, 256, 4)
    if (dtype == DLI_F32) {
      DLI_GN_SIZES(float);
    } else {
      DLI_GN_SIZES(__nv_bfloat16);
    }
#undef DLI_GN_SIZES
#undef DLI_GN_VEC
  }
  const int threads = size >= 1024 ? 256 : 128;
  if (dtype == DLI_F32)
    e = launch_pdl((gated_group_rmsnorm_kernel<float>), grid, dim3(threads), 0, stream, 1, (float*)out, y, (const float*)u, u_stride, z_col, w,
                   inner, parts, eps);
  else
    e = launch_pdl((gated_group_rmsnorm_kernel<__nv_bfloat16>), grid, dim3(threads), 0, stream, 1, (__nv_bfloat16*)out, y,
                   (const __nv_bfloat16*)u, u_stride, z_col, w, inner, parts, eps);
  return (int)e;
}
