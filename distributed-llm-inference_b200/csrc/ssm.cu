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
// to the sequence's slot of state [slots, heads, N, P].  A thread owns NPT values of n (n = nl + 4 k) of one
// column p; the four threads of a column add their shares of y by shuffles, always in the same order.
//   xbc [n, inner + 2 G N]: x | B | C after convolution and activation; dt_raw: column dt_col + head of u.
template <typename T, int NPT>
__global__ void ssm_scan_kernel(float* __restrict__ y, const T* __restrict__ xbc, const T* __restrict__ u, long long u_stride, int dt_col,
                                const float* __restrict__ dt_bias, const float* __restrict__ A_log, const float* __restrict__ D,
                                float* __restrict__ state, const int* __restrict__ q_start, const int* __restrict__ state_slot,
                                int heads, int P, int N, int groups) {
  pdl_launch_dependents();
  pdl_wait();
  const int head = blockIdx.x, s = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nl = lane >> 3;
  const int p = (blockIdx.z * (blockDim.x >> 5) + warp) * 8 + (lane & 7);
  const bool live = p < P;
  const int inner = heads * P, C = inner + 2 * groups * N;
  const int g = head / (heads / groups);
  const int first = q_start[s], last = q_start[s + 1];
  float* S0 = state + ((size_t)state_slot[s] * heads + head) * N * P;
  float S[NPT];
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int n = nl + 4 * k;
    S[k] = (live && n < N) ? S0[(size_t)n * P + p] : 0.f;
  }
  const float A = expf(A_log[head]), bias = dt_bias[head], Dh = D[head];
  const int xcol = head * P + p, bcol = inner + g * N, ccol = inner + groups * N + g * N;
  for (int t = first; t < last; ++t) {
    const T* row = xbc + (size_t)t * C;
    const float dt = softplus(to_float(u[(size_t)t * u_stride + dt_col + head]) + bias);
    const float decay = expf(-A * dt);
    const float x = live ? to_float(row[xcol]) : 0.f;
    const float dtx = dt * x;
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < NPT; ++k) {
      const int n = nl + 4 * k;
      if (n < N) {
        S[k] = fmaf(decay, S[k], to_float(row[bcol + n]) * dtx);
        acc = fmaf(S[k], to_float(row[ccol + n]), acc);
      }
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 8);
    acc += __shfl_xor_sync(0xffffffffu, acc, 16);
    if (live && nl == 0) y[(size_t)t * inner + xcol] = fmaf(Dh, x, acc);
  }
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int n = nl + 4 * k;
    if (live && n < N) S0[(size_t)n * P + p] = S[k];
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

template <typename T>
int launch_scan(float* y, const T* xbc, const T* u, long long u_stride, int dt_col, const float* dt_bias, const float* A_log,
                const float* D, float* state, const int* q_start, const int* state_slot, int num_seqs, int heads, int P, int N, int groups,
                cudaStream_t stream) {
  const int warps = (P + 7) / 8 < 8 ? (P + 7) / 8 : 8;
  const dim3 grid(heads, num_seqs, (P + warps * 8 - 1) / (warps * 8)), block(warps * 32);
#define DLI_SCAN(NPT)                                                                                                              \
  return (int)launch_pdl((ssm_scan_kernel<T, NPT>), grid, block, 0, stream, 1, y, xbc, u, u_stride, dt_col, dt_bias, A_log, D, state, \
                         q_start, state_slot, heads, P, N, groups)
  if (N <= 16) DLI_SCAN(4);
  if (N <= 32) DLI_SCAN(8);
  if (N <= 64) DLI_SCAN(16);
  if (N <= 128) DLI_SCAN(32);
  if (N <= 256) DLI_SCAN(64);
#undef DLI_SCAN
  return DLI_ERR_UNSUPPORTED;
}

}  // namespace

DLI_EXPORT int dli_causal_conv_silu(void* out, const void* u, long long u_stride, int col0, const float* w, const float* bias,
                                    const void* state, const int* seq_of_token, const int* q_start, const int* state_slot, int n, int C,
                                    int taps, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (C < 1 || taps < 1 || (C + 127) / 128 > 65535) return DLI_ERR_UNSUPPORTED;
  const dim3 grid(n, (C + 127) / 128), block(128);
  cudaError_t e;
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
  const int threads = size >= 1024 ? 256 : 128;
  const dim3 grid(n, parts);
  cudaError_t e;
  if (dtype == DLI_F32)
    e = launch_pdl((gated_group_rmsnorm_kernel<float>), grid, dim3(threads), 0, stream, 1, (float*)out, y, (const float*)u, u_stride, z_col, w,
                   inner, parts, eps);
  else
    e = launch_pdl((gated_group_rmsnorm_kernel<__nv_bfloat16>), grid, dim3(threads), 0, stream, 1, (__nv_bfloat16*)out, y,
                   (const __nv_bfloat16*)u, u_stride, z_col, w, inner, parts, eps);
  return (int)e;
}
