// The gated delta rule: a linear recurrence whose state is a matrix S (d x dv) per head,
//     S <- gamma S;   w = beta (v - S^T k);   S <- S + k w^T;   o = S^T q,
// over any mix of prompt portions and single decoded tokens, each sequence from and to its own state slot.
// Everything that enters the recurrence is float32: the unit vectors q and k, beta, gamma, the state and the sums.
#include "common.cuh"

using namespace dli;

namespace {

__device__ __forceinline__ float softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid(float x) { return 1.f / (1.f + expf(-x)); }

// A CTA owns CB value columns of one head of one sequence; NS threads share a column, thread nl holding rows
// i = (kk * NS + nl) * 4 + j (kk < DPT / 4, j < 4) of it in registers.  The step's tokens come through shared memory
// in tiles of TB tokens: q and k of the head's q/k head as float32 unit vectors (q also times d^-1/2), v of the CTA's
// columns, beta, gamma and q . k, which the warps compute token by token while staging.  With both read-outs taken
// from the state before the token's write,
//     a = S^T k,  c = S^T q   (one pass over the column, two sums, reduced over the NS threads together)
//     w = beta (v - gamma a),  o = gamma c + w (k . q),  S <- gamma S + k w
// which is the recurrence above with o = (gamma S + k w^T)^T q written out; the sums are added in an order that the
// sizes fix.  The tile's o leaves through shared memory.
//   qkv [n, 2 G d + H dv]: q | k | v after convolution and activation; b and a_raw are columns b_col + head and
//   a_col + head of u.  state [slots, H, dv, d]: a column's d numbers are contiguous.
template <typename T, int DPT, int NS, int TB>
__global__ void __launch_bounds__(256) delta_rule_scan_kernel(float* __restrict__ o, const T* __restrict__ qkv, const T* __restrict__ u,
                                                              long long u_stride, int b_col, int a_col, const float* __restrict__ dt_bias,
                                                              const float* __restrict__ A_log, float* __restrict__ state,
                                                              const int* __restrict__ q_start, const int* __restrict__ state_slot, int heads,
                                                              int kv_heads, int d, int dv, int CB, float unit_eps) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int DP = DPT * NS;  // d rounded up: rows beyond d hold zeros and stay zero
  extern __shared__ __align__(16) float smem[];
  float* ks = smem;                 // [TB][DP]
  float* qs = ks + TB * DP;         // [TB][DP]
  float* vs = qs + TB * DP;         // [TB][CB]
  float* os = vs + TB * CB;         // [TB][CB]
  float* betas = os + TB * CB;      // [TB]
  float* gammas = betas + TB;       // [TB]
  float* kqs = gammas + TB;         // [TB]
  const int head = blockIdx.x, s = blockIdx.y;
  const int tid = threadIdx.x, nl = tid & (NS - 1), cl = tid / NS;
  const int c0 = blockIdx.z * CB, col = c0 + cl;
  const bool live = col < dv;
  const int g = head / (heads / kv_heads);
  const int inner = heads * dv, C = 2 * kv_heads * d + inner;
  const int qcol = g * d, kcol = kv_heads * d + g * d, vcol = 2 * kv_heads * d + head * dv + c0;
  const int first = q_start[s], last = q_start[s + 1];
  if (first >= last) return;
  float* S0 = state + (((size_t)state_slot[s] * heads + head) * dv + (live ? col : 0)) * d;
  const bool vec = (d & 3) == 0;
  float S[DPT];
#pragma unroll
  for (int kk = 0; kk < DPT / 4; ++kk) {
    const int i0 = (kk * NS + nl) * 4;
    if (live && vec && i0 < d) {
      const float4 x = *reinterpret_cast<const float4*>(S0 + i0);
      S[4 * kk] = x.x; S[4 * kk + 1] = x.y; S[4 * kk + 2] = x.z; S[4 * kk + 3] = x.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) S[4 * kk + j] = (live && i0 + j < d) ? S0[i0 + j] : 0.f;
    }
  }
  const float A = expf(A_log[head]), bias = dt_bias[head];
  const float q_scale = 1.f / sqrtf((float)d);
  const int lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
  for (int tile = first; tile < last; tile += TB) {
    const int cnt = min(TB, last - tile);
    // ---- stage the tile: raw q, k (zero beyond d) and v
    for (int e = tid; e < cnt * DP; e += blockDim.x) {
      const int tok = e / DP, i = e - tok * DP;
      const T* row = qkv + (size_t)(tile + tok) * C;
      qs[e] = i < d ? to_float(row[qcol + i]) : 0.f;
      ks[e] = i < d ? to_float(row[kcol + i]) : 0.f;
    }
    for (int e = tid; e < cnt * CB; e += blockDim.x) {
      const int tok = e / CB, c = e - tok * CB;
      vs[e] = c0 + c < dv ? to_float(qkv[(size_t)(tile + tok) * C + vcol + c]) : 0.f;
    }
    __syncthreads();
    // ---- a warp per token: unit vectors, q . k, beta and gamma
    for (int tok = warp; tok < cnt; tok += warps) {
      float sq = 0.f, sk = 0.f, qk = 0.f;
      for (int i = lane; i < DP; i += 32) {
        const float qv = qs[tok * DP + i], kv = ks[tok * DP + i];
        sq = fmaf(qv, qv, sq);
        sk = fmaf(kv, kv, sk);
        qk = fmaf(qv, kv, qk);
      }
      sq = warp_sum(sq); sk = warp_sum(sk); qk = warp_sum(qk);
      const float rq = q_scale / sqrtf(sq + unit_eps), rk = 1.f / sqrtf(sk + unit_eps);
      for (int i = lane; i < DP; i += 32) {
        qs[tok * DP + i] *= rq;
        ks[tok * DP + i] *= rk;
      }
      if (lane == 0) {
        const T* urow = u + (size_t)(tile + tok) * u_stride;
        kqs[tok] = qk * rq * rk;
        betas[tok] = sigmoid(to_float(urow[b_col + head]));
        gammas[tok] = expf(-A * softplus(to_float(urow[a_col + head]) + bias));
      }
    }
    __syncthreads();
    // ---- the walk
#pragma unroll 2
    for (int t = 0; t < cnt; ++t) {
      const float4* k4 = reinterpret_cast<const float4*>(ks + t * DP);
      const float4* q4 = reinterpret_cast<const float4*>(qs + t * DP);
      float a0 = 0.f, a1 = 0.f, e0 = 0.f, e1 = 0.f;  // two partial sums each: shorter chains, a fixed order
#pragma unroll
      for (int kk = 0; kk < DPT / 4; ++kk) {
        const float4 k = k4[kk * NS + nl], q = q4[kk * NS + nl];
        a0 = fmaf(S[4 * kk], k.x, a0);
        a1 = fmaf(S[4 * kk + 1], k.y, a1);
        a0 = fmaf(S[4 * kk + 2], k.z, a0);
        a1 = fmaf(S[4 * kk + 3], k.w, a1);
        e0 = fmaf(S[4 * kk], q.x, e0);
        e1 = fmaf(S[4 * kk + 1], q.y, e1);
        e0 = fmaf(S[4 * kk + 2], q.z, e0);
        e1 = fmaf(S[4 * kk + 3], q.w, e1);
      }
      float sa = a0 + a1, sc = e0 + e1;
#pragma unroll
      for (int off = 1; off < NS; off <<= 1) {
        sa += __shfl_xor_sync(0xffffffffu, sa, off);
        sc += __shfl_xor_sync(0xffffffffu, sc, off);
      }
      const float gamma = gammas[t];
      const float w = betas[t] * (vs[t * CB + cl] - gamma * sa);
      if (nl == 0) os[t * CB + cl] = fmaf(w, kqs[t], gamma * sc);
#pragma unroll
      for (int kk = 0; kk < DPT / 4; ++kk) {
        const float4 k = k4[kk * NS + nl];
        S[4 * kk] = fmaf(k.x, w, gamma * S[4 * kk]);
        S[4 * kk + 1] = fmaf(k.y, w, gamma * S[4 * kk + 1]);
        S[4 * kk + 2] = fmaf(k.z, w, gamma * S[4 * kk + 2]);
        S[4 * kk + 3] = fmaf(k.w, w, gamma * S[4 * kk + 3]);
      }
    }
    __syncthreads();  // the tile has been walked: its o is complete
    for (int e = tid; e < cnt * CB; e += blockDim.x) {
      const int tok = e / CB, c = e - tok * CB;
      if (c0 + c < dv) o[(size_t)(tile + tok) * inner + head * dv + c0 + c] = os[e];
    }
    __syncthreads();  // os has been read; the next tile may be staged
  }
  if (!live) return;
#pragma unroll
  for (int kk = 0; kk < DPT / 4; ++kk) {
    const int i0 = (kk * NS + nl) * 4;
    if (vec && i0 < d) {
      *reinterpret_cast<float4*>(S0 + i0) = make_float4(S[4 * kk], S[4 * kk + 1], S[4 * kk + 2], S[4 * kk + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (i0 + j < d) S0[i0 + j] = S[4 * kk + j];
    }
  }
}

template <typename T, int DPT, int NS, int TB>
int launch_delta_shape(float* o, const T* qkv, const T* u, long long u_stride, int b_col, int a_col, const float* dt_bias, const float* A_log,
                       float* state, const int* q_start, const int* state_slot, int num_seqs, int heads, int kv_heads, int d, int dv,
                       float unit_eps, cudaStream_t stream) {
  // columns per CTA: as many as 256 threads hold, fewer for narrow heads and where it takes smaller CTAs to give every SM one
  const int most = 256 / NS;
  int CB = dv >= most ? most : ((dv + 7) / 8) * 8;
  while (CB > 8 && (long long)heads * num_seqs * ((dv + CB - 1) / CB) < sm_count()) CB /= 2;
  CB = ((CB + 7) / 8) * 8;
  const int threads = CB * NS;  // a multiple of 32
  const dim3 grid(heads, num_seqs, (dv + CB - 1) / CB), block(threads);
  const size_t smem = (size_t)(2 * TB * DPT * NS + 2 * TB * CB + 3 * TB) * sizeof(float);
  return (int)launch_pdl((delta_rule_scan_kernel<T, DPT, NS, TB>), grid, block, smem, stream, 1, o, qkv, u, u_stride, b_col, a_col, dt_bias, A_log,
                         state, q_start, state_slot, heads, kv_heads, d, dv, CB, unit_eps);
}

template <typename T>
int launch_delta(float* o, const T* qkv, const T* u, long long u_stride, int b_col, int a_col, const float* dt_bias, const float* A_log,
                 float* state, const int* q_start, const int* state_slot, int num_seqs, int heads, int kv_heads, int d, int dv, float unit_eps,
                 cudaStream_t stream) {
#define DLI_DELTA(DPT, NS, TB) \
  return launch_delta_shape<T, DPT, NS, TB>(o, qkv, u, u_stride, b_col, a_col, dt_bias, A_log, state, q_start, state_slot, num_seqs, heads, kv_heads, d, dv, unit_eps, stream)
  if (d <= 16) DLI_DELTA(4, 4, 32);
  if (d <= 32) DLI_DELTA(4, 8, 32);
  if (d <= 64) DLI_DELTA(8, 8, 32);
  if (d <= 128) DLI_DELTA(16, 8, 32);
  if (d <= 256) DLI_DELTA(32, 8, 16);
#undef DLI_DELTA
  return DLI_ERR_UNSUPPORTED;
}

}  // namespace

DLI_EXPORT int dli_delta_rule_scan(float* o, const void* qkv, const void* u, long long u_stride, int b_col, int a_col, const float* dt_bias,
                                   const float* A_log, float* state, const int* q_start, const int* state_slot, int num_seqs, int heads,
                                   int kv_heads, int d, int dv, int max_len, float unit_eps, int dtype, cudaStream_t stream) {
  (void)max_len;
  if (num_seqs == 0) return 0;
  if (heads < 1 || kv_heads < 1 || heads % kv_heads || d < 1 || dv < 1 || num_seqs > 65535 || (dv + 7) / 8 > 65535) return DLI_ERR_UNSUPPORTED;
  if (dtype == DLI_F32)
    return launch_delta<float>(o, (const float*)qkv, (const float*)u, u_stride, b_col, a_col, dt_bias, A_log, state, q_start, state_slot,
                               num_seqs, heads, kv_heads, d, dv, unit_eps, stream);
  return launch_delta<__nv_bfloat16>(o, (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)u, u_stride, b_col, a_col, dt_bias, A_log, state,
                                     q_start, state_slot, num_seqs, heads, kv_heads, d, dv, unit_eps, stream);
}
