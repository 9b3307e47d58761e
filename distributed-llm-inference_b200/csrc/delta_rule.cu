// The gated delta rule: a linear recurrence whose state is a matrix S (d x dv) per head,
//     S <- gamma S;   w = beta (v - S^T k);   S <- S + k w^T;   o = S^T q,
// over any mix of prompt portions and single decoded tokens, each sequence from and to its own state slot.
// Everything that enters the recurrence is float32: the unit vectors q and k, beta, gamma, the state and the sums.
//
// Two kernels.  The first works token by token, all tokens side by side: it makes q and k unit vectors, computes
// beta, gamma and q . k, and leaves everything the recurrence reads as float32 rows.  The second walks each
// sequence's tokens in order with the state in registers, and fetches those rows a tile of tokens ahead of its walk.
#include "common.cuh"

using namespace dli;

namespace {

__device__ __forceinline__ float softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid(float x) { return 1.f / (1.f + expf(-x)); }

// Row of the float32 buffer that the first kernel writes for a token (G q/k heads of d, H heads of dv):
//   q [G d] | k [G d] | v [H dv] | beta [H] | gamma [H] | q . k [G],   `stride` floats apart (a multiple of 4)
// q and k are unit vectors (sum of squares + unit_eps inside the root), q also times d^-1/2.
__host__ __device__ inline int prep_stride(int G, int d, int H, int dv) { return (2 * G * d + H * dv + 2 * H + G + 3) & ~3; }

// One block per token; a warp per q/k head for the unit vectors, then all threads for v, beta and gamma.
//   qkv [n, 2 G d + H dv]: q | k | v after convolution and activation; b and a_raw are columns b_col + head and
//   a_col + head of u.
template <typename T>
__global__ void delta_prep_kernel(float* __restrict__ x32, const T* __restrict__ qkv, const T* __restrict__ u, long long u_stride, int b_col,
                                  int a_col, const float* __restrict__ dt_bias, const float* __restrict__ A_log, int H, int G, int d, int dv,
                                  float unit_eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int C = 2 * G * d + H * dv;
  const T* row = qkv + (size_t)t * C;
  float* out = x32 + (size_t)t * prep_stride(G, d, H, dv);
  const float q_scale = 1.f / sqrtf((float)d);
  for (int g = warp; g < G; g += warps) {
    const T* q = row + g * d;
    const T* k = row + G * d + g * d;
    float sq = 0.f, sk = 0.f, qk = 0.f;
    for (int i = lane; i < d; i += 32) {
      const float qv = to_float(q[i]), kv = to_float(k[i]);
      sq = fmaf(qv, qv, sq);
      sk = fmaf(kv, kv, sk);
      qk = fmaf(qv, kv, qk);
    }
    sq = warp_sum(sq); sk = warp_sum(sk); qk = warp_sum(qk);
    const float rq = q_scale / sqrtf(sq + unit_eps), rk = 1.f / sqrtf(sk + unit_eps);
    for (int i = lane; i < d; i += 32) {
      out[g * d + i] = to_float(q[i]) * rq;
      out[G * d + g * d + i] = to_float(k[i]) * rk;
    }
    if (lane == 0) out[2 * G * d + H * dv + 2 * H + g] = qk * rq * rk;
  }
  for (int e = threadIdx.x; e < H * dv; e += blockDim.x) out[2 * G * d + e] = to_float(row[2 * G * d + e]);
  const T* urow = u + (size_t)t * u_stride;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    out[2 * G * d + H * dv + h] = sigmoid(to_float(urow[b_col + h]));
    out[2 * G * d + H * dv + H + h] = expf(-expf(A_log[h]) * softplus(to_float(urow[a_col + h]) + dt_bias[h]));
  }
}

__device__ __forceinline__ void cp_async16(float* smem_dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(float* smem_dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// A CTA owns CB value columns of one head of one sequence; NS threads share a column, thread nl holding rows
// i = (kk * NS + nl) * 4 + j (kk < DPT / 4, j < 4) of it in registers.  The step's tokens come through shared memory
// in tiles of TB tokens, two tiles in turn: while one is walked, asynchronous copies bring the next (16 bytes a copy
// where the sizes keep every run aligned, VEC; 4 bytes otherwise).  With both read-outs taken from the state before the
// token's write,
//     a = S^T k,  c = S^T q   (one pass over the column, two sums, reduced over the NS threads together)
//     w = beta (v - gamma a),  o = gamma c + w (k . q),  S <- gamma S + k w
// which is the recurrence above with o = (gamma S + k w^T)^T q written out; the sums are added in an order that the
// sizes fix.  The tile's o leaves through shared memory.  state [slots, H, dv, d]: a column's d numbers are contiguous.
template <int DPT, int NS, int TB, bool VEC>
__global__ void __launch_bounds__(256) delta_rule_scan_kernel(float* __restrict__ o, const float* __restrict__ x32, float* __restrict__ state,
                                                              const int* __restrict__ q_start, const int* __restrict__ state_slot, int heads,
                                                              int kv_heads, int d, int dv, int CB) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int DP = DPT * NS;  // d rounded up: rows beyond d hold zeros and stay zero
  extern __shared__ __align__(16) float smem[];
  float* ks = smem;                    // [2][TB][DP]
  float* qs = ks + 2 * TB * DP;        // [2][TB][DP]
  float* vs = qs + 2 * TB * DP;        // [2][TB][CB]
  float* sc = vs + 2 * TB * CB;        // [2][TB][4]: beta, gamma, q . k
  float* os = sc + 2 * TB * 4;         // [TB][CB]
  const int head = blockIdx.x, s = blockIdx.y;
  const int tid = threadIdx.x, nl = tid & (NS - 1), cl = tid / NS;
  const int c0 = blockIdx.z * CB, col = c0 + cl;
  const bool live = col < dv;
  const int g = head / (heads / kv_heads);
  const int inner = heads * dv, stride = prep_stride(kv_heads, d, heads, dv);
  const int first = q_start[s], last = q_start[s + 1];
  if (first >= last) return;
  const int vcnt = min(CB, dv - c0);
  const int qoff = g * d, koff = kv_heads * d + g * d, voff = 2 * kv_heads * d + head * dv + c0;
  const int boff = 2 * kv_heads * d + inner + head, goff = boff + heads, kqoff = 2 * kv_heads * d + inner + 2 * heads + g;

  // copies of one tile, shared out over the CTA's threads
  auto fetch = [&](int tile, int buf) {
    const int cnt = min(TB, last - tile);
    constexpr int U = VEC ? 4 : 1;
    const int du = d / U, vu = vcnt / U, per_tok = 2 * du + vu + 3;
    for (int e = tid; e < cnt * per_tok; e += blockDim.x) {
      const int tok = e / per_tok, it = e - tok * per_tok;
      const float* src = x32 + (size_t)(tile + tok) * stride;
      const int slot = buf * TB + tok;
      if (it < 2 * du) {
        const bool is_k = it >= du;
        const int i = (is_k ? it - du : it) * U;
        float* dst = (is_k ? ks : qs) + slot * DP + i;
        if (VEC) cp_async16(dst, src + (is_k ? koff : qoff) + i);
        else cp_async4(dst, src + (is_k ? koff : qoff) + i);
      } else if (it < 2 * du + vu) {
        const int i = (it - 2 * du) * U;
        if (VEC) cp_async16(vs + slot * CB + i, src + voff + i);
        else cp_async4(vs + slot * CB + i, src + voff + i);
      } else {
        const int j = it - 2 * du - vu;
        cp_async4(sc + slot * 4 + j, src + (j == 0 ? boff : (j == 1 ? goff : kqoff)));
      }
    }
    cp_async_commit();
  };

  // rows beyond d and columns beyond dv are never copied: zero once
  if (d < DP || vcnt < CB) {
    for (int e = tid; e < 4 * TB * DP + 2 * TB * CB; e += blockDim.x) smem[e] = 0.f;
    __syncthreads();
  }
  fetch(first, 0);

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
  int buf = 0;
  for (int tile = first; tile < last; tile += TB, buf ^= 1) {
    const int cnt = min(TB, last - tile);
    const bool more = tile + TB < last;
    if (more) {
      fetch(tile + TB, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();  // this tile's rows have landed, for every thread
    const float* kt = ks + buf * TB * DP;
    const float* qt = qs + buf * TB * DP;
    const float* vt = vs + buf * TB * CB;
    const float* st = sc + buf * TB * 4;
#pragma unroll 2
    for (int t = 0; t < cnt; ++t) {
      const float4* k4 = reinterpret_cast<const float4*>(kt + t * DP);
      const float4* q4 = reinterpret_cast<const float4*>(qt + t * DP);
      float4 k[DPT / 4];
      float a0 = 0.f, a1 = 0.f, e0 = 0.f, e1 = 0.f;  // two partial sums each: shorter chains, a fixed order
#pragma unroll
      for (int kk = 0; kk < DPT / 4; ++kk) {
        k[kk] = k4[kk * NS + nl];
        const float4 q = q4[kk * NS + nl];
        a0 = fmaf(S[4 * kk], k[kk].x, a0);
        a1 = fmaf(S[4 * kk + 1], k[kk].y, a1);
        a0 = fmaf(S[4 * kk + 2], k[kk].z, a0);
        a1 = fmaf(S[4 * kk + 3], k[kk].w, a1);
        e0 = fmaf(S[4 * kk], q.x, e0);
        e1 = fmaf(S[4 * kk + 1], q.y, e1);
        e0 = fmaf(S[4 * kk + 2], q.z, e0);
        e1 = fmaf(S[4 * kk + 3], q.w, e1);
      }
      float sa = a0 + a1, sq = e0 + e1;
#pragma unroll
      for (int off = 1; off < NS; off <<= 1) {
        sa += __shfl_xor_sync(0xffffffffu, sa, off);
        sq += __shfl_xor_sync(0xffffffffu, sq, off);
      }
      const float4 bgk = *reinterpret_cast<const float4*>(st + t * 4);  // beta, gamma, q . k
      const float gamma = bgk.y;
      const float w = bgk.x * (vt[t * CB + cl] - gamma * sa);
      if (nl == 0) os[t * CB + cl] = fmaf(w, bgk.z, gamma * sq);
#pragma unroll
      for (int kk = 0; kk < DPT / 4; ++kk) {
        S[4 * kk] = fmaf(k[kk].x, w, gamma * S[4 * kk]);
        S[4 * kk + 1] = fmaf(k[kk].y, w, gamma * S[4 * kk + 1]);
        S[4 * kk + 2] = fmaf(k[kk].z, w, gamma * S[4 * kk + 2]);
        S[4 * kk + 3] = fmaf(k[kk].w, w, gamma * S[4 * kk + 3]);
      }
    }
    __syncthreads();  // the tile has been walked: its o is complete, its rows may be overwritten
    for (int e = tid; e < cnt * CB; e += blockDim.x) {
      const int tok = e / CB, c = e - tok * CB;
      if (c < vcnt) o[(size_t)(tile + tok) * inner + head * dv + c0 + c] = os[e];
    }
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

template <int DPT, int NS, int TB>
int launch_delta_shape(float* o, const float* x32, float* state, const int* q_start, const int* state_slot, int num_seqs, int heads, int kv_heads,
                       int d, int dv, cudaStream_t stream) {
  // columns per CTA: as many as 256 threads hold, fewer for narrow heads and where it takes smaller CTAs to give every SM two
  const int most = 256 / NS;
  int CB = dv >= most ? most : ((dv + 7) / 8) * 8;
  while (CB > 8 && (long long)heads * num_seqs * ((dv + CB - 1) / CB) < 2 * sm_count()) CB /= 2;
  CB = ((CB + 7) / 8) * 8;
  const int threads = CB * NS;  // a multiple of 32
  const dim3 grid(heads, num_seqs, (dv + CB - 1) / CB), block(threads);
  const size_t smem = (size_t)(4 * TB * DPT * NS + 2 * TB * CB + 2 * TB * 4 + TB * CB) * sizeof(float);
  // 16-byte copies: every run of the float32 rows starts and ends on a 16-byte boundary
  const bool vec = (d % 4) == 0 && (dv % 4) == 0 && (((uintptr_t)x32) & 15) == 0;
  if (vec)
    return (int)launch_pdl((delta_rule_scan_kernel<DPT, NS, TB, true>), grid, block, smem, stream, 1, o, x32, state, q_start, state_slot, heads,
                           kv_heads, d, dv, CB);
  return (int)launch_pdl((delta_rule_scan_kernel<DPT, NS, TB, false>), grid, block, smem, stream, 1, o, x32, state, q_start, state_slot, heads,
                         kv_heads, d, dv, CB);
}

int launch_delta(float* o, const float* x32, float* state, const int* q_start, const int* state_slot, int num_seqs, int heads, int kv_heads, int d,
                 int dv, cudaStream_t stream) {
  // Threads per column: 8 hold the most state each (the fewest shared-memory reads per multiply-add); 16 where 8 would
  // leave an SM with fewer than four warps, as one long prompt on a few heads does.
  const long long columns = (long long)heads * num_seqs * dv;
  const bool wide = columns * 8 < 4LL * 32 * sm_count() && d > 32;
#define DLI_DELTA(DPT, NS, TB) return launch_delta_shape<DPT, NS, TB>(o, x32, state, q_start, state_slot, num_seqs, heads, kv_heads, d, dv, stream)
  if (d <= 16) DLI_DELTA(4, 4, 16);
  if (d <= 32) DLI_DELTA(4, 8, 16);
  if (wide) {
    if (d <= 64) DLI_DELTA(4, 16, 16);
    if (d <= 128) DLI_DELTA(8, 16, 16);
    if (d <= 256) DLI_DELTA(16, 16, 8);
  } else {
    if (d <= 64) DLI_DELTA(8, 8, 16);
    if (d <= 128) DLI_DELTA(16, 8, 16);
    if (d <= 256) DLI_DELTA(32, 8, 8);
  }
#undef DLI_DELTA
  return DLI_ERR_UNSUPPORTED;
}

}  // namespace

// floats of scratch a step of n tokens needs
DLI_EXPORT long long dli_delta_rule_scratch(int n, int heads, int kv_heads, int d, int dv) {
  return (long long)n * prep_stride(kv_heads, d, heads, dv);
}

DLI_EXPORT int dli_delta_rule_scan(float* o, const void* qkv, const void* u, long long u_stride, int b_col, int a_col, const float* dt_bias,
                                   const float* A_log, float* state, const int* q_start, const int* state_slot, float* scratch, int n,
                                   int num_seqs, int heads, int kv_heads, int d, int dv, int max_len, float unit_eps, int dtype,
                                   cudaStream_t stream) {
  (void)max_len;
  if (num_seqs == 0 || n == 0) return 0;
  if (heads < 1 || kv_heads < 1 || heads % kv_heads || d < 1 || d > 256 || dv < 1 || num_seqs > 65535 || (dv + 7) / 8 > 65535 || !scratch)
    return DLI_ERR_UNSUPPORTED;
  const int threads = kv_heads >= 4 ? 128 : 64;
  cudaError_t e;
  if (dtype == DLI_F32)
    e = launch_pdl((delta_prep_kernel<float>), dim3(n), dim3(threads), 0, stream, 1, scratch, (const float*)qkv, (const float*)u, u_stride, b_col,
                   a_col, dt_bias, A_log, heads, kv_heads, d, dv, unit_eps);
  else
    e = launch_pdl((delta_prep_kernel<__nv_bfloat16>), dim3(n), dim3(threads), 0, stream, 1, scratch, (const __nv_bfloat16*)qkv,
                   (const __nv_bfloat16*)u, u_stride, b_col, a_col, dt_bias, A_log, heads, kv_heads, d, dv, unit_eps);
  if (e != cudaSuccess) return (int)e;
  return launch_delta(o, scratch, state, q_start, state_slot, num_seqs, heads, kv_heads, d, dv, stream);
}
