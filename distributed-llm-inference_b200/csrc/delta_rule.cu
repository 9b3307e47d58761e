// The gated delta rule: a linear recurrence whose state is a matrix S (d x dv) per head,
//     S <- gamma S;   w = beta (v - S^T k);   S <- S + k w^T;   o = S^T q,
// over any mix of prompt portions and single decoded tokens, each sequence from and to its own state slot.
// Everything that enters the recurrence is float32: the unit vectors q and k, beta, gamma, the state and the sums.
//
// Two kernels work token by token, all tokens side by side: (1) q and k become unit vectors, beta and gamma are
// computed, and everything the recurrence reads is left as float32 rows; (2) every token's k . k and q . k with the
// tokens before it in its tile of TILE tokens, already multiplied by the decays between the two tokens.  A third
// walks each sequence with the state in registers, in one of two forms.  Steps of few tokens per sequence (decoding)
// take the recurrence as it stands, token after token.  Longer portions go tile by tile: inside a tile the recurrence
// is solved in closed form, so that no sum over the state waits for the token before it.  With G_t the product of the
// tile's gammas up to t and S0 the state at the tile's start,
//     w_t = beta_t (v_t - G_t S0^T k_t) - sum_{j<t} A_tj w_j,      A_tj = beta_t (G_t / G_j) (k_t . k_j)
//     o_t = G_t S0^T q_t + sum_{j<=t} Q_tj w_j,                    Q_tj = (G_t / G_j) (q_t . k_j)
//     S   = G_last S0 + sum_j (G_last / G_j) k_j w_j^T
// which is the recurrence written out; G_t / G_j is a running product of gammas, never a division.
#include "common.cuh"

using namespace dli;

namespace {

constexpr int TILE = 16;  // tokens of a tile: the span over which the recurrence is solved at once

__device__ __forceinline__ float softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid(float x) { return 1.f / (1.f + expf(-x)); }

// Row of the float32 buffer that the first two kernels write for a token (G q/k heads of d, H heads of dv):
//   q [G d] | k [G d] | v [H dv] | per head: beta, G_t, G_last / G_t, gamma | A_t. [H][TILE] | Q_t. [H][TILE]
// `stride` floats apart; every part starts on a 16-byte boundary.  The second index of A and Q counts the tokens of the
// token's tile (entries the formulas do not have are zero).  q and k are unit vectors (sum of squares + unit_eps inside
// the root), q also times d^-1/2.
struct RowLayout {
  int q, k, v, sc, a, qm, stride;
};
__host__ __device__ inline RowLayout row_layout(int G, int d, int H, int dv) {
  RowLayout r;
  r.q = 0;
  r.k = G * d;
  r.v = 2 * G * d;
  r.sc = (r.v + H * dv + 3) & ~3;
  r.a = r.sc + 4 * H;
  r.qm = r.a + H * TILE;
  r.stride = r.qm + H * TILE;
  return r;
}

// One block per token; a warp per q/k head for the unit vectors, then all threads for v, beta and gamma.
//   qkv [n, 2 G d + H dv]: q | k | v after convolution and activation; b and a_raw are columns b_col + head and
//   a_col + head of u.
// own_qk (steps that walk token after token and skip the second kernel): the token's own q . k goes to its place in
// the token's row of Q, for every head of the q/k head.
template <typename T>
__global__ void delta_prep_kernel(float* __restrict__ x32, const T* __restrict__ qkv, const T* __restrict__ u, long long u_stride, int b_col,
                                  int a_col, const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                  const int* __restrict__ seq_of_token, const int* __restrict__ q_start, int own_qk, int H, int G, int d, int dv,
                                  float unit_eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int C = 2 * G * d + H * dv;
  const RowLayout L = row_layout(G, d, H, dv);
  const T* row = qkv + (size_t)t * C;
  float* out = x32 + (size_t)t * L.stride;
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
      out[L.q + g * d + i] = to_float(q[i]) * rq;
      out[L.k + g * d + i] = to_float(k[i]) * rk;
    }
    if (own_qk) {
      const int first = q_start[seq_of_token[t]];
      const int r = t >= first ? (t - first) % TILE : 0;
      const int fan = H / G;
      for (int j = lane; j < fan; j += 32) out[L.qm + (g * fan + j) * TILE + r] = qk * rq * rk;
    }
  }
  for (int e = threadIdx.x; e < H * dv; e += blockDim.x) out[L.v + e] = to_float(row[2 * G * d + e]);
  const T* urow = u + (size_t)t * u_stride;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    out[L.sc + 4 * h] = sigmoid(to_float(urow[b_col + h]));
    out[L.sc + 4 * h + 3] = expf(-expf(A_log[h]) * softplus(to_float(urow[a_col + h]) + dt_bias[h]));
  }
}

// One block per token t, r-th of its tile (tiles are counted from its sequence's first token of this step).  A warp per
// (q/k head, j <= r) computes k_t . k_j and q_t . k_j from the unit vectors of the first kernel; then a thread per
// (head, j) multiplies in the decays between the two tokens, and a thread per head computes G_t and G_last / G_t.
__global__ void delta_pairs_kernel(float* __restrict__ x32, const int* __restrict__ seq_of_token, const int* __restrict__ q_start, int n, int H,
                                   int G, int d, int dv) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float dots[];  // [G][TILE] k . k, [G][TILE] q . k
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const RowLayout L = row_layout(G, d, H, dv);
  const int s = seq_of_token[t];
  const int first = q_start[s], last = q_start[s + 1];
  const int r = t >= first ? (t - first) % TILE : 0;
  // the tile's last token (rows that pad a replayed graph belong to no sequence: they only have to stay inside the buffer)
  const int tile_end = min((t < last && t - r + TILE > last) ? last - 1 : t - r + TILE - 1, n - 1);
  float* mine = x32 + (size_t)t * L.stride;
  for (int e = warp; e < G * (r + 1); e += warps) {
    const int g = e / (r + 1), j = e - g * (r + 1);
    const float* kj = x32 + (size_t)(t - r + j) * L.stride + L.k + g * d;
    const float* kt = mine + L.k + g * d;
    const float* qt = mine + L.q + g * d;
    float kk = 0.f, qk = 0.f;
    for (int i = lane; i < d; i += 32) {
      const float x = kj[i];
      kk = fmaf(kt[i], x, kk);
      qk = fmaf(qt[i], x, qk);
    }
    kk = warp_sum(kk); qk = warp_sum(qk);
    if (lane == 0) {
      dots[g * TILE + j] = kk;
      dots[(G + g) * TILE + j] = qk;
    }
  }
  __syncthreads();
  const int fan = H / G;
  for (int e = threadIdx.x; e < H * TILE; e += blockDim.x) {
    const int h = e / TILE, j = e - h * TILE;
    float a = 0.f, q = 0.f;
    if (j <= r) {
      float run = 1.f;  // G_t / G_j: the gammas of the tokens behind j up to t
      for (int i = j + 1; i <= r; ++i) run *= x32[(size_t)(t - r + i) * L.stride + L.sc + 4 * h + 3];
      q = run * dots[(G + h / fan) * TILE + j];
      if (j < r) a = mine[L.sc + 4 * h] * run * dots[(h / fan) * TILE + j];
    }
    mine[L.a + e] = a;
    mine[L.qm + e] = q;
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    float up = 1.f, behind = 1.f;
    for (int i = t - r; i <= t; ++i) up *= x32[(size_t)i * L.stride + L.sc + 4 * h + 3];
    for (int i = t + 1; i <= tile_end; ++i) behind *= x32[(size_t)i * L.stride + L.sc + 4 * h + 3];
    mine[L.sc + 4 * h + 1] = up;
    mine[L.sc + 4 * h + 2] = behind;
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

// A column's share of the state: thread nl of the NS that share column `col` holds rows i = (kk * NS + nl) * 4 + j.
template <int DPT, int NS>
__device__ __forceinline__ void load_state(float (&S)[DPT], const float* S0, int nl, int d, bool live) {
  const bool vec = (d & 3) == 0;
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
}
template <int DPT, int NS>
__device__ __forceinline__ void store_state(const float (&S)[DPT], float* S0, int nl, int d) {
  const bool vec = (d & 3) == 0;
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

// ---------------------------------------------------------------- token after token (steps of few tokens a sequence)
// A CTA owns CB value columns of one head of one sequence; NS threads share a column.  The step's tokens come through
// shared memory in groups of TB, two groups in turn: while one is walked, asynchronous copies bring the next (16 bytes
// a copy where the sizes keep every run aligned, VEC; 4 bytes otherwise).  With both read-outs taken from the state
// before the token's write,
//     a = S^T k,  c = S^T q   (one pass over the column, two sums, reduced over the NS threads together)
//     w = beta (v - gamma a),  o = gamma c + w (k . q),  S <- gamma S + k w
// The sums are added in an order that the sizes fix.  state [slots, H, dv, d]: a column's d numbers are contiguous.
template <int DPT, int NS, int TB, bool VEC>
__global__ void __launch_bounds__(256) delta_rule_walk_kernel(float* __restrict__ o, const float* __restrict__ x32, float* __restrict__ state,
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
  const int inner = heads * dv;
  const RowLayout L = row_layout(kv_heads, d, heads, dv);
  const int first = q_start[s], last = q_start[s + 1];
  if (first >= last) return;
  const int vcnt = min(CB, dv - c0);

  auto fetch = [&](int tile, int buf) {
    const int cnt = min(TB, last - tile);
    constexpr int U = VEC ? 4 : 1;
    const int du = d / U, vu = vcnt / U, per_tok = 2 * du + vu + 3;
    for (int e = tid; e < cnt * per_tok; e += blockDim.x) {
      const int tok = e / per_tok, it = e - tok * per_tok;
      const float* src = x32 + (size_t)(tile + tok) * L.stride;
      const int slot = buf * TB + tok;
      if (it < 2 * du) {
        const bool is_k = it >= du;
        const int i = (is_k ? it - du : it) * U;
        float* dst = (is_k ? ks : qs) + slot * DP + i;
        if (VEC) cp_async16(dst, src + (is_k ? L.k : L.q) + g * d + i);
        else cp_async4(dst, src + (is_k ? L.k : L.q) + g * d + i);
      } else if (it < 2 * du + vu) {
        const int i = (it - 2 * du) * U;
        if (VEC) cp_async16(vs + slot * CB + i, src + L.v + head * dv + c0 + i);
        else cp_async4(vs + slot * CB + i, src + L.v + head * dv + c0 + i);
      } else {
        const int j = it - 2 * du - vu;  // beta; gamma; q . k: the token's own entry of its row of Q
        const int at = j == 0 ? L.sc + 4 * head : (j == 1 ? L.sc + 4 * head + 3 : L.qm + head * TILE + (tile + tok - first) % TILE);
        cp_async4(sc + slot * 4 + j, src + at);
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
  float S[DPT];
  load_state<DPT, NS>(S, S0, nl, d, live);
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
    __syncthreads();  // this group's rows have landed, for every thread
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
    __syncthreads();  // the group has been walked: its o is complete, its rows may be overwritten
    for (int e = tid; e < cnt * CB; e += blockDim.x) {
      const int tok = e / CB, cc = e - tok * CB;
      if (cc < vcnt) o[(size_t)(tile + tok) * inner + head * dv + c0 + cc] = os[e];
    }
  }
  if (live) store_state<DPT, NS>(S, S0, nl, d);
}

// ---------------------------------------------------------------- tile by tile (portions)
// Sixteen threads share a column, thread nl holding rows i = (kk * 16 + nl) * 4 + j of it.  d and dv are multiples
// of 4.  Tiles of TILE = 16 tokens come through shared memory, two in turn (16-byte asynchronous copies; a token's
// copies are issued by a fixed group of threads, so no index is divided).  Per tile: every thread takes its share of
// the 2 x 16 sums over the state before the tile (all independent of one another); the sixteen threads of a column
// add them up so that thread nl ends with the sums of token nl; then, token by token, the thread of that token hands
// its w to the other fifteen by a shuffle and each subtracts (adds) its own row's coefficient times it: forward
// substitution and the read-out in sixteen short steps; last, all bring the state to the tile's end.  Rows of a last,
// partial tile are zero, which the formulas take as tokens that change nothing.
constexpr int AROW = 20;  // floats between the rows of A and Q in shared memory (16 used): spreads a column over the banks

template <int DPT>
__global__ void __launch_bounds__(256) delta_rule_tile_kernel(float* __restrict__ o, const float* __restrict__ x32, float* __restrict__ state,
                                                              const int* __restrict__ q_start, const int* __restrict__ state_slot, int heads,
                                                              int kv_heads, int d, int dv, int CB) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int NS = 16, TB = TILE;
  constexpr int DP = DPT * NS;
  extern __shared__ __align__(16) float smem[];
  float* ks = smem;                    // [2][TB][DP]
  float* qs = ks + 2 * TB * DP;        // [2][TB][DP]
  float* vs = qs + 2 * TB * DP;        // [2][TB][CB]
  float* am = vs + 2 * TB * CB;        // [2][TB][AROW]
  float* qm = am + 2 * TB * AROW;      // [2][TB][AROW]
  float* sc = qm + 2 * TB * AROW;      // [2][TB][4]: beta, G_t, G_last / G_t, gamma
  float* os = sc + 2 * TB * 4;         // [TB][CB]
  const int head = blockIdx.x, s = blockIdx.y;
  const int tid = threadIdx.x, nl = tid & (NS - 1), cl = tid / NS;
  const int c0 = blockIdx.z * CB, col = c0 + cl;
  const bool live = col < dv;
  const int g = head / (heads / kv_heads);
  const int inner = heads * dv;
  const RowLayout L = row_layout(kv_heads, d, heads, dv);
  const int first = q_start[s], last = q_start[s + 1];
  if (first >= last) return;
  const int vcnt = min(CB, dv - c0);
  const int per_tok = blockDim.x / TB, my_tok = tid / per_tok, my_sub = tid - my_tok * per_tok;  // (a CTA has a multiple of 16 threads)

  auto fetch = [&](int tile, int buf) {
    if (tile + my_tok < last) {
      const float* src = x32 + (size_t)(tile + my_tok) * L.stride;
      const int slot = buf * TB + my_tok;
      for (int i = my_sub * 4; i < d; i += per_tok * 4) {
        cp_async16(ks + slot * DP + i, src + L.k + g * d + i);
        cp_async16(qs + slot * DP + i, src + L.q + g * d + i);
      }
      for (int i = my_sub * 4; i < vcnt; i += per_tok * 4) cp_async16(vs + slot * CB + i, src + L.v + head * dv + c0 + i);
      for (int i = my_sub * 4; i < TB; i += per_tok * 4) {
        cp_async16(am + slot * AROW + i, src + L.a + head * TILE + i);
        cp_async16(qm + slot * AROW + i, src + L.qm + head * TILE + i);
      }
      if (my_sub == 0) cp_async16(sc + slot * 4, src + L.sc + 4 * head);
    }
    cp_async_commit();
  };
  // what the copies of a tile leave alone: rows beyond d, columns beyond dv, and the tokens a last tile does not have
  auto clear_rest = [&](int tile, int buf) {
    const int cnt = last - tile;
    if (cnt >= TB) return;
    for (int e = tid; e < (TB - cnt) * DP; e += blockDim.x) {
      ks[(buf * TB + cnt) * DP + e] = 0.f;
      qs[(buf * TB + cnt) * DP + e] = 0.f;
    }
    for (int e = tid; e < (TB - cnt) * CB; e += blockDim.x) vs[(buf * TB + cnt) * CB + e] = 0.f;
    for (int e = tid; e < (TB - cnt) * AROW; e += blockDim.x) {
      am[(buf * TB + cnt) * AROW + e] = 0.f;
      qm[(buf * TB + cnt) * AROW + e] = 0.f;
    }
    for (int e = tid; e < (TB - cnt) * 4; e += blockDim.x) sc[(buf * TB + cnt) * 4 + e] = 0.f;
  };

  if (d < DP || vcnt < CB) {
    for (int e = tid; e < 4 * TB * DP + 2 * TB * CB; e += blockDim.x) smem[e] = 0.f;
    __syncthreads();
  }
  clear_rest(first, 0);
  fetch(first, 0);
  float* S0 = state + (((size_t)state_slot[s] * heads + head) * dv + (live ? col : 0)) * d;
  float S[DPT];
  load_state<DPT, NS>(S, S0, nl, d, live);
  int buf = 0;
  for (int tile = first; tile < last; tile += TB, buf ^= 1) {
    const int cnt = min(TB, last - tile);
    const bool more = tile + TB < last;
    if (more) {
      clear_rest(tile + TB, buf ^ 1);
      fetch(tile + TB, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();  // this tile's rows have landed (or are zero), for every thread
    const float* kt = ks + buf * TB * DP;
    const float* qt = qs + buf * TB * DP;
    const float* st = sc + buf * TB * 4;
    // ---- the sums over the state before the tile
    float a[TB], c[TB];
#pragma unroll
    for (int t = 0; t < TB; ++t) a[t] = c[t] = 0.f;
#pragma unroll
    for (int kk = 0; kk < DPT / 4; ++kk) {
#pragma unroll
      for (int t = 0; t < TB; ++t) {
        const float4 k = reinterpret_cast<const float4*>(kt + t * DP)[kk * NS + nl];
        const float4 q = reinterpret_cast<const float4*>(qt + t * DP)[kk * NS + nl];
        a[t] = fmaf(S[4 * kk], k.x, a[t]);
        a[t] = fmaf(S[4 * kk + 1], k.y, a[t]);
        a[t] = fmaf(S[4 * kk + 2], k.z, a[t]);
        a[t] = fmaf(S[4 * kk + 3], k.w, a[t]);
        c[t] = fmaf(S[4 * kk], q.x, c[t]);
        c[t] = fmaf(S[4 * kk + 1], q.y, c[t]);
        c[t] = fmaf(S[4 * kk + 2], q.z, c[t]);
        c[t] = fmaf(S[4 * kk + 3], q.w, c[t]);
      }
    }
    // ---- sixteen sums over sixteen threads: a thread keeps the half of its sums that its bit of nl names and adds what
    // its partner had of them; after four rounds thread nl holds the sum of token nl
#pragma unroll
    for (int half = TB / 2, bit = NS / 2; half >= 1; half >>= 1, bit >>= 1) {
      const bool upper = (nl & bit) != 0;
#pragma unroll
      for (int i = 0; i < half; ++i) {
        const float give_a = upper ? a[i] : a[i + half], keep_a = upper ? a[i + half] : a[i];
        const float give_c = upper ? c[i] : c[i + half], keep_c = upper ? c[i + half] : c[i];
        a[i] = keep_a + __shfl_xor_sync(0xffffffffu, give_a, bit);
        c[i] = keep_c + __shfl_xor_sync(0xffffffffu, give_c, bit);
      }
    }
    // ---- forward substitution and read-out, a token a step
    const float4 mine = *reinterpret_cast<const float4*>(st + nl * 4);  // beta, G, G_last / G, gamma of token nl
    float rhs = mine.x * (vs[(buf * TB + nl) * CB + cl] - mine.y * a[0]);
    float out = mine.y * c[0];
    const float* arow = am + (buf * TB + nl) * AROW;
    const float* qrow = qm + (buf * TB + nl) * AROW;
    float w[TB];
    const int lane = tid & 31, base = lane & ~(NS - 1);
#pragma unroll
    for (int t = 0; t < TB; ++t) {
      w[t] = __shfl_sync(0xffffffffu, rhs, base + t);  // token t's w is final: every row before it has been subtracted
      rhs = fmaf(-arow[t], w[t], rhs);                 // (A_lt is zero unless t < l)
      out = fmaf(qrow[t], w[t], out);                  // (Q_lt is zero unless t <= l)
    }
    os[nl * CB + cl] = out;
    // ---- the state at the tile's end: S = G_last S + sum_t (G_last / G_t) w_t k_t
    const float g_last = st[(cnt - 1) * 4 + 1];
#pragma unroll
    for (int t = 0; t < TB; ++t) w[t] *= st[t * 4 + 2];
#pragma unroll
    for (int kk = 0; kk < DPT / 4; ++kk) {
      float s0 = g_last * S[4 * kk], s1 = g_last * S[4 * kk + 1], s2 = g_last * S[4 * kk + 2], s3 = g_last * S[4 * kk + 3];
#pragma unroll
      for (int t = 0; t < TB; ++t) {
        const float4 k = reinterpret_cast<const float4*>(kt + t * DP)[kk * NS + nl];
        s0 = fmaf(k.x, w[t], s0);
        s1 = fmaf(k.y, w[t], s1);
        s2 = fmaf(k.z, w[t], s2);
        s3 = fmaf(k.w, w[t], s3);
      }
      S[4 * kk] = s0; S[4 * kk + 1] = s1; S[4 * kk + 2] = s2; S[4 * kk + 3] = s3;
    }
    __syncthreads();  // the tile is done: its o is complete, its rows may be overwritten
    for (int e = tid; e < cnt * CB; e += blockDim.x) {
      const int tok = e / CB, cc = e - tok * CB;
      if (cc < vcnt) o[(size_t)(tile + tok) * inner + head * dv + c0 + cc] = os[e];
    }
  }
  if (live) store_state<DPT, NS>(S, S0, nl, d);
}

// columns per CTA: as many as 256 threads hold, fewer for narrow heads and where it takes smaller CTAs to give every SM two
inline int columns_per_cta(int ns, int heads, int num_seqs, int dv) {
  const int most = 256 / ns;
  int CB = dv >= most ? most : ((dv + 7) / 8) * 8;
  while (CB > 8 && (long long)heads * num_seqs * ((dv + CB - 1) / CB) < 2 * sm_count()) CB /= 2;
  return ((CB + 7) / 8) * 8;
}

template <typename K, typename... Args>
int launch_sized(K kernel, MaxPerDevice& set, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  if ((int)smem > 48 * 1024 && set.here() < (int)smem) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    set.here() = (int)smem;
  }
  return (int)launch_pdl(kernel, grid, block, smem, stream, 1, args...);
}

template <int DPT, int NS, int TB>
int launch_walk(float* o, const float* x32, float* state, const int* q_start, const int* state_slot, int num_seqs, int heads, int kv_heads, int d,
                int dv, cudaStream_t stream) {
  const int CB = columns_per_cta(NS, heads, num_seqs, dv);
  const dim3 grid(heads, num_seqs, (dv + CB - 1) / CB), block(CB * NS);
  const size_t smem = (size_t)(4 * TB * DPT * NS + 2 * TB * CB + 2 * TB * 4 + TB * CB) * sizeof(float);
  // 16-byte copies: every run of the float32 rows starts and ends on a 16-byte boundary
  const bool vec = (d % 4) == 0 && (dv % 4) == 0 && (((uintptr_t)x32) & 15) == 0;
  static MaxPerDevice set_vec, set_any;
  if (vec)
    return launch_sized(delta_rule_walk_kernel<DPT, NS, TB, true>, set_vec, grid, block, smem, stream, o, x32, state, q_start, state_slot, heads,
                        kv_heads, d, dv, CB);
  return launch_sized(delta_rule_walk_kernel<DPT, NS, TB, false>, set_any, grid, block, smem, stream, o, x32, state, q_start, state_slot, heads,
                      kv_heads, d, dv, CB);
}

template <int DPT>
int launch_tiles(float* o, const float* x32, float* state, const int* q_start, const int* state_slot, int num_seqs, int heads, int kv_heads, int d,
                 int dv, cudaStream_t stream) {
  const int CB = columns_per_cta(16, heads, num_seqs, dv);
  const dim3 grid(heads, num_seqs, (dv + CB - 1) / CB), block(CB * 16);
  const size_t smem = (size_t)(4 * TILE * DPT * 16 + 2 * TILE * CB + 4 * TILE * AROW + 2 * TILE * 4 + TILE * CB) * sizeof(float);
  static MaxPerDevice set;
  return launch_sized(delta_rule_tile_kernel<DPT>, set, grid, block, smem, stream, o, x32, state, q_start, state_slot, heads, kv_heads, d, dv, CB);
}

// portions go tile by tile (sizes whose float32 rows keep every copy on 16-byte boundaries); steps of few tokens a
// sequence, and other sizes, token after token
inline bool takes_tiles(const float* x32, int d, int dv, int max_len) {
  return max_len > 4 && (d % 4) == 0 && (dv % 4) == 0 && (((uintptr_t)x32) & 15) == 0;
}

int launch_delta(float* o, const float* x32, float* state, const int* q_start, const int* state_slot, int num_seqs, int heads, int kv_heads, int d,
                 int dv, int max_len, cudaStream_t stream) {
#define DLI_ARGS o, x32, state, q_start, state_slot, num_seqs, heads, kv_heads, d, dv, stream
  if (takes_tiles(x32, d, dv, max_len)) {
    if (d <= 64) return launch_tiles<4>(DLI_ARGS);
    if (d <= 128) return launch_tiles<8>(DLI_ARGS);
    if (d <= 256) return launch_tiles<16>(DLI_ARGS);
    if (d <= 512) return launch_tiles<32>(DLI_ARGS);
  }
  // few tokens a sequence: token after token.  Threads per column: 8 hold the most state each; 16 for the largest heads.
  if (d <= 16) return launch_walk<4, 4, 16>(DLI_ARGS);
  if (d <= 32) return launch_walk<4, 8, 16>(DLI_ARGS);
  if (d <= 64) return launch_walk<8, 8, 16>(DLI_ARGS);
  if (d <= 128) return launch_walk<16, 8, 16>(DLI_ARGS);
  if (d <= 256) return launch_walk<16, 16, 8>(DLI_ARGS);
  if (d <= 512) return launch_walk<32, 16, 4>(DLI_ARGS);
#undef DLI_ARGS
  return DLI_ERR_UNSUPPORTED;
}

}  // namespace

DLI_EXPORT int dli_delta_rule_scan(float* o, const void* qkv, const void* u, long long u_stride, int b_col, int a_col, const float* dt_bias,
                                   const float* A_log, float* state, const int* seq_of_token, const int* q_start, const int* state_slot,
                                   float* scratch, int n, int num_seqs, int heads, int kv_heads, int d, int dv, int max_len, float unit_eps,
                                   int dtype, cudaStream_t stream) {
  if (num_seqs == 0 || n == 0) return 0;
  if (heads < 1 || kv_heads < 1 || heads % kv_heads || d < 1 || d > 512 || dv < 1 || num_seqs > 65535 || (dv + 7) / 8 > 65535 || !scratch)
    return DLI_ERR_UNSUPPORTED;
  const int threads = kv_heads >= 4 ? 128 : 64;
  const bool tiles = takes_tiles(scratch, d, dv, max_len);  // otherwise the walk needs of the second kernel only q . k of the token itself
  cudaError_t e;
  if (dtype == DLI_F32)
    e = launch_pdl((delta_prep_kernel<float>), dim3(n), dim3(threads), 0, stream, 1, scratch, (const float*)qkv, (const float*)u, u_stride, b_col,
                   a_col, dt_bias, A_log, seq_of_token, q_start, (int)!tiles, heads, kv_heads, d, dv, unit_eps);
  else
    e = launch_pdl((delta_prep_kernel<__nv_bfloat16>), dim3(n), dim3(threads), 0, stream, 1, scratch, (const __nv_bfloat16*)qkv,
                   (const __nv_bfloat16*)u, u_stride, b_col, a_col, dt_bias, A_log, seq_of_token, q_start, (int)!tiles, heads, kv_heads, d, dv,
                   unit_eps);
  if (e != cudaSuccess) return (int)e;
  if (!tiles) return launch_delta(o, scratch, state, q_start, state_slot, num_seqs, heads, kv_heads, d, dv, max_len, stream);
  const size_t pair_smem = (size_t)2 * kv_heads * TILE * sizeof(float);
  if (pair_smem > 48 * 1024) return DLI_ERR_UNSUPPORTED;
  e = launch_pdl(delta_pairs_kernel, dim3(n), dim3(128), pair_smem, stream, 1, scratch, seq_of_token, q_start, n, heads, kv_heads, d, dv);
  if (e != cudaSuccess) return (int)e;
  return launch_delta(o, scratch, state, q_start, state_slot, num_seqs, heads, kv_heads, d, dv, max_len, stream);
}
