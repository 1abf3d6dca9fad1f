// dn_seq_moe.cuh -- routed feed-forward of the batched sequence-mixer path (libdnet_b200_seq.so).
//
// A token's router logits z = W_r h + b_r are fp32; its `top` largest pick the experts, the softmax over those
// logits alone weighs them.  An expert is a clamped GLU: g = min(W_g h, limit), u = clamp(W_u h, -limit, limit),
// y = W_d (g sigmoid(1.702 g) (u + 1)).  The (token, choice) pairs P = N top are the rows of the expert products:
//   * a few tokens (decode): pair p is row p; one warp per output feature streams the chosen expert's weight row
//   * a prompt portion: k_moe_plan sorts the pairs by expert into 64-row tiles (a tile never spans two experts)
//     and the tile kernels gather the tokens' rows; k_moe_combine adds a token's pairs in the order of its choices
// so that a token's result does not depend on what else is in the step.
//
// A second router (k_router_scored) scores with a softmax over all experts, adds a learned correction for the choice
// only, keeps the best groups of neighbouring experts, and weighs the chosen with their uncorrected scores divided by
// their sum; its last outputs may stand for identity experts, which return the token's input and have no matrices:
// the plan gives them no tiles, the row kernels skip them, and the combining kernels add the input itself.  Experts
// are a clamped GLU or silu(gate) * up (`act`); a shared expert may be scaled by a sigmoid gate, one number a token.
#pragma once
#include "dn_seq_kernels.cuh"

namespace dnseq {

// one block per token: logits, top-k (ties: the lower index), softmax over the chosen; pos[p] = p
template <class T>
__global__ void __launch_bounds__(1024) k_router(const T* __restrict__ h, const T* __restrict__ Wr, const T* __restrict__ br, int W, int E,
                                                int top, int32_t* __restrict__ idx, float* __restrict__ wt, int32_t* __restrict__ pos) {
  extern __shared__ float zl[];      // [E]
  const int n = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const T* x = h + (size_t)n * W;
  for (int e = warp; e < E; e += nw) {
    const T* wr = Wr + (size_t)e * W;
    float a = 0.f;
    constexpr int V = Vec16<T>::n;
    if (W % V == 0 && ((((uintptr_t)h | (uintptr_t)Wr) & 15) == 0)) {      // rows start on 16-byte boundaries
      for (int c = lane * V; c < W; c += 32 * V) {
        T xv[V], wv[V];
        *reinterpret_cast<uint4*>(xv) = *reinterpret_cast<const uint4*>(x + c);
        *reinterpret_cast<uint4*>(wv) = *reinterpret_cast<const uint4*>(wr + c);
#pragma unroll
        for (int j = 0; j < V; j++) a = fmaf(ldf(xv + j), ldf(wv + j), a);
      }
    } else {
      for (int c = lane; c < W; c += 32) a = fmaf(ldf(x + c), ldf(wr + c), a);
    }
    a = warp_sum(a);
    if (lane == 0) zl[e] = a + (br ? ldf(br + e) : 0.f);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float best[16];
    int32_t* id = idx + (size_t)n * top;
    for (int j = 0; j < top; j++) {
      int arg = -1;
      float m = -INFINITY;
      for (int e = 0; e < E; e++) {
        bool taken = false;
        for (int i = 0; i < j; i++) taken = taken || id[i] == e;
        if (!taken && (arg < 0 || zl[e] > m)) { m = zl[e]; arg = e; }
      }
      id[j] = arg;
      best[j] = m;
    }
    float s = 0.f;
    const float zmax = best[0];
    for (int j = 0; j < top; j++) { best[j] = expf(best[j] - zmax); s += best[j]; }
    for (int j = 0; j < top; j++) {
      wt[(size_t)n * top + j] = best[j] / s;
      pos[(size_t)n * top + j] = n * top + j;
    }
  }
}

// dot product of two rows by one warp (16-byte loads when the rows allow); every lane returns the sum
template <class T>
__device__ __forceinline__ float warp_dot(const T* __restrict__ x, const T* __restrict__ w, int W, bool vec) {
  constexpr int V = Vec16<T>::n;
  const int lane = threadIdx.x & 31;
  float a = 0.f;
  if (vec) {
    for (int c = lane * V; c < W; c += 32 * V) {
      T xv[V], wv[V];
      *reinterpret_cast<uint4*>(xv) = *reinterpret_cast<const uint4*>(x + c);
      *reinterpret_cast<uint4*>(wv) = *reinterpret_cast<const uint4*>(w + c);
#pragma unroll
      for (int j = 0; j < V; j++) a = fmaf(ldf(xv + j), ldf(wv + j), a);
    }
  } else {
    for (int c = lane; c < W; c += 32) a = fmaf(ldf(x + c), ldf(w + c), a);
  }
  return warp_sum(a);
}

// Scored router, one block per token.  Et = real + identity experts.  Logits fp32; s = softmax over all Et; choice score
// c = s + corr; with groups > 0 the Et experts form `groups` equal runs, a run's score is its largest c, and only experts
// of the `keep` best runs can be chosen (ties: the lower index, for runs and experts alike); the `top` largest c choose;
// weights = s[chosen] / (their sum + 1e-20) * scale.  sg (optional): one more row, sgate[n] = sigmoid(sg . h).
template <class T>
__global__ void __launch_bounds__(1024) k_router_scored(const T* __restrict__ h, const T* __restrict__ Wr, const T* __restrict__ corr, int W, int Et,
                                                       int top, int groups, int keep, float scale, const T* __restrict__ sg,
                                                       int32_t* __restrict__ idx, float* __restrict__ wt, int32_t* __restrict__ pos,
                                                       float* __restrict__ sgate) {
  extern __shared__ float zl[];      // [Et] scores, [Et] choice scores
  float* ch = zl + Et;
  const int n = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const T* x = h + (size_t)n * W;
  const bool vec = W % Vec16<T>::n == 0 && ((((uintptr_t)h | (uintptr_t)Wr | (uintptr_t)(sg ? sg : Wr)) & 15) == 0);
  for (int e = warp; e < Et + (sg ? 1 : 0); e += nw) {
    const float a = warp_dot(x, e < Et ? Wr + (size_t)e * W : sg, W, vec);
    if (lane == 0) {
      if (e < Et) zl[e] = a;
      else sgate[n] = sigmoid_f(a);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float zmax = -INFINITY, sum = 0.f;
    for (int e = 0; e < Et; e++) zmax = fmaxf(zmax, zl[e]);
    for (int e = 0; e < Et; e++) { zl[e] = expf(zl[e] - zmax); sum += zl[e]; }
    for (int e = 0; e < Et; e++) { zl[e] /= sum; ch[e] = zl[e] + (corr ? ldf(corr + e) : 0.f); }
    if (groups > 0 && keep < groups) {
      const int per = Et / groups;
      // drop the groups - keep worst runs: repeatedly the run with the smallest best score (ties: the higher index goes)
      unsigned long long alive[4] = {~0ull, ~0ull, ~0ull, ~0ull};      // groups <= 256
      for (int d = 0; d < groups - keep; d++) {
        int worst = -1;
        float wv = INFINITY;
        for (int g = 0; g < groups; g++) {
          if (!((alive[g >> 6] >> (g & 63)) & 1ull)) continue;
          float best = -INFINITY;
          for (int e = g * per; e < (g + 1) * per; e++) best = fmaxf(best, ch[e]);
          if (worst < 0 || best <= wv) { wv = best; worst = g; }
        }
        alive[worst >> 6] &= ~(1ull << (worst & 63));
        for (int e = worst * per; e < (worst + 1) * per; e++) ch[e] = -INFINITY;
      }
    }
    int32_t* id = idx + (size_t)n * top;
    float ssum = 0.f;
    for (int j = 0; j < top; j++) {
      int arg = -1;
      float m = -INFINITY;
      for (int e = 0; e < Et; e++) {
        bool taken = false;
        for (int i = 0; i < j; i++) taken = taken || id[i] == e;
        if (!taken && (arg < 0 || ch[e] > m)) { m = ch[e]; arg = e; }
      }
      id[j] = arg;
      ssum += zl[arg];
    }
    for (int j = 0; j < top; j++) {
      wt[(size_t)n * top + j] = zl[id[j]] / (ssum + 1e-20f) * scale;
      pos[(size_t)n * top + j] = n * top + j;
    }
  }
}

// pairs sorted by expert: pos[p] = row of pair p, row_tok[row] = its token, and the table of tiles of `rows` rows
struct MoePlan {
  int32_t* pos;        // [P]
  int32_t* row_tok;    // [P]
  int32_t* tile_e;     // [max tiles]
  int32_t* tile_r0;
  int32_t* tile_rows;
  int32_t* n_tiles;    // [1]
};
constexpr int MOE_ROWS = 64;
// E: outputs of the router; experts from Ereal on are identity experts: their pairs get rows but no tiles
__global__ void __launch_bounds__(1024) k_moe_plan(const int32_t* __restrict__ idx, int P, int top, int E, int rows, MoePlan pl, int Ereal) {
  extern __shared__ int32_t cnt[];      // [E] counts, [E + 1] offsets
  int32_t* off = cnt + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) pl.pos[p] = atomicAdd(&cnt[idx[p]], 1);     // rank among its expert's pairs
  __syncthreads();
  if (threadIdx.x == 0) {
    int a = 0, t = 0;
    for (int e = 0; e < E; e++) {
      off[e] = a;
      for (int r = 0; e < Ereal && r < cnt[e]; r += rows, t++) {
        pl.tile_e[t] = e;
        pl.tile_r0[t] = a + r;
        pl.tile_rows[t] = min(rows, cnt[e] - r);
      }
      a += cnt[e];
    }
    *pl.n_tiles = t;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int row = off[idx[p]] + pl.pos[p];
    pl.pos[p] = row;
    pl.row_tok[row] = p / top;
  }
}

// expert tables of a layer: etab[0..E) gate, [E..2E) up, [2E..3E) down
// tile products on the CUDA cores (any sizes; fp32 accumulation in ascending k).  UP: act[row] = cglu(x W_g^T, x W_u^T)
// with x the row's token gathered from X [N, K]; DOWN: out[row] = act[row] W_d^T, fp32.
template <class T, bool UP>
__global__ void __launch_bounds__(256) k_moe_tiles(const T* __restrict__ X, const void* const* __restrict__ etab, int E, MoePlan pl,
                                                   void* __restrict__ Y, int O, int K, float limit, int act) {
  constexpr int BM = MOE_ROWS, BN = 64, BK = 16;
  const int t = blockIdx.y;
  if (t >= *pl.n_tiles) return;
  __shared__ float Xs[BK][BM + 4], Ws[BK][BN + 4], Vs[BK][BN + 4];
  __shared__ int32_t src[BM];
  const int e = pl.tile_e[t], r0 = pl.tile_r0[t], rows = pl.tile_rows[t];
  const T* Wa = (const T*)etab[UP ? e : 2 * E + e];
  const T* Wb = UP ? (const T*)etab[E + e] : nullptr;
  for (int r = threadIdx.x; r < BM; r += 256) src[r] = r < rows ? (UP ? pl.row_tok[r0 + r] : r0 + r) : -1;
  __syncthreads();
  const int o0 = blockIdx.x * BN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4], acc2[4][4], cmp[4][4], cmp2[4][4];      // block sums added with compensation, as in k_linear
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = acc2[i][j] = cmp[i][j] = cmp2[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int el = threadIdx.x; el < BM * BK; el += 256) {
      const int r = el / BK, c = el % BK;
      Xs[c][r] = (src[r] >= 0 && k0 + c < K) ? ldf(X + (size_t)src[r] * K + k0 + c) : 0.f;
      Ws[c][r] = (o0 + r < O && k0 + c < K) ? ldf(Wa + (size_t)(o0 + r) * K + k0 + c) : 0.f;
      if (UP) Vs[c][r] = (o0 + r < O && k0 + c < K) ? ldf(Wb + (size_t)(o0 + r) * K + k0 + c) : 0.f;
    }
    __syncthreads();
    float part[4][4], part2[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) part[i][j] = part2[i][j] = 0.f;
#pragma unroll
    for (int k = 0; k < BK; k++) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = Xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) part[i][j] = fmaf(a[i], w[j], part[i][j]);
      if (UP) {
#pragma unroll
        for (int j = 0; j < 4; j++) w[j] = Vs[k][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
          for (int j = 0; j < 4; j++) part2[i][j] = fmaf(a[i], w[j], part2[i][j]);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) {
        kahan_add(acc[i][j], cmp[i][j], part[i][j]);
        if (UP) kahan_add(acc2[i][j], cmp2[i][j], part2[i][j]);
      }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int r = ty * 4 + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int o = o0 + tx * 4 + j;
      if (o >= O) continue;
      if (UP) stf((T*)Y + (size_t)(r0 + r) * O + o, act_apply(act, acc[i][j], acc2[i][j], limit));
      else ((float*)Y)[(size_t)(r0 + r) * O + o] = acc[i][j];
    }
  }
}

// a few tokens: pair p = blockIdx.y is row p; one warp per output feature of the pair's expert.  Rows from P on (if the
// grid has them) are the shared expert's: row P + n is token n on the shared matrices, with its own width and limit.
struct SharedExpert {
  const void *gate, *up, *down;
  int ff;
  float limit;
  void* act;       // [N, ff]
  float* out;      // [N, W]
};
template <class T, bool UP>
__global__ void __launch_bounds__(256) k_moe_rows(const T* __restrict__ X, const void* const* __restrict__ etab, int E, const int32_t* __restrict__ idx,
                                                  int top, void* __restrict__ Y, int O, int K, float limit, int P, const T* __restrict__ h,
                                                  SharedExpert sh, int act) {
  const int p = blockIdx.y;
  const int o = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (p >= P) {
    const int n = p - P;
    if (UP) {
      if (o < sh.ff) linear_row<T>(h + (size_t)n * K, (const T*)sh.gate, (const T*)sh.up, (T*)sh.act + (size_t)n * sh.ff, false, 1, sh.ff, K, act, o, sh.limit);
    } else {
      if (o < O) linear_row<T>((const T*)sh.act + (size_t)n * sh.ff, (const T*)sh.down, (const T*)nullptr, sh.out + (size_t)n * O, true, 1, O, sh.ff, ACT_NONE, o, 0.f);
    }
    return;
  }
  const int e = idx[p];
  if (o >= O || e >= E) return;      // an identity expert has no matrices: the combining kernel adds the token's input
  if (UP)
    linear_row<T>(X + (size_t)(p / top) * K, (const T*)etab[e], (const T*)etab[E + e], (T*)Y + (size_t)p * O, false, 1, O, K, act, o, limit);
  else
    linear_row<T>(X + (size_t)p * K, (const T*)etab[2 * E + e], (const T*)nullptr, (float*)Y + (size_t)p * O, true, 1, O, K, ACT_NONE, o, 0.f);
}

// the tokens' rows in the order of the plan (the tensor-core tiles read them with one TMA descriptor): xg[row] = h[row_tok[row]]
template <class T>
__global__ void k_moe_gather(const T* __restrict__ h, const int32_t* __restrict__ row_tok, int W, T* __restrict__ xg) {
  const int row = blockIdx.x;
  const T* src = h + (size_t)row_tok[row] * W;
  T* dst = xg + (size_t)row * W;
  if ((W * (int)sizeof(T)) % 16 == 0) {
    for (int c = threadIdx.x; c < W * (int)sizeof(T) / 16; c += blockDim.x) reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
  } else {
    for (int c = threadIdx.x; c < W; c += blockDim.x) dst[c] = src[c];
  }
}

// y[n] = sum_j wt[n, j] out[pos[n, j]], the pairs of a token in the order of its choices.  With x: the sum (plus the
// shared expert's output y2, if any) goes through the dynamic-tanh norm after the sublayer straight into the plain
// residual, x[n] += dyt(y[n] + y2[n]), and y is not written.  idx / E / hid: pairs whose expert is >= E add the token's
// input instead of a row of eo; sgate: the shared expert's output is scaled per token.
template <class T>
__global__ void k_moe_combine(const float* __restrict__ eo, const float* __restrict__ wt, const int32_t* __restrict__ pos, int N, int W, int top,
                              float* __restrict__ y, float* __restrict__ x, const float* __restrict__ y2, const T* __restrict__ nw,
                              const T* __restrict__ nb, const T* __restrict__ nalpha, NextNorm<T> nx, const int32_t* __restrict__ idx, int E,
                              const T* __restrict__ hid, const float* __restrict__ sgate) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)N * W) return;
  const size_t n = i / W;
  const int c = (int)(i % W);
  float a = 0.f;
  for (int j = 0; j < top; j++) {
    const bool ident = idx && idx[n * top + j] >= E;      // an identity expert: the token's input itself
    a = fmaf(wt[n * top + j], ident ? ldf(hid + i) : eo[(size_t)pos[n * top + j] * W + c], a);
  }
  if (x) {
    const float xn = x[i] + dyt_f(a + (y2 ? (sgate ? sgate[n] : 1.f) * y2[i] : 0.f), ldf(nalpha), nw, nb, c);
    x[i] = xn;
    if (nx.alpha) stf(nx.h + i, dyt_f(xn, ldf(nx.alpha), nx.w, nx.b, c));      // the norm before the next sublayer, while x is at hand
  } else y[i] = a;
}

}  // namespace dnseq
