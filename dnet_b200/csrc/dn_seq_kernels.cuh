// dn_seq_kernels.cuh -- kernels of the batched sequence-mixer path (libdnet_b200_seq.so).
//
// A step is a ragged batch: N tokens of E entries (one entry = the next tokens of one live sequence, a portion of
// a prompt or a single decoded token).  Entry e owns the rows [ent_start[e], ent_start[e+1]) of every [N, *]
// buffer; its tokens sit at positions ent_pos0[e].. of the sequence in state slot ent_slot[e].  Everything a token
// computes depends only on its own row, its sequence's cache pages and its slot's recurrent state, and every
// reduction runs in an order that does not depend on N, E or the page / slot numbers.
//
// Mechanisms (each with its constants as arguments, none tied to one model family):
//   * residual streams ("hyper-connections"): S fp32 copies of the residual, a learned read-out before a sublayer
//     and a learned S x S mix + write-back after it; S = 0 is the plain residual sum
//   * RMS norm with a one-plus or a plain weight, over a row or over a whole projection
//   * short causal depthwise convolution over time with the last taps-1 inputs carried per sequence
//   * rotary embedding, interleaved pairs, on the first `rot` dims of each head
//   * paged softmax attention with a causal mask restricted to the query's own block of `chunk` positions
//     (chunk = 0: plain causal), GQA, separate key and value widths, optional reuse of another layer's pages
//   * gated delta rule: per head a [dk, dv] fp32 state with decay, delta-rule write and read-out
//   * dynamic-tanh norm (no statistics), capped scores, a sink term in the softmax denominator, per-head output gates
//   * (dn_seq_recur.cuh) decayed outer-product recurrences with a decay per key channel, token-shift mixing
//   * (dn_seq_moe.cuh) routed GLU experts, chosen by logits or by corrected, group-limited softmax scores
//   * (dn_seq_latent.cuh) latent attention: one compressed row per token in the cache, queries absorbed into it
//   * a sliding-window mask beside the block mask; rotary pairs interleaved or half apart
//   * RMS norm on a sublayer's output only (the sublayers read the residual itself)
//   * layer norm with weight and bias; a causal convolution over time on every sublayer's input with carried rows; a
//     hashed bigram row added to the embedding; RMS norm per head on q and k; rotary frequencies scaled by
//     interpolation; a query scale that grows with the logarithm of the position; values that are the keys
//   * a sliding window followed by mean-pooled blocks of the tokens that have left it (one softmax over both)
//   * (dn_seq_gdelta.cuh) generalized delta rule with a decay and a removal rate per key channel
// T is the storage type of weights and activations (bf16 or float); sums, norms, scores, positions, gates and
// states are fp32 in both.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dnseq {

typedef __nv_bfloat16 bf16;
constexpr int PAGE = 64;
constexpr int MAX_STREAMS = 8;

template <class T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <class T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
// v as the storage type holds it
template <class T> __device__ __forceinline__ float round_to(float v);
template <> __device__ __forceinline__ float round_to<float>(float v) { return v; }
template <> __device__ __forceinline__ float round_to<bf16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
// 16 bytes of the storage type (8 bf16 or 4 floats) from / to a 16-byte aligned address, as floats
template <class T> struct Vec16 { static constexpr int n = 16 / sizeof(T); };      // elements of 16 bytes
__device__ __forceinline__ void ldv(const float* p, float* o) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
__device__ __forceinline__ void ldv(const bf16* p, float* o) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; i++) { const float2 f = __bfloat1622float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void stv(float* p, const float* o) { *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]); }
__device__ __forceinline__ void stv(bf16* p, const float* o) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// sum over the block in a fixed order (warp partials added by index); red: >= 33 floats of shared memory
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
// clamped GLU: g = min(gate, limit), u = clamp(up, -limit, limit); g sigmoid(1.702 g) (u + 1)
__device__ __forceinline__ float clamped_glu_f(float g, float u, float limit) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * sigmoid_f(1.702f * g) * (u + 1.f);
}
// activation of a product's epilogue: 0 none; 1 gelu_tanh(a) * b; 2 tanh(a); 3 clamped GLU of (a, b) with `lim`;
// 4 silu(a) * b; 5 relu(a)^2.  A bias, where a product has one, is added to a before the activation.
constexpr int ACT_NONE = 0, ACT_GEGLU = 1, ACT_TANH = 2, ACT_CGLU = 3, ACT_SWIGLU = 4, ACT_RELU2 = 5;
__host__ __device__ __forceinline__ bool act_two(int act) { return act == ACT_GEGLU || act == ACT_CGLU || act == ACT_SWIGLU; }
__device__ __forceinline__ float act_apply(int act, float a, float b, float lim) {
  if (act == ACT_GEGLU) return gelu_tanh_f(a) * b;
  if (act == ACT_TANH) return tanhf(a);
  if (act == ACT_CGLU) return clamped_glu_f(a, b, lim);
  if (act == ACT_SWIGLU) return silu_f(a) * b;
  if (act == ACT_RELU2) { const float r = fmaxf(a, 0.f); return r * r; }
  return a;
}
// sum += v with the rounding error of the addition carried in c (compensated summation)
__device__ __forceinline__ void kahan_add(float& sum, float& c, float v) {
  const float y = __fsub_rn(v, c), t = __fadd_rn(sum, y);
  c = __fsub_rn(__fsub_rn(t, sum), y);
  sum = t;
}
// dynamic tanh: tanh(alpha x) w + b
template <class T>
__device__ __forceinline__ float dyt_f(float x, float alpha, const T* __restrict__ w, const T* __restrict__ b, int c) {
  return tanhf(alpha * x) * ldf(w + c) + ldf(b + c);
}

// the batch of one step, all device pointers
struct Batch {
  const int32_t* tok;        // [N]
  const int32_t* slot;       // [N]   state slot of the token's sequence
  const int32_t* pos;        // [N]   position in its sequence
  const int32_t* first;      // [N]   row of the first token of the token's entry
  const int32_t* ent_start;  // [E+1]
  const int32_t* ent_slot;   // [E]
  const int32_t* ent_pos0;   // [E]
  const int32_t* bt;         // [slots][max_pages] page of each 64-token block
  int N, E, max_pages;
  int max_len, row_tiles;    // longest entry of the step; sum over entries of ceil(tokens / 64)
  const int32_t* brow;       // [N]   row of the bigram table the token's embedding adds (null: the model has none)
};

// ---------------------------------------------------------------------------------------------------------------
// embedding -> residual streams
// nalpha != null: the embedding is dynamic-tanh normed; x0 != null: it is also kept aside (the loop's injection reads it);
// hout != null: also in the products' number format (models whose sublayers read the residual without a norm)
template <class T>
__global__ void k_embed(const T* __restrict__ embed, Batch b, float scale, int W, int S1, float* __restrict__ xs, const T* __restrict__ nw,
                        const T* __restrict__ nb, const T* __restrict__ nalpha, float* __restrict__ x0, T* __restrict__ hout,
                        const T* __restrict__ bigram) {
  const int n = blockIdx.x;
  const size_t row = (size_t)b.tok[n] * W;
  const float alpha = nalpha ? ldf(nalpha) : 0.f;
  const T* brow = bigram ? bigram + (size_t)b.brow[n] * W : nullptr;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float v = ldf(embed + row + c) * scale;
    if (brow) v += ldf(brow + c);      // the hashed (previous token, token) row, summed in fp32
    if (nalpha) v = dyt_f(v, alpha, nw, nb, c);
    for (int s = 0; s < S1; s++) xs[((size_t)s * b.N + n) * W + c] = v;
    if (x0) x0[(size_t)n * W + c] = v;
    if (hout) stf(hout + (size_t)n * W + c, v);      // the first sublayer reads the residual itself
  }
}

// ---------------------------------------------------------------------------------------------------------------
// the sublayers' input convolution, for V = 16 bytes of adjacent columns a thread: the V x TAPS weights of the columns
// c .. c + V - 1 are TAPS adjacent 16-byte vectors of cw [W, TAPS]; wl[i * TAPS + j] is column c + i, tap j
#define DN_TAPS_SWITCH(taps, CALL) \
  switch (taps) { case 1: { CALL(1); } break; case 2: { CALL(2); } break; case 3: { CALL(3); } break; case 4: { CALL(4); } break; case 5: { CALL(5); } break; \
                  case 6: { CALL(6); } break; case 7: { CALL(7); } break; case 8: { CALL(8); } break; default: { CALL(9); } break; }
template <class T, int TAPS>
__device__ __forceinline__ void canon_weights(const T* __restrict__ cw, int c, float* wl) {
  constexpr int V = Vec16<T>::n;
#pragma unroll
  for (int jj = 0; jj < TAPS; jj++) ldv(cw + (size_t)c * TAPS + jj * V, wl + jj * V);
}
// one token whose older rows are all carried rows st[0 .. TAPS - 2] (st[TAPS - 2] the newest): u is the token's normed row
// in shared memory; writes h = u + conv and moves the row into the carried ones.  Taps in ascending order, the token's own last.
template <class T, int TAPS>
__device__ __forceinline__ void canon_tail(const float* __restrict__ u, const T* __restrict__ cw, T* __restrict__ st, T* __restrict__ hrow, int W) {
  constexpr int V = Vec16<T>::n;
  for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {
    float wl[V * TAPS], a[V], x[V];
    canon_weights<T, TAPS>(cw, c, wl);
#pragma unroll
    for (int i = 0; i < V; i++) a[i] = 0.f;
#pragma unroll
    for (int j = 0; j + 1 < TAPS; j++) {
      ldv(st + (size_t)j * W + c, x);
#pragma unroll
      for (int i = 0; i < V; i++) a[i] += wl[i * TAPS + j] * x[i];
      if (j > 0) stv(st + (size_t)(j - 1) * W + c, x);      // row j moves to j - 1
    }
#pragma unroll
    for (int i = 0; i < V; i++) { x[i] = u[c + i]; a[i] = x[i] + (a[i] + wl[i * TAPS + TAPS - 1] * x[i]); }
    stv(hrow + c, a);
    if (TAPS > 1) stv(st + (size_t)(TAPS - 2) * W + c, x);
  }
}

// stream read-out (u = sum_s in[s] x_s, or x_0) + RMS norm with weight (1 + w) or w; rows[] optionally gathers.
// 16-byte loads of the streams when the width allows; a thread's partial sum of squares runs over its own columns in
// ascending order and the block adds the partials by index, so the result depends on W and the block size only.
template <class T>
__global__ void k_read_norm(const float* __restrict__ xs, int N, int W, int S, const T* __restrict__ hc_in, const T* __restrict__ nw,
                            int one_plus, int sum_all, float eps, const int32_t* __restrict__ rows, T* __restrict__ h,
                            const T* __restrict__ nb, const T* __restrict__ nalpha, int layer_norm,
                            const T* __restrict__ cw = nullptr, int taps = 0, const int32_t* __restrict__ slot_of = nullptr,
                            T* __restrict__ cstate = nullptr, size_t slot_stride = 0) {
  extern __shared__ __align__(16) float sm[];
  float* u = sm;            // [W]
  float* red = sm + W;      // [33]
  const int r = blockIdx.x, n = rows ? rows[r] : r;
  float cin[MAX_STREAMS];
  const int S1 = S > 0 ? S : 1;
  for (int s = 0; s < S1; s++) cin[s] = (S > 0 && !sum_all) ? ldf(hc_in + s) : 1.f;
  float ss = 0.f;
  if ((W & 3) == 0) {
    for (int c = threadIdx.x * 4; c < W; c += blockDim.x * 4) {
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < S1; s++) {
        const float4 x = *reinterpret_cast<const float4*>(xs + ((size_t)s * N + n) * W + c);
        a.x += cin[s] * x.x; a.y += cin[s] * x.y; a.z += cin[s] * x.z; a.w += cin[s] * x.w;
      }
      *reinterpret_cast<float4*>(u + c) = a;
      ss += a.x * a.x; ss += a.y * a.y; ss += a.z * a.z; ss += a.w * a.w;
    }
  } else {
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      float a = 0.f;
      for (int s = 0; s < S1; s++) a += cin[s] * xs[((size_t)s * N + n) * W + c];
      u[c] = a;
      ss += a * a;
    }
  }
  if (nalpha) {        // dynamic tanh: no statistics of the row enter
    __syncthreads();
    const float alpha = ldf(nalpha);
    for (int c = threadIdx.x; c < W; c += blockDim.x) stf(h + (size_t)r * W + c, dyt_f(u[c], alpha, nw, nb, c));
    return;
  }
  if (layer_norm) {    // (u - mean) / sqrt(variance + eps) * w + b: the mean first, then the mean of the squared deviations
    __syncthreads();
    float su = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) su += u[c];
    const float mean = block_sum(su, red) / (float)W;
    float sd = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) { const float d = u[c] - mean; sd += d * d; }
    const float rinv = 1.f / sqrtf(block_sum(sd, red) / (float)W + eps);
    if (cw) {
      for (int c = threadIdx.x; c < W; c += blockDim.x) u[c] = round_to<T>((u[c] - mean) * rinv * ldf(nw + c) + ldf(nb + c));
    } else {
      for (int c = threadIdx.x; c < W; c += blockDim.x) stf(h + (size_t)r * W + c, (u[c] - mean) * rinv * ldf(nw + c) + ldf(nb + c));
      return;
    }
  } else {
    ss = block_sum(ss, red);
    const float rinv = 1.f / sqrtf(ss / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      const float g = ldf(nw + c) + (one_plus ? 1.f : 0.f);
      if (cw) u[c] = round_to<T>(u[c] * rinv * g);
      else stf(h + (size_t)r * W + c, u[c] * rinv * g);
    }
    if (!cw) return;
  }
  // cw != null (steps whose entries bring one token each): the sublayer's input convolution in the same pass.  u holds the
  // normed row as the storage type rounds it; older rows come from the slot's carried rows st[0 .. taps - 2] (st[taps - 2] the
  // newest), which then take the row in.  Taps in ascending order, the token's own last, as k_canon.
  __syncthreads();
  T* st = cstate + (size_t)slot_of[n] * slot_stride;
  constexpr int V = Vec16<T>::n;
  if (W % V == 0 && ((((uintptr_t)st | (uintptr_t)cw) & 15) == 0)) {
#define DN_CALL(K) canon_tail<T, K>(u, cw, st, h + (size_t)r * W, W)
    DN_TAPS_SWITCH(taps, DN_CALL)
#undef DN_CALL
  } else {
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      const float v = u[c];
      float a = 0.f;
      for (int j = 0; j + 1 < taps; j++) {
        const float x = ldf(st + (size_t)j * W + c);
        a += ldf(cw + (size_t)c * taps + j) * x;
        if (j > 0) stf(st + (size_t)(j - 1) * W + c, x);
      }
      a += ldf(cw + (size_t)c * taps + taps - 1) * v;
      stf(h + (size_t)r * W + c, v + a);
      if (taps > 1) stf(st + (size_t)(taps - 2) * W + c, v);
    }
  }
}

// stream write-back: x_t <- sum_s mix[s][t] x_s + out[t] y   (S = 0: x <- x + y); VEC elements per thread
template <class T, int VEC>
__global__ void k_write_back(float* __restrict__ xs, int N, int W, int S, const T* __restrict__ mix, const T* __restrict__ out,
                             const float* __restrict__ y) {
  __shared__ float cm[MAX_STREAMS * MAX_STREAMS + MAX_STREAMS];
  for (int i = threadIdx.x; i < S * S + S; i += blockDim.x) cm[i] = i < S * S ? ldf(mix + i) : ldf(out + (i - S * S));
  __syncthreads();
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC, NW = (size_t)N * W;
  if (i >= NW) return;
  float yy[VEC], x[MAX_STREAMS][VEC];
  if (VEC == 4) *reinterpret_cast<float4*>(yy) = *reinterpret_cast<const float4*>(y + i);
  else yy[0] = y[i];
  if (S <= 0) {
    float* xp = xs + i;
    if (VEC == 4) {
      float4 v = *reinterpret_cast<float4*>(xp);
      v.x += yy[0]; v.y += yy[1]; v.z += yy[2]; v.w += yy[3];
      *reinterpret_cast<float4*>(xp) = v;
    } else xp[0] += yy[0];
    return;
  }
#pragma unroll
  for (int s = 0; s < MAX_STREAMS; s++) {
    if (s < S) {
      if (VEC == 4) *reinterpret_cast<float4*>(x[s]) = *reinterpret_cast<const float4*>(xs + (size_t)s * NW + i);
      else x[s][0] = xs[(size_t)s * NW + i];
    }
  }
  for (int t = 0; t < S; t++) {
    float a[VEC];
#pragma unroll
    for (int v = 0; v < VEC; v++) a[v] = 0.f;
#pragma unroll
    for (int s = 0; s < MAX_STREAMS; s++) {
      if (s < S) {
        const float m = cm[s * S + t];
#pragma unroll
        for (int v = 0; v < VEC; v++) a[v] += m * x[s][v];
      }
    }
    const float ot = cm[S * S + t];
#pragma unroll
    for (int v = 0; v < VEC; v++) a[v] += ot * yy[v];
    if (VEC == 4) *reinterpret_cast<float4*>(xs + (size_t)t * NW + i) = *reinterpret_cast<float4*>(a);
    else xs[(size_t)t * NW + i] = a[0];
  }
}

// a sublayer's output normed again (dynamic tanh) before it joins the plain residual:
//   x <- x + dyt(a y + b y2)        (y2 optional: two branches of a mixer, or routed + shared experts)
// and, since the norm before the next sublayer is elementwise too, its output in the same pass: h <- dyt'(x)
template <class T>
struct NextNorm { const T *w, *b, *alpha; T* h; };      // alpha == null: none
template <class T>
__global__ void k_dyt_add(float* __restrict__ x, size_t NW, int W, const float* __restrict__ y, float a, const float* __restrict__ y2, float b,
                          const T* __restrict__ nw, const T* __restrict__ nb, const T* __restrict__ nalpha, NextNorm<T> nx) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= NW) return;
  const int c = (int)(i % W);
  float v = a * y[i];
  if (y2) v += b * y2[i];
  const float xn = x[i] + dyt_f(v, ldf(nalpha), nw, nb, c);
  x[i] = xn;
  if (nx.alpha) stf(nx.h + i, dyt_f(xn, ldf(nx.alpha), nx.w, nx.b, c));
}
// the same, in place, for models with residual streams (the write-back follows): y <- dyt(a y + b y2)
template <class T>
__global__ void k_dyt_inplace(float* __restrict__ y, size_t NW, int W, float a, const float* __restrict__ y2, float b, const T* __restrict__ nw,
                              const T* __restrict__ nb, const T* __restrict__ nalpha) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= NW) return;
  float v = a * y[i];
  if (y2) v += b * y2[i];
  y[i] = dyt_f(v, ldf(nalpha), nw, nb, (int)(i % W));
}
// y <- a y + b y2 (two branches of a mixer joined without a norm)
__global__ void k_axpby(float* __restrict__ y, size_t NW, float a, const float* __restrict__ y2, float b) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < NW) y[i] = a * y[i] + b * y2[i];
}
// the loop's injection operand: cat[n] = [T(x[n]); T(x0[n])]
template <class T>
__global__ void k_loop_cat(const float* __restrict__ x, const float* __restrict__ x0, int N, int W, T* __restrict__ cat) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)N * 2 * W) return;
  const size_t n = i / (2 * W);
  const int c = (int)(i % (2 * W));
  stf(cat + i, c < W ? x[n * W + c] : x0[n * W + c - W]);
}
// logits <- s logits
__global__ void k_scale(float* __restrict__ z, size_t n, float s) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) z[i] *= s;
}
// logits <- cap tanh(logits / cap)
__global__ void k_softcap(float* __restrict__ z, size_t n, float cap) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) z[i] = cap * tanhf(z[i] / cap);
}

// h <- T(x): the input of a sublayer that reads the residual itself
template <class T>
__global__ void k_cast(const float* __restrict__ x, size_t n, T* __restrict__ h) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) stf(h + i, x[i]);
}

// A sublayer's output joins the plain residual through an RMS norm of its own:
//   v = a y + b y2 + sum_j wt[j] (expert output j | the token's input, for an identity expert) + gate sh      (all optional)
//   x <- x + v / sqrt(mean(v^2) + eps) * (w or 1 + w);   hout <- T(x), the input of the sublayer that follows
// One block per token; a thread's partial sum of squares runs over its own columns in ascending order and the block adds
// the partials by index, so a row's result depends on W and the block size only.
template <class T>
struct MoeSrc {
  const float* eo;          // [pairs, W] expert outputs (null: no routed part)
  const float* wt;          // [N, top]
  const int32_t* pos;       // [N, top] row of a pair in eo
  const int32_t* idx;       // [N, top] chosen expert; >= E: an identity expert
  int top, E;
  const T* hid;             // [N, W] the feed-forward's input
  const float* sh;          // [N, W] the shared expert's output (null: none)
  const float* sgate;       // [N] its gate, already through the sigmoid (null: 1)
};
template <class T>
__global__ void k_rms_join(float* __restrict__ x, int W, const float* __restrict__ y, float a, const float* __restrict__ y2, float b, MoeSrc<T> ms,
                           const T* __restrict__ nw, int one_plus, float eps, T* __restrict__ hout) {
  extern __shared__ __align__(16) float sm[];
  float* v = sm;            // [W]
  float* red = sm + W;      // [33]
  const size_t n = blockIdx.x, base = n * W;
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float u = y ? a * y[base + c] : 0.f;
    if (y2) u += b * y2[base + c];
    if (ms.eo) {
      for (int j = 0; j < ms.top; j++) {
        const int e = ms.idx[n * ms.top + j];
        const float src = e < ms.E ? ms.eo[(size_t)ms.pos[n * ms.top + j] * W + c] : ldf(ms.hid + base + c);
        u = fmaf(ms.wt[n * ms.top + j], src, u);
      }
    }
    if (ms.sh) u = fmaf(ms.sgate ? ms.sgate[n] : 1.f, ms.sh[base + c], u);
    v[c] = u;
    ss += u * u;
  }
  ss = block_sum(ss, red);
  const float rinv = 1.f / sqrtf(ss / (float)W + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float xn = x[base + c] + v[c] * rinv * (ldf(nw + c) + (one_plus ? 1.f : 0.f));
    x[base + c] = xn;
    if (hout) stf(hout + base + c, xn);
  }
}

// The two halves of a parallel mixer join the plain residual, each through an RMS norm of its own over the width:
//   x <- x + a y / rms(y) w1 + b y2 / rms(y2) w2        (plain weights)
// One block per token, sums in the fixed order of k_rms_join.
template <class T>
__global__ void k_rms2_join(float* __restrict__ x, int W, const float* __restrict__ y, float a, const T* __restrict__ w1, const float* __restrict__ y2,
                            float b, const T* __restrict__ w2, float eps) {
  __shared__ float red[33];
  const size_t base = (size_t)blockIdx.x * W;
  float s1 = 0.f, s2 = 0.f;
  // a thread's partial sums run over its own columns in ascending order, four adjacent ones at a time when the width allows
  const int V = (W & 3) == 0 ? 4 : 1;
  for (int c = threadIdx.x * V; c < W; c += blockDim.x * V)
    for (int i = 0; i < V; i++) {
      const float u = y[base + c + i], v = y2[base + c + i];
      s1 += u * u;
      s2 += v * v;
    }
  s1 = block_sum(s1, red);
  s2 = block_sum(s2, red);
  const float r1 = a / sqrtf(s1 / (float)W + eps), r2 = b / sqrtf(s2 / (float)W + eps);
  if (V == 4) {
    for (int c = threadIdx.x * 4; c < W; c += blockDim.x * 4) {
      const float4 u = *reinterpret_cast<const float4*>(y + base + c), v = *reinterpret_cast<const float4*>(y2 + base + c);
      float4 o = *reinterpret_cast<float4*>(x + base + c);
      o.x += u.x * r1 * ldf(w1 + c) + v.x * r2 * ldf(w2 + c);
      o.y += u.y * r1 * ldf(w1 + c + 1) + v.y * r2 * ldf(w2 + c + 1);
      o.z += u.z * r1 * ldf(w1 + c + 2) + v.z * r2 * ldf(w2 + c + 2);
      o.w += u.w * r1 * ldf(w1 + c + 3) + v.w * r2 * ldf(w2 + c + 3);
      *reinterpret_cast<float4*>(x + base + c) = o;
    }
    return;
  }
  for (int c = threadIdx.x; c < W; c += blockDim.x)
    x[base + c] += y[base + c] * r1 * ldf(w1 + c) + y2[base + c] * r2 * ldf(w2 + c);
}

// sum of the streams (inspection hook)
__global__ void k_stream_sum(const float* __restrict__ xs, int N, int W, int S1, float* __restrict__ o) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)N * W) return;
  float a = 0.f;
  for (int s = 0; s < S1; s++) a += xs[(size_t)s * N * W + i];
  o[i] = a;
}

// ---------------------------------------------------------------------------------------------------------------
// Y[N, O] = X[N, K] W[O, K]^T on CUDA-core tiles (any N, O, K).  fp32 accumulation: the 16 products of a k-block are
// summed from zero in ascending k, and the blocks' sums are added with a compensation term (Kahan), so the rounding
// error of a long reduction stays that of one block -- the fp32 mode's products then match the few-row kernel's
// (lane partials + tree) to the last bits, whatever the step's size.
// OUT32: write fp32 (residual-side outputs), else T.  act: ACT_* (the two-operand ones read W2 as well).
template <class T, bool OUT32>
__global__ void __launch_bounds__(256) k_linear(const T* __restrict__ X, const T* __restrict__ Wt, const T* __restrict__ W2,
                                                void* __restrict__ Y, int N, int O, int K, int act, float alim,
                                                const T* __restrict__ bias) {
  const bool two = act_two(act);
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float Xs[BK][BM + 4], Ws[BK][BN + 4], Vs[BK][BN + 4];
  const int n0 = blockIdx.y * BM, o0 = blockIdx.x * BN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4], acc2[4][4], cmp[4][4], cmp2[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = acc2[i][j] = cmp[i][j] = cmp2[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int e = threadIdx.x; e < BM * BK; e += 256) {
      const int r = e / BK, c = e % BK;
      Xs[c][r] = (n0 + r < N && k0 + c < K) ? ldf(X + (size_t)(n0 + r) * K + k0 + c) : 0.f;
      Ws[c][r] = (o0 + r < O && k0 + c < K) ? ldf(Wt + (size_t)(o0 + r) * K + k0 + c) : 0.f;
      if (two) Vs[c][r] = (o0 + r < O && k0 + c < K) ? ldf(W2 + (size_t)(o0 + r) * K + k0 + c) : 0.f;
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
      if (two) {
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
        if (two) kahan_add(acc2[i][j], cmp2[i][j], part2[i][j]);
      }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int n = n0 + ty * 4 + i;
    if (n >= N) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int o = o0 + tx * 4 + j;
      if (o >= O) continue;
      const float v = act_apply(act, acc[i][j] + (bias ? ldf(bias + o) : 0.f), acc2[i][j], alim);
      if (OUT32) ((float*)Y)[(size_t)n * O + o] = v;
      else stf((T*)Y + (size_t)n * O + o, v);
    }
  }
}

// Y[N, O] = X[N, K] W[O, K]^T for a few rows (N <= 8: decode steps): one warp per output feature streams its weight
// row once (16-byte loads when the row allows) against all N activations; lane partials in ascending k, one
// shuffle reduction.  The weights are read exactly once: HBM-bound.
// one warp, one output feature o of one product
template <class T>
__device__ __forceinline__ void linear_row(const T* __restrict__ X, const T* __restrict__ Wt, const T* __restrict__ W2, void* __restrict__ Y,
                                           bool out32, int N, int O, int K, int actc, int o, float alim = 0.f,
                                           const T* __restrict__ bias = nullptr) {
  constexpr int V = Vec16<T>::n;
  const bool act = act_two(actc);
  const int lane = threadIdx.x & 31;
  float acc[8], acc2[8];
#pragma unroll
  for (int i = 0; i < 8; i++) acc[i] = acc2[i] = 0.f;
  const T* wr = Wt + (size_t)o * K;
  const T* ur = act ? W2 + (size_t)o * K : nullptr;
  const bool vec = (K % V == 0) && ((((uintptr_t)Wt | (uintptr_t)X | (uintptr_t)(act ? W2 : Wt)) & 15) == 0);
  if (vec) {
    for (int k = lane * V; k < K; k += 32 * V) {
      T wv[V], uv[V];
      *reinterpret_cast<uint4*>(wv) = *reinterpret_cast<const uint4*>(wr + k);
      if (act) *reinterpret_cast<uint4*>(uv) = *reinterpret_cast<const uint4*>(ur + k);
#pragma unroll
      for (int i = 0; i < 8; i++) {
        if (i < N) {
          T xv[V];
          *reinterpret_cast<uint4*>(xv) = *reinterpret_cast<const uint4*>(X + (size_t)i * K + k);
#pragma unroll
          for (int j = 0; j < V; j++) {
            const float x = ldf(xv + j);
            acc[i] = fmaf(x, ldf(wv + j), acc[i]);
            if (act) acc2[i] = fmaf(x, ldf(uv + j), acc2[i]);
          }
        }
      }
    }
  } else {
    for (int k = lane; k < K; k += 32) {
      const float w = ldf(wr + k), u = act ? ldf(ur + k) : 0.f;
#pragma unroll
      for (int i = 0; i < 8; i++)
        if (i < N) {
          const float x = ldf(X + (size_t)i * K + k);
          acc[i] = fmaf(x, w, acc[i]);
          acc2[i] = fmaf(x, u, acc2[i]);
        }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; i++) {
    if (i < N) {
      float v = warp_sum(acc[i]) + (bias ? ldf(bias + o) : 0.f);
      v = act_apply(actc, v, act ? warp_sum(acc2[i]) : 0.f, alim);
      if (lane == 0) {
        if (out32) ((float*)Y)[(size_t)i * O + o] = v;
        else stf((T*)Y + (size_t)i * O + o, v);
      }
    }
  }
}
template <class T, bool OUT32>
__global__ void __launch_bounds__(256) k_linear_rows(const T* __restrict__ X, const T* __restrict__ Wt, const T* __restrict__ W2,
                                                     void* __restrict__ Y, int N, int O, int K, int act, float alim,
                                                     const T* __restrict__ bias) {
  const int o = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (o >= O) return;
  linear_row<T>(X, Wt, W2, Y, OUT32, N, O, K, act, o, alim, bias);
}
// several products of the same few rows in one launch (the projections of a mixer in a decode step): blocks are
// dealt to the products in order, 8 output features each
constexpr int MAX_SEGS = 8;
struct LinSegs {
  const void* X[MAX_SEGS];   // null: the launch's common input
  const void* W[MAX_SEGS];
  void* Y[MAX_SEGS];
  int O[MAX_SEGS];
  int out32[MAX_SEGS];
  int act[MAX_SEGS];         // ACT_NONE or ACT_TANH
  int n;
};
template <class T>
__global__ void __launch_bounds__(256) k_linear_rows_multi(const T* __restrict__ X, LinSegs sg, int N, int K) {
  int blk = blockIdx.x, i = 0;
  for (; i < sg.n; i++) {
    const int nb = (sg.O[i] + 7) / 8;
    if (blk < nb) break;
    blk -= nb;
  }
  if (i >= sg.n) return;
  const int o = blk * 8 + (threadIdx.x >> 5);
  if (o >= sg.O[i]) return;
  linear_row<T>(sg.X[i] ? (const T*)sg.X[i] : X, (const T*)sg.W[i], (const T*)nullptr, sg.Y[i], sg.out32[i] != 0, N, sg.O[i], K, sg.act[i], o);
}

// ---------------------------------------------------------------------------------------------------------------
// short causal convolution: value of input channel c at `back` steps before row n of its entry
template <class T>
__device__ __forceinline__ float conv_in(const T* __restrict__ U, int ldu, int c, int n, int local, int back, const T* __restrict__ st,
                                         int ldst, int taps) {
  if (back <= local) return ldf(U + (size_t)(n - back) * ldu + c);
  return ldf(st + (size_t)(taps - 1 - (back - local)) * ldst + c);   // carried inputs: st[taps-2] is the newest
}
template <class T>
__device__ __forceinline__ float conv_at(const T* __restrict__ U, int ldu, const T* __restrict__ cw, int c, int n, int local,
                                         const T* __restrict__ st, int ldst, int taps) {
  if (taps <= 0) return ldf(U + (size_t)n * ldu + c);
  float a = 0.f;
  for (int j = 0; j < taps; j++) a += ldf(cw + (size_t)c * taps + j) * conv_in(U, ldu, c, n, local, taps - 1 - j, st, ldst, taps);
  return a;
}

// after a step: the last taps-1 inputs of every entry become its slot's carried inputs; blockIdx.z picks the
// projection (q, k, v; a width of 0 means the layer has none of its own)
template <class T>
struct CarrySrc { const T* U[3]; int C[3]; };
template <class T>
__global__ void k_conv_carry(CarrySrc<T> src, int taps, Batch b, T* __restrict__ state, size_t slot_stride) {
  const int z = blockIdx.z, C = src.C[z];
  const int e = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const T* U = src.U[z];
  const int ldst = src.C[0] + src.C[1] + src.C[2], coff = z == 0 ? 0 : z == 1 ? src.C[0] : src.C[0] + src.C[1];
  const int s0 = b.ent_start[e], len = b.ent_start[e + 1] - s0;
  T* st = state + (size_t)b.ent_slot[e] * slot_stride + coff;
  T keep[8];
  const int m = taps - 1;
  for (int j = 0; j < m; j++) {
    const int idx = len - m + j;   // local index of the input that lands in st[j]
    keep[j] = idx >= 0 ? U[(size_t)(s0 + idx) * C + c] : st[(size_t)(m + idx) * ldst + c];
  }
  for (int j = 0; j < m; j++) st[(size_t)j * ldst + c] = keep[j];
}

// A sublayer's input passes a causal convolution over time: h[n] = hn[n] + sum_j w[:, j] hn[n - taps + 1 + j], rows
// before the entry's first one from the slot's carried rows (zeros in a fresh slot); taps in ascending order.  Grid
// (groups of CANON_TOK tokens, column groups); a thread takes 16 bytes of columns when the width allows, keeps their
// weights in registers and walks the group's tokens.  k_conv_carry afterwards makes the step's last rows the carried
// ones.  (Steps whose entries bring one token each run the convolution inside k_read_norm.)
constexpr int CANON_TOK = 8;
template <class T, int TAPS>
__device__ __forceinline__ void canon_tokens(const T* __restrict__ hn, const T* __restrict__ cw, const Batch& b, int W, const T* __restrict__ state,
                                             size_t slot_stride, T* __restrict__ h, int n0, int n1, int c) {
  constexpr int V = Vec16<T>::n;
  float wl[V * TAPS];
  canon_weights<T, TAPS>(cw, c, wl);
  for (int n = n0; n < n1; n++) {
    const int local = n - b.first[n];
    const T* st = state + (size_t)b.slot[n] * slot_stride;
    float a[V], x[V];
#pragma unroll
    for (int i = 0; i < V; i++) a[i] = 0.f;
#pragma unroll
    for (int j = 0; j < TAPS; j++) {
      const int back = TAPS - 1 - j;
      ldv(back <= local ? hn + (size_t)(n - back) * W + c : st + (size_t)(TAPS - 1 - (back - local)) * W + c, x);
#pragma unroll
      for (int i = 0; i < V; i++) a[i] += wl[i * TAPS + j] * x[i];
    }
#pragma unroll
    for (int i = 0; i < V; i++) a[i] = x[i] + a[i];      // x: the token's own row (the last tap)
    stv(h + (size_t)n * W + c, a);
  }
}
template <class T>
__global__ void k_canon(const T* __restrict__ hn, const T* __restrict__ cw, int taps, Batch b, int W, const T* __restrict__ state,
                        size_t slot_stride, T* __restrict__ h) {
  const int n0 = blockIdx.x * CANON_TOK, n1 = min(b.N, n0 + CANON_TOK);
  constexpr int V = Vec16<T>::n;
  if (W % V == 0 && slot_stride % V == 0 && ((((uintptr_t)state | (uintptr_t)cw) & 15) == 0)) {
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    if (c >= W) return;
#define DN_CALL(K) canon_tokens<T, K>(hn, cw, b, W, state, slot_stride, h, n0, n1, c)
    DN_TAPS_SWITCH(taps, DN_CALL)
#undef DN_CALL
    return;
  }
  for (int n = n0; n < n1; n++) {
    const int local = n - b.first[n];
    const T* st = state + (size_t)b.slot[n] * slot_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < W; c += gridDim.y * blockDim.x) {
      float a = 0.f;
      for (int j = 0; j < taps; j++) a += ldf(cw + (size_t)c * taps + j) * conv_in(hn, W, c, n, local, taps - 1 - j, st, W, taps);
      stf(h + (size_t)n * W + c, ldf(hn + (size_t)n * W + c) + a);
    }
  }
}

struct AttnPrep {
  int H, G, dk, dv, taps, rot;       // heads, kv heads, key dim, value dim, conv taps (0: none), rotated dims
  int own_kv;                        // 0: keys / values come from another layer's pages
  int norm;                          // 0: q and k pass without the RMS norm; 1: over the whole projection; 2: per head, one weight [dk]
  float eps;
  const float* inv_freq;             // [rot/2]
  int own_v;                         // 0: the values are the keys (nothing goes to the value pool)
  int half;                          // 1: rotary pairs (i, i + rot / 2), else (2i, 2i + 1)
  float mscale;                      // cos and sin are multiplied by this
  float qt_coef; int qt_every;       // q times 1 + qt_coef ln(floor((p + 1) / qt_every) + 1) (qt_every 0: no)
};

// attention mixer, between the projections and the scores: conv -> RMS norm (over the whole q / k projection or per
// head) -> rotary (angles, cos and sin fp32, one table a token) -> query scale -> q to scratch, k / v into the
// sequence's pages.  One block per token.  Shared memory: Cq + Ck + 34 + H + G + rot floats.
template <class T>
__global__ void k_attn_prep(AttnPrep a, Batch b, const T* __restrict__ Uq, const T* __restrict__ Uk, const T* __restrict__ Uv,
                            const T* __restrict__ cwq, const T* __restrict__ cwk, const T* __restrict__ cwv, const T* __restrict__ nq,
                            const T* __restrict__ nk, const T* __restrict__ cstate, size_t slot_stride, T* __restrict__ qout,
                            T* __restrict__ kpool, T* __restrict__ vpool) {
  extern __shared__ float sm[];
  // a layer that borrows its keys and values projects and carries q only
  const int Cq = a.H * a.dk, Ck = a.own_kv ? a.G * a.dk : 0, Cv = (a.own_kv && a.own_v) ? a.G * a.dv : 0, ldst = Cq + Ck + Cv;
  const int HG = a.H + (a.own_kv ? a.G : 0);
  float* qs = sm;
  float* ks = sm + Cq;
  float* red = ks + Ck;           // [34]
  float* hinv = red + 34;         // [H + G] inverse RMS of each head (norm 2)
  float* cst = hinv + a.H + a.G;  // [rot / 2] cos, then [rot / 2] sin
  float* snt = cst + a.rot / 2;
  const int n = blockIdx.x, slot = b.slot[n], p = b.pos[n];
  const int local = n - b.first[n];   // rows of this step that precede the token in its sequence
  const T* st = cstate + (size_t)slot * slot_stride;
  float sq = 0.f, sk = 0.f;
  for (int c = threadIdx.x; c < Cq; c += blockDim.x) {
    const float v = conv_at(Uq, Cq, cwq, c, n, local, st, ldst, a.taps);
    qs[c] = v;
    sq += v * v;
  }
  sq = block_sum(sq, red);
  if (a.own_kv) {
    for (int c = threadIdx.x; c < Ck; c += blockDim.x) {
      const float v = conv_at(Uk, Ck, cwk, c, n, local, st + Cq, ldst, a.taps);
      ks[c] = v;
      sk += v * v;
    }
    sk = block_sum(sk, red);
  }
  for (int i = threadIdx.x; i < a.rot / 2; i += blockDim.x) {
    float sn, cs;
    sincosf((float)p * a.inv_freq[i], &sn, &cs);
    cst[i] = cs * a.mscale;
    snt[i] = sn * a.mscale;
  }
  if (a.norm == 2) {      // one warp a head: lanes over the head's dims in ascending order, then the lanes pairwise
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int hh = w; hh < HG; hh += nw) {
      const float* src = hh < a.H ? qs + hh * a.dk : ks + (hh - a.H) * a.dk;
      float ss = 0.f;
      for (int d = lane; d < a.dk; d += 32) ss += src[d] * src[d];
      ss = warp_sum(ss);
      if (lane == 0) hinv[hh] = 1.f / sqrtf(ss / (float)a.dk + a.eps);
    }
  }
  __syncthreads();
  const float rq = a.norm == 1 ? 1.f / sqrtf(sq / (float)Cq + a.eps) : 1.f, rk = (a.norm == 1 && a.own_kv) ? 1.f / sqrtf(sk / (float)Ck + a.eps) : 1.f;
  const float qt = a.qt_every > 0 ? 1.f + a.qt_coef * logf((float)((p + 1) / a.qt_every + 1)) : 1.f;
  const int page = b.bt[(size_t)slot * b.max_pages + p / PAGE], prow = p % PAGE;
  T* krow = kpool + ((size_t)page * PAGE + prow) * Ck;
  // element d of head hh (q heads first, then k heads) after the norm
  auto val = [&](int hh, int d) -> float {
    const bool isq = hh < a.H;
    const int c = (isq ? hh : hh - a.H) * a.dk + d;
    const float x = isq ? qs[c] : ks[c];
    if (a.norm == 0) return x;
    if (a.norm == 1) return isq ? x * rq * ldf(nq + c) : x * rk * ldf(nk + c);
    return x * hinv[hh] * ldf((isq ? nq : nk) + d);
  };
  auto put = [&](int hh, int d, float y) {
    if (hh < a.H) stf(qout + (size_t)n * Cq + hh * a.dk + d, a.qt_every > 0 ? y * qt : y);
    else stf(krow + (hh - a.H) * a.dk + d, y);
  };
  if (a.half) {       // pairs (i, i + rot / 2); dims from rot up pass
    const int hr = a.rot / 2;
    for (int e = threadIdx.x; e < HG * a.dk; e += blockDim.x) {
      const int hh = e / a.dk, d = e % a.dk;
      float y = val(hh, d);
      if (d < hr) y = y * cst[d] - val(hh, d + hr) * snt[d];
      else if (d < a.rot) y = y * cst[d - hr] + val(hh, d - hr) * snt[d - hr];
      put(hh, d, y);
    }
  } else {
    const int halfk = a.dk / 2;
    // pairs (2i, 2i+1) of every head; odd dk leaves its last dim to the tail loop below
    for (int e = threadIdx.x; e < HG * halfk; e += blockDim.x) {
      const int hh = e / halfk, i = e % halfk;
      float x0 = val(hh, 2 * i), x1 = val(hh, 2 * i + 1);
      if (2 * i + 1 < a.rot) {
        const float y0 = x0 * cst[i] - x1 * snt[i], y1 = x1 * cst[i] + x0 * snt[i];
        x0 = y0; x1 = y1;
      }
      put(hh, 2 * i, x0);
      put(hh, 2 * i + 1, x1);
    }
    if (a.dk & 1)
      for (int hh = threadIdx.x; hh < HG; hh += blockDim.x) put(hh, a.dk - 1, val(hh, a.dk - 1));
  }
  if (Cv > 0) {
    T* vr = vpool + ((size_t)page * PAGE + prow) * Cv;
    for (int c = threadIdx.x; c < Cv; c += blockDim.x)
      stf(vr + c, conv_at(Uv, Cv, cwv, c, n, local, st + Cq + Ck, ldst, a.taps));
  }
}

// Mean-pooled blocks behind a sliding window.  Block j of a sequence holds the positions j P .. j P + P - 1; its pooled
// key (value) is the mean of the P keys (values) as the pages hold them.  A pooled row lives with the page of the
// block's last position e = j P + P - 1: row j - floor(64 (e / 64) / P) of that page's POOL_ROWS(P) = ceil(64 / P) rows
// in a pool of its own, so the sequence's block table finds it and a freed page frees its pooled rows.  A query at p
// with a window of `size` positions sees the blocks j < pooled_seen(p, size, P): those with j P + P - 1 <= p - size.
__host__ __device__ __forceinline__ int pool_rows(int P) { return (PAGE + P - 1) / P; }
__device__ __forceinline__ int pooled_seen(int p, int size, int P) { return (P > 0 && p - size + 1 > 0) ? (p - size + 1) / P : 0; }
__device__ __forceinline__ size_t pooled_row(const int32_t* __restrict__ bt, int j, int P) {
  const int pg = (j * P + P - 1) / PAGE;
  return (size_t)bt[pg] * pool_rows(P) + (j - (pg * PAGE) / P);
}
// after the step's keys and values are in their pages: the block of every token that ends one ((p + 1) % P == 0) pools
// it, positions in ascending order.  One block per token.
template <class T>
__global__ void k_pool_rows(Batch b, int P, int Ck, int Cv, const T* __restrict__ kpool, const T* __restrict__ vpool, T* __restrict__ pk,
                            T* __restrict__ pv) {
  const int n = blockIdx.x, p = b.pos[n];
  if ((p + 1) % P) return;
  const int32_t* bt = b.bt + (size_t)b.slot[n] * b.max_pages;
  const size_t row = pooled_row(bt, (p + 1) / P - 1, P);
  for (int c = threadIdx.x; c < Ck + Cv; c += blockDim.x) {
    const bool isk = c < Ck;
    const int cc = isk ? c : c - Ck, ld = isk ? Ck : Cv;
    const T* src = isk ? kpool : vpool;
    float a = 0.f;
    for (int j = p - P + 1; j <= p; j++) a += ldf(src + ((size_t)bt[j / PAGE] * PAGE + (j % PAGE)) * ld + cc);
    stf((isk ? pk : pv) + row * ld + cc, a / (float)P);
  }
}

// paged attention of one (token, head): keys lo..p with lo the start of the query's block of `chunk` positions
// (0: the sequence's start); fp32 scores and weights.  One block per (token, head); its AT_WARPS warps take the
// 32-key tiles (counted from lo) round-robin, each with its own running maximum, sum and output, and the block
// merges the warps' partials in warp order -- a row's result depends on its own position only.  A lane scores
// one key of the tile (its K row in 16-byte loads when the head size allows) and owns ceil(dv / 32) adjacent
// output dims.
// Extras of the scores (all optional): softcap > 0 caps a scaled score to softcap tanh(score / softcap); sink (one
// number per head) adds exp(sink_h) to the softmax denominator -- a key without a value, neither scaled nor capped;
// gate ([N, H] fp32 pre-activations) multiplies head h's output by sigmoid(gate[n, h]).
struct AttnExtra {
  float softcap;
  const void* sink;
  const float* gate;
  int window;      // 1: `chunk` is a sliding window -- a query at p sees the keys p - chunk + 1 .. p
  int v_ld;        // row stride of the value pool in elements (0: G dv); latent attention reads its values out of the key rows
  int pool;        // > 0 (with window): blocks of this many tokens wholly before the window are seen as one mean key / value each
  const void* pk;  // their pools [pages][pool_rows(pool)][row], strides as the token pools'
  const void* pv;
};
// keys a query at p sees: the pooled blocks first (virtual indices 0 .. nb - 1), then the tokens lo .. p
__device__ __forceinline__ int attn_pooled(int p, int chunk, const AttnExtra& ex) { return ex.pool > 0 ? pooled_seen(p, chunk, ex.pool) : 0; }
// first key a query at position p sees
__device__ __forceinline__ int attn_lo(int p, int chunk, int window) {
  if (chunk <= 0) return 0;
  return window ? max(0, p - chunk + 1) : (p / chunk) * chunk;
}
// Long rows of a small step are split over gridDim.z blocks: a row that sees n keys uses ceil(n / AT_SPLIT_KEYS) of
// them (at most gridDim.z), split z taking every nz-th group of AT_WARPS tiles; each writes its partial (maximum,
// sum, output) to scratch and k_attn_merge joins them in the order of z.  The split depends on the row's own
// position only.
constexpr int AT_MAX_SPLITS = 16, AT_SPLIT_ROWS = 64;
constexpr int AT_WARPS = 16;
constexpr int AT_SPLIT_KEYS = AT_WARPS * 32;
__device__ __forceinline__ int attn_splits(int keys, int zmax) { return min(zmax, max(1, (keys + AT_SPLIT_KEYS - 1) / AT_SPLIT_KEYS)); }
template <class T>
__device__ __forceinline__ void ld_vals(float (&v)[8], const T* p, int cnt, bool vec) {
  if (vec) {
    const int bytes = cnt * (int)sizeof(T);
    if (bytes == 16) {
      uint4 raw = *reinterpret_cast<const uint4*>(p);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int i = 0; i < 16 / (int)sizeof(T); i++) v[i] = ldf(e + i);
      return;
    }
    if (bytes == 8) {
      uint2 raw = *reinterpret_cast<const uint2*>(p);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int i = 0; i < 8 / (int)sizeof(T); i++) v[i] = ldf(e + i);
      return;
    }
  }
#pragma unroll
  for (int i = 0; i < 8; i++) if (i < cnt) v[i] = ldf(p + i);
}
template <class T, int MAXV>      // MAXV: value dims a lane owns at most (8: dv <= 256, 16: dv <= 512)
__global__ void __launch_bounds__(AT_WARPS * 32) k_attn(Batch b, const T* __restrict__ q, const T* __restrict__ kpool,
                                                        const T* __restrict__ vpool, int H, int G, int dk, int dv, int chunk, float scale,
                                                        AttnExtra ex, T* __restrict__ out, float* __restrict__ part_g) {
  extern __shared__ __align__(16) float sm[];
  constexpr int V = 16 / (int)sizeof(T);
  const int VPL = (dv + 31) / 32, dvp = VPL * 32;
  float* qs = sm;                                   // [dk rounded up to 4]
  float* part = sm + ((dk + 3) & ~3);               // [AT_WARPS][2 + dvp]
  const int n = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = h / (H / G), slot = b.slot[n], p = b.pos[n];
  const int lo = attn_lo(p, chunk, ex.window);
  const int nb = attn_pooled(p, chunk, ex), nkeys = nb + p - lo + 1;
  const int nz = attn_splits(nkeys, (int)gridDim.z), z = blockIdx.z;
  if (z >= nz) return;
  const int Ck = G * dk, Cv = ex.v_ld > 0 ? ex.v_ld : G * dv;
  for (int d = threadIdx.x; d < dk; d += blockDim.x) qs[d] = ldf(q + ((size_t)n * H + h) * dk + d);
  __syncthreads();
  const int32_t* bt = b.bt + (size_t)slot * b.max_pages;
  const bool kvec = (dk % V) == 0;                  // K rows start on 16-byte boundaries
  const int vcnt = min(VPL, max(0, dv - lane * VPL));
  // 8- or 16-byte value loads: a lane's run of VPL numbers must start on such a boundary in every row
  const bool vvec = (dv % 32) == 0 && ((size_t)Cv * sizeof(T)) % 16 == 0 && ((VPL * sizeof(T)) % 16 == 0 || VPL * sizeof(T) == 8);
  const int vbytes = VPL * (int)sizeof(T);
  const bool vraw = (dv % 32) == 0 && (vbytes == 4 || vbytes == 8 || vbytes == 16) && ((size_t)Cv * sizeof(T)) % vbytes == 0 &&
                    ((((uintptr_t)vpool | (uintptr_t)ex.pv) & 15) == 0);
  float m = -INFINITY, l = 0.f, acc[MAXV];
#pragma unroll
  for (int i = 0; i < MAXV; i++) acc[i] = 0.f;
  // virtual key v (pooled blocks first, then the tokens lo .. p) lives in row row_of(v) of the token pools, or, with bit 31
  // set, of the pooled pools; a lane finds its own key's row once and the value loop takes the rows from the lanes
  auto row_of = [&](int v) -> uint32_t {
    if (v < nb) return 0x80000000u | (uint32_t)pooled_row(bt, v, ex.pool);
    const int j = lo + v - nb;
    return (uint32_t)bt[j / PAGE] * PAGE + (uint32_t)(j % PAGE);
  };
  const T* kpl = (const T*)ex.pk;
  const T* vpl = (const T*)ex.pv;
  for (int j0 = (z * AT_WARPS + warp) * 32; j0 < nkeys; j0 += nz * AT_WARPS * 32) {
    const int j = j0 + lane;
    float s = -INFINITY;
    uint32_t myrow = 0;
    if (j < nkeys) {
      myrow = row_of(j);
      const T* kr = ((myrow >> 31) ? kpl : kpool) + (size_t)(myrow & 0x7fffffffu) * Ck + g * dk;
      {   // the key's value row is needed after the scores: ask for its lines now, so that the value loop finds them in L2
        const char* vrow = reinterpret_cast<const char*>(((myrow >> 31) ? vpl : vpool) + (size_t)(myrow & 0x7fffffffu) * Cv + g * dv);
        if (vrow != reinterpret_cast<const char*>(kr))
          for (int o = 0; o < dv * (int)sizeof(T); o += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(vrow + o));
      }
      float d0 = 0.f;
      if (kvec) {
#pragma unroll 8
        for (int d = 0; d < dk; d += V) {      // (unrolled: the loads of a long key row are issued ahead of the sums)
          uint4 raw = *reinterpret_cast<const uint4*>(kr + d);
          const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
          for (int x = 0; x < V; x++) d0 = fmaf(qs[d + x], ldf(e + x), d0);
        }
      } else {
        for (int d = 0; d < dk; d++) d0 = fmaf(qs[d], ldf(kr + d), d0);
      }
      s = d0 * scale;
      if (ex.softcap > 0.f) s = ex.softcap * tanhf(s / ex.softcap);
    }
    const float mn = fmaxf(m, warp_max(s));
    const float corr = expf(m - mn);      // exp(-inf) = 0 on the warp's first tile
    const float pj = j < nkeys ? expf(s - mn) : 0.f;
    l = l * corr + warp_sum(pj);
#pragma unroll
    for (int i = 0; i < MAXV; i++) acc[i] *= corr;
    const int cnt = min(32, nkeys - j0);
    if (vraw) {
      // a lane's run of values is one 4-, 8- or 16-byte load a row: the loads of eight rows are issued together, then
      // their sums run in the rows' order (rows beyond the tile repeat its last row with weight zero)
      for (int t0 = 0; t0 < cnt; t0 += 8) {
        uint4 raw[8];
        float pt[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
          const int t = min(t0 + u, cnt - 1);
          const uint32_t rw = __shfl_sync(0xffffffffu, myrow, t);
          pt[u] = t0 + u < cnt ? __shfl_sync(0xffffffffu, pj, t) : 0.f;
          const T* vr = ((rw >> 31) ? vpl : vpool) + (size_t)(rw & 0x7fffffffu) * Cv + g * dv + lane * VPL;
          if (vbytes == 16) raw[u] = *reinterpret_cast<const uint4*>(vr);
          else if (vbytes == 8) { const uint2 r2 = *reinterpret_cast<const uint2*>(vr); raw[u] = make_uint4(r2.x, r2.y, 0u, 0u); }
          else raw[u] = make_uint4(*reinterpret_cast<const uint32_t*>(vr), 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
          const T* e = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
          for (int i = 0; i < 16 / (int)sizeof(T); i++)
            if (i < MAXV && i < VPL) acc[i] = fmaf(pt[u], ldf(e + i), acc[i]);
        }
      }
      m = mn;
      continue;
    }
#pragma unroll 8
    for (int t = 0; t < cnt; t++) {
      const float pt = __shfl_sync(0xffffffffu, pj, t);
      const uint32_t rw = __shfl_sync(0xffffffffu, myrow, t);
      const T* vr = ((rw >> 31) ? vpl : vpool) + (size_t)(rw & 0x7fffffffu) * Cv + g * dv + lane * VPL;
#pragma unroll
      for (int i0 = 0; i0 < MAXV; i0 += 8) {
        if (i0 < vcnt) {
          float vv[8];
          ld_vals(vv, vr + i0, min(8, vcnt - i0), vvec);
#pragma unroll
          for (int i = 0; i < 8; i++)
            if (i0 + i < vcnt) acc[i0 + i] = fmaf(pt, vv[i], acc[i0 + i]);
        }
      }
    }
    m = mn;
  }
  float* mine = part + (size_t)warp * (2 + dvp);
  if (lane == 0) { mine[0] = m; mine[1] = l; }
#pragma unroll
  for (int i = 0; i < MAXV; i++)
    if (i < VPL) mine[2 + lane * VPL + i] = acc[i];
  __syncthreads();
  const bool split = nz > 1;      // the sink and the gate then wait for the merge
  const float snk = (ex.sink && !split) ? ldf((const T*)ex.sink + h) : -INFINITY;
  const float og = ex.gate ? sigmoid_f(ex.gate[(size_t)n * H + h]) : 1.f;
  float* pg = split ? part_g + (((size_t)n * H + h) * gridDim.z + z) * (2 + dvp) : nullptr;
  for (int d = threadIdx.x; d < dv; d += blockDim.x) {
    float M = snk;
    for (int w = 0; w < AT_WARPS; w++) M = fmaxf(M, part[(size_t)w * (2 + dvp)]);
    float L = (ex.sink && !split) ? expf(snk - M) : 0.f, a = 0.f;
    for (int w = 0; w < AT_WARPS; w++) {
      const float* pw = part + (size_t)w * (2 + dvp);
      const float f = expf(pw[0] - M);     // a warp that saw no tile has maximum -inf and weight 0
      L += pw[1] * f;
      a += pw[2 + d] * f;
    }
    if (split) {
      pg[2 + d] = a;
      if (d == 0) { pg[0] = M; pg[1] = L; }
    } else stf(out + ((size_t)n * H + h) * dv + d, a / L * og);
  }
}
// joins the partials of the rows that k_attn split (rows with one split are complete already); grid (N, H, 1)
template <class T>
__global__ void k_attn_merge(Batch b, int H, int dv, int chunk, int zmax, AttnExtra ex, const float* __restrict__ part_g, T* __restrict__ out) {
  const int n = blockIdx.x, h = blockIdx.y, p = b.pos[n];
  const int lo = attn_lo(p, chunk, ex.window);
  const int nz = attn_splits(attn_pooled(p, chunk, ex) + p - lo + 1, zmax);
  if (nz <= 1) return;
  const int dvp = (dv + 31) / 32 * 32;
  const float* pg = part_g + ((size_t)n * H + h) * zmax * (2 + dvp);
  const float snk = ex.sink ? ldf((const T*)ex.sink + h) : -INFINITY;
  const float og = ex.gate ? sigmoid_f(ex.gate[(size_t)n * H + h]) : 1.f;
  float M = snk;
  for (int z = 0; z < nz; z++) M = fmaxf(M, pg[(size_t)z * (2 + dvp)]);
  for (int d = threadIdx.x; d < dv; d += blockDim.x) {
    float L = ex.sink ? expf(snk - M) : 0.f, a = 0.f;
    for (int z = 0; z < nz; z++) {
      const float* pz = pg + (size_t)z * (2 + dvp);
      const float f = expf(pz[0] - M);
      L += pz[1] * f;
      a += pz[2 + d] * f;
    }
    stf(out + ((size_t)n * H + h) * dv + d, a / L * og);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// The same attention for prompt portions, bf16, on the warp-level tensor-core MMA (m16n8k16, fp32 accumulation).
// A block owns 64 consecutive query rows of one entry and one query head; its four warps take 16 rows each.  Keys
// and values come page by page (a 64-key tile is exactly one page) through shared memory.  Scores, the running
// maximum and the running sum are fp32; the weights enter the P V product as a bf16 pair (p = hi + lo, both
// products accumulated in fp32), which keeps 16 bits of each weight's mantissa.  Per row the key tiles are
// visited in ascending absolute position and a tile that the row does not see changes nothing, so a row's result
// does not depend on how the prompt was cut or what else is in the batch.
// DKP / DVP: head sizes rounded up to the template's; the padding is zero in shared memory.
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// rows x cols bf16 from global (row stride ld) into a padded shared tile [64][LDS]; rows >= valid and columns >= cols are zero
template <int LDS>
__device__ __forceinline__ void load_tile64(bf16* __restrict__ dst, const bf16* __restrict__ src, size_t ld, int cols, int valid) {
  const int vec = LDS / 8 - 1;     // 16-byte groups per row, the pad group left out
  for (int e = threadIdx.x; e < 64 * vec; e += blockDim.x) {
    const int r = e / vec, c = (e % vec) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < valid && c < cols) v = *reinterpret_cast<const uint4*>(src + (size_t)r * ld + c);
    *reinterpret_cast<uint4*>(dst + r * LDS + c) = v;
  }
}

// the same for pooled rows j0 .. j0 + valid - 1 of a sequence, each found through the block table (src: the pool's base plus
// the head group's offset)
template <int LDS>
__device__ __forceinline__ void load_tile64_rows(bf16* __restrict__ dst, const bf16* __restrict__ src, size_t ld, int cols, int valid,
                                                 const int32_t* __restrict__ bt, int j0, int P) {
  const int vec = LDS / 8 - 1;
  for (int e = threadIdx.x; e < 64 * vec; e += blockDim.x) {
    const int r = e / vec, c = (e % vec) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < valid && c < cols) v = *reinterpret_cast<const uint4*>(src + pooled_row(bt, j0 + r, P) * ld + c);
    *reinterpret_cast<uint4*>(dst + r * LDS + c) = v;
  }
}

constexpr int AT_ROWS = 64;      // query rows of a block, and keys of a tile (= PAGE)
template <int DKP, int DVP>
__global__ void __launch_bounds__(128) k_attn_tiles(Batch b, const bf16* __restrict__ q, const bf16* __restrict__ kpool,
                                                    const bf16* __restrict__ vpool, int H, int G, int dk, int dv, int chunk, float scale,
                                                    AttnExtra ex, bf16* __restrict__ out) {
  static_assert(PAGE == AT_ROWS, "a key tile is one page");
  constexpr int LQ = DKP + 8, LV = DVP + 8;
  extern __shared__ __align__(16) unsigned char smraw[];
  bf16* Qs = reinterpret_cast<bf16*>(smraw);
  bf16* Ks = Qs + AT_ROWS * LQ;
  // values that are the keys (one pool, equal tile shapes): the key tile is the value tile, nothing is staged twice
  const bool vk = DKP == DVP && dk == dv && vpool == kpool && ex.pv == ex.pk;
  bf16* Vs = vk ? Ks : Ks + AT_ROWS * LQ;
  // which entry and which of its 64-row tiles
  int e = 0, t = blockIdx.x;
  for (; e < b.E; e++) {
    const int nt = (b.ent_start[e + 1] - b.ent_start[e] + AT_ROWS - 1) / AT_ROWS;
    if (t < nt) break;
    t -= nt;
  }
  if (e >= b.E) return;
  const int h = blockIdx.y, g = h / (H / G);
  const int s0 = b.ent_start[e] + t * AT_ROWS, s1 = b.ent_start[e + 1];
  const int rows = min(AT_ROWS, s1 - s0);
  const int p_first = b.ent_pos0[e] + t * AT_ROWS, p_last = p_first + rows - 1;
  const int Ck = G * dk, Cv = ex.v_ld > 0 ? ex.v_ld : G * dv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  load_tile64<LQ>(Qs, q + ((size_t)s0 * H + h) * dk, (size_t)H * dk, dk, rows);
  __syncthreads();
  // this thread's two rows of its warp's 16
  const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
  const int p0 = r0 < rows ? p_first + r0 : -1, p1 = r1 < rows ? p_first + r1 : -1;
  const int lo0 = p0 >= 0 ? attn_lo(p0, chunk, ex.window) : 0, lo1 = p1 >= 0 ? attn_lo(p1, chunk, ex.window) : 0;
  const bool warp_live = warp * 16 < rows;
  uint32_t qf[DKP / 16][4];
#pragma unroll
  for (int kk = 0; kk < DKP / 16; kk++) ldsm_x4(qf[kk], Qs + (warp * 16 + (lane & 15)) * LQ + kk * 16 + (lane >> 4) * 8);
  float o[DVP / 8][4];
#pragma unroll
  for (int j = 0; j < DVP / 8; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const int32_t* bt = b.bt + (size_t)b.ent_slot[e] * b.max_pages;
  const int lo_tile = attn_lo(p_first, chunk, ex.window);
  // pooled blocks behind the window come first, 64 to a tile, in ascending block order; then the pages of the tokens
  const int nb0 = p0 >= 0 ? attn_pooled(p0, chunk, ex) : 0, nb1 = p1 >= 0 ? attn_pooled(p1, chunk, ex) : 0;
  const int nb_last = attn_pooled(p_last, chunk, ex), pool_tiles = (nb_last + AT_ROWS - 1) / AT_ROWS;
  const int tok0 = (lo_tile / PAGE) * PAGE, tok_tiles = p_last >= tok0 ? (p_last - tok0) / PAGE + 1 : 0;
  for (int it = 0; it < pool_tiles + tok_tiles; it++) {
    const bool pooled = it < pool_tiles;
    const int j0 = pooled ? it * AT_ROWS : tok0 + (it - pool_tiles) * PAGE;
    __syncthreads();
    if (pooled) {
      load_tile64_rows<LQ>(Ks, (const bf16*)ex.pk + (size_t)g * dk, (size_t)Ck, dk, min(AT_ROWS, nb_last - j0), bt, j0, ex.pool);
      if (!vk) load_tile64_rows<LV>(Vs, (const bf16*)ex.pv + (size_t)g * dv, (size_t)Cv, dv, min(AT_ROWS, nb_last - j0), bt, j0, ex.pool);
    } else {
      const size_t prow = (size_t)bt[j0 / PAGE] * PAGE;
      const int kvalid = min(PAGE, p_last - j0 + 1);      // rows of the page beyond the last query's position are not read
      load_tile64<LQ>(Ks, kpool + prow * Ck + (size_t)g * dk, (size_t)Ck, dk, kvalid);
      if (!vk) load_tile64<LV>(Vs, vpool + prow * Cv + (size_t)g * dv, (size_t)Cv, dv, kvalid);
    }
    __syncthreads();
    if (!warp_live) continue;
    float sc[8][4];
#pragma unroll
    for (int j = 0; j < 8; j++) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < DKP / 16; kk++) {
#pragma unroll
      for (int jj = 0; jj < 4; jj++) {     // two 8-key tiles per ldmatrix
        uint32_t kf[4];
        ldsm_x4(kf, Ks + (jj * 16 + (lane >> 4) * 8 + (lane & 7)) * LQ + kk * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(sc[2 * jj], qf[kk], kf[0], kf[1]);
        mma_bf16(sc[2 * jj + 1], qf[kk], kf[2], kf[3]);
      }
    }
    // scale, mask, running maximum
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; j++) {
#pragma unroll
      for (int i = 0; i < 2; i++) {
        const int key = j0 + j * 8 + (lane & 3) * 2 + i;
        float a0 = sc[j][i] * scale, a1 = sc[j][2 + i] * scale;
        if (ex.softcap > 0.f) { a0 = ex.softcap * tanhf(a0 / ex.softcap); a1 = ex.softcap * tanhf(a1 / ex.softcap); }
        sc[j][i] = (pooled ? key < nb0 : (key <= p0 && key >= lo0)) ? a0 : -INFINITY;
        sc[j][2 + i] = (pooled ? key < nb1 : (key <= p1 && key >= lo1)) ? a1 : -INFINITY;
        mx0 = fmaxf(mx0, sc[j][i]);
        mx1 = fmaxf(mx1, sc[j][2 + i]);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    const float u0 = n0 == -INFINITY ? 0.f : n0, u1 = n1 == -INFINITY ? 0.f : n1;   // nothing seen yet: weights are 0
    const float c0 = expf(m0 - u0), c1 = expf(m1 - u1);
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
#pragma unroll
      for (int i = 0; i < 2; i++) {
        sc[j][i] = expf(sc[j][i] - u0);
        sc[j][2 + i] = expf(sc[j][2 + i] - u1);
        ps0 += sc[j][i];
        ps1 += sc[j][2 + i];
      }
    }
    ps0 += __shfl_xor_sync(0xffffffffu, ps0, 1); ps0 += __shfl_xor_sync(0xffffffffu, ps0, 2);
    ps1 += __shfl_xor_sync(0xffffffffu, ps1, 1); ps1 += __shfl_xor_sync(0xffffffffu, ps1, 2);
    l0 = l0 * c0 + ps0; l1 = l1 * c1 + ps1;
    m0 = n0; m1 = n1;
#pragma unroll
    for (int j = 0; j < DVP / 8; j++) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
    // O += P V with P = hi + lo
#pragma unroll
    for (int kk = 0; kk < 4; kk++) {       // 16 keys per step
      uint32_t ph[4], pl[4];
#pragma unroll
      for (int x = 0; x < 4; x++) {
        const float a = sc[2 * kk + (x >> 1)][(x & 1) * 2], c = sc[2 * kk + (x >> 1)][(x & 1) * 2 + 1];
        const float ah = __bfloat162float(__float2bfloat16_rn(a)), ch = __bfloat162float(__float2bfloat16_rn(c));
        ph[x] = pack_bf16(ah, ch);
        pl[x] = pack_bf16(a - ah, c - ch);
      }
#pragma unroll
      for (int jj = 0; jj < DVP / 16; jj++) {
        uint32_t vf[4];
        ldsm_x4_t(vf, Vs + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LV + jj * 16 + (lane >> 4) * 8);
        mma_bf16(o[2 * jj], ph, vf[0], vf[1]);
        mma_bf16(o[2 * jj + 1], ph, vf[2], vf[3]);
        mma_bf16(o[2 * jj], pl, vf[0], vf[1]);
        mma_bf16(o[2 * jj + 1], pl, vf[2], vf[3]);
      }
    }
  }
  if (!warp_live) return;
  if (ex.sink) {       // one more term of the denominator, with no value: fold it in as a last key
    const float snk = __bfloat162float(((const bf16*)ex.sink)[h]);
    const float n0 = fmaxf(m0, snk), n1 = fmaxf(m1, snk);
    const float c0 = expf(m0 - n0), c1 = expf(m1 - n1);
    l0 = l0 * c0 + expf(snk - n0); l1 = l1 * c1 + expf(snk - n1);
#pragma unroll
    for (int j = 0; j < DVP / 8; j++) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
  }
  float i0 = p0 >= 0 ? 1.f / l0 : 0.f, i1 = p1 >= 0 ? 1.f / l1 : 0.f;
  if (ex.gate) {
    if (p0 >= 0) i0 *= sigmoid_f(ex.gate[(size_t)(s0 + r0) * H + h]);
    if (p1 >= 0) i1 *= sigmoid_f(ex.gate[(size_t)(s0 + r1) * H + h]);
  }
#pragma unroll
  for (int j = 0; j < DVP / 8; j++) {
    const int d = j * 8 + (lane & 3) * 2;
    if (d < dv) {
      if (p0 >= 0) *reinterpret_cast<uint32_t*>(out + ((size_t)(s0 + r0) * H + h) * dv + d) = pack_bf16(o[j][0] * i0, o[j][1] * i0);
      if (p1 >= 0) *reinterpret_cast<uint32_t*>(out + ((size_t)(s0 + r1) * H + h) * dv + d) = pack_bf16(o[j][2] * i1, o[j][3] * i1);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// gated delta rule
struct DeltaPrep {
  int H, G, dk, dv, taps;
};
// conv + silu on q, k, v; unit-norm q (times dk^-1/2) and k per head; beta = sigmoid(b), decay = exp(-exp(A) softplus(a + dt))
template <class T>
__global__ void k_delta_prep(DeltaPrep a, Batch b, const T* __restrict__ Uq, const T* __restrict__ Uk, const T* __restrict__ Uv,
                             const T* __restrict__ cwq, const T* __restrict__ cwk, const T* __restrict__ cwv, const float* __restrict__ pa,
                             const float* __restrict__ pb, const T* __restrict__ A_log, const T* __restrict__ dt_bias,
                             const T* __restrict__ cstate, size_t slot_stride, float* __restrict__ qn, float* __restrict__ kn,
                             float* __restrict__ vv, float* __restrict__ beta, float* __restrict__ decay) {
  extern __shared__ float sm[];
  const int Cq = a.G * a.dk, Cv = a.H * a.dv, ldst = 2 * Cq + Cv;
  float* qs = sm;
  float* ks = sm + Cq;
  const int n = blockIdx.x, slot = b.slot[n], p = b.pos[n];
  const int local = n - b.first[n];
  const T* st = cstate + (size_t)slot * slot_stride;
  for (int c = threadIdx.x; c < Cq; c += blockDim.x) {
    qs[c] = silu_f(conv_at(Uq, Cq, cwq, c, n, local, st, ldst, a.taps));
    ks[c] = silu_f(conv_at(Uk, Cq, cwk, c, n, local, st + Cq, ldst, a.taps));
  }
  for (int c = threadIdx.x; c < Cv; c += blockDim.x) {
    vv[(size_t)n * Cv + c] = silu_f(conv_at(Uv, Cv, cwv, c, n, local, st + 2 * Cq, ldst, a.taps));
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int hh = w; hh < 2 * a.G; hh += nw) {
    const bool isq = hh < a.G;
    const int g = isq ? hh : hh - a.G;
    const float* src = (isq ? qs : ks) + g * a.dk;
    float ss = 0.f;
    for (int d = lane; d < a.dk; d += 32) ss += src[d] * src[d];
    ss = warp_sum(ss);
    const float r = (1.f / sqrtf(ss + 1e-6f)) * (isq ? 1.f / sqrtf((float)a.dk) : 1.f);
    float* dst = (isq ? qn : kn) + (size_t)n * Cq + g * a.dk;
    for (int d = lane; d < a.dk; d += 32) dst[d] = src[d] * r;
  }
  for (int h = threadIdx.x; h < a.H; h += blockDim.x) {
    beta[(size_t)n * a.H + h] = 1.f / (1.f + expf(-pb[(size_t)n * a.H + h]));
    decay[(size_t)n * a.H + h] = expf(-expf(ldf(A_log + h)) * softplus_f(pa[(size_t)n * a.H + h] + ldf(dt_bias + h)));
  }
}

// The recurrence, token by token:  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.
// Columns of S are independent: a block owns 32 columns of one (entry, head); P adjacent lanes share a column,
// each holding R consecutive rows (P R >= dk) in registers.  State [slot][head][dk][dv] fp32.
// The tokens' inputs (k, q, the block's 32 values, decay, beta) come through shared memory in tiles of TB tokens,
// copied asynchronously one tile ahead, so that the serial chain of a token is registers, shared memory and the
// lane shuffles only.  k and q lie there as P runs of R values, each run padded by 4 floats: the 16-byte reads of
// the P lanes of a column then fall into different banks; rows from dk up are zero, so the token loop has no
// bounds checks.  Sums run in an order fixed by (dk, P): four interleaved partial sums over a thread's rows,
// then the lanes of a column pairwise -- nothing depends on the tile size or on where a portion was cut.
__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

template <int R, int P>
__global__ void __launch_bounds__(32 * P) k_delta_rule(Batch b, int H, int G, int dk, int dv, int TB, const float* __restrict__ qn, const float* __restrict__ kn,
                             const float* __restrict__ vv, const float* __restrict__ beta, const float* __restrict__ decay,
                             float* __restrict__ state, size_t slot_stride, float* __restrict__ o) {
  extern __shared__ __align__(16) float dsm[];      // 2 x TB x per
  constexpr int KP = P * (R + 4);                   // padded extent of k (and of q)
  constexpr int per = 2 * KP + 36;                      // k q v[32] decay beta, rounded to 16 bytes
  const int e = blockIdx.x / H, h = blockIdx.x % H, g = h / (H / G);
  const int part = threadIdx.x % P, colb = threadIdx.x / P, col = blockIdx.y * 32 + colb;
  const int s0 = b.ent_start[e], s1 = b.ent_start[e + 1];
  const bool live = col < dv;
  float* Sg = state + (size_t)b.ent_slot[e] * slot_stride + (size_t)h * dk * dv;
  const int r0 = part * R;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; r++) S[r] = (live && r0 + r < dk) ? Sg[(size_t)(r0 + r) * dv + col] : 0.f;
  const int Cq = G * dk, Cv = H * dv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int nwarp = P;
  auto stage = [&](int buf, int n0) {
    const int cnt = min(TB, s1 - n0);
    for (int t = warp; t < cnt; t += nwarp) {
      const int n = n0 + t;
      float* dst = dsm + ((size_t)buf * TB + t) * per;
      const float* kr = kn + (size_t)n * Cq + g * dk;
      const float* qr = qn + (size_t)n * Cq + g * dk;
      for (int c = lane; c < P * R; c += 32) {
        const int idx = (c / R) * (R + 4) + (c % R);
        if (c < dk) { cp_async4(dst + idx, kr + c); cp_async4(dst + KP + idx, qr + c); }
        else dst[idx] = dst[KP + idx] = 0.f;
      }
      const int vc = blockIdx.y * 32 + lane;
      if (vc < dv) cp_async4(dst + 2 * KP + lane, vv + (size_t)n * Cv + h * dv + vc);
      else dst[2 * KP + lane] = 0.f;
      if (lane == 0) cp_async4(dst + 2 * KP + 32, decay + (size_t)n * H + h);
      if (lane == 1) cp_async4(dst + 2 * KP + 33, beta + (size_t)n * H + h);
    }
    cp_async_commit();
  };
  stage(0, s0);
  int buf = 0;
  // the read-out of token t is summed over the lanes of its column together with the dot product of token t + 1:
  // two independent shuffle chains in flight instead of one after the other
  float odp = 0.f;
  for (int n0 = s0; n0 < s1; n0 += TB, buf ^= 1) {
    if (n0 + TB < s1) { stage(buf ^ 1, n0 + TB); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    const int cnt = min(TB, s1 - n0);
    for (int t = 0; t < cnt; t++) {
      const float* in = dsm + ((size_t)buf * TB + t) * per;
      const float4* k4 = reinterpret_cast<const float4*>(in + part * (R + 4));
      const float4* q4 = reinterpret_cast<const float4*>(in + KP + part * (R + 4));
      const float gd = in[2 * KP + 32], bt = in[2 * KP + 33], v = in[2 * KP + colb];
      float kk[R], qq[R], d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < R / 4; j++) {
        const float4 kv = k4[j], qv = q4[j];
        kk[4 * j] = kv.x; kk[4 * j + 1] = kv.y; kk[4 * j + 2] = kv.z; kk[4 * j + 3] = kv.w;
        qq[4 * j] = qv.x; qq[4 * j + 1] = qv.y; qq[4 * j + 2] = qv.z; qq[4 * j + 3] = qv.w;
#pragma unroll
        for (int i = 0; i < 4; i++) {
          S[4 * j + i] *= gd;
          d4[i] = fmaf(S[4 * j + i], kk[4 * j + i], d4[i]);
        }
      }
      float dot = (d4[0] + d4[1]) + (d4[2] + d4[3]);
#pragma unroll
      for (int x = 1; x < P; x <<= 1) {
        const float a = __shfl_xor_sync(0xffffffffu, dot, x), c = __shfl_xor_sync(0xffffffffu, odp, x);
        dot += a;
        odp += c;
      }
      if (live && part == 0 && n0 + t > s0) o[(size_t)(n0 + t - 1) * Cv + h * dv + col] = odp;
      const float u = bt * (v - dot);
      float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < R; r++) {
        S[r] = fmaf(kk[r], u, S[r]);
        o4[r & 3] = fmaf(S[r], qq[r], o4[r & 3]);
      }
      odp = (o4[0] + o4[1]) + (o4[2] + o4[3]);
    }
    __syncthreads();      // the tile is read out before the copy after next lands in it
  }
#pragma unroll
  for (int x = 1; x < P; x <<= 1) odp += __shfl_xor_sync(0xffffffffu, odp, x);
  if (live && part == 0 && s1 > s0) o[(size_t)(s1 - 1) * Cv + h * dv + col] = odp;
#pragma unroll
  for (int r = 0; r < R; r++)
    if (live && r0 + r < dk) Sg[(size_t)(r0 + r) * dv + col] = S[r];
}

// read-out of the recurrence: per head o / rms(o) * w * silu(gate) -> T.  One warp per (token, head).
// wstride: 0 when the heads share one weight [dv], dv when every head has its own ([H, dv]); gate_sigmoid: the gate
// goes through a sigmoid instead of silu
template <class T>
__global__ void __launch_bounds__(32) k_delta_out(const float* __restrict__ o, const T* __restrict__ gate, const T* __restrict__ nw, int H,
                                                  int dv, float eps, T* __restrict__ out, int wstride, int gate_sigmoid = 0) {
  const int n = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
  const size_t base = ((size_t)n * H + h) * dv;
  float ss = 0.f;
  for (int d = lane; d < dv; d += 32) ss += o[base + d] * o[base + d];
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)dv + eps);
  for (int d = lane; d < dv; d += 32) {
    const float gz = ldf(gate + base + d);
    stf(out + base + d, o[base + d] * r * ldf(nw + (size_t)h * wstride + d) * (gate_sigmoid ? sigmoid_f(gz) : silu_f(gz)));
  }
}

}  // namespace dnseq
