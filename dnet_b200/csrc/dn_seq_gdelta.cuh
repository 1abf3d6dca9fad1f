// dn_seq_gdelta.cuh -- the generalized delta rule (libdnet_b200_seq.so).
//
// Per head and sequence an fp32 state S [dk, dv].  A token brings a read vector r, a key k and a value v (projections
// in the storage type), a decay w and a removal rate a per key channel (fp32), and with the unit key u = k / sqrt(|k|^2 + 1e-6)
//     S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T          (both terms read the old state)
//     o_t = S_t^T r_t
// The delta rule of dn_seq_kernels.cuh removes beta (k^T S) along k from every row alike; here every key channel decays
// and gives up what lies along u at its own rate.  Columns of S are independent, so the recurrence has the column-
// parallel form of the other two: s <- w * s - (a * u) (u . s) + k v_c, o_c = s . r.
#pragma once
#include "dn_seq_kernels.cuh"

namespace dnseq {

// between the projections and the recurrence; grid (tokens, groups of heads), one warp a head.  In: r, k, v [N, C] (storage type); zw [N, C] the
// decay's pre-activation and za [N, C] the removal rate's (fp32 products, biases not yet added).  Out, all fp32:
// rn = r, kn = k, vv = v, zw <- w = exp(-exp(-1/2) sigmoid(zw + w0)), un = u, za <- a * u with a = sigmoid(za + ab).
// One warp a head for the unit norm: lanes over the head's dims in ascending order, then the lanes pairwise.
template <class T>
__global__ void k_gdelta_prep(int H, int dk, const T* __restrict__ Ur, const T* __restrict__ Uk, const T* __restrict__ Uv,
                              const T* __restrict__ w0, const T* __restrict__ ab, float* __restrict__ rn, float* __restrict__ kn,
                              float* __restrict__ vv, float* __restrict__ zw, float* __restrict__ un, float* __restrict__ za) {
  const int n = blockIdx.x, C = H * dk;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const float dmax = 0.6065306597126334f;      // exp(-1/2)
  for (int h = blockIdx.y * nw + warp; h < H; h += gridDim.y * nw) {
    const size_t base = (size_t)n * C + (size_t)h * dk;
    float ss = 0.f;
    for (int d = lane; d < dk; d += 32) { const float k = ldf(Uk + base + d); ss += k * k; }
    ss = warp_sum(ss);
    const float rinv = 1.f / sqrtf(ss + 1e-6f);
    for (int d = lane; d < dk; d += 32) {
      const size_t i = base + d;
      const int c = h * dk + d;
      const float k = ldf(Uk + i), u = k * rinv;
      rn[i] = ldf(Ur + i);
      kn[i] = k;
      vv[i] = ldf(Uv + i);
      un[i] = u;
      zw[i] = expf(-dmax * sigmoid_f(zw[i] + ldf(w0 + c)));
      za[i] = sigmoid_f(za[i] + ldf(ab + c)) * u;
    }
  }
}

// The recurrence, token by token.  A block owns COLS columns of one (entry, head); P adjacent lanes share a column, each
// holding R consecutive rows (P R >= dk) in registers.  State [slot][head][dk][dv] fp32, read once and written once per
// step.  A token's u, a * u, w, k, r and the block's COLS values come through shared memory in tiles of TB tokens, copied
// asynchronously one tile ahead; each vector lies there as P runs of R values, padded by 4 floats where R > 4 (the 16-byte
// reads of a column's P lanes fall into different banks); rows from dk up are zero.  The sums u . s and s . r run over a
// thread's rows in four interleaved partial sums, then over the lanes of a column pairwise: an order fixed by (dk, P),
// whatever the tile size or the cut of a prompt.  The read-out of token t is reduced over the lanes together with
// u . s of token t + 1 (two independent shuffle chains in flight).
template <int R, int P, int COLS>
__global__ void __launch_bounds__(COLS * P) k_gdelta_rule(Batch b, int H, int dk, int dv, int TB, const float* __restrict__ rn,
                                                          const float* __restrict__ kn, const float* __restrict__ vv,
                                                          const float* __restrict__ wd, const float* __restrict__ un,
                                                          const float* __restrict__ au, float* __restrict__ state, size_t slot_stride,
                                                          float* __restrict__ o) {
  static_assert(COLS * P >= 32 && (COLS * P) % 32 == 0 && COLS <= 32, "whole warps");
  extern __shared__ __align__(16) float dsm[];      // 2 x TB x per
  constexpr int RS = R == 4 ? 4 : R + 4;            // a lane's run with its padding (none for runs of one 16-byte read)
  constexpr int KP = P * RS;
  constexpr int per = 5 * KP + COLS;                // u, a u, w, k, r, v[COLS]
  const int e = blockIdx.x / H, h = blockIdx.x % H;
  const int part = threadIdx.x % P, colb = threadIdx.x / P, col = blockIdx.y * COLS + colb;
  const int s0 = b.ent_start[e], s1 = b.ent_start[e + 1];
  const bool live = col < dv;
  float* Sg = state + (size_t)b.ent_slot[e] * slot_stride + (size_t)h * dk * dv;
  const int r0 = part * R;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; r++) S[r] = (live && r0 + r < dk) ? Sg[(size_t)(r0 + r) * dv + col] : 0.f;
  const int C = H * dk, Cv = H * dv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int nwarp = COLS * P / 32;
  auto stage = [&](int buf, int n0) {
    const int cnt = min(TB, s1 - n0);
    for (int t = warp; t < cnt; t += nwarp) {
      const int n = n0 + t;
      float* dst = dsm + ((size_t)buf * TB + t) * per;
      const size_t base = (size_t)n * C + (size_t)h * dk;
      for (int c = lane; c < P * R; c += 32) {
        const int idx = (c / R) * RS + (c % R);
        if (c < dk) {
          cp_async4(dst + idx, un + base + c); cp_async4(dst + KP + idx, au + base + c); cp_async4(dst + 2 * KP + idx, wd + base + c);
          cp_async4(dst + 3 * KP + idx, kn + base + c); cp_async4(dst + 4 * KP + idx, rn + base + c);
        } else dst[idx] = dst[KP + idx] = dst[2 * KP + idx] = dst[3 * KP + idx] = dst[4 * KP + idx] = 0.f;
      }
      if (lane < COLS) {
        const int vc = blockIdx.y * COLS + lane;
        if (vc < dv) cp_async4(dst + 5 * KP + lane, vv + (size_t)n * Cv + h * dv + vc);
        else dst[5 * KP + lane] = 0.f;
      }
    }
    cp_async_commit();
  };
  stage(0, s0);
  int buf = 0;
  float odp = 0.f;
  for (int n0 = s0; n0 < s1; n0 += TB, buf ^= 1) {
    if (n0 + TB < s1) { stage(buf ^ 1, n0 + TB); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    const int cnt = min(TB, s1 - n0);
    for (int t = 0; t < cnt; t++) {
      const float* in = dsm + ((size_t)buf * TB + t) * per + part * RS;
      const float4* u4 = reinterpret_cast<const float4*>(in);
      const float4* a4 = reinterpret_cast<const float4*>(in + KP);
      const float4* w4 = reinterpret_cast<const float4*>(in + 2 * KP);
      const float4* k4 = reinterpret_cast<const float4*>(in + 3 * KP);
      const float4* r4 = reinterpret_cast<const float4*>(in + 4 * KP);
      const float v = dsm[((size_t)buf * TB + t) * per + 5 * KP + colb];
      float d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < R / 4; j++) {
        const float4 uv = u4[j];
        d4[0] = fmaf(S[4 * j], uv.x, d4[0]); d4[1] = fmaf(S[4 * j + 1], uv.y, d4[1]);
        d4[2] = fmaf(S[4 * j + 2], uv.z, d4[2]); d4[3] = fmaf(S[4 * j + 3], uv.w, d4[3]);
      }
      float dot = (d4[0] + d4[1]) + (d4[2] + d4[3]);
#pragma unroll
      for (int x = 1; x < P; x <<= 1) {
        const float a = __shfl_xor_sync(0xffffffffu, dot, x), c = __shfl_xor_sync(0xffffffffu, odp, x);
        dot += a;
        odp += c;
      }
      if (live && part == 0 && n0 + t > s0) o[(size_t)(n0 + t - 1) * Cv + h * dv + col] = odp;
      float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < R / 4; j++) {
        const float4 av = a4[j], wv = w4[j], kv = k4[j], rv = r4[j];
        const float aa[4] = {av.x, av.y, av.z, av.w}, ww[4] = {wv.x, wv.y, wv.z, wv.w}, kk[4] = {kv.x, kv.y, kv.z, kv.w}, rr[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
          float& Sr = S[4 * j + i];
          Sr = fmaf(kk[i], v, fmaf(-aa[i], dot, ww[i] * Sr));
          o4[i] = fmaf(Sr, rr[i], o4[i]);
        }
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

}  // namespace dnseq
