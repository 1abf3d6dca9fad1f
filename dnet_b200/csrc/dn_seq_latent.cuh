// dn_seq_latent.cuh -- latent attention of the batched sequence-mixer path (libdnet_b200_seq.so).
//
// Per token the layer projects the input to one latent row [c; r]: c (kv_rank numbers, RMS-normed) and r (rot_part
// numbers, rotated by the position), and that row is all the cache keeps.  Head h's key is [W_uk,h c; r] and its
// value W_uv,h c, with the query laid out as [dn unrotated; rot_part rotated].  Nothing per head is ever written:
//
//   score(i, j) = q_un,i . (W_uk,h c_j) + q_rot,i . r_j  =  (W_uk,h^T q_un,i) . c_j + q_rot,i . r_j
//   out_i       = sum_j p_ij W_uv,h c_j                    =  W_uv,h (sum_j p_ij c_j)
//
// so the query is *absorbed* into the latent space (k_linear_heads with the transposed up-projection), attention runs
// as multi-query attention of H heads over the one cached row per token -- key size kv_rank + rot_part, value = the
// first kv_rank numbers of the same row (the attention kernels of dn_seq_kernels.cuh with G = 1 and the value pool
// aliased to the key pool) -- and the result is taken out of the latent space per head afterwards.  The same code
// serves prompt portions and decode steps, whatever the cut.
//
// Rotary pairs are (2i, 2i + 1) or (i, i + rot / 2), on the first `rot` numbers of the rotated part; angles are fp32.
#pragma once
#include "dn_seq_kernels.cuh"

namespace dnseq {

struct LatentPrep {
  int H, dn, dr, R;        // heads; unrotated and rotated query dims per head; latent size
  int rot, half;           // rotated numbers of the rotated part; 1: pairs half apart
  float eps;
  const float* inv_freq;   // [rot / 2]
};

// pair i of a rotated part: its two indices
__device__ __forceinline__ void rot_pair(int i, int rot, int half, int* a, int* b) {
  if (half) { *a = i; *b = i + rot / 2; }
  else { *a = 2 * i; *b = 2 * i + 1; }
}

// One block per token: the latent row [rmsnorm(c) w; rot(r)] into the sequence's page, and the rotated parts of the
// queries into the absorbed-query buffer qout [N, H, R + dr] (its first R numbers per head come from k_linear_heads).
template <class T>
__global__ void k_latent_prep(LatentPrep a, Batch b, const T* __restrict__ Uq, const T* __restrict__ Ukv, const T* __restrict__ cnorm,
                              T* __restrict__ qout, T* __restrict__ kpool) {
  __shared__ float red[33];
  const int n = blockIdx.x, slot = b.slot[n], p = b.pos[n];
  const int Ck = a.R + a.dr, dq = a.dn + a.dr;
  const T* kv = Ukv + (size_t)n * Ck;
  float ss = 0.f;
  for (int c = threadIdx.x; c < a.R; c += blockDim.x) { const float v = ldf(kv + c); ss += v * v; }
  ss = block_sum(ss, red);
  const float rinv = 1.f / sqrtf(ss / (float)a.R + a.eps);
  const int page = b.bt[(size_t)slot * b.max_pages + p / PAGE], prow = p % PAGE;
  T* row = kpool + ((size_t)page * PAGE + prow) * Ck;
  for (int c = threadIdx.x; c < a.R; c += blockDim.x) stf(row + c, ldf(kv + c) * rinv * ldf(cnorm + c));
  // rotated parts: source 0 is the shared key part, sources 1..H the heads' query parts
  const int np = a.rot / 2, per = np + (a.dr - a.rot);      // work items a source: the pairs, then the numbers that do not turn
  for (int e = threadIdx.x; e < (a.H + 1) * per; e += blockDim.x) {
    const int src = e / per, i = e % per;
    const T* in = src == 0 ? kv + a.R : Uq + (size_t)n * a.H * dq + (size_t)(src - 1) * dq + a.dn;
    T* out = src == 0 ? row + a.R : qout + ((size_t)n * a.H + (src - 1)) * Ck + a.R;
    if (i < np) {
      int ia, ib;
      rot_pair(i, a.rot, a.half, &ia, &ib);
      const float u = ldf(in + ia), v = ldf(in + ib);
      float sn, cs;
      sincosf((float)p * a.inv_freq[i], &sn, &cs);
      stf(out + ia, u * cs - v * sn);
      stf(out + ib, v * cs + u * sn);
    } else {
      const int c = a.rot + (i - np);
      stf(out + c, ldf(in + c));
    }
  }
}

// RMS norm of every row of X [N, C] with a plain weight, in place (the query latent)
template <class T>
__global__ void k_rms_rows(T* __restrict__ X, int C, const T* __restrict__ w, float eps) {
  __shared__ float red[33];
  T* x = X + (size_t)blockIdx.x * C;
  float ss = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) { const float v = ldf(x + c); ss += v * v; }
  ss = block_sum(ss, red);
  const float rinv = 1.f / sqrtf(ss / (float)C + eps);
  for (int c = threadIdx.x; c < C; c += blockDim.x) stf(x + c, ldf(x + c) * rinv * ldf(w + c));
}

// One product per head z = blockIdx.z on CUDA-core tiles:  Y[n, z ldyz + o] = sum_k X[n ldx + z ldxz + k] Wz(o, k) with
// Wz(o, k) = W[z wz + o wo + k wk].  The strides let one kernel read an up-projection as stored (wo = K, wk = 1: values
// out of the latent space) or transposed (wo = 1, wk = O: queries into it).  fp32 accumulation as in k_linear: a
// k-block's 16 products from zero in ascending k, the blocks' sums added with compensation.
struct HeadsGeom {
  int ldx, ldxz;       // row stride of X, offset of head z inside a row
  int ldy, ldyz;
  size_t wz;           // offset of head z's matrix
  int wo, wk;
};
template <class T>
__global__ void __launch_bounds__(256) k_linear_heads(const T* __restrict__ X, const T* __restrict__ Wt, T* __restrict__ Y, int N, int O, int K,
                                                      HeadsGeom g) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float Xs[BK][BM + 4], Ws[BK][BN + 4];
  const int z = blockIdx.z;
  const T* Xz = X + (size_t)z * g.ldxz;
  const T* Wz = Wt + (size_t)z * g.wz;
  T* Yz = Y + (size_t)z * g.ldyz;
  const int n0 = blockIdx.y * BM, o0 = blockIdx.x * BN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4], cmp[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = cmp[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int e = threadIdx.x; e < BM * BK; e += 256) {
      const int r = e / BK, c = e % BK;
      Xs[c][r] = (n0 + r < N && k0 + c < K) ? ldf(Xz + (size_t)(n0 + r) * g.ldx + k0 + c) : 0.f;
      // adjacent threads read adjacent addresses of the weight whichever way it lies
      const int wr = g.wo == 1 ? e % BN : r, wc = g.wo == 1 ? e / BN : c;
      Ws[wc][wr] = (o0 + wr < O && k0 + wc < K) ? ldf(Wz + (size_t)(o0 + wr) * g.wo + (size_t)(k0 + wc) * g.wk) : 0.f;
    }
    __syncthreads();
    float part[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) part[i][j] = 0.f;
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
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) kahan_add(acc[i][j], cmp[i][j], part[i][j]);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int n = n0 + ty * 4 + i;
    if (n >= N) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int o = o0 + tx * 4 + j;
      if (o < O) stf(Yz + (size_t)n * g.ldy + o, acc[i][j]);
    }
  }
}

}  // namespace dnseq
