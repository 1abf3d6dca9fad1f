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
#include "dn_seq_moe.cuh"      // warp_dot

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


// The same two products for a few tokens (N <= 8: decode steps), each weight read once.
// Into the latent space: a block owns 32 latent numbers of one head; its four warps split the rows of W_uk,h (lane r reads
// column r of a row: adjacent lanes, adjacent numbers) against the tokens' unrotated query parts in shared memory, and
// the warps' partial sums are added in warp order.
template <class T>
__global__ void __launch_bounds__(128) k_absorb_few(const T* __restrict__ Uq, const T* __restrict__ Wuk, T* __restrict__ qout, int N, int H, int dn,
                                                    int dq, int R, int Ck) {
  extern __shared__ float qs[];      // [N][dn], then [4][8][32] partial sums
  float* part = qs + N * dn;
  const int h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, r = blockIdx.x * 32 + lane;
  for (int i = threadIdx.x; i < N * dn; i += blockDim.x) qs[i] = ldf(Uq + ((size_t)(i / dn) * H + h) * dq + i % dn);
  __syncthreads();
  float acc[8];
#pragma unroll
  for (int n = 0; n < 8; n++) acc[n] = 0.f;
  const int per = (dn + 3) / 4, d0 = warp * per, d1 = min(dn, d0 + per);
  if (r < R) {
    const T* w = Wuk + (size_t)h * dn * R + r;
#pragma unroll 8
    for (int d = d0; d < d1; d++) {
      const float wv = ldf(w + (size_t)d * R);
#pragma unroll
      for (int n = 0; n < 8; n++)
        if (n < N) acc[n] = fmaf(qs[n * dn + d], wv, acc[n]);
    }
  }
#pragma unroll
  for (int n = 0; n < 8; n++) part[(warp * 8 + n) * 32 + lane] = acc[n];
  __syncthreads();
  if (warp == 0 && r < R) {
#pragma unroll
    for (int n = 0; n < 8; n++)
      if (n < N) stf(qout + ((size_t)n * H + h) * Ck + r, ((part[n * 32 + lane] + part[(8 + n) * 32 + lane]) + part[(16 + n) * 32 + lane]) + part[(24 + n) * 32 + lane]);
  }
}
// Out of the latent space: one warp per output feature (head h, value dim j) streams its row of W_uv
template <class T>
__global__ void __launch_bounds__(256) k_upv_few(const T* __restrict__ X, const T* __restrict__ Wuv, T* __restrict__ Y, int N, int H, int dv, int R) {
  const int o = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (o >= H * dv) return;
  const int h = o / dv;
  const T* w = Wuv + (size_t)o * R;
  const bool vec = R % Vec16<T>::n == 0 && ((((uintptr_t)X | (uintptr_t)Wuv) & 15) == 0);
  for (int n = 0; n < N; n++) {
    const float a = warp_dot(X + ((size_t)n * H + h) * R, w, R, vec);
    if (lane == 0) stf(Y + (size_t)n * H * dv + o, a);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Latent attention of prompt portions, bf16, on the warp-level tensor-core MMA (m16n8k16, fp32 accumulation).
// A block owns 64 consecutive query rows of one entry and one head.  A key tile is one page of cached rows, staged
// once through shared memory and used twice: all R + rot numbers of a row as the key, its first R numbers as the value
// (ldmatrix.trans on the same tile), so a page is read once per (row tile, head).  Eight warps: warp w takes the 16 rows
// (w & 3) and the half (w >> 2) of the value columns -- with a latent of 512 the output accumulators of 16 rows x 256
// columns are 128 registers a thread; both halves compute the same scores.  The query tile stays in shared memory
// (its fragments are re-read per key tile: 576 numbers a row do not fit the registers beside the accumulators).
// Shared memory holds the query tile and two key tiles (219 KB for a latent of 512 + 64): the next page is copied
// (cp.async) while the current one is multiplied.
// Scores, running maximum and sum are fp32; the weights enter P V as a bf16 pair (hi + lo).  Per row the key tiles are
// visited in ascending position and a tile the row does not see changes nothing: the result does not depend on the cut.
// DVH: value columns a warp owns (the block covers 2 DVH >= R).  LD: shared row pitch = max(padded key size, 2 DVH) + 8.
//
// DEC (decode steps): the 64 rows of a block are up to 64 *heads* of one token -- all heads read the same cached rows, so
// a page is staged once for all of them -- and the pages a token sees are dealt round-robin to gridDim.z blocks, each
// writing its partial (maximum, sum, unnormalised output) for k_latent_merge, which joins them in the order of z.
// The split is a function of the token's own position.  grid (tokens, ceil(H / 64), splits).  MODE 1: up to 64 heads a
// block, warps as for prompts; MODE 2 (at most 16 heads): one row group, so all eight warps take an eighth of the value
// columns each (every warp computes the 16 x 64 scores).
__device__ __forceinline__ int latent_splits(int p, int lo, int zmax) { return min(zmax, p / PAGE - lo / PAGE + 1); }
// A 64-row tile into shared memory by asynchronous 16-byte copies (no registers, all of a thread's copies in flight at
// once); rows >= valid and columns >= cols are filled with zeros (a copy of 0 source bytes).  The caller commits and waits.
__device__ __forceinline__ void cp_async16(bf16* dst, const bf16* src, int src_bytes) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void load_tile_rt(bf16* __restrict__ dst, const bf16* __restrict__ src, size_t ld, int cols, int valid, int LD) {
  const int vec = LD / 8 - 1;      // 16-byte groups per row, the pad group left out
  for (int e = threadIdx.x; e < 64 * vec; e += blockDim.x) {
    const int r = e / vec, c = (e % vec) * 8;
    const bool in = r < valid && c < cols;
    cp_async16(dst + (size_t)r * LD + c, in ? src + (size_t)r * ld + c : src, in ? 16 : 0);
  }
}
template <int DVH, int MODE>
__global__ void __launch_bounds__(256, 1) k_latent_tiles(Batch b, const bf16* __restrict__ q, const bf16* __restrict__ kpool, int H, int Ck, int R,
                                                         int DKP, int LD, int chunk, float scale, AttnExtra ex, bf16* __restrict__ out,
                                                         float* __restrict__ part_g, int part_ld) {
  constexpr bool DEC = MODE != 0;
  constexpr int CW = MODE == 2 ? DVH / 4 : DVH;      // value columns a warp owns
  extern __shared__ __align__(16) unsigned char smraw[];
  bf16* Qs = reinterpret_cast<bf16*>(smraw);
  bf16* Kbuf = Qs + 64 * LD;      // two tiles
  int e = 0, t = blockIdx.x, h = blockIdx.y, s0, rows, p_first, p_last, slot, page_step = PAGE, page0 = 0;
  if (DEC) {
    const int n = blockIdx.x;
    h = blockIdx.y * 64;                        // first head of the block's rows
    rows = min(64, H - h);
    s0 = n;
    p_first = p_last = b.pos[n];
    slot = b.slot[n];
    const int nz = latent_splits(p_last, attn_lo(p_last, chunk, ex.window), (int)gridDim.z);
    if ((int)blockIdx.z >= nz) return;
    page0 = blockIdx.z * PAGE;
    page_step = nz * PAGE;
  } else {
    for (; e < b.E; e++) {
      const int nt = (b.ent_start[e + 1] - b.ent_start[e] + 63) / 64;
      if (t < nt) break;
      t -= nt;
    }
    if (e >= b.E) return;
    s0 = b.ent_start[e] + t * 64;
    rows = min(64, b.ent_start[e + 1] - s0);
    p_first = b.ent_pos0[e] + t * 64;
    p_last = p_first + rows - 1;
    slot = b.ent_slot[e];
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, rg = MODE == 2 ? 0 : (warp & 3), hv = MODE == 2 ? warp : (warp >> 2);
  if (DEC) load_tile_rt(Qs, q + ((size_t)s0 * H + h) * Ck, (size_t)Ck, Ck, rows, LD);
  else load_tile_rt(Qs, q + ((size_t)s0 * H + h) * Ck, (size_t)H * Ck, Ck, rows, LD);
  const int r0 = rg * 16 + (lane >> 2), r1 = r0 + 8;
  const int p0 = r0 < rows ? (DEC ? p_first : p_first + r0) : -1, p1 = r1 < rows ? (DEC ? p_first : p_first + r1) : -1;
  const int lo0 = p0 >= 0 ? attn_lo(p0, chunk, ex.window) : 0, lo1 = p1 >= 0 ? attn_lo(p1, chunk, ex.window) : 0;
  const bool warp_live = rg * 16 < rows;
  float o[CW / 8][4];
#pragma unroll
  for (int j = 0; j < CW / 8; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const int32_t* bt = b.bt + (size_t)slot * b.max_pages;
  const int lo_tile = attn_lo(p_first, chunk, ex.window);
  const bf16* qrow = Qs + (size_t)(rg * 16 + (lane & 15)) * LD + (lane >> 4) * 8;
  auto stage = [&](int j0, int buf) {      // rows of the page beyond the last query's position are not read
    load_tile_rt(Kbuf + (size_t)buf * 64 * LD, kpool + (size_t)bt[j0 / PAGE] * PAGE * Ck, (size_t)Ck, Ck, min(PAGE, p_last - j0 + 1), LD);
    cp_async_commit();
  };
  const int j_first = (lo_tile / PAGE) * PAGE + page0;
  if (j_first <= p_last) stage(j_first, 0);      // (the query tile's copies are in this group too)
  int buf = 0;
  for (int j0 = j_first; j0 <= p_last; j0 += page_step, buf ^= 1) {
    if (j0 + page_step <= p_last) { stage(j0 + page_step, buf ^ 1); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    const bf16* Ks = Kbuf + (size_t)buf * 64 * LD;
    if (!warp_live) { __syncthreads(); continue; }
    float sc[8][4];
#pragma unroll
    for (int j = 0; j < 8; j++) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll 2
    for (int kk = 0; kk < DKP / 16; kk++) {
      uint32_t qf[4];
      ldsm_x4(qf, qrow + kk * 16);
#pragma unroll
      for (int jj = 0; jj < 4; jj++) {
        uint32_t kf[4];
        ldsm_x4(kf, Ks + (size_t)(jj * 16 + (lane >> 4) * 8 + (lane & 7)) * LD + kk * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(sc[2 * jj], qf, kf[0], kf[1]);
        mma_bf16(sc[2 * jj + 1], qf, kf[2], kf[3]);
      }
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; j++) {
#pragma unroll
      for (int i = 0; i < 2; i++) {
        const int key = j0 + j * 8 + (lane & 3) * 2 + i;
        float a0 = sc[j][i] * scale, a1 = sc[j][2 + i] * scale;
        if (ex.softcap > 0.f) { a0 = ex.softcap * tanhf(a0 / ex.softcap); a1 = ex.softcap * tanhf(a1 / ex.softcap); }
        sc[j][i] = (key <= p0 && key >= lo0) ? a0 : -INFINITY;
        sc[j][2 + i] = (key <= p1 && key >= lo1) ? a1 : -INFINITY;
        mx0 = fmaxf(mx0, sc[j][i]);
        mx1 = fmaxf(mx1, sc[j][2 + i]);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    const float u0 = n0 == -INFINITY ? 0.f : n0, u1 = n1 == -INFINITY ? 0.f : n1;      // nothing seen yet: weights are 0
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
    for (int j = 0; j < CW / 8; j++) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
    // O += P V with P = hi + lo; V = the first columns of the key tile
#pragma unroll
    for (int kk = 0; kk < 4; kk++) {
      uint32_t ph[4], pl[4];
#pragma unroll
      for (int x = 0; x < 4; x++) {
        const float a = sc[2 * kk + (x >> 1)][(x & 1) * 2], c = sc[2 * kk + (x >> 1)][(x & 1) * 2 + 1];
        const float ah = __bfloat162float(__float2bfloat16_rn(a)), ch = __bfloat162float(__float2bfloat16_rn(c));
        ph[x] = pack_bf16(ah, ch);
        pl[x] = pack_bf16(a - ah, c - ch);
      }
      const bf16* vrow = Ks + (size_t)(kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LD + hv * CW + (lane >> 4) * 8;
#pragma unroll
      for (int jj = 0; jj < CW / 16; jj++) {
        uint32_t vf[4];
        ldsm_x4_t(vf, vrow + jj * 16);
        mma_bf16(o[2 * jj], ph, vf[0], vf[1]);
        mma_bf16(o[2 * jj + 1], ph, vf[2], vf[3]);
        mma_bf16(o[2 * jj], pl, vf[0], vf[1]);
        mma_bf16(o[2 * jj + 1], pl, vf[2], vf[3]);
      }
    }
    __syncthreads();      // the tile is read out before the copy after next lands in it
  }
  if (!warp_live) return;
  if (DEC) {      // the block's partial of every head: [maximum, sum, unnormalised output]
    float* g0 = part_g + (((size_t)s0 * H + h + r0) * gridDim.z + blockIdx.z) * part_ld;
    float* g1 = part_g + (((size_t)s0 * H + h + r1) * gridDim.z + blockIdx.z) * part_ld;
    if (hv == 0 && (lane & 3) == 0) {
      if (p0 >= 0) { g0[0] = m0; g0[1] = l0; }
      if (p1 >= 0) { g1[0] = m1; g1[1] = l1; }
    }
#pragma unroll
    for (int j = 0; j < CW / 8; j++) {
      const int d = hv * CW + j * 8 + (lane & 3) * 2;
      if (d < R) {
        if (p0 >= 0) { g0[2 + d] = o[j][0]; g0[3 + d] = o[j][1]; }
        if (p1 >= 0) { g1[2 + d] = o[j][2]; g1[3 + d] = o[j][3]; }
      }
    }
    return;
  }
  float i0 = p0 >= 0 ? 1.f / l0 : 0.f, i1 = p1 >= 0 ? 1.f / l1 : 0.f;
  if (ex.gate) {
    if (p0 >= 0) i0 *= sigmoid_f(ex.gate[(size_t)(s0 + r0) * H + h]);
    if (p1 >= 0) i1 *= sigmoid_f(ex.gate[(size_t)(s0 + r1) * H + h]);
  }
#pragma unroll
  for (int j = 0; j < CW / 8; j++) {
    const int d = hv * CW + j * 8 + (lane & 3) * 2;
    if (d < R) {
      if (p0 >= 0) *reinterpret_cast<uint32_t*>(out + ((size_t)(s0 + r0) * H + h) * R + d) = pack_bf16(o[j][0] * i0, o[j][1] * i0);
      if (p1 >= 0) *reinterpret_cast<uint32_t*>(out + ((size_t)(s0 + r1) * H + h) * R + d) = pack_bf16(o[j][2] * i1, o[j][3] * i1);
    }
  }
}

// joins the partials of k_latent_tiles<., true> in the order of the splits, applies the head's gate; grid (tokens, H).
// One warp turns the splits' maxima and sums into a weight per split; every thread then adds its value numbers over
// the splits with all loads in flight at once (zmax <= 32).
__global__ void k_latent_merge(Batch b, int H, int R, int chunk, int zmax, AttnExtra ex, const float* __restrict__ part_g, int part_ld,
                               bf16* __restrict__ out) {
  __shared__ float f[32];
  __shared__ float scale;
  const int n = blockIdx.x, h = blockIdx.y, p = b.pos[n];
  const int nz = latent_splits(p, attn_lo(p, chunk, ex.window), zmax);
  const float* pg = part_g + ((size_t)n * H + h) * zmax * part_ld;
  if (threadIdx.x < 32) {
    const int z = threadIdx.x;
    const float m = z < nz ? pg[(size_t)z * part_ld] : -INFINITY;
    const float M = warp_max(m);
    const float fz = z < nz ? expf(m - M) : 0.f;
    const float L = warp_sum(z < nz ? pg[(size_t)z * part_ld + 1] * fz : 0.f);
    f[z] = fz;
    if (z == 0) scale = (ex.gate ? sigmoid_f(ex.gate[(size_t)n * H + h]) : 1.f) / L;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < R; d += blockDim.x) {
    float v[32];
#pragma unroll
    for (int z = 0; z < 32; z++) v[z] = z < nz ? pg[(size_t)z * part_ld + 2 + d] : 0.f;
    float a = 0.f;
#pragma unroll
    for (int z = 0; z < 32; z++) a = fmaf(v[z], f[z], a);
    out[((size_t)n * H + h) * R + d] = __float2bfloat16_rn(a * scale);
  }
}

// The two per-head products of a prompt portion, bf16, on the warp-level MMA (m16n8k16, fp32 accumulation): the geometry of
// k_linear_heads, a block = 64 tokens x 128 output features of one head, four warps of 16 rows each, operands staged
// through shared memory in k-chunks of 64.  WT: the weight lies [k][o] (o contiguous: the key up-projection read
// transposed, ldmatrix.trans), else [o][k].  Needs 16-byte aligned rows: every stride a multiple of 8 numbers.
template <bool WT>
__global__ void __launch_bounds__(128) k_heads_mma(const bf16* __restrict__ X, const bf16* __restrict__ Wt, bf16* __restrict__ Y, int N, int O, int K,
                                                   HeadsGeom g) {
  constexpr int KC = 64, LDX = KC + 8, LDW = WT ? 128 + 8 : KC + 8;
  __shared__ __align__(16) bf16 Xs[64 * LDX];
  __shared__ __align__(16) bf16 Ws[(WT ? KC : 128) * LDW];
  const int z = blockIdx.z, n0 = blockIdx.y * 64, o0 = blockIdx.x * 128;
  const bf16* Xz = X + (size_t)z * g.ldxz;
  const bf16* Wz = Wt + (size_t)z * g.wz;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float acc[16][4];
#pragma unroll
  for (int j = 0; j < 16; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  for (int k0 = 0; k0 < K; k0 += KC) {
    __syncthreads();
    for (int e = threadIdx.x; e < 64 * (KC / 8); e += 128) {
      const int r = e / (KC / 8), c = (e % (KC / 8)) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (n0 + r < N && k0 + c < K) v = *reinterpret_cast<const uint4*>(Xz + (size_t)(n0 + r) * g.ldx + k0 + c);
      *reinterpret_cast<uint4*>(Xs + r * LDX + c) = v;
    }
    if (WT) {
      for (int e = threadIdx.x; e < KC * 16; e += 128) {
        const int r = e / 16, c = (e % 16) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (k0 + r < K && o0 + c < O) v = *reinterpret_cast<const uint4*>(Wz + (size_t)(k0 + r) * g.wk + o0 + c);
        *reinterpret_cast<uint4*>(Ws + r * LDW + c) = v;
      }
    } else {
      for (int e = threadIdx.x; e < 128 * (KC / 8); e += 128) {
        const int r = e / (KC / 8), c = (e % (KC / 8)) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (o0 + r < O && k0 + c < K) v = *reinterpret_cast<const uint4*>(Wz + (size_t)(o0 + r) * g.wo + k0 + c);
        *reinterpret_cast<uint4*>(Ws + r * LDW + c) = v;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < KC / 16; kk++) {
      uint32_t af[4];
      ldsm_x4(af, Xs + (warp * 16 + (lane & 15)) * LDX + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int jj = 0; jj < 8; jj++) {
        uint32_t bfr[4];
        if (WT) ldsm_x4_t(bfr, Ws + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LDW + jj * 16 + (lane >> 4) * 8);
        else ldsm_x4(bfr, Ws + (jj * 16 + (lane >> 4) * 8 + (lane & 7)) * LDW + kk * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(acc[2 * jj], af, bfr[0], bfr[1]);
        mma_bf16(acc[2 * jj + 1], af, bfr[2], bfr[3]);
      }
    }
  }
  bf16* Yz = Y + (size_t)z * g.ldyz;
  const int r0 = n0 + warp * 16 + (lane >> 2), r1 = r0 + 8;
#pragma unroll
  for (int j = 0; j < 16; j++) {
    const int o = o0 + j * 8 + (lane & 3) * 2;
    if (o < O) {      // O is even and the rows are 4-byte aligned (checked by the caller)
      if (r0 < N) *reinterpret_cast<uint32_t*>(Yz + (size_t)r0 * g.ldy + o) = pack_bf16(acc[j][0], acc[j][1]);
      if (r1 < N) *reinterpret_cast<uint32_t*>(Yz + (size_t)r1 * g.ldy + o) = pack_bf16(acc[j][2], acc[j][3]);
    }
  }
}

}  // namespace dnseq
