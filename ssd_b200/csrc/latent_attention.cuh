// latent_attention.cuh — attention over a compressed (latent) KV cache with a learned softmax sink.
//
// What is cached per token and layer is one row [kv_rank + rot_dim] of storage type T in a paged pool: the RMS-normed
// latent c and the ONE rotated key part shared by all heads.  Keys and values are never materialised: with
//   k_h = W_uk,h c,   v_h = W_uv,h c       the score is   q_h . k_h = (W_uk,h^T q_h) . c
// so the queries are taken into latent space once per token (a per-head GEMM against W_uk^T, "absorption"), attention
// runs multi-query style over the latent rows (every head reads the same row), and the per-head value projection is
// applied to the attention's latent output (a per-head GEMM against W_uv).
//
//   latent_prep_kernel   splits the fused down-projection: RMS-norm -> query latent (T); RMS-norm -> c and
//                        rotate-half RoPE (fp32 angles) -> rotated key part, both scattered into the page slot
//   latent_q_kernel      per head: unrotated query part -> T (operand of the absorption GEMM), rotated part -> RoPE, fp32
//   latent_attn_kernel   one CTA per (row, head group): causal over the cache up to the row's own position; scores,
//                        online softmax and the accumulators are fp32; the running maximum starts at the sink logit and
//                        the running sum at 1, i.e. the sink is one more term of the denominator with no key and no value
#pragma once
#include "layer_ops.cuh"

namespace ssdk {

SSDK_DEVINL size_t page_row(const Ragged& rg, int s, int pos) {
  const int page = rg.tables[(size_t)s * rg.max_blocks + pos / rg.block_size];
  return (size_t)page * rg.block_size + pos % rg.block_size;
}

struct LatentPrepArgs {
  const float* z;     // [M, ldz]: q latent [q_rank] | kv latent [kv_rank] | key rot part [rot_dim]
  int ldz;
  const void* qn_w;   // [q_rank] T
  const void* kvn_w;  // [kv_rank] T
  void* cq;           // [M, q_rank] T
  void* cache;        // [rows, kv_rank + rot_dim] T (this layer's pool)
  const float* inv_freq;  // [rot_dims / 2]
  int q_rank, kv_rank, rot_dim, rot_dims;
  float eps;
};

template <typename T>
__global__ void latent_prep_kernel(const LatentPrepArgs p, const Ragged rg) {
  __shared__ float red[33];
  const int m = blockIdx.x, s = rg.tok_seq[m];
  const int pos = rg.pos0[s] + (m - rg.cu[s]);
  const float* z = p.z + (size_t)m * p.ldz;
  float ss = 0.f;
  for (int c = threadIdx.x; c < p.q_rank; c += blockDim.x) ss = fmaf(z[c], z[c], ss);
  ss = block_sum(ss, red);
  float inv = 1.0f / sqrtf(ss / (float)p.q_rank + p.eps);
  for (int c = threadIdx.x; c < p.q_rank; c += blockDim.x)
    st_f<T>((T*)p.cq + (size_t)m * p.q_rank + c, z[c] * inv * ld_f<T>((const T*)p.qn_w + c));
  const float* zk = z + p.q_rank;
  ss = 0.f;
  for (int c = threadIdx.x; c < p.kv_rank; c += blockDim.x) ss = fmaf(zk[c], zk[c], ss);
  ss = block_sum(ss, red);
  inv = 1.0f / sqrtf(ss / (float)p.kv_rank + p.eps);
  T* row = (T*)p.cache + page_row(rg, s, pos) * (size_t)(p.kv_rank + p.rot_dim);
  for (int c = threadIdx.x; c < p.kv_rank; c += blockDim.x) st_f<T>(row + c, zk[c] * inv * ld_f<T>((const T*)p.kvn_w + c));
  const float* zr = zk + p.kv_rank;
  const int half = p.rot_dims / 2;
  for (int c = threadIdx.x; c < p.rot_dim; c += blockDim.x) {
    float out = zr[c];
    if (c < p.rot_dims) {
      const int i = c < half ? c : c - half;
      float sn, cs;
      sincosf((float)pos * p.inv_freq[i], &sn, &cs);
      out = c < half ? zr[c] * cs - zr[c + half] * sn : zr[c] * cs + zr[c - half] * sn;
    }
    st_f<T>(row + p.kv_rank + c, out);
  }
}

// q [M, H, D + R] fp32 -> qn [M, H, D] (T), qr [M, H, R] fp32 rotated
template <typename T>
__global__ void latent_q_kernel(const float* __restrict__ q, T* __restrict__ qn, float* __restrict__ qr,
                                const float* __restrict__ inv_freq, const Ragged rg, int H, int D, int R, int rot_dims) {
  const int m = blockIdx.x, hd = blockIdx.y, s = rg.tok_seq[m];
  const int pos = rg.pos0[s] + (m - rg.cu[s]);
  const float* src = q + ((size_t)m * H + hd) * (D + R);
  for (int c = threadIdx.x; c < D; c += blockDim.x) st_f<T>(qn + ((size_t)m * H + hd) * D + c, src[c]);
  const float* zr = src + D;
  const int half = rot_dims / 2;
  for (int c = threadIdx.x; c < R; c += blockDim.x) {
    float out = zr[c];
    if (c < rot_dims) {
      const int i = c < half ? c : c - half;
      float sn, cs;
      sincosf((float)pos * inv_freq[i], &sn, &cs);
      out = c < half ? zr[c] * cs - zr[c + half] * sn : zr[c] * cs + zr[c - half] * sn;
    }
    qr[((size_t)m * H + hd) * R + c] = out;
  }
}

struct LatentAttnArgs {
  const float* qlat;  // [M, H, kv_rank] fp32 absorbed queries
  const float* qr;    // [M, H, R] fp32 rotated queries
  const void* cache;  // [rows, kv_rank + R] T
  const void* sink;   // [H] T
  void* out;          // [M, H, kv_rank] T
  int H, kv_rank, R, hg;  // hg = heads per CTA
  float scale;
};
constexpr int kLatKC = 32;       // keys per chunk
constexpr int kLatThreads = 256;

// dynamic shared memory: q [hg][W] | keys [KC][Wp] | acc [hg][kv_rank] | sc [hg][KC] | m, l, f [hg] each;  W = kv_rank + R,
// Wp = W | 1 (odd row stride: the score loop reads one key row per thread)
template <typename T>
__global__ void __launch_bounds__(kLatThreads) latent_attn_kernel(const LatentAttnArgs p, const Ragged rg) {
  SSDK_DYN_SMEM(float, sm);
  const int m = blockIdx.x, h0 = blockIdx.y * p.hg, nh = min(p.hg, p.H - h0);
  const int s = rg.tok_seq[m], pos = rg.pos0[s] + (m - rg.cu[s]);
  const int KR = p.kv_rank, R = p.R, W = KR + R, Wp = W | 1;
  const int tid = threadIdx.x;
  float* s_q = sm;
  float* s_key = s_q + p.hg * W;
  float* s_acc = s_key + kLatKC * Wp;
  float* s_sc = s_acc + p.hg * KR;
  float* s_m = s_sc + p.hg * kLatKC;
  float* s_l = s_m + p.hg;
  float* s_f = s_l + p.hg;
  for (int e = tid; e < nh * W; e += kLatThreads) {
    const int h = e / W, d = e % W;
    s_q[e] = d < KR ? p.qlat[((size_t)m * p.H + h0 + h) * KR + d] : p.qr[((size_t)m * p.H + h0 + h) * R + (d - KR)];
  }
  for (int e = tid; e < nh * KR; e += kLatThreads) s_acc[e] = 0.f;
  if (tid < nh) { s_m[tid] = ld_f<T>((const T*)p.sink + h0 + tid); s_l[tid] = 1.0f; }
  const int ctx = pos + 1;
  const int warp = tid >> 5, lane = tid & 31;
  for (int c0 = 0; c0 < ctx; c0 += kLatKC) {
    const int nk = min(kLatKC, ctx - c0);
    __syncthreads();
    for (int e = tid; e < nk * W; e += kLatThreads) {
      const int jk = e / W, d = e % W;
      s_key[jk * Wp + d] = ld_f<T>((const T*)p.cache + page_row(rg, s, c0 + jk) * (size_t)W + d);
    }
    __syncthreads();
    for (int e = tid; e < nh * kLatKC; e += kLatThreads) {
      const int h = e / kLatKC, jk = e % kLatKC;
      float sc = -INFINITY;
      if (jk < nk) {
        float a = 0.f;
        const float* qv = s_q + h * W;
        const float* kv = s_key + jk * Wp;
        for (int d = 0; d < W; ++d) a = fmaf(qv[d], kv[d], a);
        sc = a * p.scale;
      }
      s_sc[e] = sc;
    }
    __syncthreads();
    for (int h = warp; h < nh; h += kLatThreads / 32) {   // kLatKC == 32: one key per lane
      const float sc = s_sc[h * kLatKC + lane];
      const float mo = s_m[h], mn = fmaxf(mo, warp_max(sc));
      const float pr = lane < nk ? expf(sc - mn) : 0.f;
      const float sum = warp_sum(pr);
      s_sc[h * kLatKC + lane] = pr;
      if (lane == 0) {
        const float f = expf(mo - mn);
        s_f[h] = f;
        s_l[h] = fmaf(s_l[h], f, sum);
        s_m[h] = mn;
      }
    }
    __syncthreads();
    for (int e = tid; e < nh * KR; e += kLatThreads) {
      const int h = e / KR, r = e % KR;
      float a = s_acc[e] * s_f[h];
      const float* pr = s_sc + h * kLatKC;
      for (int jk = 0; jk < nk; ++jk) a = fmaf(pr[jk], s_key[jk * Wp + r], a);
      s_acc[e] = a;
    }
  }
  __syncthreads();
  for (int e = tid; e < nh * KR; e += kLatThreads) {
    const int h = e / KR, r = e % KR;
    st_f<T>((T*)p.out + ((size_t)m * p.H + h0 + h) * KR + r, s_acc[e] / s_l[h]);
  }
}

}  // namespace ssdk
