// gqa_attention.cuh — grouped-query causal softmax attention over a paged key/value cache, for the layered (hybrid)
// models.  H query heads share G key/value heads (query head h reads head h / (H / G)); key size D and value size V are
// independent.  A page row holds, for one token, the keys of all G heads (rotated, optionally unit-RMS) and then their
// values: [G D | G V] of storage type T.  The softmax denominator may carry a constant (`sink`: 1 = a sink of score 0
// that has no value), on top of or instead of the learned per-head sink of latent attention.
//
//   gqa_prep_kernel      per (token, head): interleaved-pair rotation of the first rot_dims dimensions (angle = position *
//                        frequency in fp32, cos and sin times a constant), optional unit RMS over D; queries go to a
//                        group-major buffer [G, M, H/G, D] (T), keys and raw values into the token's page row
//   kv_gather_kernel     one sequence's pages -> contiguous keys [G, ctx_pad, D] and transposed values [G, V, ctx_pad]
//   portions (>= 2 rows) two batched GEMMs per query block around sink_softmax_kernel (HybRun::gqa_attention)
//   single-token rows    gqa_decode_partial_kernel (all decoding sequences in one launch, context split flash-decoding
//                        style, fp32 weights) + gqa_decode_merge_kernel
//   attn_gate_kernel     group-major fp32 output x sigmoid(gate pre-activation) -> [M, H V] (T) for the output projection
#pragma once
#include "latent_attention.cuh"

namespace ssdk {

struct GqaPrepArgs {
  const float* z; int ldz;     // [M, ldz]: q [H D] | k [G D] | v [G V] (fp32 projections)
  void* q;                     // [G, M, H/G, D] T
  void* cache;                 // [rows, G (D + V)] T (this layer's pool)
  const float* inv_freq;       // [rot_dims / 2] or nullptr
  int H, G, D, V, rot_dims, qk_norm;
  float rot_mult, eps;
};

// grid (M, H + G), one warp: units 0 .. H-1 are query heads, H .. H+G-1 key heads (which also copy their value head)
template <typename T>
__global__ void gqa_prep_kernel(const GqaPrepArgs p, const Ragged rg) {
  const int m = blockIdx.x, unit = blockIdx.y, lane = threadIdx.x, s = rg.tok_seq[m];
  const int pos = rg.pos0[s] + (m - rg.cu[s]);
  const int H = p.H, G = p.G, D = p.D, V = p.V;
  const bool is_q = unit < H;
  const int hd = is_q ? unit : unit - H;
  const float* src = p.z + (size_t)m * p.ldz + (is_q ? (size_t)hd * D : (size_t)H * D + (size_t)hd * D);
  T* dst;
  if (is_q) {
    const int hpg = H / G, g = hd / hpg;
    dst = (T*)p.q + (((size_t)g * rg.M + m) * hpg + (hd - g * hpg)) * D;
  } else {
    dst = (T*)p.cache + page_row(rg, s, pos) * (size_t)(G * (D + V)) + (size_t)hd * D;
  }
  // pass 1: rotate pairs, accumulate the square sum; pass 2: scale and store (the pair values are recomputed)
  float ss = 0.f;
  const int rd = p.inv_freq ? p.rot_dims : 0;
  auto value = [&](int d) -> float {
    if (d >= rd) return src[d];
    const int i = d >> 1;
    float sn, cs;
    sincosf((float)pos * p.inv_freq[i], &sn, &cs);
    sn *= p.rot_mult; cs *= p.rot_mult;
    const float a = src[2 * i], b = src[2 * i + 1];
    return (d & 1) ? b * cs + a * sn : a * cs - b * sn;
  };
  float inv = 1.0f;
  if (p.qk_norm) {
    for (int d = lane; d < D; d += 32) { const float v = value(d); ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    inv = 1.0f / sqrtf(ss / (float)D + p.eps);
  }
  for (int d = lane; d < D; d += 32) st_f<T>(dst + d, value(d) * inv);
  if (!is_q) {
    const float* vsrc = p.z + (size_t)m * p.ldz + (size_t)(H + G) * D + (size_t)hd * V;
    T* vdst = (T*)p.cache + page_row(rg, s, pos) * (size_t)(G * (D + V)) + (size_t)G * D + (size_t)hd * V;
    for (int d = lane; d < V; d += 32) st_f<T>(vdst + d, vsrc[d]);
  }
}

// grid (ctx_pad): position j of sequence s -> keys[g][j][:] and vt[g][:][j]; zero from ctx up to ctx_pad
template <typename T>
__global__ void kv_gather_kernel(const T* __restrict__ cache, T* __restrict__ keys, T* __restrict__ vt, const Ragged rg, int s,
                                 int ctx, int ctx_pad, int G, int D, int V) {
  const int j = blockIdx.x;
  const T* row = j < ctx ? cache + page_row(rg, s, j) * (size_t)(G * (D + V)) : nullptr;
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    keys[((size_t)g * ctx_pad + j) * D + d] = row ? row[i] : T(0.f);
  }
  for (int i = threadIdx.x; i < G * V; i += blockDim.x) vt[(size_t)i * ctx_pad + j] = row ? row[(size_t)G * D + i] : T(0.f);
}

struct GqaDecodeArgs {
  const void* q;      // [G, M, H/G, D] T
  const void* cache;  // [rows, G (D + V)] T
  float* part;        // [n_seqs, H, splits, V + 2] fp32: unnormalised P V | running maximum | running sum
  float* out;         // [G, M, H/G, V] fp32
  int H, G, D, V, splits;
  float scale, sink;
};

constexpr int kGqaDecWarps = 4;

inline size_t gqa_decode_smem(int D, int V) { return ((size_t)D + (size_t)kGqaDecWarps * (V + 2)) * 4; }

// grid (n_seqs, H, splits), kGqaDecWarps warps.  A warp takes 32 keys at a time: first every lane scores ONE key (a
// thread-local dot product over D), then every lane owns value columns lane, lane + 32, .. and the 32 weights are
// passed around by shuffle.  VPL = ceil(V / 32) accumulators per lane.
template <typename T, int VPL>
__global__ void __launch_bounds__(kGqaDecWarps * 32) gqa_decode_partial_kernel(const GqaDecodeArgs p, const Ragged rg) {
  extern __shared__ float gd_sm[];
  const int s = blockIdx.x, hd = blockIdx.y, sp = blockIdx.z;
  const int row = rg.cu[s];
  if (rg.cu[s + 1] - row != 1) return;
  const int H = p.H, G = p.G, D = p.D, V = p.V, hpg = H / G, g = hd / hpg;
  float* qs = gd_sm;                      // [D] query times scale
  float* wp = gd_sm + D;                  // [warps][V + 2]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* q = (const T*)p.q + (((size_t)g * rg.M + row) * hpg + (hd - g * hpg)) * D;
  for (int d = tid; d < D; d += blockDim.x) qs[d] = ld_f<T>(q + d) * p.scale;
  __syncthreads();
  const int ctx = rg.pos0[s] + 1, per = (ctx + p.splits - 1) / p.splits;
  const int k_lo = sp * per, k_hi = min(ctx, k_lo + per);
  const size_t roww = (size_t)G * (D + V);
  float mx = -INFINITY, sum = 0.f, acc[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) acc[i] = 0.f;
  for (int k0 = k_lo + warp * 32; k0 < k_hi; k0 += kGqaDecWarps * 32) {
    const int key = k0 + lane;
    const bool ok = key < k_hi;
    const size_t prow = ok ? page_row(rg, s, key) : 0;
    float sc = -INFINITY;
    if (ok) {
      const T* kr = (const T*)p.cache + prow * roww + (size_t)g * D;
      float a0 = 0.f, a1 = 0.f;
      int d = 0;
      for (; d + 1 < D; d += 2) { a0 = fmaf(qs[d], ld_f<T>(kr + d), a0); a1 = fmaf(qs[d + 1], ld_f<T>(kr + d + 1), a1); }
      if (d < D) a0 = fmaf(qs[d], ld_f<T>(kr + d), a0);
      sc = a0 + a1;
    }
    const float m_new = fmaxf(mx, warp_max(sc));
    const float r = mx == -INFINITY ? 0.f : expf(mx - m_new);
    const float w = ok ? expf(sc - m_new) : 0.f;
    sum = sum * r + warp_sum(w);
#pragma unroll
    for (int i = 0; i < VPL; ++i) acc[i] *= r;
    mx = m_new;
    const int nk = min(32, k_hi - k0);
    for (int kk = 0; kk < nk; ++kk) {
      const float wk = __shfl_sync(0xffffffffu, w, kk);
      const unsigned long long pr = __shfl_sync(0xffffffffu, (unsigned long long)prow, kk);
      const T* vr = (const T*)p.cache + (size_t)pr * roww + (size_t)G * D + (size_t)g * V;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int c = lane + 32 * i;
        if (c < V) acc[i] = fmaf(wk, ld_f<T>(vr + c), acc[i]);
      }
    }
  }
  float* mine = wp + (size_t)warp * (V + 2);
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = lane + 32 * i;
    if (c < V) mine[c] = acc[i];
  }
  if (lane == 0) { mine[V] = mx; mine[V + 1] = sum; }
  __syncthreads();
  // the warps' parts are joined in warp order
  float m = -INFINITY;
  for (int w = 0; w < kGqaDecWarps; ++w) m = fmaxf(m, wp[(size_t)w * (V + 2) + V]);
  float* dst = p.part + (((size_t)s * H + hd) * p.splits + sp) * (V + 2);
  for (int c = tid; c < V + 1; c += blockDim.x) {
    float a = 0.f;
    for (int w = 0; w < kGqaDecWarps; ++w) {
      const float mw = wp[(size_t)w * (V + 2) + V];
      if (mw != -INFINITY) a = fmaf(expf(mw - m), wp[(size_t)w * (V + 2) + (c < V ? c : V + 1)], a);
    }
    dst[c < V ? c : V + 1] = a;
  }
  if (tid == 0) dst[V] = m;
}

// grid (n_seqs, H): out = sum_j e^(m_j - m) acc_j / (sink e^(-m) + sum_j e^(m_j - m) l_j)
__global__ void gqa_decode_merge_kernel(const GqaDecodeArgs p, const Ragged rg) {
  const int s = blockIdx.x, hd = blockIdx.y;
  const int row = rg.cu[s];
  if (rg.cu[s + 1] - row != 1) return;
  const int V = p.V, hpg = p.H / p.G, g = hd / hpg;
  const float* part = p.part + ((size_t)s * p.H + hd) * p.splits * (V + 2);
  float m = p.sink > 0.f ? 0.f : -INFINITY;
  for (int j = 0; j < p.splits; ++j) m = fmaxf(m, part[(size_t)j * (V + 2) + V]);
  float den = p.sink > 0.f ? p.sink * expf(-m) : 0.f;
  for (int j = 0; j < p.splits; ++j) {
    const float mj = part[(size_t)j * (V + 2) + V];
    if (mj != -INFINITY) den += expf(mj - m) * part[(size_t)j * (V + 2) + V + 1];
  }
  const float inv = 1.0f / den;
  float* out = p.out + (((size_t)g * rg.M + row) * hpg + (hd - g * hpg)) * V;
  for (int c = threadIdx.x; c < V; c += blockDim.x) {
    float a = 0.f;
    for (int j = 0; j < p.splits; ++j) {
      const float mj = part[(size_t)j * (V + 2) + V];
      if (mj != -INFINITY) a = fmaf(expf(mj - m), part[(size_t)j * (V + 2) + c], a);
    }
    out[c] = a * inv;
  }
}

// o [G, M, H/G, V] fp32 (group-major) and gate pre-activations gz[m * ldg + h * V + v] -> y [M, H V] (T) = o * sigmoid(gz)
template <typename T>
__global__ void attn_gate_kernel(const float* __restrict__ o, const float* __restrict__ gz, int ldg, T* __restrict__ y, int M, int H,
                                 int G, int V) {
  const int m = blockIdx.x, hpg = H / G;
  for (int i = threadIdx.x; i < H * V; i += blockDim.x) {
    const int hd = i / V, v = i - hd * V, g = hd / hpg;
    const float ov = o[(((size_t)g * M + m) * hpg + (hd - g * hpg)) * V + v];
    st_f<T>(y + (size_t)m * H * V + i, gz ? ov * sigmoid_f(gz[(size_t)m * ldg + i]) : ov);
  }
}

}  // namespace ssdk
