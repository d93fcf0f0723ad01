// recurrent.cuh — matrix-state recurrences of the layered (hybrid) models.  One CTA per (sequence, head) walks the
// rows that this step brings for the sequence, in order, with the head's state matrix S [K, V] resident in shared
// memory (thread j owns column j: S[i][j] at s_S[i * V + j], so a warp's accesses are conflict free) and writes it
// back to the sequence's state slot.  Everything that enters the recurrence (decays, gates, stabiliser, state, the
// read-out) is fp32; the projections arrive as fp32 GEMM outputs.
//
//   wkv_scan_kernel   (RWKV-style, per-channel data-dependent decay, bonus u for the current token)
//       o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t ;  S_t = diag(w_t) S_{t-1} + k_t v_t^T ;  w_t = exp(-exp(z_t + w0))
//   mlstm_scan_kernel (xLSTM matrix memory with exponential gating and a running stabiliser m, m_0 = 0)
//       m_t = max(f_t + m_{t-1}, i_t);  S_t = e^{f_t + m_{t-1} - m_t} S_{t-1} + e^{i_t - m_t} k_t v_t^T;  n_t likewise with k_t
//       o_t = S_t^T q_t / (max(|n_t . q_t|, e^{-m_t}) + 1e-6)
//       i_t = cap tanh(i_raw / cap),  f_t = logsigmoid(cap tanh(f_raw / cap))
// A slot's content is read only when the sequence has run tokens before (pos0 > 0): a reused slot needs no clearing.
#pragma once
#include "layer_ops.cuh"

namespace ssdk {

struct WkvArgs {
  const float* r; const float* k; const float* v; const float* zw;  // [M, ld] each, head h at column h * D
  int ld;
  const void* w0;    // [H * D] T   decay bias
  const void* u;     // [H, D] T    bonus
  float* o;          // [M, H * D]
  float* state;      // per slot: S [H, D, D]
  size_t slot_stride;
  // token-shift carry: the portion's last row of h goes to the slot (written by the head-0 CTA)
  const void* h; float* h_prev; int width;
  int H, D;
};

template <typename T>
__global__ void wkv_scan_kernel(const WkvArgs p, const Ragged rg) {
  SSDK_DYN_SMEM(float, sm);
  const int s = blockIdx.x, hd = blockIdx.y, D = p.D, j = threadIdx.x;
  float* s_S = sm;            // [D][D]
  float* s_r = s_S + D * D;   // [D]
  float* s_k = s_r + D;
  float* s_w = s_k + D;
  float* s_u = s_w + D;
  float* s_w0 = s_u + D;
  const int row_lo = rg.cu[s], row_hi = rg.cu[s + 1];
  if (row_hi <= row_lo) return;
  float* S_g = p.state + (size_t)rg.slot[s] * p.slot_stride + (size_t)hd * D * D;
  const bool fresh = rg.pos0[s] == 0;
  for (int e = j; e < D * D; e += blockDim.x) s_S[e] = fresh ? 0.f : S_g[e];
  if (j < D) {
    s_u[j] = ld_f<T>((const T*)p.u + hd * D + j);
    s_w0[j] = ld_f<T>((const T*)p.w0 + hd * D + j);
  }
  for (int t = row_lo; t < row_hi; ++t) {
    __syncthreads();
    const size_t base = (size_t)t * p.ld + hd * D;
    float vj = 0.f;
    if (j < D) {
      s_r[j] = p.r[base + j];
      s_k[j] = p.k[base + j];
      s_w[j] = expf(-expf(p.zw[base + j] + s_w0[j]));
      vj = p.v[base + j];
    }
    __syncthreads();
    if (j < D) {
      float acc = 0.f;
      for (int i = 0; i < D; ++i) {
        const float st = s_S[i * D + j];
        const float kv = s_k[i] * vj;
        acc = fmaf(s_r[i], fmaf(s_u[i], kv, st), acc);
        s_S[i * D + j] = fmaf(s_w[i], st, kv);
      }
      p.o[(size_t)t * p.H * D + hd * D + j] = acc;
    }
  }
  __syncthreads();
  for (int e = j; e < D * D; e += blockDim.x) S_g[e] = s_S[e];
  if (hd == 0) {
    float* hp = p.h_prev + (size_t)rg.slot[s] * p.slot_stride;
    for (int c = j; c < p.width; c += blockDim.x) hp[c] = ld_f<T>((const T*)p.h + (size_t)(row_hi - 1) * p.width + c);
  }
}

struct MlstmArgs {
  const float* q; const float* k; const float* v;  // [M, ld]; q/k head h at column h * D, v at h * V
  const float* ig; const float* fg;                // [M, ld] raw gate projections (bias not yet added), head h at column h
  int ld;
  const void* ib; const void* fb;                  // [H] T gate biases
  float* o;                                        // [M, H * V]
  float* S; float* n; float* m;                    // slot-relative bases: S [H, D, V], n [H, D], m [H]
  size_t slot_stride;
  int H, D, V;
  float cap, q_scale;
};

SSDK_DEVINL float log_sigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

template <typename T>
__global__ void mlstm_scan_kernel(const MlstmArgs p, const Ragged rg) {
  SSDK_DYN_SMEM(float, sm);
  const int s = blockIdx.x, hd = blockIdx.y, D = p.D, V = p.V, j = threadIdx.x;
  float* s_S = sm;            // [D][V]
  float* s_q = s_S + D * V;   // [D]
  float* s_k = s_q + D;
  float* s_n = s_k + D;
  const int row_lo = rg.cu[s], row_hi = rg.cu[s + 1];
  if (row_hi <= row_lo) return;
  const size_t slot = (size_t)rg.slot[s] * p.slot_stride;
  float* S_g = p.S + slot + (size_t)hd * D * V;
  float* n_g = p.n + slot + (size_t)hd * D;
  float* m_g = p.m + slot + hd;
  const bool fresh = rg.pos0[s] == 0;
  for (int e = j; e < D * V; e += blockDim.x) s_S[e] = fresh ? 0.f : S_g[e];
  for (int e = j; e < D; e += blockDim.x) s_n[e] = fresh ? 0.f : n_g[e];
  float m = fresh ? 0.f : *m_g;
  const float ib = ld_f<T>((const T*)p.ib + hd), fb = ld_f<T>((const T*)p.fb + hd);
  for (int t = row_lo; t < row_hi; ++t) {
    const float iraw = p.ig[(size_t)t * p.ld + hd] + ib, fraw = p.fg[(size_t)t * p.ld + hd] + fb;
    const float ig = p.cap * tanhf(iraw / p.cap);
    const float fg = log_sigmoid_f(p.cap * tanhf(fraw / p.cap));
    const float mn = fmaxf(fg + m, ig);
    const float a = expf(fg + m - mn), b = expf(ig - mn);
    m = mn;
    __syncthreads();  // the previous row's readers of s_q / s_k / s_n are done
    for (int e = j; e < D; e += blockDim.x) {
      const float kk = p.k[(size_t)t * p.ld + hd * D + e];
      s_q[e] = p.q[(size_t)t * p.ld + hd * D + e] * p.q_scale;
      s_k[e] = kk;
      s_n[e] = fmaf(a, s_n[e], b * kk);
    }
    __syncthreads();
    if (j < V) {
      const float bv = b * p.v[(size_t)t * p.ld + hd * V + j];
      float acc = 0.f, dot = 0.f;
      for (int i = 0; i < D; ++i) {
        const float st = fmaf(a, s_S[i * V + j], s_k[i] * bv);
        s_S[i * V + j] = st;
        acc = fmaf(st, s_q[i], acc);
        dot = fmaf(s_n[i], s_q[i], dot);
      }
      const float den = fmaxf(fabsf(dot), expf(-m)) + 1e-6f;
      p.o[(size_t)t * p.H * V + hd * V + j] = acc / den;
    }
  }
  __syncthreads();
  for (int e = j; e < D * V; e += blockDim.x) S_g[e] = s_S[e];
  for (int e = j; e < D; e += blockDim.x) n_g[e] = s_n[e];
  if (j == 0) *m_g = m;
}

}  // namespace ssdk
