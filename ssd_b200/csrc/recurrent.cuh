// recurrent.cuh — matrix-state recurrences of the layered (hybrid) models.  One CTA per (sequence, head) walks the
// rows that this step brings for the sequence, in order, with the head's state matrix S [K, V] resident in shared
// memory (a thread owns a run of rows of ONE column: S[i][j] at s_S[i * V + j], so a warp's accesses are conflict
// free) and writes it back to the sequence's state slot.  Everything that enters the recurrence (decays, gates, stabiliser, state, the
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

// Thread layout of both scans: tid = g * Vr + j, Vr = V rounded up to a warp: column j of the state, row group g of G
// (rows [g * Dg, (g + 1) * Dg)).  The G partial read-outs of a column meet in shared memory and are summed in the
// fixed order g = 0 .. G-1.  The next row's operands are requested from global memory before the current row's
// arithmetic starts, so their latency hides behind it.
struct ScanShape {
  int Vr, G, Dg;
};
constexpr int kScanPF = 4;  // rows of operands in flight in the register-resident scans

template <typename T>
__global__ void wkv_scan_kernel(const WkvArgs p, const Ragged rg, const ScanShape sh) {
  SSDK_DYN_SMEM(float, sm);
  const int s = blockIdx.x, hd = blockIdx.y, D = p.D, tid = threadIdx.x, nt = blockDim.x;
  const int j = tid % sh.Vr, g = tid / sh.Vr, i_lo = g * sh.Dg, i_hi = min(D, i_lo + sh.Dg);
  float* s_S = sm;            // [D][D]
  float* s_r = s_S + D * D;   // [D]
  float* s_k = s_r + D;
  float* s_w = s_k + D;
  float* s_u = s_w + D;
  float* s_w0 = s_u + D;
  float* s_part = s_w0 + D;   // [G][Vr]
  const int row_lo = rg.cu[s], row_hi = rg.cu[s + 1];
  if (row_hi <= row_lo) return;
  float* S_g = p.state + (size_t)rg.slot[s] * p.slot_stride + (size_t)hd * D * D;
  const bool fresh = rg.pos0[s] == 0;
  for (int e = tid; e < D * D; e += nt) s_S[e] = fresh ? 0.f : S_g[e];
  for (int e = tid; e < D; e += nt) {
    s_u[e] = ld_f<T>((const T*)p.u + hd * D + e);
    s_w0[e] = ld_f<T>((const T*)p.w0 + hd * D + e);
  }
  // prefetched operands of the coming row: element `tid` of r, k, z (threads below D) and v[j]
  float nr = 0.f, nk = 0.f, nz = 0.f, nv = 0.f;
  {
    const size_t base = (size_t)row_lo * p.ld + hd * D;
    if (tid < D) { nr = p.r[base + tid]; nk = p.k[base + tid]; nz = p.zw[base + tid]; }
    if (j < D) nv = p.v[base + j];
  }
  for (int t = row_lo; t < row_hi; ++t) {
    __syncthreads();
    const size_t base = (size_t)t * p.ld + hd * D;
    if (tid < D) { s_r[tid] = nr; s_k[tid] = nk; s_w[tid] = expf(-expf(nz + s_w0[tid])); }
    for (int e = tid + nt; e < D; e += nt) {   // heads wider than the CTA
      s_r[e] = p.r[base + e]; s_k[e] = p.k[base + e]; s_w[e] = expf(-expf(p.zw[base + e] + s_w0[e]));
    }
    const float vj = nv;
    __syncthreads();
    if (t + 1 < row_hi) {
      const size_t nb = base + p.ld;
      if (tid < D) { nr = p.r[nb + tid]; nk = p.k[nb + tid]; nz = p.zw[nb + tid]; }
      if (j < D) nv = p.v[nb + j];
    }
    float acc = 0.f;
    if (j < D) {
#pragma unroll 4
      for (int i = i_lo; i < i_hi; ++i) {
        const float st = s_S[i * D + j];
        const float kv = s_k[i] * vj;
        acc = fmaf(s_r[i], fmaf(s_u[i], kv, st), acc);
        s_S[i * D + j] = fmaf(s_w[i], st, kv);
      }
    }
    if (sh.G > 1) {
      s_part[g * sh.Vr + j] = acc;
      __syncthreads();
      if (g == 0) {
        acc = s_part[j];
        for (int q = 1; q < sh.G; ++q) acc += s_part[q * sh.Vr + j];
      }
    }
    if (g == 0 && j < D) p.o[(size_t)t * p.H * D + hd * D + j] = acc;
  }
  __syncthreads();
  for (int e = tid; e < D * D; e += nt) S_g[e] = s_S[e];
  if (hd == 0) {
    float* hp = p.h_prev + (size_t)rg.slot[s] * p.slot_stride;
    for (int c = tid; c < p.width; c += nt) hp[c] = ld_f<T>((const T*)p.h + (size_t)(row_hi - 1) * p.width + c);
  }
}

// Register-resident variant: every thread keeps its DG rows of its column in registers for the whole portion (the state
// never touches shared memory), the per-row operands {r, k, w, u} travel as ONE float4 per state row (rows beyond the
// head size are zero operands), so a state row costs one broadcast shared-memory load instead of six accesses.
// Launched when G * DG >= D with DG in {8, 16, 32} fits a CTA; the shared-memory kernel above serves every other size.
template <typename T, int DG>
__global__ void __launch_bounds__(512) wkv_scan_reg_kernel(const WkvArgs p, const Ragged rg, const ScanShape sh) {
  SSDK_DYN_SMEM(float4, sm4);
  const int s = blockIdx.x, hd = blockIdx.y, D = p.D, tid = threadIdx.x;
  const int j = tid % sh.Vr, g = tid / sh.Vr, i_lo = g * DG, rows = sh.G * DG;
  float4* s_op = sm4;                                        // [rows] {r, k, w, u}
  float* s_part = reinterpret_cast<float*>(s_op + rows);     // [G][Vr]
  const int row_lo = rg.cu[s], row_hi = rg.cu[s + 1];
  if (row_hi <= row_lo) return;
  float* S_g = p.state + (size_t)rg.slot[s] * p.slot_stride + (size_t)hd * D * D;
  const bool fresh = rg.pos0[s] == 0;
  float S[DG];
#pragma unroll
  for (int ii = 0; ii < DG; ++ii) S[ii] = (!fresh && j < D && i_lo + ii < D) ? S_g[(size_t)(i_lo + ii) * D + j] : 0.f;
  float my_u = 0.f, my_w0 = 0.f;
  if (tid < D) { my_u = ld_f<T>((const T*)p.u + hd * D + tid); my_w0 = ld_f<T>((const T*)p.w0 + hd * D + tid); }
  // the operands of the next kScanPF rows are in flight (registers) while a row is computed: a row's arithmetic is far
  // shorter than a trip to L2
  float nr[kScanPF], nk[kScanPF], nz[kScanPF], nv[kScanPF];
#pragma unroll
  for (int u = 0; u < kScanPF; ++u) {
    nr[u] = nk[u] = nz[u] = nv[u] = 0.f;
    if (row_lo + u < row_hi) {
      const size_t base = (size_t)(row_lo + u) * p.ld + hd * D;
      if (tid < D) { nr[u] = p.r[base + tid]; nk[u] = p.k[base + tid]; nz[u] = p.zw[base + tid]; }
      if (j < D) nv[u] = p.v[base + j];
    }
  }
  for (int t0 = row_lo; t0 < row_hi; t0 += kScanPF) {
#pragma unroll
    for (int u = 0; u < kScanPF; ++u) {
      const int t = t0 + u;
      if (t >= row_hi) break;
      __syncthreads();
      if (tid < rows) s_op[tid] = tid < D ? make_float4(nr[u], nk[u], expf(-expf(nz[u] + my_w0)), my_u) : make_float4(0.f, 0.f, 0.f, 0.f);
      const float vj = nv[u];
      __syncthreads();
      if (t + kScanPF < row_hi) {
        const size_t nb = (size_t)(t + kScanPF) * p.ld + hd * D;
        if (tid < D) { nr[u] = p.r[nb + tid]; nk[u] = p.k[nb + tid]; nz[u] = p.zw[nb + tid]; }
        if (j < D) nv[u] = p.v[nb + j];
      }
      float acc = 0.f;
#pragma unroll
      for (int ii = 0; ii < DG; ++ii) {
        const float4 o = s_op[i_lo + ii];
        const float kv = o.y * vj;
        acc = fmaf(o.x, fmaf(o.w, kv, S[ii]), acc);
        S[ii] = fmaf(o.z, S[ii], kv);
      }
      if (sh.G > 1) {
        s_part[g * sh.Vr + j] = acc;
        __syncthreads();
        if (g == 0) {
          acc = s_part[j];
          for (int q = 1; q < sh.G; ++q) acc += s_part[q * sh.Vr + j];
        }
      }
      if (g == 0 && j < D) p.o[(size_t)t * p.H * D + hd * D + j] = acc;
    }
  }
#pragma unroll
  for (int ii = 0; ii < DG; ++ii)
    if (j < D && i_lo + ii < D) S_g[(size_t)(i_lo + ii) * D + j] = S[ii];
  if (hd == 0) {
    float* hp = p.h_prev + (size_t)rg.slot[s] * p.slot_stride;
    for (int c = tid; c < p.width; c += blockDim.x) hp[c] = ld_f<T>((const T*)p.h + (size_t)(row_hi - 1) * p.width + c);
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
__global__ void mlstm_scan_kernel(const MlstmArgs p, const Ragged rg, const ScanShape sh) {
  SSDK_DYN_SMEM(float, sm);
  const int s = blockIdx.x, hd = blockIdx.y, D = p.D, V = p.V, tid = threadIdx.x, nt = blockDim.x;
  const int j = tid % sh.Vr, g = tid / sh.Vr, i_lo = g * sh.Dg, i_hi = min(D, i_lo + sh.Dg);
  float* s_S = sm;            // [D][V]
  float* s_q = s_S + D * V;   // [D]
  float* s_k = s_q + D;
  float* s_n = s_k + D;
  float* s_part = s_n + D;    // [G][Vr] read-out partials
  float* s_dot = s_part + sh.G * sh.Vr;  // [G] partial n . q
  const int row_lo = rg.cu[s], row_hi = rg.cu[s + 1];
  if (row_hi <= row_lo) return;
  const size_t slot = (size_t)rg.slot[s] * p.slot_stride;
  float* S_g = p.S + slot + (size_t)hd * D * V;
  float* n_g = p.n + slot + (size_t)hd * D;
  float* m_g = p.m + slot + hd;
  const bool fresh = rg.pos0[s] == 0;
  for (int e = tid; e < D * V; e += nt) s_S[e] = fresh ? 0.f : S_g[e];
  for (int e = tid; e < D; e += nt) s_n[e] = fresh ? 0.f : n_g[e];
  float m = fresh ? 0.f : *m_g;
  const float ib = ld_f<T>((const T*)p.ib + hd), fb = ld_f<T>((const T*)p.fb + hd);
  float nq = 0.f, nk = 0.f, nv = 0.f, ni, nf;
  {
    const size_t base = (size_t)row_lo * p.ld;
    if (tid < D) { nq = p.q[base + hd * D + tid]; nk = p.k[base + hd * D + tid]; }
    if (j < V) nv = p.v[base + hd * V + j];
    ni = p.ig[base + hd]; nf = p.fg[base + hd];
  }
  for (int t = row_lo; t < row_hi; ++t) {
    const size_t base = (size_t)t * p.ld;
    const float ig = p.cap * tanhf((ni + ib) / p.cap);
    const float fg = log_sigmoid_f(p.cap * tanhf((nf + fb) / p.cap));
    const float mn = fmaxf(fg + m, ig);
    const float a = expf(fg + m - mn), b = expf(ig - mn);
    m = mn;
    __syncthreads();  // the previous row's readers of s_q / s_k / s_n / s_part are done
    if (tid < D) { s_q[tid] = nq * p.q_scale; s_k[tid] = nk; s_n[tid] = fmaf(a, s_n[tid], b * nk); }
    for (int e = tid + nt; e < D; e += nt) {   // heads wider than the CTA
      const float kk = p.k[base + hd * D + e];
      s_q[e] = p.q[base + hd * D + e] * p.q_scale; s_k[e] = kk; s_n[e] = fmaf(a, s_n[e], b * kk);
    }
    const float bv = b * nv;
    __syncthreads();
    if (t + 1 < row_hi) {
      const size_t nb = base + p.ld;
      if (tid < D) { nq = p.q[nb + hd * D + tid]; nk = p.k[nb + hd * D + tid]; }
      if (j < V) nv = p.v[nb + hd * V + j];
      ni = p.ig[nb + hd]; nf = p.fg[nb + hd];
    }
    float acc = 0.f, dot = 0.f;
    if (j < V) {
#pragma unroll 4
      for (int i = i_lo; i < i_hi; ++i) {
        const float st = fmaf(a, s_S[i * V + j], s_k[i] * bv);
        s_S[i * V + j] = st;
        acc = fmaf(st, s_q[i], acc);
      }
    }
    if (j == 0) {
      for (int i = i_lo; i < i_hi; ++i) dot = fmaf(s_n[i], s_q[i], dot);
      s_dot[g] = dot;
    }
    s_part[g * sh.Vr + j] = acc;
    __syncthreads();
    if (g == 0 && j < V) {
      acc = s_part[j];
      dot = s_dot[0];
      for (int q = 1; q < sh.G; ++q) { acc += s_part[q * sh.Vr + j]; dot += s_dot[q]; }
      const float den = fmaxf(fabsf(dot), expf(-m)) + 1e-6f;
      p.o[(size_t)t * p.H * V + hd * V + j] = acc / den;
    }
  }
  __syncthreads();
  for (int e = tid; e < D * V; e += nt) S_g[e] = s_S[e];
  for (int e = tid; e < D; e += nt) n_g[e] = s_n[e];
  if (tid == 0) *m_g = m;
}

// Register-resident variant of the mLSTM scan (see wkv_scan_reg_kernel): {q, k} travel as one float2 per state row.
template <typename T, int DG>
__global__ void __launch_bounds__(512) mlstm_scan_reg_kernel(const MlstmArgs p, const Ragged rg, const ScanShape sh) {
  SSDK_DYN_SMEM(float2, sm2);
  const int s = blockIdx.x, hd = blockIdx.y, D = p.D, V = p.V, tid = threadIdx.x;
  const int j = tid % sh.Vr, g = tid / sh.Vr, i_lo = g * DG, rows = sh.G * DG;
  float2* s_op = sm2;                                      // [rows] {q, k}
  float* s_n = reinterpret_cast<float*>(s_op + rows);      // [rows]
  float* s_part = s_n + rows;                              // [G][Vr]
  float* s_dot = s_part + sh.G * sh.Vr;                    // [G]
  const int row_lo = rg.cu[s], row_hi = rg.cu[s + 1];
  if (row_hi <= row_lo) return;
  const size_t slot = (size_t)rg.slot[s] * p.slot_stride;
  float* S_g = p.S + slot + (size_t)hd * D * V;
  float* n_g = p.n + slot + (size_t)hd * D;
  float* m_g = p.m + slot + hd;
  const bool fresh = rg.pos0[s] == 0;
  float S[DG];
#pragma unroll
  for (int ii = 0; ii < DG; ++ii) S[ii] = (!fresh && j < V && i_lo + ii < D) ? S_g[(size_t)(i_lo + ii) * V + j] : 0.f;
  if (tid < rows) s_n[tid] = (!fresh && tid < D) ? n_g[tid] : 0.f;
  float m = fresh ? 0.f : *m_g;
  const float ib = ld_f<T>((const T*)p.ib + hd), fb = ld_f<T>((const T*)p.fb + hd);
  float nq[kScanPF], nk[kScanPF], nv[kScanPF], ni[kScanPF], nf[kScanPF];
#pragma unroll
  for (int u = 0; u < kScanPF; ++u) {
    nq[u] = nk[u] = nv[u] = ni[u] = nf[u] = 0.f;
    if (row_lo + u < row_hi) {
      const size_t base = (size_t)(row_lo + u) * p.ld;
      if (tid < D) { nq[u] = p.q[base + hd * D + tid]; nk[u] = p.k[base + hd * D + tid]; }
      if (j < V) nv[u] = p.v[base + hd * V + j];
      ni[u] = p.ig[base + hd]; nf[u] = p.fg[base + hd];
    }
  }
  for (int t0 = row_lo; t0 < row_hi; t0 += kScanPF) {
#pragma unroll
    for (int u = 0; u < kScanPF; ++u) {
      const int t = t0 + u;
      if (t >= row_hi) break;
      const float ig = p.cap * tanhf((ni[u] + ib) / p.cap);
      const float fg = log_sigmoid_f(p.cap * tanhf((nf[u] + fb) / p.cap));
      const float mn = fmaxf(fg + m, ig);
      const float a = expf(fg + m - mn), b = expf(ig - mn);
      m = mn;
      __syncthreads();
      if (tid < rows) {
        s_op[tid] = tid < D ? make_float2(nq[u] * p.q_scale, nk[u]) : make_float2(0.f, 0.f);
        s_n[tid] = fmaf(a, s_n[tid], b * (tid < D ? nk[u] : 0.f));
      }
      const float bv = b * nv[u];
      __syncthreads();
      if (t + kScanPF < row_hi) {
        const size_t nb = (size_t)(t + kScanPF) * p.ld;
        if (tid < D) { nq[u] = p.q[nb + hd * D + tid]; nk[u] = p.k[nb + hd * D + tid]; }
        if (j < V) nv[u] = p.v[nb + hd * V + j];
        ni[u] = p.ig[nb + hd]; nf[u] = p.fg[nb + hd];
      }
      float acc = 0.f;
#pragma unroll
      for (int ii = 0; ii < DG; ++ii) {
        const float2 o = s_op[i_lo + ii];
        S[ii] = fmaf(a, S[ii], o.y * bv);
        acc = fmaf(S[ii], o.x, acc);
      }
      if (j == 0) {
        float dot = 0.f;
#pragma unroll
        for (int ii = 0; ii < DG; ++ii) dot = fmaf(s_n[i_lo + ii], s_op[i_lo + ii].x, dot);
        s_dot[g] = dot;
      }
      s_part[g * sh.Vr + j] = acc;
      __syncthreads();
      if (g == 0 && j < V) {
        acc = s_part[j];
        float dot = s_dot[0];
        for (int q = 1; q < sh.G; ++q) { acc += s_part[q * sh.Vr + j]; dot += s_dot[q]; }
        const float den = fmaxf(fabsf(dot), expf(-m)) + 1e-6f;
        p.o[(size_t)t * p.H * V + hd * V + j] = acc / den;
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int ii = 0; ii < DG; ++ii)
    if (j < V && i_lo + ii < D) S_g[(size_t)(i_lo + ii) * V + j] = S[ii];
  if (tid < D) n_g[tid] = s_n[tid];
  if (tid == 0) *m_g = m;
}

}  // namespace ssdk
