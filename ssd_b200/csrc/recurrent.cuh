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
// never touches shared memory).  Rows are taken in chunks of kScanChunk: the chunk's raw operands arrive by cp.async while
// the previous chunk is computed, all threads turn them into one float4 {r, k, w = exp(-exp(z + w0)), u} per (row, state
// row) at once, and then every thread walks the chunk with nothing but broadcast shared-memory loads and FMAs; the G
// partial read-outs of a column are summed (fixed order g = 0 .. G-1) for the whole chunk afterwards.  Four CTA barriers
// per chunk instead of three per row.  Launched when G * DG >= D with DG in {8, 16, 32} fits a CTA and its shared
// memory; the shared-memory kernel above serves every other size.
constexpr int kScanChunk = 16;

SSDK_DEVINL void cp_async4(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}

inline size_t wkv_scan_reg_smem(int D, const ScanShape& sh, int DG) {
  const size_t C = kScanChunk, rows = (size_t)sh.G * DG;
  return C * rows * 16 + (C * sh.Vr + C * sh.G * sh.Vr + 4 * C * D + 2 * rows) * 4;
}

template <typename T, int DG>
__global__ void __launch_bounds__(512) wkv_scan_reg_kernel(const WkvArgs p, const Ragged rg, const ScanShape sh) {
  SSDK_DYN_SMEM(float4, sm4);
  constexpr int C = kScanChunk;
  const int s = blockIdx.x, hd = blockIdx.y, D = p.D, tid = threadIdx.x, nt = blockDim.x;
  const int Vr = sh.Vr, G = sh.G, j = tid % Vr, g = tid / Vr, i_lo = g * DG, rows = G * DG;
  float4* s_op = sm4;                                          // [C][rows] {r, k, w, u}
  float* s_v = reinterpret_cast<float*>(s_op + C * rows);      // [C][Vr]
  float* s_part = s_v + C * Vr;                                // [C][G][Vr]
  float* raw = s_part + C * G * Vr;                            // r | k | z | v, each [C][D], as the projections left them
  float* s_w0 = raw + 4 * C * D;                               // [rows]
  float* s_u = s_w0 + rows;                                    // [rows]
  const int row_lo = rg.cu[s], row_hi = rg.cu[s + 1];
  if (row_hi <= row_lo) return;
  float* S_g = p.state + (size_t)rg.slot[s] * p.slot_stride + (size_t)hd * D * D;
  const bool fresh = rg.pos0[s] == 0;
  float S[DG];
#pragma unroll
  for (int ii = 0; ii < DG; ++ii) S[ii] = (!fresh && j < D && i_lo + ii < D) ? S_g[(size_t)(i_lo + ii) * D + j] : 0.f;
  for (int i = tid; i < rows; i += nt) {
    s_w0[i] = i < D ? ld_f<T>((const T*)p.w0 + hd * D + i) : 0.f;
    s_u[i] = i < D ? ld_f<T>((const T*)p.u + hd * D + i) : 0.f;
  }
  auto issue = [&](int t0) {
    const int n = min(C, row_hi - t0);
    for (int e = tid; e < n * D; e += nt) {
      const int c = e / D, i = e - c * D;
      const size_t src = (size_t)(t0 + c) * p.ld + hd * D + i;
      cp_async4(raw + e, p.r + src);
      cp_async4(raw + C * D + e, p.k + src);
      cp_async4(raw + 2 * C * D + e, p.zw + src);
      cp_async4(raw + 3 * C * D + e, p.v + src);
    }
    cp_async_commit();
  };
  issue(row_lo);
  for (int t0 = row_lo; t0 < row_hi; t0 += C) {
    const int n = min(C, row_hi - t0);
    cp_async_wait<0>();
    __syncthreads();  // the chunk's operands have landed; the previous chunk's readers of s_op / s_v / s_part are done
    for (int e = tid; e < n * rows; e += nt) {
      const int c = e / rows, i = e - c * rows;
      s_op[e] = i < D ? make_float4(raw[c * D + i], raw[C * D + c * D + i], expf(-expf(raw[2 * C * D + c * D + i] + s_w0[i])), s_u[i])
                      : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int e = tid; e < n * Vr; e += nt) {
      const int c = e / Vr, jj = e - c * Vr;
      s_v[e] = jj < D ? raw[3 * C * D + c * D + jj] : 0.f;
    }
    __syncthreads();
    if (t0 + C < row_hi) issue(t0 + C);
    for (int c = 0; c < n; ++c) {
      const float vj = s_v[c * Vr + j];
      const float4* op = s_op + c * rows + i_lo;
      float acc = 0.f;
#pragma unroll
      for (int ii = 0; ii < DG; ++ii) {
        const float4 o = op[ii];
        const float kv = o.y * vj;
        acc = fmaf(o.x, fmaf(o.w, kv, S[ii]), acc);
        S[ii] = fmaf(o.z, S[ii], kv);
      }
      if (G > 1) s_part[(c * G + g) * Vr + j] = acc;
      else if (j < D) p.o[(size_t)(t0 + c) * p.H * D + hd * D + j] = acc;
    }
    if (G > 1) {
      __syncthreads();
      for (int e = tid; e < n * Vr; e += nt) {
        const int c = e / Vr, jj = e - c * Vr;
        if (jj >= D) continue;
        float acc = s_part[(c * G) * Vr + jj];
        for (int q = 1; q < G; ++q) acc += s_part[(c * G + q) * Vr + jj];
        p.o[(size_t)(t0 + c) * p.H * D + hd * D + jj] = acc;
      }
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

// Register-resident, chunked variant of the mLSTM scan (see wkv_scan_reg_kernel): {q, k} travel as one float2 per (row,
// state row).  The gates of a chunk are evaluated by warp 0 — capped gates in parallel, the stabiliser's max-chain row
// by row with exactly the sequential arithmetic, then the two exponentials in parallel.  The normaliser n lives in the
// registers of each row group's first thread, which updates it beside its state column.
inline size_t mlstm_scan_reg_smem(int D, int V, const ScanShape& sh, int DG) {
  const size_t C = kScanChunk, rows = (size_t)sh.G * DG;
  return C * rows * 8 + (C * sh.Vr + C * sh.G * sh.Vr + C * sh.G + 3 * C + 2 * C * D + C * V + 2 * C) * 4 + 16;
}

template <typename T, int DG>
__global__ void __launch_bounds__(512) mlstm_scan_reg_kernel(const MlstmArgs p, const Ragged rg, const ScanShape sh) {
  SSDK_DYN_SMEM(float2, sm2);
  constexpr int C = kScanChunk;
  const int s = blockIdx.x, hd = blockIdx.y, D = p.D, V = p.V, tid = threadIdx.x, nt = blockDim.x;
  const int Vr = sh.Vr, G = sh.G, j = tid % Vr, g = tid / Vr, i_lo = g * DG, rows = G * DG;
  float2* s_op = sm2;                                      // [C][rows] {q * scale, k}
  float* s_v = reinterpret_cast<float*>(s_op + C * rows);  // [C][Vr]
  float* s_part = s_v + C * Vr;                            // [C][G][Vr]
  float* s_dot = s_part + C * G * Vr;                      // [C][G]
  float* s_a = s_dot + C * G;                              // [C] decay of the row
  float* s_b = s_a + C;                                    // [C] input weight of the row
  float* s_m = s_b + C;                                    // [C] stabiliser after the row
  float* raw_q = s_m + C;                                  // [C][D]
  float* raw_k = raw_q + C * D;                            // [C][D]
  float* raw_v = raw_k + C * D;                            // [C][V]
  float* raw_i = raw_v + C * V;                            // [C]
  float* raw_f = raw_i + C;                                // [C]
  const int row_lo = rg.cu[s], row_hi = rg.cu[s + 1];
  if (row_hi <= row_lo) return;
  const size_t slot = (size_t)rg.slot[s] * p.slot_stride;
  float* S_g = p.S + slot + (size_t)hd * D * V;
  float* n_g = p.n + slot + (size_t)hd * D;
  float* m_g = p.m + slot + hd;
  const bool fresh = rg.pos0[s] == 0;
  float S[DG], nn[DG];
#pragma unroll
  for (int ii = 0; ii < DG; ++ii) {
    S[ii] = (!fresh && j < V && i_lo + ii < D) ? S_g[(size_t)(i_lo + ii) * V + j] : 0.f;
    nn[ii] = (!fresh && j == 0 && i_lo + ii < D) ? n_g[i_lo + ii] : 0.f;
  }
  float m = fresh ? 0.f : *m_g;  // tracked by warp 0
  const float ib = ld_f<T>((const T*)p.ib + hd), fb = ld_f<T>((const T*)p.fb + hd);
  auto issue = [&](int t0) {
    const int n = min(C, row_hi - t0);
    for (int e = tid; e < n * D; e += nt) {
      const int c = e / D, i = e - c * D;
      const size_t src = (size_t)(t0 + c) * p.ld + hd * D + i;
      cp_async4(raw_q + e, p.q + src);
      cp_async4(raw_k + e, p.k + src);
    }
    for (int e = tid; e < n * V; e += nt) {
      const int c = e / V, jj = e - c * V;
      cp_async4(raw_v + e, p.v + (size_t)(t0 + c) * p.ld + hd * V + jj);
    }
    if (tid < n) {
      cp_async4(raw_i + tid, p.ig + (size_t)(t0 + tid) * p.ld + hd);
      cp_async4(raw_f + tid, p.fg + (size_t)(t0 + tid) * p.ld + hd);
    }
    cp_async_commit();
  };
  issue(row_lo);
  for (int t0 = row_lo; t0 < row_hi; t0 += C) {
    const int n = min(C, row_hi - t0);
    cp_async_wait<0>();
    __syncthreads();
    for (int e = tid; e < n * rows; e += nt) {
      const int c = e / rows, i = e - c * rows;
      s_op[e] = i < D ? make_float2(raw_q[c * D + i] * p.q_scale, raw_k[c * D + i]) : make_float2(0.f, 0.f);
    }
    for (int e = tid; e < n * Vr; e += nt) {
      const int c = e / Vr, jj = e - c * Vr;
      s_v[e] = jj < V ? raw_v[c * V + jj] : 0.f;
    }
    if (tid < 32) {
      static_assert(C <= 32, "a chunk's gates are one warp's lanes");
      const int c = tid;
      float ig = 0.f, fg = 0.f;
      if (c < n) {
        ig = p.cap * tanhf((raw_i[c] + ib) / p.cap);
        fg = log_sigmoid_f(p.cap * tanhf((raw_f[c] + fb) / p.cap));
      }
      float m_prev = 0.f, m_new = 0.f;
      for (int cc = 0; cc < n; ++cc) {
        const float ic = __shfl_sync(0xffffffffu, ig, cc), fc = __shfl_sync(0xffffffffu, fg, cc);
        const float mn = fmaxf(fc + m, ic);
        if (c == cc) { m_prev = m; m_new = mn; }
        m = mn;
      }
      if (c < n) {
        s_a[c] = expf(fg + m_prev - m_new);
        s_b[c] = expf(ig - m_new);
        s_m[c] = m_new;
      }
    }
    __syncthreads();
    if (t0 + C < row_hi) issue(t0 + C);
    for (int c = 0; c < n; ++c) {
      const float a = s_a[c], b = s_b[c];
      const float bv = b * s_v[c * Vr + j];
      const float2* op = s_op + c * rows + i_lo;
      float acc = 0.f;
#pragma unroll
      for (int ii = 0; ii < DG; ++ii) {
        const float2 o = op[ii];
        S[ii] = fmaf(a, S[ii], o.y * bv);
        acc = fmaf(S[ii], o.x, acc);
      }
      if (j == 0) {
        float dot = 0.f;
#pragma unroll
        for (int ii = 0; ii < DG; ++ii) {
          const float2 o = op[ii];
          nn[ii] = fmaf(a, nn[ii], b * o.y);
          dot = fmaf(nn[ii], o.x, dot);
        }
        s_dot[c * G + g] = dot;
      }
      s_part[(c * G + g) * Vr + j] = acc;
    }
    __syncthreads();
    for (int e = tid; e < n * Vr; e += nt) {
      const int c = e / Vr, jj = e - c * Vr;
      if (jj >= V) continue;
      float acc = s_part[(c * G) * Vr + jj], dot = s_dot[c * G];
      for (int q = 1; q < G; ++q) { acc += s_part[(c * G + q) * Vr + jj]; dot += s_dot[c * G + q]; }
      const float den = fmaxf(fabsf(dot), expf(-s_m[c])) + 1e-6f;
      p.o[(size_t)(t0 + c) * p.H * V + hd * V + jj] = acc / den;
    }
  }
#pragma unroll
  for (int ii = 0; ii < DG; ++ii) {
    if (j < V && i_lo + ii < D) S_g[(size_t)(i_lo + ii) * V + j] = S[ii];
    if (j == 0 && i_lo + ii < D) n_g[i_lo + ii] = nn[ii];
  }
  if (tid == 0) *m_g = m;
}

}  // namespace ssdk
