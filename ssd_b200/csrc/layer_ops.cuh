// layer_ops.cuh — the element-wise steps of a layered (hybrid) model's block.  The residual stream, every norm
// statistic and every gate are fp32; T (bf16 or float) is the storage type of the activations that feed a linear layer.
//   embed_rows_kernel         x = embed[token]                                  (fp32 residual)
//   unit_offset_rmsnorm_kernel y = x / sqrt(mean(x^2) + eps) * (1 + w)           (unit-offset weight: the scale is 1 + w)
//   token_shift_kernel        RWKV token shift: S mixes h + (h_prev - h) * mu_s, h_prev carried in the state slot
//   head_rmsnorm_gate_kernel  per-head unit RMS, times a channel weight, times silu / sigmoid of a gate pre-activation
//   clamped_glu_kernel        y = g * sigmoid(1.702 g) * (u + 1) with g = min(g, lim), u = clamp(u, -lim, lim)
//   unary_kernel              tanh (decay low-rank bottleneck)
//   block_combine_kernel      parallel block: x += ls1 * mixer + ls2 * (sum_k w_k expert_k + sigmoid(sg) * shared)
#pragma once
#include "common.cuh"
#include "linear.cuh"

namespace ssdk {

// per-step description of a ragged batch, all on the device
struct Ragged {
  const int* cu;        // [n_seqs + 1] first row of every sequence's portion
  const int* pos0;      // [n_seqs] tokens of the sequence that earlier steps already ran
  const int* slot;      // [n_seqs] recurrent-state slot
  const int* tok_seq;   // [M] sequence of a row
  const int* tables;    // [n_seqs, max_blocks] page table
  int n_seqs, M, max_blocks, block_size;
};

template <typename T>
__global__ void embed_rows_kernel(const int* __restrict__ ids, const T* __restrict__ embed, float* __restrict__ x, int width,
                                  int vocab) {
  const int m = blockIdx.x;
  int id = ids[m];
  id = min(max(id, 0), vocab - 1);
  for (int c = threadIdx.x; c < width; c += blockDim.x) x[(size_t)m * width + c] = ld_f<T>(embed + (size_t)id * width + c);
}

// rows: optional gather (row r of the output reads x[rows[r]])
template <typename T>
__global__ void unit_offset_rmsnorm_kernel(const float* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                                           const int* __restrict__ rows, int width, float eps) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) { const float v = xr[c]; ss = fmaf(v, v, ss); }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    st_f<T>(y + (size_t)r * width + c, xr[c] * inv * (1.0f + ld_f<T>(w + c)));
}

// mixes[s][m][c] = h[m][c] + (prev[m][c] - h[m][c]) * mu[s][c]; prev of a portion's first row comes from the slot
// (zero at position 0).  h_prev is NOT written here: the scan kernel of the same layer saves the portion's last row after
// every row of this kernel has read the old one (stream order).
template <typename T>
__global__ void token_shift_kernel(const T* __restrict__ h, const T* __restrict__ mu, const float* __restrict__ h_prev,
                                   size_t slot_stride, T* __restrict__ mixes, Ragged rg, int width, int n_mix) {
  const int m = blockIdx.x, s = rg.tok_seq[m];
  const bool first = m == rg.cu[s];
  const float* prev_state = (first && rg.pos0[s] > 0) ? h_prev + (size_t)rg.slot[s] * slot_stride : nullptr;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float cur = ld_f<T>(h + (size_t)m * width + c);
    const float prev = first ? (prev_state ? prev_state[c] : 0.f) : ld_f<T>(h + (size_t)(m - 1) * width + c);
    const float d = prev - cur;
    for (int k = 0; k < n_mix; ++k)
      st_f<T>(mixes + ((size_t)k * rg.M + m) * width + c, fmaf(d, ld_f<T>(mu + (size_t)k * width + c), cur));
  }
}

SSDK_DEVINL float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// o [M, H, V] fp32 -> y [M, H*V] (T): o / rms(o) * w * act(g);  GATE: 0 = silu, 1 = sigmoid
template <typename T, int GATE>
__global__ void head_rmsnorm_gate_kernel(const float* __restrict__ o, const float* __restrict__ g, int ldg,
                                         const T* __restrict__ w, T* __restrict__ y, int H, int V, float eps) {
  __shared__ float red[33];
  const int m = blockIdx.x, hd = blockIdx.y;
  const float* orow = o + ((size_t)m * H + hd) * V;
  float ss = 0.f;
  for (int j = threadIdx.x; j < V; j += blockDim.x) ss = fmaf(orow[j], orow[j], ss);
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)V + eps);
  for (int j = threadIdx.x; j < V; j += blockDim.x) {
    const float gz = g[(size_t)m * ldg + hd * V + j];
    const float ga = GATE == 0 ? gz * sigmoid_f(gz) : sigmoid_f(gz);
    st_f<T>(y + (size_t)m * H * V + hd * V + j, orow[j] * inv * ld_f<T>(w + hd * V + j) * ga);
  }
}

// z [rows, ldz] fp32 with gate columns [0, ff) and up columns [ff, 2 ff) -> y [rows, ff] (T)
template <typename T>
__global__ void clamped_glu_kernel(const float* __restrict__ z, int ldz, T* __restrict__ y, int ff, float limit,
                                   const int* __restrict__ n_rows) {
  const int r = blockIdx.x;
  if (n_rows && r >= *n_rows) return;
  for (int c = threadIdx.x; c < ff; c += blockDim.x) {
    const float g = fminf(z[(size_t)r * ldz + c], limit);
    const float u = fminf(fmaxf(z[(size_t)r * ldz + ff + c], -limit), limit);
    st_f<T>(y + (size_t)r * ff + c, g * sigmoid_f(1.702f * g) * (u + 1.0f));
  }
}

template <typename T>
__global__ void tanh_rows_kernel(const float* __restrict__ z, T* __restrict__ y, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    st_f<T>(y + i, tanhf(z[i]));
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ z, __nv_bfloat16* __restrict__ y, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    y[i] = __float2bfloat16_rn(z[i]);
}

// out[i] = sum over s of partials[s][i] in the fixed order s = 0 .. S-1 (split-K of the tcgen05 GEMM, fp32)
__global__ void splitk_sum_kernel(const float* __restrict__ partials, float* __restrict__ out, int S, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float a = partials[i];
  for (int s = 1; s < S; ++s) a += partials[(size_t)s * n + i];
  out[i] = a;
}

struct CombineArgs {
  float* x;              // [M, width] residual, updated in place
  const float* mix;      // [M, width] mixer output (after its output projection)
  const void* ls1;       // [width] T
  const void* ls2;       // [width] T or nullptr (no feed-forward)
  const float* routed;   // [M * top, width] expert outputs in assignment order, or nullptr
  const int* apos;       // [M * top] row of (token, k) in `routed`
  const float* wts;      // [M * top] routing weights
  int top;
  const float* shared;   // [M, width] shared expert output or nullptr
  const float* sg;       // shared gate pre-activation: sg[m * ld_sg]
  int ld_sg;
  int width;
};
template <typename T>
__global__ void block_combine_kernel(const CombineArgs p) {
  const int m = blockIdx.x;
  const float sgate = p.shared ? sigmoid_f(p.sg[(size_t)m * p.ld_sg]) : 0.f;
  for (int c = threadIdx.x; c < p.width; c += blockDim.x) {
    float y = ld_f<T>((const T*)p.ls1 + c) * p.mix[(size_t)m * p.width + c];
    if (p.ls2) {
      float f = 0.f;
      if (p.routed)
        for (int k = 0; k < p.top; ++k)
          f = fmaf(p.wts[(size_t)m * p.top + k], p.routed[(size_t)p.apos[(size_t)m * p.top + k] * p.width + c], f);
      if (p.shared) f = fmaf(sgate, p.shared[(size_t)m * p.width + c], f);
      y = fmaf(ld_f<T>((const T*)p.ls2 + c), f, y);
    }
    p.x[(size_t)m * p.width + c] += y;
  }
}

}  // namespace ssdk
