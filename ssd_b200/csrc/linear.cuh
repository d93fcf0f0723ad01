// linear.cuh — shape-generic linear layers for the layered (hybrid) models: C[M,N] = A[M,K] · W[N,K]^T with fp32
// accumulation for ANY M, N, K (head sizes such as 40 or 48 have no 64-column TMA box), in two storage types:
//   T = bf16 : operands bf16, products exact in fp32, fp32 accumulate (the rounding contract of a tensor-core GEMM);
//              tile products on mma.sync.m16n8k16 when rows are 16-byte aligned (K, strides multiples of 8),
//              CUDA-core FMA otherwise
//   T = float: true fp32 FMA (no TF32), used by the exact mode
// Three addressing modes share one kernel: dense, batched (blockIdx.z walks per-head slices by strides) and grouped
// (a tile list made on the device by the router maps tile -> expert / first row / row count; the rows of A may be
// gathered through an index).  The accumulation order of an output element depends on K alone, never on M or on which
// other rows share the tile, so a token's result is independent of the batch it ran in.
// Dense bf16 products with K a multiple of 64 take the tcgen05 path of gemm.cuh instead (HybRun::lin in
// hybrid_engine.cuh); this file serves the shapes a 64-column TMA box cannot: odd sizes, per-head slices, gathered rows.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "attention.cuh"
#include "common.cuh"

namespace ssdk {

template <typename T> SSDK_DEVINL float ld_f(const T* p);
template <> SSDK_DEVINL float ld_f<float>(const float* p) { return *p; }
template <> SSDK_DEVINL float ld_f<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> SSDK_DEVINL void st_f(T* p, float v);
template <> SSDK_DEVINL void st_f<float>(float* p, float v) { *p = v; }
template <> SSDK_DEVINL void st_f<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

struct LinearArgs {
  const void* A;   // [*, lda]  storage type T
  const void* W;   // [N, ldw]  storage type T
  void* C;         // [*, ldc]  fp32 or T
  int M, N, K;
  int lda, ldw, ldc;
  long long sA, sW, sC;    // element strides per blockIdx.z (batched mode)
  const int* a_rows;       // optional gather: logical row r of A lives at row a_rows[r]
  // grouped mode (tile_expert != nullptr): blockIdx.y indexes the tile list
  const int* tile_expert;
  const int* tile_row0;
  const int* tile_rows;
  const int* n_tiles;
  long long sW_expert;     // elements between two experts' matrices
};

constexpr int kLinBM = 64, kLinBN = 64, kLinBK = 16, kLinThreads = 256;

// CUDA-core tile: 64 x 64 outputs per CTA, 4 x 4 per thread, operands staged as fp32 in shared memory.
template <typename T, typename OutT>
__global__ void __launch_bounds__(kLinThreads) linear_kernel(const LinearArgs p) {
  __shared__ float As[kLinBK][kLinBM + 4];
  __shared__ float Ws[kLinBK][kLinBN + 4];
  int row0, nrows;
  const T* W = (const T*)p.W + (long long)blockIdx.z * p.sW;
  const T* A = (const T*)p.A + (long long)blockIdx.z * p.sA;
  OutT* C = (OutT*)p.C + (long long)blockIdx.z * p.sC;
  if (p.tile_expert) {
    if ((int)blockIdx.y >= *p.n_tiles) return;
    W += (long long)p.tile_expert[blockIdx.y] * p.sW_expert;
    row0 = p.tile_row0[blockIdx.y];
    nrows = p.tile_rows[blockIdx.y];
  } else {
    row0 = blockIdx.y * kLinBM;
    nrows = min(kLinBM, p.M - row0);
    if (nrows <= 0) return;
  }
  const int col0 = blockIdx.x * kLinBN;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  // each thread stages 4 elements of A and 4 of W per k-step: element e -> (row e / 16, k e % 16)
  long long a_off[4], w_off[4];
  bool a_ok[4], w_ok[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int e = tid + i * kLinThreads, r = e >> 4;
    a_ok[i] = r < nrows;
    int ar = row0 + r;
    if (a_ok[i] && p.a_rows) ar = p.a_rows[ar];
    a_off[i] = (long long)ar * p.lda;
    w_ok[i] = col0 + r < p.N;
    w_off[i] = (long long)(col0 + r) * p.ldw;
  }
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < p.K; k0 += kLinBK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * kLinThreads, r = e >> 4, kk = e & 15;
      const bool kin = k0 + kk < p.K;
      As[kk][r] = (a_ok[i] && kin) ? ld_f<T>(A + a_off[i] + k0 + kk) : 0.f;
      Ws[kk][r] = (w_ok[i] && kin) ? ld_f<T>(W + w_off[i] + k0 + kk) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kLinBK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (r >= nrows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx * 4 + j;
      if (c < p.N) st_f<OutT>(C + (long long)(row0 + r) * p.ldc + c, acc[i][j]);
    }
  }
}

// Tensor-core tile for bf16 (legacy mma.sync path; operands need 16-byte aligned rows: K, lda, ldw and the batch strides
// multiples of 8).  64 x 64 outputs per CTA, four warps of 32 x 32, k-steps of 32 through a three-stage cp.async ring of
// padded shared-memory tiles (row stride 80 B: ldmatrix rows fall into distinct 16-byte bank groups): two k-steps of
// global loads are in flight under the one being multiplied, which is what a few-row (decode) call needs to stream
// weights and what a prefill call needs to hide latency.  One __syncthreads per k-step.
constexpr int kMmaThreads = 128, kMmaBK = 32, kMmaLd = kMmaBK + 8, kMmaStages = 3;

template <typename OutT>
__global__ void __launch_bounds__(kMmaThreads) linear_mma_kernel(const LinearArgs p) {
  typedef __nv_bfloat16 T;
  __shared__ __align__(16) T As[kMmaStages][kLinBM][kMmaLd];
  __shared__ __align__(16) T Ws[kMmaStages][kLinBN][kMmaLd];
  int row0, nrows;
  const T* W = (const T*)p.W + (long long)blockIdx.z * p.sW;
  const T* A = (const T*)p.A + (long long)blockIdx.z * p.sA;
  OutT* C = (OutT*)p.C + (long long)blockIdx.z * p.sC;
  if (p.tile_expert) {
    if ((int)blockIdx.y >= *p.n_tiles) return;
    W += (long long)p.tile_expert[blockIdx.y] * p.sW_expert;
    row0 = p.tile_row0[blockIdx.y];
    nrows = p.tile_rows[blockIdx.y];
  } else {
    row0 = blockIdx.y * kLinBM;
    nrows = min(kLinBM, p.M - row0);
    if (nrows <= 0) return;
  }
  const int col0 = blockIdx.x * kLinBN;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, wm = warp >> 1, wn = warp & 1;
  // staging: vector v = tid + i * 128 -> row v / 4, k offset (v % 4) * 8; a row outside the tile is zero-filled
  const T* a_src[2];
  const T* w_src[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int v = tid + i * kMmaThreads, r = v >> 2, kv = (v & 3) * 8;
    int ar = row0 + r;
    const bool aok = r < nrows;
    if (aok && p.a_rows) ar = p.a_rows[ar];
    a_src[i] = aok ? A + (long long)ar * p.lda + kv : nullptr;
    w_src[i] = (col0 + r < p.N) ? W + (long long)(col0 + r) * p.ldw + kv : nullptr;
  }
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[i][j][k] = 0.f;
  const int nk = (p.K + kMmaBK - 1) / kMmaBK;
  auto issue = [&](int kt) {
    if (kt < nk) {
      const int k0 = kt * kMmaBK, st = kt % kMmaStages;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int v = tid + i * kMmaThreads, r = v >> 2, kv = (v & 3) * 8;
        const bool kin = k0 + kv < p.K;
        const bool av = a_src[i] && kin, wv = w_src[i] && kin;
        cp_async16(&As[st][r][kv], av ? (const void*)(a_src[i] + k0) : (const void*)A, av);
        cp_async16(&Ws[st][r][kv], wv ? (const void*)(w_src[i] + k0) : (const void*)W, wv);
      }
    }
    cp_async_commit();
  };
  issue(0);
  issue(1);
  for (int kt = 0; kt < nk; ++kt) {
    cp_async_wait<1>();
    __syncthreads();
    issue(kt + 2);
    const int st = kt % kMmaStages;
#pragma unroll
    for (int kk = 0; kk < kMmaBK; kk += 16) {
      uint32_t a[2][4], b[2][4];
#pragma unroll
      for (int mi = 0; mi < 2; ++mi) ldmatrix_x4(a[mi], &As[st][wm * 32 + mi * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
      for (int nj = 0; nj < 2; ++nj)
        ldmatrix_x4(b[nj], &Ws[st][wn * 32 + nj * 16 + (lane >> 4) * 8 + (lane & 7)][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
      for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int ni = 0; ni < 4; ++ni) mma_bf16_16816(acc[mi][ni], a[mi], b[ni >> 1][(ni & 1) * 2], b[ni >> 1][(ni & 1) * 2 + 1]);
    }
  }
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wm * 32 + mi * 16 + g + half * 8;
      if (r >= nrows) continue;
#pragma unroll
      for (int ni = 0; ni < 4; ++ni) {
        const int c = col0 + wn * 32 + ni * 8 + 2 * t;
        OutT* dst = C + (long long)(row0 + r) * p.ldc + c;
        if (c < p.N) st_f<OutT>(dst, acc[mi][ni][half * 2]);
        if (c + 1 < p.N) st_f<OutT>(dst + 1, acc[mi][ni][half * 2 + 1]);
      }
    }
}

}  // namespace ssdk
