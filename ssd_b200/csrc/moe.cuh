// moe.cuh — routing of a sigmoid-scored, group-limited mixture of experts.
//
//   group_topk_router_kernel  one warp per token.  scores = sigmoid(router logits) (fp32).  The experts form `groups`
//       equal, contiguous groups; a group scores the sum of its two best experts (one, if a group has one expert);
//       only experts of the `keep` best groups compete; the `top` best of those are chosen; their scores, divided by
//       their sum (+ 1e-20) and multiplied by `route_scale`, are the combination weights.  Ties go to the lower index.
//   expert_plan_kernel        one CTA: counting sort of the (token, k) assignments by expert -> for every assignment
//       its row in expert order (apos) and the token each sorted row reads (arow), plus the list of row tiles
//       (expert, first row, rows) that the grouped linear kernel walks.  The order of rows inside one expert is
//       arbitrary; every row is computed independently, so results do not depend on it.
// The expert matrices themselves run through linear_kernel in grouped mode (linear.cuh) and clamped_glu_kernel.
#pragma once
#include "layer_ops.cuh"

namespace ssdk {

struct RouterArgs {
  const float* z;   // [M, E] router logits
  int* sel;         // [M, top]
  float* wts;       // [M, top]
  int M, E, top, groups, keep;
  float route_scale;
};
constexpr int kRouterMaxE = 512;
constexpr int kRouterWarps = 4;

__global__ void __launch_bounds__(kRouterWarps * 32) group_topk_router_kernel(const RouterArgs p) {
  __shared__ float s_score[kRouterWarps][kRouterMaxE];   // < 0 once taken or shut out
  __shared__ float s_group[kRouterWarps][kRouterMaxE];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x * kRouterWarps + warp;
  if (m >= p.M) return;
  float* sc = s_score[warp];
  float* gs = s_group[warp];
  const int E = p.E, G = p.groups, per = E / G;
  for (int e = lane; e < E; e += 32) sc[e] = sigmoid_f(p.z[(size_t)m * E + e]);
  __syncwarp();
  for (int g = lane; g < G; g += 32) {
    float b1 = -1.f, b2 = -1.f;
    for (int e = g * per; e < (g + 1) * per; ++e) {
      const float v = sc[e];
      if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) { b2 = v; }
    }
    gs[g] = b1 + (b2 >= 0.f ? b2 : 0.f);
  }
  __syncwarp();
  // keep the `keep` best groups: mark them with -1 after picking, then shut out the experts of all unmarked groups
  for (int r = 0; r < p.keep; ++r) {
    ArgMax a{-2.f, 0x7fffffff};
    for (int g = lane; g < G; g += 32) a = argmax_better(a, ArgMax{gs[g], g});
    a = warp_argmax(a);
    __syncwarp();
    if (lane == 0) gs[a.i] = -1.f;
    __syncwarp();
  }
  for (int e = lane; e < E; e += 32)
    if (gs[e / per] != -1.f) sc[e] = -1.f;
  __syncwarp();
  float mine = 0.f, total = 0.f;   // lane r keeps the r-th chosen score (top <= 32)
  int mine_i = 0;
  for (int r = 0; r < p.top; ++r) {
    ArgMax a{-2.f, 0x7fffffff};
    for (int e = lane; e < E; e += 32) a = argmax_better(a, ArgMax{sc[e], e});
    a = warp_argmax(a);
    __syncwarp();
    if (lane == 0) sc[a.i] = -1.f;
    __syncwarp();
    if (lane == r) { mine = a.v; mine_i = a.i; }
    total += a.v;
  }
  if (lane < p.top) {
    p.sel[(size_t)m * p.top + lane] = mine_i;
    p.wts[(size_t)m * p.top + lane] = mine / (total + 1e-20f) * p.route_scale;
  }
}

struct PlanArgs {
  const int* sel;    // [A] expert of assignment a = token * top + k
  int* apos;         // [A] row of assignment a in expert order
  int* arow;         // [A] token of sorted row
  int* tile_expert; int* tile_row0; int* tile_rows; int* n_tiles;
  int* n_rows;       // = A (device copy for kernels that bound their grid by it)
  int A, E, top, tile;
};

__global__ void __launch_bounds__(1024) expert_plan_kernel(const PlanArgs p) {
  __shared__ int s_cnt[kRouterMaxE];
  __shared__ int s_off[kRouterMaxE + 1];
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) s_cnt[e] = 0;
  __syncthreads();
  for (int a = threadIdx.x; a < p.A; a += blockDim.x) atomicAdd(&s_cnt[p.sel[a]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0, nt = 0;
    for (int e = 0; e < p.E; ++e) {
      s_off[e] = off;
      for (int r0 = 0; r0 < s_cnt[e]; r0 += p.tile) {
        p.tile_expert[nt] = e;
        p.tile_row0[nt] = off + r0;
        p.tile_rows[nt] = min(p.tile, s_cnt[e] - r0);
        ++nt;
      }
      off += s_cnt[e];
    }
    s_off[p.E] = off;
    *p.n_tiles = nt;
    *p.n_rows = p.A;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) s_cnt[e] = 0;
  __syncthreads();
  for (int a = threadIdx.x; a < p.A; a += blockDim.x) {
    const int e = p.sel[a];
    const int row = s_off[e] + atomicAdd(&s_cnt[e], 1);
    p.apos[a] = row;
    p.arow[row] = a / p.top;
  }
}

}  // namespace ssdk
