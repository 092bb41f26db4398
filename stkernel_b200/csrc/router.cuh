// Top-k expert selection for one token by one warp, shared by the stand-alone router kernel (moe.cu) and by the
// gate projection's epilogue (skinny.cu: the CTA that finishes the projection last routes the tokens, so a decode
// step needs no router launch).
//
// scores = sigmoid | sqrt(softplus) of the fp32 gate logits; selection by score + bias (or by a token-id hash table
// with bounds checks); weights from the unbiased score, renormalised and scaled (topkGatingSoftplusSqrt /
// fused_topk_bias and the hash-MoE lookup of overlay/nvidia_model.py:806-827).
#pragma once
#include "common.cuh"

namespace stk {

struct RouterArgs {
  const float* bias;          // [E] or nullptr
  const int* tid2eid;         // [vocab, topk] or nullptr
  const int64_t* token_ids;   // [T] (hash routing)
  int vocab;
  int* ids;                   // [T, topk]
  float* weights;             // [T, topk]
  int E, topk, scoring, renorm;
  float scaling;
  int* status;
};

// float -> unsigned key with the same order (so that the warp-wide integer max instruction finds the float max)
__device__ __forceinline__ uint32_t ordered_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// `row` = the token's E logits.  kCg: read them around L1 (they were written by other CTAs of the same kernel).
// kPer = experts per lane (E <= 32 * kPer).
template <bool kCg, int kPer>
__device__ __forceinline__ void route_token_impl(const RouterArgs& r, const float* __restrict__ row, int t, int lane) {
  float sc[kPer], sel[kPer];
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int e = i * 32 + lane;
    if (e < r.E) {
      const float x = kCg ? __ldcg(row + e) : row[e];
      float s;
      if (r.scoring == 0) s = 1.f / (1.f + __expf(-x));
      else s = sqrtf(x > 20.f ? x : log1pf(__expf(x)));
      sc[i] = s;
      sel[i] = s + (r.bias ? r.bias[e] : 0.f);
    } else {
      sc[i] = 0.f;
      sel[i] = -INFINITY;
    }
  }
  float wsum = 0.f;
  float my_w = 0.f;      // lane j keeps the j-th selected weight
  int my_id = -1;
  if (r.tid2eid != nullptr) {
    const long long tok = r.token_ids[t];
    const bool ok = tok >= 0 && tok < r.vocab;
    if (!ok && lane == 0) set_status(r.status, kBadIndex, t);
    for (int j = 0; j < r.topk; ++j) {
      int e = ok ? r.tid2eid[tok * r.topk + j] : 0;
      if (e < 0 || e >= r.E) {
        if (lane == 0) set_status(r.status, kBadIndex, t);
        e = 0;
      }
      // static indexing only (a dynamic index would push sc[] and sel[] to local memory)
      float pick = 0.f;
#pragma unroll
      for (int i = 0; i < kPer; ++i) pick = (i == (e >> 5)) ? sc[i] : pick;
      const float s = __shfl_sync(0xffffffffu, pick, e & 31);
      wsum += s;
      if (lane == j) { my_w = s; my_id = e; }
    }
  } else {
    for (int j = 0; j < r.topk; ++j) {
      // lane-local best as a tree over the kPer candidates (a serial scan is kPer dependent compare/selects;
      // one warp runs this code alone, so its time is the depth of the dependency chain, not the instruction count)
      float bv[kPer];
      int be[kPer];
#pragma unroll
      for (int i = 0; i < kPer; ++i) { bv[i] = sel[i]; be[i] = i * 32 + lane; }
#pragma unroll
      for (int w = kPer / 2; w > 0; w >>= 1) {
#pragma unroll
        for (int i = 0; i < w; ++i) {
          const bool take = bv[i + w] > bv[i];          // equal values keep the lower expert id (i < i + w)
          bv[i] = take ? bv[i + w] : bv[i];
          be[i] = take ? be[i + w] : be[i];
        }
      }
      const float best = bv[0];
      int best_e = best == -INFINITY ? 0x7fffffff : be[0];
      // warp-wide arg-max in two hardware reductions: the largest key, then the lowest expert id among its holders
      const uint32_t key = ordered_key(best);
      const uint32_t kmax = __reduce_max_sync(0xffffffffu, key);
      best_e = __reduce_min_sync(0xffffffffu, key == kmax ? best_e : 0x7fffffff);
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < kPer; ++i) {
        if (i * 32 + lane == best_e) { s = sc[i]; sel[i] = -INFINITY; }
      }
      s = __shfl_sync(0xffffffffu, s, best_e & 31);
      wsum += s;
      if (lane == j) { my_w = s; my_id = best_e; }
    }
  }
  if (lane < r.topk) {
    float w = my_w;
    if (r.renorm) w = w / fmaxf(wsum, 1e-20f);
    r.ids[t * r.topk + lane] = my_id;
    r.weights[t * r.topk + lane] = w * r.scaling;
  }
}

template <bool kCg = false>
__device__ __forceinline__ void route_token(const RouterArgs& r, const float* __restrict__ row, int t, int lane) {
  if (r.E <= 256) route_token_impl<kCg, 8>(r, row, t, lane);
  else route_token_impl<kCg, 16>(r, row, t, lane);
}

}  // namespace stk
