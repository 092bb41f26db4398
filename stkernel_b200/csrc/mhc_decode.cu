// Hyper-connection pre-mix for decode-sized batches (hc = 4, H <= 4096), with the previous sub-block's post-mix and
// the tensor-parallel all-reduce of that sub-block's output folded in.
//
// One 8-CTA cluster per token.  Every CTA owns H/8 columns of all four residual streams, so a value is loaded once and
// serves the mix projection (24 dot products against fn), the stream sum and the RMSNorm:
//
//   X'[j]  = post_old[j] * fa + sum_k comb_old[j, k] * res_old[k]            (bf16; written out as the new streams)
//   mix[m] = sum_{j,h} X'[j][h] * fn[m][j*H + h],   G[j][k] = sum_h X'[j][h] * X'[k][h]
//   pre, post, comb (Sinkhorn) from mix and rms = rsqrt(tr(G) / 4H + eps)     (overlay/mhc_tilelang.py:206-325)
//   y = rmsnorm(sum_j pre[j] * X'[j]) * w,  with  sum_h y0[h]^2 = pre^T G pre  -- so the norm needs no second
//   reduction over the cluster.
//
// The dependency chain is: one round of global loads (everything a thread needs is requested up front), one
// reduction, one exchange through distributed shared memory (each CTA writes its 40 partial sums into every peer's
// shared memory and waits on the cluster barrier once), Sinkhorn in one warp beside the output of y.
//
// `fa` comes either from memory or, under tensor parallelism, from the ranks' receive slots of the folded
// all-reduce (symm.cuh): this kernel then *is* the reduction -- it polls the words it needs (bounded), adds the ranks
// in a fixed order and rounds to bf16 as the stand-alone all-reduce kernel would.
//
// Takes the place of the reference's fused post+pre path for M <= 16 (overlay/mhc_tilelang.py:672-850) and of the
// all-reduce in front of it (overlay/cuda_communicator.py:255-268).
#define STK_PDL_CLASS 4
#include <cooperative_groups.h>

#include "common.cuh"
#include "symm.cuh"

namespace stk {
namespace cg = cooperative_groups;

constexpr int kDcCluster = 8;
constexpr int kDcThreads = 512;
constexpr int kDcWarps = kDcThreads / 32;
constexpr int kDcMix = 24;
constexpr int kDcVals = kDcMix + 16;      // mix partials + the 4x4 Gram matrix of the streams

struct MhcDecodeArgs {
  const __nv_bfloat16* x;         // [T, 4, H] streams as given (direct mode), else nullptr
  const __nv_bfloat16* fa;        // [T, H] output of the previous sub-block (fused mode, already reduced), or nullptr
  const __nv_bfloat16* res_old;   // [T, 4, H]
  const float* post_old;          // [T, 4]
  const float* comb_old;          // [T, 16]
  __nv_bfloat16* x_out;           // [T, 4, H] new streams (fused mode)
  const float* fn;                // [24, 4H]
  const float* base;              // [24]
  const float* scale;             // [3]
  const __nv_bfloat16* norm_w;    // [H] or nullptr
  float* post;                    // [T, 4]
  float* comb;                    // [T, 16]
  __nv_bfloat16* y;               // [T, H]
  int H;
  float rms_eps, hc_eps;
  int sinkhorn_iters;
  float post_mult;
  int use_ll;                     // fused mode: fa is the sum of the ranks' slots of `ll`
  LLAr ll;
  int stage_fn;                   // copy this thread's mix weights into (dynamic) shared memory ahead of the wait
  int* status;
};

__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

__global__ void __launch_bounds__(kDcThreads)
mhc_decode_kernel(const MhcDecodeArgs a) {
  cg::cluster_group cluster = cg::this_cluster();
  const int crank = static_cast<int>(cluster.block_rank());
  const int t = blockIdx.x / kDcCluster;
  const int H = a.H, HC = 4 * a.H;
  const int cols = H / kDcCluster;                    // multiple of 4, at most 512
  const int j = threadIdx.x >> 7;                     // the stream whose dot products this thread accumulates
  const int cgi = threadIdx.x & 127;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool active = cgi * 4 < cols;
  const int h = crank * cols + cgi * 4;
  __shared__ float red[kDcWarps][kDcMix + 4];
  __shared__ float recv[kDcCluster][kDcVals];         // row r is written by cluster rank r
  __shared__ float tot[kDcVals];
  __shared__ float s_pre[4];
  __shared__ float s_r;
  __shared__ __align__(16) float s_fa[4][512];                      // per-thread-group partial sums of the ranks' slots

  extern __shared__ __align__(16) float4 s_fn[];                    // [24][512] when stage_fn, else empty

  cluster_arrive();                                   // phase 0: "this CTA runs" (its shared memory may be written)
  // Ahead of the previous kernel's completion: this thread's 24 x 16 bytes of the (immutable) mix weights.  Few tokens:
  // asynchronous copies into shared memory, so that the dot products below start without a memory round trip (196 KB
  // per CTA, one CTA per SM).  Many tokens: a prefetch towards L2 only, which keeps several CTAs resident per SM.
  if (a.stage_fn) {
    if (active) {
      const float* fbase = a.fn + static_cast<long long>(j) * H + h;
#pragma unroll
      for (int m = 0; m < kDcMix; ++m) {
        const uint32_t dst = smem_u32(&s_fn[m * kDcThreads + threadIdx.x]);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(fbase + static_cast<long long>(m) * HC) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  } else if (cols * 4 >= 128) {
    const int lines = cols * 4 / 128;
    for (int idx = threadIdx.x; idx < kDcMix * 4 * lines; idx += kDcThreads) {
      const int row = idx / lines, ln = idx % lines;          // row = m * 4 + stream
      prefetch_l2(a.fn + static_cast<long long>(row >> 2) * HC + (row & 3) * H + crank * cols + ln * 32);
    }
  }
  pdl_wait();
  pdl_trigger();

  const bool fused = a.x == nullptr;
  float xs[4][4];                                     // X'[stream][column], already rounded to bf16
#pragma unroll
  for (int s = 0; s < 4; ++s)
#pragma unroll
    for (int c = 0; c < 4; ++c) xs[s][c] = 0.f;
  uint2 nw = make_uint2(0, 0);
  uint32_t epoch = 0;
  if (fused && a.use_ll) epoch = ll_read_epoch(a.ll);
  if (active) {
    if (a.norm_w != nullptr && j == 0) nw = __ldg(reinterpret_cast<const uint2*>(a.norm_w + h));
    if (!fused) {
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const uint2 v = *reinterpret_cast<const uint2*>(a.x + (static_cast<long long>(t) * 4 + s) * H + h);
        const float2 p = unpack_bf16x2(v.x), q = unpack_bf16x2(v.y);
        xs[s][0] = p.x; xs[s][1] = p.y; xs[s][2] = q.x; xs[s][3] = q.y;
      }
    }
  }
  if (fused) {
    float ro[4][4];
    float po[4], co[16];
    uint2 rv[4];
    if (active) {
#pragma unroll
      for (int s = 0; s < 4; ++s) rv[s] = *reinterpret_cast<const uint2*>(a.res_old + (static_cast<long long>(t) * 4 + s) * H + h);
      const float4 p4 = *reinterpret_cast<const float4*>(a.post_old + t * 4);
      po[0] = p4.x; po[1] = p4.y; po[2] = p4.z; po[3] = p4.w;
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const float4 c4 = *reinterpret_cast<const float4*>(a.comb_old + t * 16 + s * 4);
        co[s * 4] = c4.x; co[s * 4 + 1] = c4.y; co[s * 4 + 2] = c4.z; co[s * 4 + 3] = c4.w;
      }
    }
    float fa4[4] = {0.f, 0.f, 0.f, 0.f};
    if (a.use_ll) {
      // this thread group adds the slots of ranks j and j + 4; the four groups' sums meet in shared memory
      float part[4] = {0.f, 0.f, 0.f, 0.f};
      if (active) {
        const long long w0 = (static_cast<long long>(t) * H + h) >> 1;
        for (int r = j; r < a.ll.world; r += 4) {
          uint32_t d0, d1;
          ll_wait_word(a.ll, epoch, r, w0, d0, a.status);
          ll_wait_word(a.ll, epoch, r, w0 + 1, d1, a.status);
          const float2 p = unpack_bf16x2(d0), q = unpack_bf16x2(d1);
          part[0] += p.x; part[1] += p.y; part[2] += q.x; part[3] += q.y;
        }
        *reinterpret_cast<float4*>(&s_fa[j][cgi * 4]) = make_float4(part[0], part[1], part[2], part[3]);
      }
      __syncthreads();
      if (active) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float v = (s_fa[0][cgi * 4 + c] + s_fa[1][cgi * 4 + c]) + (s_fa[2][cgi * 4 + c] + s_fa[3][cgi * 4 + c]);
          fa4[c] = bf16_to_f(__float2bfloat16(v));
        }
      }
    } else if (active) {
      const uint2 v = *reinterpret_cast<const uint2*>(a.fa + static_cast<long long>(t) * H + h);
      const float2 p = unpack_bf16x2(v.x), q = unpack_bf16x2(v.y);
      fa4[0] = p.x; fa4[1] = p.y; fa4[2] = q.x; fa4[3] = q.y;
    }
    if (active) {
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const float2 p = unpack_bf16x2(rv[s].x), q = unpack_bf16x2(rv[s].y);
        ro[s][0] = p.x; ro[s][1] = p.y; ro[s][2] = q.x; ro[s][3] = q.y;
      }
#pragma unroll
      for (int s = 0; s < 4; ++s) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float v = po[s] * fa4[c];
#pragma unroll
          for (int k = 0; k < 4; ++k) v = fmaf(co[s * 4 + k], ro[k][c], v);
          xs[s][c] = bf16_to_f(__float2bfloat16(v));
        }
      }
      // this thread's own stream goes out as the new residual
      float own[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) own[c] = j == 0 ? xs[0][c] : j == 1 ? xs[1][c] : j == 2 ? xs[2][c] : xs[3][c];
      const uint2 o = make_uint2(pack_bf16x2(own[0], own[1]), pack_bf16x2(own[2], own[3]));
      *reinterpret_cast<uint2*>(a.x_out + (static_cast<long long>(t) * 4 + j) * H + h) = o;
    }
  }

  // ---- partial dot products of this thread's stream, and its row of the Gram matrix ----
  float acc[kDcMix];
  float g[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int m = 0; m < kDcMix; ++m) acc[m] = 0.f;
  if (active) {
    float mine[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) mine[c] = j == 0 ? xs[0][c] : j == 1 ? xs[1][c] : j == 2 ? xs[2][c] : xs[3][c];
    const float* fbase = a.fn + static_cast<long long>(j) * H + h;
    if (a.stage_fn) {
      asm volatile("cp.async.wait_group 0;" ::: "memory");      // this thread reads only what it copied itself
#pragma unroll
      for (int m = 0; m < kDcMix; ++m) {
        const float4 f = s_fn[m * kDcThreads + threadIdx.x];
        acc[m] = fmaf(mine[0], f.x, fmaf(mine[1], f.y, fmaf(mine[2], f.z, mine[3] * f.w)));
      }
    } else {
#pragma unroll
      for (int m = 0; m < kDcMix; ++m) {
        const float4 f = __ldg(reinterpret_cast<const float4*>(fbase + static_cast<long long>(m) * HC));
        acc[m] = fmaf(mine[0], f.x, fmaf(mine[1], f.y, fmaf(mine[2], f.z, mine[3] * f.w)));
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k)
      g[k] = fmaf(mine[0], xs[k][0], fmaf(mine[1], xs[k][1], fmaf(mine[2], xs[k][2], mine[3] * xs[k][3])));
  }
#pragma unroll
  for (int m = 0; m < kDcMix; ++m) {
    const float v = warp_sum(acc[m]);
    if (lane == 0) red[warp][m] = v;
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float v = warp_sum(g[k]);
    if (lane == 0) red[warp][kDcMix + k] = v;
  }
  __syncthreads();
  cluster_wait();                                     // phase 0 complete: every CTA of the cluster is running
  if (threadIdx.x < kDcVals) {
    const int i = threadIdx.x;
    float s = 0.f;
    if (i < kDcMix) {
      for (int w = 0; w < kDcWarps; ++w) s += red[w][i];
    } else {
      const int jj = (i - kDcMix) >> 2, k = (i - kDcMix) & 3;     // the four warps of stream jj hold row jj
      for (int w = 0; w < 4; ++w) s += red[jj * 4 + w][kDcMix + k];
    }
    for (int r = 0; r < kDcCluster; ++r) cluster.map_shared_rank(&recv[crank][i], r)[0] = s;
  }
  cluster_arrive();                                   // phase 1: the partial sums are in every peer's shared memory
  cluster_wait();
  if (threadIdx.x < kDcVals) {
    float s = 0.f;
    for (int r = 0; r < kDcCluster; ++r) s += recv[r][threadIdx.x];
    tot[threadIdx.x] = s;
  }
  __syncthreads();
  const float* G = tot + kDcMix;
  const float rms = rsqrtf((G[0] + G[5] + G[10] + G[15]) / static_cast<float>(HC) + a.rms_eps);
  if (warp == 0) {
    float p = 0.f;
    if (lane < 4) {
      p = 1.f / (1.f + __expf(-(tot[lane] * rms * a.scale[0] + a.base[lane]))) + a.hc_eps;
      s_pre[lane] = p;
    }
    // sum_h y0[h]^2 = pre^T G pre
    float q = 0.f;
    if (lane < 16) q = __shfl_sync(0xffffu, p, lane >> 2) * __shfl_sync(0xffffu, p, lane & 3) * G[lane];
    q = warp_sum(q);
    if (lane == 0) s_r = a.norm_w != nullptr ? rsqrtf(fmaxf(q, 0.f) / static_cast<float>(H) + a.rms_eps) : 1.f;
  } else if (warp == kDcWarps - 1 && crank == 0) {
    // the last warp: nothing below waits for it
    constexpr int hc = 4;
    if (lane < hc)
      a.post[t * hc + lane] = a.post_mult / (1.f + __expf(-(tot[hc + lane] * rms * a.scale[1] + a.base[hc + lane])));
    const int rj = lane / hc, rk = lane % hc;
    const bool act = lane < hc * hc;
    float c = act ? tot[2 * hc + lane] * rms * a.scale[2] + a.base[2 * hc + lane] : -INFINITY;
    int row_src[4], col_src[4];
#pragma unroll
    for (int o = 1; o < 4; ++o) {
      row_src[o] = (rj * hc + ((rk + o) % hc)) & 31;
      col_src[o] = (((rj + o) % hc) * hc + rk) & 31;
    }
    float rmax = c;
#pragma unroll
    for (int o = 1; o < 4; ++o) {
      const float other = __shfl_sync(0xffffffffu, c, row_src[o]);
      if (act) rmax = fmaxf(rmax, other);
    }
    const float e = act ? __expf(c - rmax) : 0.f;
    float rs = e;
#pragma unroll
    for (int o = 1; o < 4; ++o) rs += __shfl_sync(0xffffffffu, e, row_src[o]);
    c = act ? e / rs + a.hc_eps : 0.f;
    for (int it = 0; it < 2 * a.sinkhorn_iters - 1; ++it) {
      const bool col = (it & 1) == 0;                 // even steps normalise columns, odd steps rows
      const float a1 = __shfl_sync(0xffffffffu, c, col ? col_src[1] : row_src[1]);
      const float a2 = __shfl_sync(0xffffffffu, c, col ? col_src[2] : row_src[2]);
      const float a3 = __shfl_sync(0xffffffffu, c, col ? col_src[3] : row_src[3]);
      const float s = (c + a1) + (a2 + a3);
      if (act) c = __fdividef(c, s + a.hc_eps);
    }
    if (act) a.comb[t * hc * hc + lane] = c;
  }
  // the stream-0 thread group (warps 0..3) writes y as soon as warp 0 has pre and r; the Sinkhorn warp is not waited for
  if (j == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
  if (active && j == 0) {
    const float r = s_r;
    const float2 w01 = unpack_bf16x2(nw.x), w23 = unpack_bf16x2(nw.y);
    const float wv[4] = {w01.x, w01.y, w23.x, w23.y};
    float o[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      float v = 0.f;
#pragma unroll
      for (int s = 0; s < 4; ++s) v = fmaf(s_pre[s], xs[s][c], v);
      v = bf16_to_f(__float2bfloat16(v));
      o[c] = a.norm_w != nullptr ? v * r * wv[c] : v;
    }
    *reinterpret_cast<uint2*>(a.y + static_cast<long long>(t) * H + h) =
        make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
  }
  if (fused && a.use_ll && threadIdx.x == 0) ll_read_done(a.ll, epoch);
}

// ---- the folded all-reduce on its own: consumer that only sums (for call sites whose consumer is not fused) -------
// out[t, h] = bf16(sum over ranks of the slots); grid (T, ceil(H / 1024)).
__global__ void __launch_bounds__(256)
ll_reduce_kernel(const LLAr ll, __nv_bfloat16* __restrict__ out, long long ldo, int H, int* status) {
  pdl_wait();
  pdl_trigger();
  const uint32_t e = ll_read_epoch(ll);
  const int t = blockIdx.x;
  const int h = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (h < H) {
    const long long w0 = (static_cast<long long>(t) * H + h) >> 1;
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    float part[4][4];
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
      for (int c = 0; c < 4; ++c) part[q][c] = 0.f;
    for (int r = 0; r < ll.world; ++r) {          // same association as the fused consumer: ranks r and r + 4 first
      uint32_t d0, d1;
      ll_wait_word(ll, e, r, w0, d0, status);
      ll_wait_word(ll, e, r, w0 + 1, d1, status);
      const float2 p = unpack_bf16x2(d0), q = unpack_bf16x2(d1);
      part[r & 3][0] += p.x; part[r & 3][1] += p.y; part[r & 3][2] += q.x; part[r & 3][3] += q.y;
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) s[c] = (part[0][c] + part[1][c]) + (part[2][c] + part[3][c]);
    *reinterpret_cast<uint2*>(out + t * ldo + h) = make_uint2(pack_bf16x2(s[0], s[1]), pack_bf16x2(s[2], s[3]));
  }
  if (threadIdx.x == 0) ll_read_done(ll, e);
}

// Producer on its own: pushes a finished [T, H] bf16 tensor into every rank's slot (for producers that are not fused).
__global__ void __launch_bounds__(256)
ll_push_kernel(const LLAr ll, const __nv_bfloat16* __restrict__ in, long long ldi, int H) {
  pdl_wait();
  pdl_trigger();
  const uint32_t e = ll_push_epoch(ll);
  const int t = blockIdx.x;
  const int h = (blockIdx.y * blockDim.x + threadIdx.x) * 2;
  if (h < H) {
    const uint32_t d = *reinterpret_cast<const uint32_t*>(in + t * ldi + h);
    const long long w = (static_cast<long long>(t) * H + h) >> 1;
    for (int p = 0; p < ll.world; ++p) ll_store(ll, e, (ll.rank + p) % ll.world, w, d);
  }
  if (threadIdx.x == 0) ll_push_done(ll, e);
}

}  // namespace stk

using namespace stk;

STK_API int stk_ll_ctx_size() { return static_cast<int>(sizeof(LLAr)); }

// bases[r] = address (in this process) of rank r's receive region; counters: two zero-initialised uint32 in local memory.
STK_API int stk_ll_ctx_fill(void* ctx, const long long* bases, void* counters, long long words, int rank, int world,
                            int spin_budget) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || words <= 0 || counters == nullptr) return -1;
  LLAr l;
  memset(&l, 0, sizeof(l));
  for (int i = 0; i < world; ++i) {
    if (bases[i] == 0 || (bases[i] & 7)) return -2;
    l.slots[i] = reinterpret_cast<uint2*>(bases[i]);
  }
  l.counters = reinterpret_cast<uint32_t*>(counters);
  l.words = words;
  l.rank = rank;
  l.world = world;
  l.spin_budget = static_cast<uint32_t>(spin_budget);
  memcpy(ctx, &l, sizeof(l));
  return 0;
}

// Pre-mix of a decode-sized batch (T clusters of 8 CTAs).  Direct mode: x != nullptr.  Fused mode: x == nullptr and the
// streams are formed from (fa | the slots of ll_ctx), res_old, post_old, comb_old and written to x_out.
STK_API int stk_mhc_decode(const void* x, const void* fa, const void* res_old, const float* post_old,
                           const float* comb_old, void* x_out, const float* fn, const float* base, const float* scale,
                           const void* norm_w, float* post, float* comb, void* y, int T, int H, float rms_eps,
                           float hc_eps, int sinkhorn_iters, float post_mult, const void* ll_ctx, int* status,
                           void* stream) {
  if (T <= 0) return 0;
  if (H % 32 || H > 4096) return -1;
  MhcDecodeArgs a;
  memset(&a, 0, sizeof(a));
  a.x = (const __nv_bfloat16*)x;
  a.fa = (const __nv_bfloat16*)fa;
  a.res_old = (const __nv_bfloat16*)res_old;
  a.post_old = post_old;
  a.comb_old = comb_old;
  a.x_out = (__nv_bfloat16*)x_out;
  a.fn = fn; a.base = base; a.scale = scale;
  a.norm_w = (const __nv_bfloat16*)norm_w;
  a.post = post; a.comb = comb;
  a.y = (__nv_bfloat16*)y;
  a.H = H; a.rms_eps = rms_eps; a.hc_eps = hc_eps; a.sinkhorn_iters = sinkhorn_iters; a.post_mult = post_mult;
  a.status = status;
  if (x == nullptr) {
    if (res_old == nullptr || post_old == nullptr || comb_old == nullptr || x_out == nullptr || x_out == res_old) return -2;
    if (ll_ctx != nullptr) {
      memcpy(&a.ll, ll_ctx, sizeof(a.ll));
      if (static_cast<long long>(T) * H / 2 > a.ll.words) return -3;
      a.use_ll = 1;
    } else if (fa == nullptr) {
      return -2;
    }
  }
  // few tokens: one CTA per SM anyway, so each stages its mix weights in shared memory ahead of its predecessor's end
  constexpr int kStageBytes = kDcMix * kDcThreads * 16;
  static int stage_ok = 0;             // 0 unknown, 1 yes, -1 no
  if (stage_ok == 0) {
    stage_ok = cudaFuncSetAttribute(mhc_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kStageBytes) == cudaSuccess ? 1 : -1;
    if (stage_ok < 0) cudaGetLastError();
  }
  a.stage_fn = (stage_ok > 0 && T <= 16) ? 1 : 0;          // 16 clusters of 8 = 128 CTAs: at most one per SM
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(T * kDcCluster);
  cfg.blockDim = dim3(kDcThreads);
  cfg.dynamicSmemBytes = a.stage_fn ? kStageBytes : 0;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kDcCluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // a kernel that polls on peers' stores is still safe under programmatic launch: it waits for its predecessor first
  cfg.numAttrs = pdl_use((cudaStream_t)stream, STK_PDL_CLASS) ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, mhc_decode_kernel, a) == cudaSuccess ? 0 : -4;
}

STK_API int stk_ll_reduce(const void* ll_ctx, void* out, long long ldo, int T, int H, int* status, void* stream) {
  if (T <= 0) return 0;
  LLAr l;
  memcpy(&l, ll_ctx, sizeof(l));
  if (H % 4 || static_cast<long long>(T) * H / 2 > l.words || ldo % 4 || (reinterpret_cast<uintptr_t>(out) & 7)) return -1;
  launch_pdl(ll_reduce_kernel, dim3(T, (H / 4 + 255) / 256), dim3(256), 0, (cudaStream_t)stream, l, (__nv_bfloat16*)out, ldo, H, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_ll_push(const void* ll_ctx, const void* in, long long ldi, int T, int H, void* stream) {
  if (T <= 0) return 0;
  LLAr l;
  memcpy(&l, ll_ctx, sizeof(l));
  if (H % 2 || static_cast<long long>(T) * H / 2 > l.words || ldi % 2 || (reinterpret_cast<uintptr_t>(in) & 3)) return -1;
  launch_pdl(ll_push_kernel, dim3(T, (H / 2 + 255) / 256), dim3(256), 0, (cudaStream_t)stream, l, (const __nv_bfloat16*)in, ldi, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
