// Lightning-indexer scoring over the paged indexer-K cache and radix top-k selection.
//
//   score[t, s] = sum_h w[t, h] * relu(q[t, h, :] . k[s, :]) * k_scale[s]      s < n_valid[t]
//
// (the reference reaches this through DeepGEMM fp8_fp4_(paged_)mqa_logits followed by
// persistent_topk: probes/sai_probe.py:2316-2337,2535-2595).  This file holds the exact
// CUDA-core scorer used for decode-sized batches and as the numerics check of the
// tensor-core scorer, and the top-k kernel shared by both.
#define STK_PDL_CLASS 64      // bit of this file's kernels in the PDL mask (STK_PDL, stk_set_pdl_mask)
#include "common.cuh"

namespace stk {

struct IdxCache {
  const uint8_t* base;
  long long page_stride;
  int fp8;                 // 1: [64 x d fp8][64 x fp32 scale]; 0: [64 x d bf16]
};

// grid (T, ceil(max_rows/128)); 128 threads, one K row each.
template <int DI>
__global__ void __launch_bounds__(128)
indexer_scores_kernel(const void* __restrict__ q, const float* __restrict__ w, IdxCache kc,
                      const int* __restrict__ block_table, int bt_stride, const int* __restrict__ tok_req,
                      const int* __restrict__ n_valid, float* __restrict__ scores, long long ld_scores, int ih,
                      int q_fp8) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float sm[];     // ih * DI floats + ih weights
  float* qs = sm;
  float* ws = sm + ih * DI;
  const int t = blockIdx.x;
  const int nv = n_valid[t];
  const int s0 = blockIdx.y * 128;
  if (s0 >= nv) {
    return;
  }
  for (int i = threadIdx.x; i < ih * DI; i += blockDim.x) {
    qs[i] = q_fp8 ? fp8_to_f(reinterpret_cast<const uint8_t*>(q)[static_cast<long long>(t) * ih * DI + i])
                  : bf16_to_f(reinterpret_cast<const __nv_bfloat16*>(q)[static_cast<long long>(t) * ih * DI + i]);
  }
  for (int i = threadIdx.x; i < ih; i += blockDim.x) ws[i] = w[t * ih + i];
  __syncthreads();
  const int s = s0 + threadIdx.x;
  if (s >= nv) return;
  const int page = block_table[static_cast<long long>(tok_req[t]) * bt_stride + (s >> 6)];
  const int r = s & 63;
  const uint8_t* pbase = kc.base + static_cast<long long>(page) * kc.page_stride;
  float k[DI];
  float kscale = 1.f;
  if (kc.fp8) {
    const uint4* src = reinterpret_cast<const uint4*>(pbase + static_cast<long long>(r) * DI);
#pragma unroll
    for (int i = 0; i < DI / 16; ++i) {
      const uint4 v = src[i];
      const uint32_t wds[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int b = 0; b < 4; ++b) k[i * 16 + j * 4 + b] = fp8_to_f((wds[j] >> (8 * b)) & 0xff);
      }
    }
    kscale = *reinterpret_cast<const float*>(pbase + 64LL * DI + r * 4);
  } else {
    const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(pbase + static_cast<long long>(r) * DI * 2);
#pragma unroll
    for (int i = 0; i < DI; ++i) k[i] = bf16_to_f(src[i]);
  }
  float acc = 0.f;
  for (int h = 0; h < ih; ++h) {
    const float4* qh = reinterpret_cast<const float4*>(qs + h * DI);
    float d0 = 0.f, d1 = 0.f;
#pragma unroll
    for (int i = 0; i < DI / 4; ++i) {
      const float4 v = qh[i];
      d0 = fmaf(v.x, k[i * 4], fmaf(v.y, k[i * 4 + 1], d0));
      d1 = fmaf(v.z, k[i * 4 + 2], fmaf(v.w, k[i * 4 + 3], d1));
    }
    acc = fmaf(ws[h], fmaxf(d0 + d1, 0.f), acc);
  }
  scores[t * ld_scores + s] = acc * kscale;
}

// ---- top-k ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t float_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One CTA (1024 threads) per row.  out[t, :k]: indices of the k largest scores among the first
// n_valid[t] entries (all of them, ascending, when n_valid <= k), -1 padded.  Elements above the
// threshold come first in index order, then threshold ties in index order: deterministic.
// Register-resident variant for rows of up to PER * 1024 scores: every thread keeps PER consecutive keys, so the row
// is read once; the four radix passes use per-warp histograms (no cross-warp atomic contention) and a warp-parallel
// suffix search; the compaction is one block-wide exclusive scan.  Same output order as the generic kernel.
template <int PER>
__global__ void __launch_bounds__(1024)
topk_rows_reg_kernel(const float* __restrict__ scores, long long ld, const int* __restrict__ n_valid,
                     int* __restrict__ out, int k, int out_ld) {
  pdl_wait();
  pdl_trigger();
  __shared__ int whist[32][256];
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining;
  __shared__ int warp_gt[32], warp_eq[32];
  const int t = blockIdx.x;
  const int n = n_valid[t];
  const float* row = scores + t * ld;
  int* orow = out + static_cast<long long>(t) * out_ld;
  if (n <= k) {
    for (int i = threadIdx.x; i < k; i += blockDim.x) orow[i] = i < n ? i : -1;
    return;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int i0 = threadIdx.x * PER;
  uint32_t key[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) key[j] = (i0 + j) < n ? float_key(row[i0 + j]) : 0u;
  const int mine = max(0, min(PER, n - i0));            // valid keys of this thread
  if (threadIdx.x == 0) {
    s_prefix = 0;
    s_remaining = k;
  }
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < 32 * 256; i += blockDim.x) (&whist[0][0])[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
#pragma unroll
    for (int j = 0; j < PER; ++j)
      if (j < mine && (key[j] & mask) == prefix) atomicAdd(&whist[warp][(key[j] >> shift) & 0xff], 1);
    __syncthreads();
    if (threadIdx.x < 256) {
      int sum = 0;
#pragma unroll 8
      for (int w = 0; w < 32; ++w) sum += whist[w][threadIdx.x];
      hist[threadIdx.x] = sum;
    }
    __syncthreads();
    if (warp == 0) {
      // lane l owns bins [8l, 8l+8); suffix sums over lanes locate the lane, a short scan the bin
      int part = 0;
#pragma unroll
      for (int b = 0; b < 8; ++b) part += hist[lane * 8 + b];
      int suf = part;                                     // inclusive suffix sum (lanes >= this one)
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_down_sync(0xffffffffu, suf, o);
        if (lane + o < 32) suf += v;
      }
      const int rem0 = s_remaining;
      const int above = suf - part;                       // count in bins above this lane's range
      const bool here = above < rem0 && suf >= rem0;      // the k-th largest falls into this lane's bins
      const uint32_t who = __ballot_sync(0xffffffffu, here);
      const int sel = who ? (31 - __clz(who)) : 0;        // exactly one lane when n > k; highest as a guard
      if (lane == sel) {
        int rem = rem0 - above;
        int b = 7;
        for (; b > 0; --b) {
          const int h = hist[lane * 8 + b];
          if (h >= rem) break;
          rem -= h;
        }
        s_prefix = prefix | (static_cast<uint32_t>(lane * 8 + b) << shift);
        s_remaining = rem;
      }
    }
    __syncthreads();
  }
  const uint32_t thr = s_prefix;
  const int need_eq = s_remaining;
  const int count_gt = k - need_eq;
  int cg = 0, ce = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    if (j < mine) {
      cg += key[j] > thr;
      ce += key[j] == thr;
    }
  }
  // block-wide exclusive scan of (cg, ce) in thread order = index order
  int sg = cg, se = ce;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int vg = __shfl_up_sync(0xffffffffu, sg, o);
    const int ve = __shfl_up_sync(0xffffffffu, se, o);
    if (lane >= o) { sg += vg; se += ve; }
  }
  if (lane == 31) { warp_gt[warp] = sg; warp_eq[warp] = se; }
  __syncthreads();
  if (warp == 0) {
    int g = warp_gt[lane], e = warp_eq[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int vg = __shfl_up_sync(0xffffffffu, g, o);
      const int ve = __shfl_up_sync(0xffffffffu, e, o);
      if (lane >= o) { g += vg; e += ve; }
    }
    warp_gt[lane] = g;
    warp_eq[lane] = e;
  }
  __syncthreads();
  int og = (warp ? warp_gt[warp - 1] : 0) + sg - cg;
  int oe = (warp ? warp_eq[warp - 1] : 0) + se - ce;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    if (j < mine) {
      if (key[j] > thr) orow[og++] = i0 + j;
      else if (key[j] == thr) {
        if (oe < need_eq) orow[count_gt + oe] = i0 + j;
        ++oe;
      }
    }
  }
}

__global__ void __launch_bounds__(1024)
topk_rows_kernel(const float* __restrict__ scores, long long ld, const int* __restrict__ n_valid,
                 int* __restrict__ out, int k, int out_ld) {
  pdl_wait();
  pdl_trigger();
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining;
  __shared__ int warp_gt[32], warp_eq[32];
  __shared__ int base_gt, base_eq;
  const int t = blockIdx.x;
  const int n = n_valid[t];
  const float* row = scores + t * ld;
  int* orow = out + static_cast<long long>(t) * out_ld;
  if (n <= k) {
    for (int i = threadIdx.x; i < k; i += blockDim.x) orow[i] = i < n ? i : -1;
    return;
  }
  if (threadIdx.x == 0) {
    s_prefix = 0;
    s_remaining = k;
  }
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const uint32_t key = float_key(row[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int rem = s_remaining;
      int b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= rem) break;
        rem -= hist[b];
      }
      s_prefix = prefix | (static_cast<uint32_t>(b) << shift);
      s_remaining = rem;
    }
    __syncthreads();
  }
  const uint32_t thr = s_prefix;
  const int need_eq = s_remaining;          // ties to take (>= 1)
  const int count_gt = k - need_eq;
  if (threadIdx.x == 0) {
    base_gt = 0;
    base_eq = 0;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i0 = 0; i0 < n; i0 += blockDim.x) {
    const int i = i0 + threadIdx.x;
    uint32_t key = 0;
    const bool in = i < n;
    if (in) key = float_key(row[i]);
    const bool gt = in && key > thr;
    const bool eq = in && key == thr;
    const uint32_t bg = __ballot_sync(0xffffffffu, gt);
    const uint32_t be = __ballot_sync(0xffffffffu, eq);
    if (lane == 0) {
      warp_gt[warp] = __popc(bg);
      warp_eq[warp] = __popc(be);
    }
    __syncthreads();
    int og = base_gt, oe = base_eq;
    for (int w = 0; w < warp; ++w) {
      og += warp_gt[w];
      oe += warp_eq[w];
    }
    og += __popc(bg & ((1u << lane) - 1));
    oe += __popc(be & ((1u << lane) - 1));
    if (gt) orow[og] = i;
    if (eq && oe < need_eq) orow[count_gt + oe] = i;
    __syncthreads();
    if (threadIdx.x == 0) {
      int tg = 0, te = 0;
      for (int w = 0; w < 32; ++w) {
        tg += warp_gt[w];
        te += warp_eq[w];
      }
      base_gt += tg;
      base_eq += te;
    }
    __syncthreads();
  }
}

// local compressed index -> physical slot of the compressed cache; counts valid entries.
// (overlay/ops_cache_utils.py:506-554)
__global__ void topk_to_slots_kernel(const int* __restrict__ topk, int k, int topk_ld,
                                     const int* __restrict__ block_table, int bt_stride,
                                     const int* __restrict__ tok_req, int* __restrict__ slots, int slots_ld,
                                     int* __restrict__ lens, int max_rows, int* status) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  __shared__ int cnt;
  if (threadIdx.x == 0) cnt = 0;
  __syncthreads();
  int local = 0;
  const int req = tok_req[t];
  for (int i = threadIdx.x; i < k; i += blockDim.x) {
    const int idx = topk[static_cast<long long>(t) * topk_ld + i];
    int slot = -1;
    if (req >= 0 && idx >= 0) {
      if (idx >= max_rows) {
        set_status(status, kBadIndex, t);
      } else {
        const int page = block_table[static_cast<long long>(req) * bt_stride + (idx >> 6)];
        if (page >= 0) {
          slot = page * 64 + (idx & 63);
          ++local;
        }
      }
    }
    slots[static_cast<long long>(t) * slots_ld + i] = slot;
  }
  atomicAdd(&cnt, local);
  __syncthreads();
  if (threadIdx.x == 0) lens[t] = cnt;
}

}  // namespace stk

using namespace stk;

STK_API int stk_indexer_scores(const void* q, const float* w, const void* kcache, long long page_stride, int k_fp8,
                               const int* block_table, int bt_stride, const int* tok_req, const int* n_valid,
                               float* scores, long long ld_scores, int T, int max_rows, int ih, int di, int q_fp8,
                               void* stream) {
  if (T <= 0 || max_rows <= 0) return 0;
  IdxCache kc{(const uint8_t*)kcache, page_stride, k_fp8};
  dim3 grid(T, (max_rows + 127) / 128);
  const size_t smem = (static_cast<size_t>(ih) * di + ih) * sizeof(float);
  cudaStream_t st = (cudaStream_t)stream;
#define STK_IDX(DI_)                                                                                          \
  {                                                                                                           \
    static bool configured = false;                                                                           \
    if (!configured && smem > 48 * 1024) {                                                                    \
      cudaFuncSetAttribute(indexer_scores_kernel<DI_>, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024); \
      configured = true;                                                                                      \
    }                                                                                                         \
    launch_pdl(indexer_scores_kernel<DI_>, dim3(grid), dim3(128), smem, st, q, w, kc, block_table, bt_stride, tok_req, n_valid,    \
                                                        scores, ld_scores, ih, q_fp8);                        \
  }
  if (di == 128) STK_IDX(128)
  else if (di == 64) STK_IDX(64)
  else if (di == 32) STK_IDX(32)
  else return -1;
#undef STK_IDX
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_topk_rows(const float* scores, long long ld, const int* n_valid, int* out, int out_ld, int T, int k,
                          void* stream) {
  if (T <= 0) return 0;
  // ld bounds every row's valid length: rows that fit in registers take the single-read kernel
  if (ld <= 8 * 1024) {
    launch_pdl(topk_rows_reg_kernel<8>, dim3(T), dim3(1024), 0, (cudaStream_t)stream, scores, ld, n_valid, out, k, out_ld);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  if (ld <= 16 * 1024) {
    launch_pdl(topk_rows_reg_kernel<16>, dim3(T), dim3(1024), 0, (cudaStream_t)stream, scores, ld, n_valid, out, k, out_ld);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  launch_pdl(topk_rows_kernel, dim3(T), dim3(1024), 0, (cudaStream_t)stream, scores, ld, n_valid, out, k, out_ld);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_topk_to_slots(const int* topk, int k, int topk_ld, const int* block_table, int bt_stride,
                              const int* tok_req, int* slots, int slots_ld, int* lens, int T, int max_rows,
                              int* status, void* stream) {
  if (T <= 0) return 0;
  launch_pdl(topk_to_slots_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream, topk, k, topk_ld, block_table, bt_stride, tok_req, slots,
                                                            slots_ld, lens, max_rows, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
