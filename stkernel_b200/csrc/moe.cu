// Mixture-of-experts routing and the weight-streaming (decode-sized) expert path.
//
//   router        scores = sigmoid | sqrt(softplus) of fp32 gate logits; selection by score + bias
//                 (or by a token-id hash table with bounds checks); weights from the unbiased
//                 score, renormalised and scaled.   (topkGatingSoftplusSqrt / fused_topk_bias and
//                 the hash-MoE lookup of overlay/nvidia_model.py:806-827)
//   moe_align     (token, k) pairs sorted by expert, stable in pair order
//   expert_fc1    act[pair, i] = silu(min(g, lim)) * clamp(u) with g/u = x . W1/W3 rows   (NVFP4)
//   expert_fc2    y[pair, n]   = act . W2 rows                                              (NVFP4)
//
// NVFP4 = e2m1 codes packed two per byte (low nibble first), one e4m3 scale per 16 values and one
// fp32 scale per expert matrix.  With a handful of tokens per expert the work is bounded by the
// bytes of the weight rows, so each warp streams whole rows with 16-byte loads and dots them in
// half2 against activations held in shared memory (fp32 accumulation per 16-value group).
// Prefill-sized batches use the tcgen05 grouped GEMM instead.
#include <cuda_fp4.h>

#define STK_PDL_CLASS 1024      // bit of this file's kernels in the PDL mask (STK_PDL, stk_set_pdl_mask)
#include "common.cuh"
#include "router.cuh"

namespace stk {

// ---- router ------------------------------------------------------------------------
// One warp per token, E <= 512 (the selection itself lives in router.cuh, shared with the gate projection's epilogue).
__global__ void router_kernel(const float* __restrict__ logits, long long ldl, const float* __restrict__ bias,
                              const int* __restrict__ tid2eid, const int64_t* __restrict__ token_ids, int vocab,
                              int* __restrict__ ids, float* __restrict__ weights, int T, int E, int topk, int scoring,
                              int renorm, float scaling, int* status) {
  pdl_wait();
  pdl_trigger();
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (t >= T) return;
  RouterArgs r{bias, tid2eid, token_ids, vocab, ids, weights, E, topk, scoring, renorm, scaling, status};
  route_token(r, logits + t * ldl, t, threadIdx.x & 31);
}

// ---- pair sort by expert ------------------------------------------------------------
// Single CTA.  sorted[q] = pair index, pair_row[p] = q (or -1 when the expert is not local),
// offsets[e] = first row of local expert e, offsets[E_local] = total rows.
// The pair list is staged in shared memory; a pair's row is its expert's offset plus the number of earlier pairs of
// the same expert (stable order, so results do not depend on thread scheduling), counted by a broadcast scan.
__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ ids, int n_pairs, int e_start, int e_local, int* __restrict__ sorted,
                 int* __restrict__ pair_row, int* __restrict__ offsets, int* __restrict__ sorted_expert) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ int sh[];          // counts[e_local + 1] | local expert of every pair (or -1)
  int* counts = sh;
  int* ids_s = sh + e_local + 1;
  for (int i = threadIdx.x; i <= e_local; i += blockDim.x) counts[i] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    int e = ids[p] - e_start;
    if (e < 0 || e >= e_local) e = -1;
    ids_s[p] = e;
    if (e >= 0) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    // exclusive scan of the expert counts by one warp
    int run = 0;
    for (int e0 = 0; e0 < e_local; e0 += 32) {
      const int e = e0 + threadIdx.x;
      const int c = e < e_local ? counts[e] : 0;
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (static_cast<int>(threadIdx.x) >= o) incl += v;
      }
      if (e < e_local) {
        counts[e] = run + incl - c;
        offsets[e] = run + incl - c;
      }
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (threadIdx.x == 0) {
      counts[e_local] = run;
      offsets[e_local] = run;
    }
  }
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = ids_s[p];
    if (e < 0) {
      pair_row[p] = -1;
      continue;
    }
    int rank = 0;
    for (int q = 0; q < p; ++q) rank += (ids_s[q] == e) ? 1 : 0;
    const int pos = counts[e] + rank;
    sorted[pos] = p;
    sorted_expert[pos] = e;
    pair_row[p] = pos;
  }
}

// ---- parallel pair sort for large batches (three small launches) ---------------------------
constexpr int kAlignChunk = 256;

// counts[c][e] = pairs of chunk c routed to local expert e
__global__ void moe_align_count_kernel(const int* __restrict__ ids, int n_pairs, int e_start, int e_local,
                                       int* __restrict__ counts) {
  extern __shared__ int sh[];
  for (int i = threadIdx.x; i < e_local; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const int p = blockIdx.x * kAlignChunk + threadIdx.x;
  if (p < n_pairs) {
    const int e = ids[p] - e_start;
    if (e >= 0 && e < e_local) atomicAdd(&sh[e], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < e_local; i += blockDim.x) counts[blockIdx.x * e_local + i] = sh[i];
}

// per expert: exclusive scan of its counts over the chunks (in place) and the expert offsets
__global__ void moe_align_scan_kernel(int* __restrict__ counts, int n_chunks, int e_local, int* __restrict__ offsets) {
  extern __shared__ int tot[];
  for (int e = threadIdx.x; e < e_local; e += blockDim.x) {
    int run = 0;
    for (int c = 0; c < n_chunks; ++c) {
      const int v = counts[c * e_local + e];
      counts[c * e_local + e] = run;
      run += v;
    }
    tot[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < e_local; ++e) {
      offsets[e] = run;
      run += tot[e];
    }
    offsets[e_local] = run;
  }
}

// stable placement: row = offsets[e] + (pairs of e in earlier chunks) + (earlier pairs of e in this chunk)
__global__ void moe_align_place_kernel(const int* __restrict__ ids, int n_pairs, int e_start, int e_local,
                                       const int* __restrict__ counts, const int* __restrict__ offsets,
                                       int* __restrict__ sorted, int* __restrict__ pair_row,
                                       int* __restrict__ sorted_expert) {
  __shared__ int se[kAlignChunk];
  const int p = blockIdx.x * kAlignChunk + threadIdx.x;
  int e = -1;
  if (p < n_pairs) {
    e = ids[p] - e_start;
    if (e < 0 || e >= e_local) e = -1;
  }
  se[threadIdx.x] = e;
  __syncthreads();
  if (p >= n_pairs) return;
  if (e < 0) {
    pair_row[p] = -1;
    return;
  }
  int rank = 0;
  for (int j = 0; j < static_cast<int>(threadIdx.x); ++j) rank += (se[j] == e) ? 1 : 0;
  const int row = offsets[e] + counts[blockIdx.x * e_local + e] + rank;
  sorted[row] = p;
  sorted_expert[row] = e;
  pair_row[p] = row;
}

// ---- NVFP4 row dot --------------------------------------------------------------------
// xs: activations as half, permuted so that (iteration k, quarter i, lane) is one uint4:
//   chunk c = lane + 32*k covers values [32c, 32c+32); uint4 index = (k*4 + i)*32 + lane.
// A row is read in two steps so that several rows' loads can be in flight before any arithmetic.
template <int ITERS>
struct Fp4Row {
  uint4 w[ITERS];
  uint32_t s[ITERS];
};

template <int ITERS>
__device__ __forceinline__ void fp4_row_load(Fp4Row<ITERS>& r, const uint8_t* __restrict__ wrow,
                                             const uint8_t* __restrict__ srow, int n_chunks, int lane) {
#pragma unroll
  for (int k = 0; k < ITERS; ++k) {
    const int c = k * 32 + lane;
    r.w[k] = make_uint4(0, 0, 0, 0);
    r.s[k] = 0;
    if (c < n_chunks) {
      r.w[k] = __ldg(reinterpret_cast<const uint4*>(wrow) + c);
      r.s[k] = __ldg(reinterpret_cast<const uint16_t*>(srow) + c);
    }
  }
}

// One 32-value chunk: 16 bytes of e2m1 pairs, two e4m3 block scales, activations at (iteration k, lane) of `xs`.
__device__ __forceinline__ float fp4_chunk_dot(const uint4& wv, uint32_t sc, const uint4* __restrict__ xs, int k, int lane) {
  const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
  float part[2];
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    __half2 hs = __floats2half2_rn(0.f, 0.f);
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const uint4 xv = xs[(k * 4 + g * 2 + q) * 32 + lane];
      const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
      const uint32_t w = words[g * 2 + q];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const __half2_raw hr = __nv_cvt_fp4x2_to_halfraw2(static_cast<__nv_fp4x2_storage_t>((w >> (8 * b)) & 0xff), __NV_E2M1);
        hs = __hfma2(*reinterpret_cast<const __half2*>(&hr), *reinterpret_cast<const __half2*>(&xw[b]), hs);
      }
    }
    part[g] = __low2float(hs) + __high2float(hs);
  }
  return fmaf(part[0], fp8_to_f(sc & 0xff), part[1] * fp8_to_f((sc >> 8) & 0xff));
}

template <int ITERS>
__device__ __forceinline__ float fp4_row_dot(const Fp4Row<ITERS>& r, const uint4* __restrict__ xs, int n_chunks, int lane) {
  float acc = 0.f;
#pragma unroll
  for (int k = 0; k < ITERS; ++k) {
    const int c = k * 32 + lane;
    if (c < n_chunks) acc += fp4_chunk_dot(r.w[k], r.s[k], xs, k, lane);
  }
  return warp_sum(acc);
}

__device__ __forceinline__ float src_to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float src_to_f(__half v) { return __half2float(v); }

// Fill the permuted half activation buffer from a bf16 or half row.  The buffer holds
// ceil(K / 1024) * 1024 halfs (the permutation leaves holes when K < 1024).  Eight consecutive
// values move as one 16-byte load and one 16-byte store.
__device__ __forceinline__ uint4 to_half8(const uint4& v, const __nv_bfloat16*) {
  uint4 o;
  __half2* oh = reinterpret_cast<__half2*>(&o);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) oh[j] = __float22half2_rn(__bfloat1622float2(b[j]));
  return o;
}
__device__ __forceinline__ uint4 to_half8(const uint4& v, const __half*) { return v; }

template <typename SrcT>
__device__ __forceinline__ void fill_xs(__half* xs_h, const SrcT* x, int K) {
  uint4* xs4 = reinterpret_cast<uint4*>(xs_h);
  if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    for (int k8 = threadIdx.x; k8 < (K >> 3); k8 += blockDim.x) {
      const uint4 v = *reinterpret_cast<const uint4*>(x + k8 * 8);
      const int c = k8 >> 2;                               // 32-value chunk
      xs4[((c >> 5) * 4 + (k8 & 3)) * 32 + (c & 31)] = to_half8(v, x);
    }
  } else {
    for (int e = threadIdx.x; e < K; e += blockDim.x) {
      const int c = e >> 5, within = e & 31;
      xs_h[(((c >> 5) * 4 + (within >> 3)) * 32 + (c & 31)) * 8 + (within & 7)] = __float2half(src_to_f(x[e]));
    }
  }
}

struct ExpertW {
  const uint8_t* w;       // [E, rows, K/2]
  const uint8_t* s;       // [E, rows, K/16] e4m3
  const float* gscale;    // [E]
};

// grid (ceil(I / 16), n_rows); CTA = 8 warps, 2 outputs per warp.
template <int ITERS>
__global__ void __launch_bounds__(256)
expert_fc1_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, ExpertW w13, const int* __restrict__ sorted,
                  const int* __restrict__ sorted_expert, const int* __restrict__ offsets, int e_local, int topk,
                  __half* __restrict__ act, int H, int I, float limit, const int* __restrict__ direct_ids,
                  int e_start) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ uint4 xs[];
  const int row = blockIdx.y;
  int pair, e;
  if (direct_ids != nullptr) {
    // direct mode (a handful of pairs): row = pair index, no sort; non-local experts are skipped.
    // Under expert parallelism most pairs belong to other ranks: their CTAs leave as soon as the id has arrived, before
    // any staging (they would otherwise hold an SM slot for a full activation copy each).
    pair = row;
    e = __ldg(direct_ids + row) - e_start;
    if (e < 0 || e >= e_local) return;
    fill_xs(reinterpret_cast<__half*>(xs), x + (pair / topk) * ldx, H);
  } else {
    if (row >= offsets[e_local]) return;
    pair = sorted[row];
    e = sorted_expert[row];
    fill_xs(reinterpret_cast<__half*>(xs), x + (pair / topk) * ldx, H);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_chunks = H / 32;
  const float gs = w13.gscale[e];
  const long long wstride = static_cast<long long>(H) / 2, sstride = static_cast<long long>(H) / 16;
  const uint8_t* wbase = w13.w + static_cast<long long>(e) * 2 * I * wstride;
  const uint8_t* sbase = w13.s + static_cast<long long>(e) * 2 * I * sstride;
  // the four weight rows of this warp (gate and up of two outputs) are all requested before the barrier that
  // publishes the staged activations, and before any arithmetic
  Fp4Row<ITERS> rg[2], ru[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int i = min(blockIdx.x * 16 + warp * 2 + j, I - 1);
    fp4_row_load<ITERS>(rg[j], wbase + i * wstride, sbase + i * sstride, n_chunks, lane);
    fp4_row_load<ITERS>(ru[j], wbase + (I + i) * wstride, sbase + (I + i) * sstride, n_chunks, lane);
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int i = blockIdx.x * 16 + warp * 2 + j;
    float g = fp4_row_dot<ITERS>(rg[j], xs, n_chunks, lane) * gs;
    float u = fp4_row_dot<ITERS>(ru[j], xs, n_chunks, lane) * gs;
    if (lane == 0 && i < I) {
      if (limit > 0.f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
      }
      act[static_cast<long long>(row) * I + i] = __float2half(g / (1.f + __expf(-g)) * u);
    }
  }
}

// FC2 for narrow experts (I <= 512: the slices of tensor-parallel decode): a row is L = I / 32 chunks, so L lanes per
// row and 32 / L rows per warp pass; four passes per warp, 8 warps: 128 * (8 / L) ... rows per CTA = 8 * (32 / L) * 4.
// Direct mode only (row = pair index).  grid (ceil(H / rows_per_cta), n_pairs).
template <int L>
__global__ void __launch_bounds__(256)
expert_fc2_narrow_kernel(const __half* __restrict__ act, ExpertW w2, int e_local, __nv_bfloat16* __restrict__ y, int H, int I,
                         const int* __restrict__ direct_ids, int e_start) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ uint4 xs[];
  constexpr int R = 32 / L, kJ = 4;
  constexpr int kRowsPerCta = 8 * R * kJ;
  const int row = blockIdx.y;
  const int e = __ldg(direct_ids + row) - e_start;
  if (e < 0 || e >= e_local) {
    for (int n = blockIdx.x * kRowsPerCta + threadIdx.x; n < min(H, (static_cast<int>(blockIdx.x) + 1) * kRowsPerCta); n += blockDim.x)
      y[static_cast<long long>(row) * H + n] = __float2bfloat16(0.f);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / L, cl = lane % L;
  const float gs = w2.gscale[e];
  const long long wstride = static_cast<long long>(I) / 2, sstride = static_cast<long long>(I) / 16;
  const uint8_t* wbase = w2.w + static_cast<long long>(e) * H * wstride;
  const uint8_t* sbase = w2.s + static_cast<long long>(e) * H * sstride;
  const int n0 = blockIdx.x * kRowsPerCta + warp * R * kJ;
  uint4 wv[kJ];
  uint32_t sc[kJ];
#pragma unroll
  for (int j = 0; j < kJ; ++j) {
    const int n = min(n0 + j * R + sub, H - 1);
    wv[j] = __ldg(reinterpret_cast<const uint4*>(wbase + n * wstride) + cl);
    sc[j] = __ldg(reinterpret_cast<const uint16_t*>(sbase + n * sstride) + cl);
  }
  fill_xs(reinterpret_cast<__half*>(xs), act + static_cast<long long>(row) * I, I);
  __syncthreads();
#pragma unroll
  for (int j = 0; j < kJ; ++j) {
    float v = fp4_chunk_dot(wv[j], sc[j], xs, 0, cl);
#pragma unroll
    for (int o = L / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int n = n0 + j * R + sub;
    if (cl == 0 && n < H) y[static_cast<long long>(row) * H + n] = __float2bfloat16(v * gs);
  }
}

// grid (ceil(H / 32), n_rows); 4 outputs per warp.
template <int ITERS>
__global__ void __launch_bounds__(256)
expert_fc2_kernel(const __half* __restrict__ act, ExpertW w2, const int* __restrict__ sorted_expert,
                  const int* __restrict__ offsets, int e_local, __nv_bfloat16* __restrict__ y, int H, int I,
                  const int* __restrict__ direct_ids, int e_start) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ uint4 xs[];
  const int row = blockIdx.y;
  int e;
  if (direct_ids != nullptr) {
    e = __ldg(direct_ids + row) - e_start;
    if (e < 0 || e >= e_local) {
      // not a local expert: this pair contributes nothing on this rank
      for (int n = blockIdx.x * 32 + threadIdx.x; n < min(H, blockIdx.x * 32 + 32); n += blockDim.x)
        y[static_cast<long long>(row) * H + n] = __float2bfloat16(0.f);
      return;
    }
    fill_xs(reinterpret_cast<__half*>(xs), act + static_cast<long long>(row) * I, I);
  } else {
    if (row >= offsets[e_local]) return;
    e = sorted_expert[row];
    fill_xs(reinterpret_cast<__half*>(xs), act + static_cast<long long>(row) * I, I);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_chunks = I / 32;
  const float gs = w2.gscale[e];
  const long long wstride = static_cast<long long>(I) / 2, sstride = static_cast<long long>(I) / 16;
  const uint8_t* wbase = w2.w + static_cast<long long>(e) * H * wstride;
  const uint8_t* sbase = w2.s + static_cast<long long>(e) * H * sstride;
  Fp4Row<ITERS> rw[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int n = min(blockIdx.x * 32 + warp * 4 + j, H - 1);
    fp4_row_load<ITERS>(rw[j], wbase + n * wstride, sbase + n * sstride, n_chunks, lane);
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int n = blockIdx.x * 32 + warp * 4 + j;
    const float v = fp4_row_dot<ITERS>(rw[j], xs, n_chunks, lane) * gs;
    if (lane == 0 && n < H) y[static_cast<long long>(row) * H + n] = __float2bfloat16(v);
  }
}

}  // namespace stk

using namespace stk;

STK_API int stk_router(const float* logits, long long ldl, const float* bias, const int* tid2eid,
                       const int64_t* token_ids, int vocab, int* ids, float* weights, int T, int E, int topk,
                       int scoring, int renorm, float scaling, int* status, void* stream) {
  if (T <= 0) return 0;
  if (E > 512 || topk > 32) return -1;
  launch_pdl(router_kernel, dim3((T + 7) / 8), dim3(256), 0, (cudaStream_t)stream, logits, ldl, bias, tid2eid, token_ids, vocab, ids,
                                                               weights, T, E, topk, scoring, renorm, scaling, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// counts: scratch of ceil(n_pairs / 256) * e_local ints (only used for large batches; may be null for
// n_pairs <= 2048).
STK_API int stk_moe_align(const int* ids, int n_pairs, int e_start, int e_local, int* sorted, int* pair_row,
                          int* offsets, int* sorted_expert, int* counts, void* stream) {
  if (n_pairs <= 0) return 0;
  if (n_pairs > 2048 && counts != nullptr) {
    const int n_chunks = (n_pairs + kAlignChunk - 1) / kAlignChunk;
    cudaStream_t st = (cudaStream_t)stream;
    moe_align_count_kernel<<<n_chunks, kAlignChunk, e_local * sizeof(int), st>>>(ids, n_pairs, e_start, e_local, counts);
    moe_align_scan_kernel<<<1, 256, e_local * sizeof(int), st>>>(counts, n_chunks, e_local, offsets);
    moe_align_place_kernel<<<n_chunks, kAlignChunk, 0, st>>>(ids, n_pairs, e_start, e_local, counts, offsets, sorted,
                                                             pair_row, sorted_expert);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  launch_pdl(moe_align_kernel, dim3(1), dim3(1024), (e_local + 1 + n_pairs) * sizeof(int), (cudaStream_t)stream, ids, n_pairs, e_start, e_local,
                                                                                   sorted, pair_row, offsets,
                                                                                   sorted_expert);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// max_rows bounds the grid (rows beyond offsets[e_local] exit at once).
STK_API int stk_moe_expert_fc1(const void* x, long long ldx, const void* w13, const void* s13, const float* g13,
                               const int* sorted, const int* sorted_expert, const int* offsets, int e_local, int topk,
                               void* act, int max_rows, int H, int I, float limit, const int* direct_ids, int e_start,
                               void* stream) {
  if (max_rows <= 0) return 0;
  if (H % 32 || H > 16384) return -1;
  ExpertW w{(const uint8_t*)w13, (const uint8_t*)s13, g13};
  dim3 grid((I + 15) / 16, max_rows);
  const size_t smem = ((H + 1023) / 1024) * 2048;
  cudaStream_t st = (cudaStream_t)stream;
  const int iters = (H / 32 + 31) / 32;
#define STK_FC1(I_) launch_pdl(expert_fc1_kernel<I_>, dim3(grid), dim3(256), smem, st, (const __nv_bfloat16*)x, ldx, w, sorted, sorted_expert, offsets, e_local, topk, (__half*)act, H, I, limit, direct_ids, e_start)
  if (iters <= 1) STK_FC1(1); else if (iters <= 2) STK_FC1(2); else if (iters <= 4) STK_FC1(4); else if (iters <= 8) STK_FC1(8); else STK_FC1(16);
#undef STK_FC1
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_moe_expert_fc2(const void* act, const void* w2, const void* s2, const float* g2,
                               const int* sorted_expert, const int* offsets, int e_local, void* y, int max_rows, int H,
                               int I, const int* direct_ids, int e_start, void* stream) {
  if (max_rows <= 0) return 0;
  if (I % 32 || I > 16384) return -1;
  ExpertW w{(const uint8_t*)w2, (const uint8_t*)s2, g2};
  const size_t smem = ((I + 1023) / 1024) * 2048;
  cudaStream_t st = (cudaStream_t)stream;
  if (direct_ids != nullptr && I <= 512 && (I & (I - 1)) == 0) {
    // narrow experts: several rows per warp pass
    const int L = I / 32;
#define STK_FC2N(L_)                                                                                              \
  launch_pdl(expert_fc2_narrow_kernel<L_>, dim3((H + 8 * (32 / L_) * 4 - 1) / (8 * (32 / L_) * 4), max_rows), dim3(256), smem, st, \
             (const __half*)act, w, e_local, (__nv_bfloat16*)y, H, I, direct_ids, e_start)
    if (L == 1) STK_FC2N(1); else if (L == 2) STK_FC2N(2); else if (L == 4) STK_FC2N(4); else if (L == 8) STK_FC2N(8); else STK_FC2N(16);
#undef STK_FC2N
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  dim3 grid((H + 31) / 32, max_rows);
  const int iters = (I / 32 + 31) / 32;
#define STK_FC2(I_) launch_pdl(expert_fc2_kernel<I_>, dim3(grid), dim3(256), smem, st, (const __half*)act, w, sorted_expert, offsets, e_local, (__nv_bfloat16*)y, H, I, direct_ids, e_start)
  if (iters <= 1) STK_FC2(1); else if (iters <= 2) STK_FC2(2); else if (iters <= 4) STK_FC2(4); else if (iters <= 8) STK_FC2(8); else STK_FC2(16);
#undef STK_FC2
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
