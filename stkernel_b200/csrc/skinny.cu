// Weight-streaming linear layer for one to four tokens (single-request decode):
//   out[t, n] = sum_k x[t, k] * W[n, k]
// One warp per output feature streams the weight row with 16-byte loads; the activations sit in
// shared memory (fp16, laid out so that a warp's reads are conflict free); fp32 accumulation.
// With so few tokens the layer is bounded by the bytes of W, and this single-pass form has a much
// shorter dependency chain than a tensor-core tile pipeline with split-K: no workspace, no second
// reduction pass.  Larger token counts use the tcgen05 GEMM.
//
// FP8 weights carry 128x128 block scales (applied per 16-value chunk); activations are used
// unquantised, which is at least as accurate as the quantised tensor-core path.
//
// Three optional fusions take neighbouring launches of the decode chain into this kernel:
//   * prologue RMSNorm: the activation row is normalised (weight, eps; rounded to bf16 like a separate norm kernel's
//     output) while it is staged into shared memory -- every CTA redoes the few-KB reduction, no CTA waits for another;
//   * folded all-reduce (row-parallel layers): the output words go straight into every rank's receive slot
//     (symm.cuh, LLAr) instead of to `out`; the consumer kernel adds the ranks;
//   * router epilogue (gate projection): the CTA that finishes last selects the experts of every token.
#define STK_PDL_CLASS 2      // bit of this file's kernels in the PDL mask (STK_PDL, stk_set_pdl_mask)
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "router.cuh"
#include "symm.cuh"

namespace stk {

constexpr int kSkinnyMaxT = 8;

struct SkinnyExtra {
  const __nv_bfloat16* norm_w;   // prologue RMSNorm weight [K] (nullptr: off)
  float norm_eps;
  int use_ll;                    // push the result into the slots of `ll` instead of writing `out`
  LLAr ll;
  int k_split;                   // 1, or 2: two CTAs per row block each take half of K and add into a zeroed fp32 `out`
                                 // (two addends commute, so the result does not depend on arrival order)
  int route;                     // run the router over `out` (fp32 logits [T, N]) in the last CTA
  int* route_counter;            // zero on entry, zero again on exit
  RouterArgs router;
};

// x: [T, K] bf16 -> xs: half, permuted: chunk c = lane + 32*k holds values [16c, 16c+16) as two uint4
// at index ((t * kIters + k) * 2 + i) * 32 + lane.
// kPrescale: each token's row is multiplied by 2^-e with e chosen so that |x| <= 8 (e >= 0 only); xscale[t] = 2^e is
// folded back in by the caller.  Raw e4m3 codes reach 448, so a product stays below 3584 and a sum of eight below
// 28672: the packed fp16 partial sums of the fp8 path cannot overflow.
template <int T, bool kPrescale>
__device__ __forceinline__ void skinny_fill_x(__half* xs, const __nv_bfloat16* x, long long ldx, int K, int iters,
                                              float* xscale, float* red, int t_valid,
                                              const __nv_bfloat16* norm_w = nullptr, float norm_eps = 0.f) {
  // eight consecutive values = one 16-byte load, one conversion, one 16-byte store
  uint4* xs4 = reinterpret_cast<uint4*>(xs);
  const int k8n = K >> 3;
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((ldx & 7) == 0);
  float mul[T];
  float nr[T];             // prologue RMSNorm: 1/rms of each row
#pragma unroll
  for (int t = 0; t < T; ++t) { mul[t] = 1.f; nr[t] = 1.f; }
  if (norm_w != nullptr) {
    // one pass over the row for both reductions: sum x^2 (the norm) and max |x * w| (the fp8 pre-scale bound: the
    // normalised row is x * w times one scalar)
#pragma unroll
    for (int t = 0; t < T; ++t) {
      float ss = 0.f, am = 0.f;
      if (t < t_valid)
        for (int k = threadIdx.x; k < K; k += blockDim.x) {
          const float v = bf16_to_f(x[t * ldx + k]);
          ss = fmaf(v, v, ss);
          if constexpr (kPrescale) am = fmaxf(am, fabsf(v * bf16_to_f(norm_w[k])));
        }
      ss = warp_sum(ss);
      am = warp_max(am);
      __syncthreads();
      if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5] = ss; red[16 + (threadIdx.x >> 5)] = am; }
      __syncthreads();
      float s2 = 0.f, a2 = 0.f;
      for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) { s2 += red[w]; a2 = fmaxf(a2, red[16 + w]); }
      nr[t] = rsqrtf(s2 / static_cast<float>(K) + norm_eps);
      if constexpr (kPrescale) {
        const float amax = a2 * nr[t] * 1.01f;          // the rounding of each normalised value to bf16 stays inside
        int e = 0;
        if (amax > 8.f) e = static_cast<int>(ceilf(log2f(amax * 0.125f)));
        if (threadIdx.x == 0) xscale[t] = exp2f(static_cast<float>(e));
        mul[t] = exp2f(static_cast<float>(-e));
      }
    }
    __syncthreads();
  } else if constexpr (kPrescale) {
#pragma unroll
    for (int t = 0; t < T; ++t) {
      float amax = 0.f;
      if (t >= t_valid) {
        // a template instance may be wider than the batch: the surplus rows are zeros
      } else if (((reinterpret_cast<uintptr_t>(x) & 3) == 0) && ((ldx & 1) == 0)) {
        for (int k2 = threadIdx.x; k2 < (K >> 1); k2 += blockDim.x) {
          const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(x + t * ldx + 2 * k2);
          amax = fmaxf(amax, fmaxf(fabsf(__low2float(v)), fabsf(__high2float(v))));
        }
      } else {
        for (int k = threadIdx.x; k < K; k += blockDim.x) amax = fmaxf(amax, fabsf(bf16_to_f(x[t * ldx + k])));
      }
      amax = block_max(amax, red);
      int e = 0;
      if (amax > 8.f) e = static_cast<int>(ceilf(log2f(amax * 0.125f)));
      if (threadIdx.x == 0) xscale[t] = exp2f(static_cast<float>(e));
      mul[t] = exp2f(static_cast<float>(-e));
      __syncthreads();
    }
  }
#pragma unroll
  for (int t = 0; t < T; ++t) {
    for (int k8 = threadIdx.x; k8 < k8n; k8 += blockDim.x) {
      const __nv_bfloat16* src = x + t * ldx + k8 * 8;
      __nv_bfloat162 b[4];
      if (t >= t_valid) {
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = __floats2bfloat162_rn(0.f, 0.f);
      } else if (aligned) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(src));
        b[0] = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
        b[1] = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
        b[2] = *reinterpret_cast<const __nv_bfloat162*>(&v.z);
        b[3] = *reinterpret_cast<const __nv_bfloat162*>(&v.w);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = __halves2bfloat162(src[2 * j], src[2 * j + 1]);
      }
      uint4 o;
      __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(b[j]);
        if (norm_w != nullptr) {
          const float2 w = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(norm_w + k8 * 8 + 2 * j));
          f = __bfloat1622float2(__floats2bfloat162_rn(f.x * nr[t] * w.x, f.y * nr[t] * w.y));
        }
        if constexpr (kPrescale) { f.x *= mul[t]; f.y *= mul[t]; }
        oh[j] = __float22half2_rn(f);
      }
      const int c = k8 >> 1;
      xs4[((t * iters + (c >> 5)) * 2 + (k8 & 1)) * 32 + (c & 31)] = o;
    }
  }
}

// ITERS = ceil(chunks per row / 32): every lane issues all of its 16-byte weight loads (and block
// scales) for a row before the first multiply, so a row costs one memory round trip, not ITERS.
// kSwiglu: W holds [gate rows (N) | up rows (N)]; the warp streams rows n and N + n and writes
// silu(min(g, limit)) * clamp(u, -limit, limit) — the shared-expert FC1 with its activation fused.
template <int T, bool kFp8, int ITERS, bool kSwiglu>
__global__ void __launch_bounds__(256)
skinny_linear_kernel(const uint8_t* __restrict__ W, long long ldw_bytes, const float* __restrict__ w_scale,
                     int w_scale_ld, const __nv_bfloat16* __restrict__ x, long long ldx, void* __restrict__ out,
                     long long ldo, int N, int K, int out_fp32, int rows_per_warp, int group_rows, float limit, int t_valid,
                     const SkinnyExtra ex) {
  extern __shared__ uint4 xs4[];
  constexpr int kVals = kFp8 ? 16 : 8;                  // values per 16-byte weight chunk
  const int n_chunks = K / kVals;
  const int iters16 = ((K / 16) + 31) / 32;             // x layout is always in 16-value chunks
  // grouped (block-diagonal) mode: all rows of this CTA belong to one group, whose activations start at g*K
  const int ksp = ex.k_split > 1 ? ex.k_split : 1;
  const int rblk = static_cast<int>(blockIdx.x) / ksp, kh = static_cast<int>(blockIdx.x) % ksp;
  const int c_per = (n_chunks + ksp - 1) / ksp;
  const int c_lo = kh * c_per, c_hi = min(n_chunks, c_lo + c_per);        // this CTA's 16-byte chunks of every row
  const int grp = group_rows > 0 ? (rblk * 8 * rows_per_warp) / group_rows : 0;
  __shared__ float s_xscale[kSkinnyMaxT];
  __shared__ float s_red[32];
  // Ahead of the previous kernel's completion: pull this CTA's weight rows (immutable) towards L2, one request per
  // 128-byte line, so that the row loop below starts on L2 hits while the activations are still being produced.
  {
    const int pw = threadIdx.x >> 5, pl = threadIdx.x & 31;
    const int pn0 = (rblk * 8 + pw) * rows_per_warp;
    const int row_bytes = kFp8 ? K : 2 * K;
    for (int pass = 0; pass < (kSwiglu ? 2 : 1); ++pass)
      for (int r = 0; r < rows_per_warp; ++r) {
        const int n = pn0 + r;
        if (n >= N) break;
        const uint8_t* wrow = W + static_cast<long long>(n + pass * N) * ldw_bytes;
        for (int b = pl * 128; b < row_bytes; b += 32 * 128) prefetch_l2(wrow + b);
      }
  }
  // ... and this warp's first row goes all the way into registers: weights are immutable, so the loads may be in
  // flight while the previous kernel finishes; the row loop then starts without a memory round trip.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (rblk * 8 + warp) * rows_per_warp;
  uint4 wv[ITERS];
  float sc[ITERS];
  auto load_row = [&](int wn) {
    const uint4* wrow = reinterpret_cast<const uint4*>(W + wn * ldw_bytes);
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int c = c_lo + it * 32 + lane;
      wv[it] = make_uint4(0, 0, 0, 0);
      sc[it] = 0.f;
      if (c < c_hi) {
        wv[it] = __ldg(wrow + c);
        if constexpr (kFp8) sc[it] = __ldg(w_scale + (wn >> 7) * w_scale_ld + (c >> 3));
      }
    }
  };
  constexpr bool kPreload = ITERS <= 8;
  if (kPreload && n0 < N) load_row(n0);
  pdl_wait();
  pdl_trigger();
  uint32_t ll_epoch = 0;
  if (ex.use_ll) ll_epoch = ll_push_epoch(ex.ll);
  skinny_fill_x<T, kFp8>(reinterpret_cast<__half*>(xs4), x + static_cast<long long>(grp) * K, ldx, K, iters16, s_xscale, s_red,
                         t_valid, ex.norm_w, ex.norm_eps);
  __syncthreads();
  float xsc[T];
#pragma unroll
  for (int t = 0; t < T; ++t) xsc[t] = kFp8 ? s_xscale[t] : 1.f;
  float prev[T];           // folded all-reduce: the even row's results wait for the odd row to share a word
#pragma unroll
  for (int t = 0; t < T; ++t) prev[t] = 0.f;
  for (int r = 0; r < rows_per_warp; ++r) {
    const int n = n0 + r;
    if (n >= N) break;
    float res[kSwiglu ? 2 : 1][T];
#pragma unroll
    for (int pass = 0; pass < (kSwiglu ? 2 : 1); ++pass) {
      const int wn = n + pass * N;                       // weight row (and scale row) of this pass
      if (!(kPreload && r == 0 && pass == 0)) load_row(wn);
      float acc[T];
#pragma unroll
      for (int t = 0; t < T; ++t) acc[t] = 0.f;
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        const int c = c_lo + it * 32 + lane;
        if (c < c_hi) {
          const uint32_t ww[4] = {wv[it].x, wv[it].y, wv[it].z, wv[it].w};
          if constexpr (kFp8) {
            // Sixteen raw e4m3 codes -> eight half2; the eight products per token are summed in packed fp16 (activations
            // are pre-scaled, see skinny_fill_x), widened once, and the 128x128 block scale is applied to that partial.
            __half2 w2[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __half2_raw h01 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(ww[j] & 0xffff), __NV_E4M3);
              const __half2_raw h23 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(ww[j] >> 16), __NV_E4M3);
              w2[2 * j] = *reinterpret_cast<const __half2*>(&h01);
              w2[2 * j + 1] = *reinterpret_cast<const __half2*>(&h23);
            }
#pragma unroll
            for (int t = 0; t < T; ++t) {
              const uint4 xa = xs4[((t * iters16 + (c >> 5)) * 2 + 0) * 32 + (c & 31)];
              const uint4 xb = xs4[((t * iters16 + (c >> 5)) * 2 + 1) * 32 + (c & 31)];
              const __half2* ha = reinterpret_cast<const __half2*>(&xa);
              const __half2* hb = reinterpret_cast<const __half2*>(&xb);
              __half2 p = __hmul2(w2[0], ha[0]);
              p = __hfma2(w2[1], ha[1], p);
              p = __hfma2(w2[2], ha[2], p);
              p = __hfma2(w2[3], ha[3], p);
              __half2 q = __hmul2(w2[4], hb[0]);
              q = __hfma2(w2[5], hb[1], q);
              q = __hfma2(w2[6], hb[2], q);
              q = __hfma2(w2[7], hb[3], q);
              const float2 pf = __half22float2(p), qf = __half22float2(q);
              acc[t] = fmaf(sc[it], (pf.x + pf.y) + (qf.x + qf.y), acc[t]);
            }
          } else {
            float wf[kVals];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&ww[j]);
              wf[2 * j] = __low2float(b);
              wf[2 * j + 1] = __high2float(b);
            }
#pragma unroll
            for (int t = 0; t < T; ++t) {
              // bf16 chunk c covers 8 values = half of 16-value chunk c/2
              const int c16 = c >> 1, it16 = c16 >> 5, lane16 = c16 & 31;
              const uint4 xv = xs4[((t * iters16 + it16) * 2 + (c & 1)) * 32 + lane16];
              const __half2* xh = reinterpret_cast<const __half2*>(&xv);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 xf = __half22float2(xh[j]);
                acc[t] = fmaf(wf[2 * j], xf.x, fmaf(wf[2 * j + 1], xf.y, acc[t]));
              }
            }
          }
        }
      }
#pragma unroll
      for (int t = 0; t < T; ++t) res[pass][t] = warp_sum(acc[t]) * xsc[t];
    }
#pragma unroll
    for (int t = 0; t < T; ++t) {
      float v = res[0][t];
      if constexpr (kSwiglu) {
        float g = v, u = res[1][t];
        if (limit > 0.f) {
          g = fminf(g, limit);
          u = fminf(fmaxf(u, -limit), limit);
        }
        v = g / (1.f + __expf(-g)) * u;
      }
      if (ex.use_ll) {
        // every lane holds the sums; rows n-1 and n share a word, lane p stores it to rank (rank + p) % world
        if ((n & 1) == 0 && n + 1 < N) {
          prev[t] = v;
        } else if (t < t_valid && lane < ex.ll.world) {
          const uint32_t d = (n & 1) ? pack_bf16x2(prev[t], v) : pack_bf16x2(v, 0.f);
          ll_store(ex.ll, ll_epoch, (ex.ll.rank + lane) % ex.ll.world, (static_cast<long long>(t) * N + (n & ~1)) >> 1, d);
        }
      } else if (lane == 0 && t < t_valid) {
        if (ksp > 1) atomicAdd(reinterpret_cast<float*>(out) + t * ldo + n, v);
        else if (out_fp32) reinterpret_cast<float*>(out)[t * ldo + n] = v;
        else reinterpret_cast<__nv_bfloat16*>(out)[t * ldo + n] = __float2bfloat16(v);
      }
    }
  }
  if (ex.use_ll && threadIdx.x == 0) ll_push_done(ex.ll, ll_epoch);
  if (ex.route) {
    // the CTA that finishes last has every logit in reach: it routes the tokens, one warp each
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const int done = atomicAdd(ex.route_counter, 1);
      s_last = done == static_cast<int>(gridDim.x) - 1;
      if (s_last) *ex.route_counter = 0;
    }
    __syncthreads();
    if (s_last) {
      __threadfence();
      for (int t = warp; t < t_valid; t += 8) route_token<true>(ex.router, reinterpret_cast<const float*>(out) + t * ldo, t, lane);
      if (ksp > 1) {
        // the halves add into `out`: leave it zero for the next call
        __syncthreads();
        for (int i = threadIdx.x; i < t_valid * N; i += blockDim.x) reinterpret_cast<float*>(out)[(i / N) * ldo + i % N] = 0.f;
      }
    }
  }
}

}  // namespace stk

#include "skinny_mma.cuh"

using namespace stk;

// T <= 8.  K must be a multiple of 16 (fp8) / 8 (bf16); rows 16-byte aligned.
// STK_SKINNY_MMA=0 keeps five to eight tokens on the CUDA-core kernel (A/B runs)
static bool stk_skinny_mma_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("STK_SKINNY_MMA");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

static int skinny_launch(const void* W, long long ldw, int is_fp8, const float* w_scale, int w_scale_ld,
                         const void* x, long long ldx, void* out, long long ldo, int T, int N, int K,
                         int out_fp32, int sm_count, int groups, int swiglu, float limit, const SkinnyExtra& ex,
                         void* stream) {
  if (T <= 0 || N <= 0) return 0;
  if (T > kSkinnyMaxT && !(T <= kSkinnyMmaMaxTokens && !ex.route && stk_skinny_mma_enabled())) return -1;
  if (K % 16 || K > 16384) return -1;
  const long long ldw_bytes = ldw * (is_fp8 ? 1 : 2);
  if (ldw_bytes % 16 || (reinterpret_cast<uintptr_t>(W) & 15)) return -2;
  // five to eight tokens: the eight-token warp-level tensor-core stream (skinny_mma.cuh)
  if (T > 4 && !ex.route && stk_skinny_mma_enabled())
    return skinny_mma_launch(W, ldw_bytes, is_fp8, w_scale, w_scale_ld, x, ldx, out, ldo, T, N, K, out_fp32, groups, swiglu,
                             limit, ex, (cudaStream_t)stream);
  const int iters16 = ((K / 16) + 31) / 32;
  const int t_inst = T <= 4 ? T : (T <= 6 ? 6 : 8);                // template instance that serves this batch
  const size_t smem = static_cast<size_t>(t_inst) * iters16 * 2 * 32 * 16;
  if (smem > 160 * 1024) return -6;
  // about four CTAs per SM; each warp takes `rpw` consecutive rows
  int rpw = ex.use_ll ? 2 : 1;                                      // the folded all-reduce packs two adjacent rows per word
  while ((N + 8 * rpw - 1) / (8 * rpw) > sm_count * 3 && rpw < 16) rpw *= 2;
  if ((ex.use_ll || ex.norm_w != nullptr || ex.route) && (groups > 1 || swiglu)) return -7;
  if (ex.use_ll && ((N & 1) || static_cast<long long>(T) * N / 2 > ex.ll.words)) return -8;
  if (ex.route && (!out_fp32 || N > 512 || N != ex.router.E || ex.route_counter == nullptr)) return -9;
  int group_rows = 0;
  if (groups > 1) {
    group_rows = N / groups;
    while (rpw > 1 && group_rows % (8 * rpw)) rpw /= 2;
    if (group_rows % (8 * rpw)) return -3;
  }
  const int ksp = ex.k_split > 1 ? 2 : 1;
  const int n_chunks = K / (is_fp8 ? 16 : 8);
  if (ksp > 1 && (!out_fp32 || !ex.route || (n_chunks / 2) % 32 || groups > 1 || swiglu)) return -10;
  const int grid = ((N + 8 * rpw - 1) / (8 * rpw)) * ksp;
  cudaStream_t st = (cudaStream_t)stream;
  const int iters = ((n_chunks + ksp - 1) / ksp + 31) / 32;
#define STK_SK3(T_, F_, I_, S_)                                                                                           \
  {                                                                                                                    \
    static bool configured = false;                                                                                    \
    if (!configured) {                                                                                                 \
      cudaFuncSetAttribute(skinny_linear_kernel<T_, F_, I_, S_>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); \
      configured = true;                                                                                               \
    }                                                                                                                  \
    launch_pdl(skinny_linear_kernel<T_, F_, I_, S_>, dim3(grid), dim3(256), smem, st, (const uint8_t*)W, ldw_bytes,     \
               w_scale, w_scale_ld, (const __nv_bfloat16*)x, ldx, out, ldo, N, K, out_fp32, rpw, group_rows, limit, T, ex); \
  }
#define STK_SK2(T_, F_)                                                                                 \
  {                                                                                                     \
    if (swiglu) {                                                                                       \
      if (iters <= 4) STK_SK3(T_, F_, 4, true)                                                          \
      else if (iters <= 8) STK_SK3(T_, F_, 8, true)                                                     \
      else if (iters <= 16) STK_SK3(T_, F_, 16, true)                                                   \
      else return -5;                                                                                   \
    } else {                                                                                            \
      if (iters <= 4) STK_SK3(T_, F_, 4, false)                                                         \
      else if (iters <= 8) STK_SK3(T_, F_, 8, false)                                                    \
      else if (iters <= 16) STK_SK3(T_, F_, 16, false)                                                  \
      else if (iters <= 32) STK_SK3(T_, F_, 32, false)                                                  \
      else return -5;                                                                                   \
    }                                                                                                   \
  }
  if (is_fp8) {
    switch (T) { case 1: STK_SK2(1, true) break; case 2: STK_SK2(2, true) break; case 3: STK_SK2(3, true) break; case 4: STK_SK2(4, true) break;
                 case 5: case 6: STK_SK2(6, true) break; default: STK_SK2(8, true) }
  } else {
    switch (T) { case 1: STK_SK2(1, false) break; case 2: STK_SK2(2, false) break; case 3: STK_SK2(3, false) break; case 4: STK_SK2(4, false) break;
                 case 5: case 6: STK_SK2(6, false) break; default: STK_SK2(8, false) }
  }
#undef STK_SK2
#undef STK_SK3
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_skinny_linear(const void* W, long long ldw, int is_fp8, const float* w_scale, int w_scale_ld,
                              const void* x, long long ldx, void* out, long long ldo, int T, int N, int K,
                              int out_fp32, int sm_count, int groups, int swiglu, float limit, void* stream) {
  SkinnyExtra ex;
  memset(&ex, 0, sizeof(ex));
  return skinny_launch(W, ldw, is_fp8, w_scale, w_scale_ld, x, ldx, out, ldo, T, N, K, out_fp32, sm_count, groups, swiglu,
                       limit, ex, stream);
}

// The same projection with its neighbours fused in (see the head of this file):
//   norm_w != nullptr   x is RMS-normalised (norm_w, norm_eps) on the way in;
//   ll_ctx != nullptr   the bf16 result goes into every rank's all-reduce slot (N even) and `out` is not written;
//   route != 0          `out` is fp32 gate logits [T, N = E]; the last CTA writes the experts and weights of every token
//                       (route_counter: one zero-initialised int that the kernel leaves at zero).  route == 2: K is
//                       split over two CTAs per row block that add into `out`, which must be zero on entry and is
//                       left zero (the logits are consumed by the routing inside the kernel).
STK_API int stk_skinny_linear_fused(const void* W, long long ldw, int is_fp8, const float* w_scale, int w_scale_ld,
                                    const void* x, long long ldx, void* out, long long ldo, int T, int N, int K,
                                    int out_fp32, int sm_count, const void* norm_w, float norm_eps, const void* ll_ctx,
                                    int route, int* route_counter, const float* bias, const int* tid2eid,
                                    const int64_t* token_ids, int vocab, int* ids, float* weights, int topk, int scoring,
                                    int renorm, float scaling, int* status, void* stream) {
  SkinnyExtra ex;
  memset(&ex, 0, sizeof(ex));
  ex.norm_w = (const __nv_bfloat16*)norm_w;
  ex.norm_eps = norm_eps;
  if (ll_ctx != nullptr) {
    memcpy(&ex.ll, ll_ctx, sizeof(ex.ll));
    ex.use_ll = 1;
  }
  if (route) {
    if (topk > 32) return -9;
    // a narrow projection (a few hundred rows) leaves most SMs idle: two CTAs per row block, half of K each
    const int n_chunks = K / (is_fp8 ? 16 : 8);
    ex.k_split = (route == 2 && (n_chunks / 2) % 32 == 0) ? 2 : 1;
    ex.route = 1;
    ex.route_counter = route_counter;
    ex.router = RouterArgs{bias, tid2eid, token_ids, vocab, ids, weights, N, topk, scoring, renorm, scaling, status};
  }
  return skinny_launch(W, ldw, is_fp8, w_scale, w_scale_ld, x, ldx, out, ldo, T, N, K, out_fp32, sm_count, 1, 0, 0.f, ex,
                       stream);
}
