// Memory-bound glue kernels: embedding fan-out into hyper-connection streams, RMSNorm
// (single and the fused q/kv pair), per-token-group FP8 quantisation (optionally fused
// behind a norm), SwiGLU with clamp, MoE combine.
//
// Replaces the reference's RMSNorm / fused_q_kv_rmsnorm (overlay/attention.py:779-785),
// per_token_group_quant "armada" and SiluAndMulWithClamp (MEASUREMENTS.md:544-546).
#include <stdlib.h>

#define STK_PDL_CLASS 1      // bit of this file's kernels in the PDL mask (STK_PDL, stk_set_pdl_mask)
#include <string.h>

#include "common.cuh"
#include "symm.cuh"

namespace stk {

// out[t, j, :] = embed[ids[t], :] for j < hc.  Ids outside [0, vocab) write zeros and flag status.
__global__ void embed_hc_kernel(const int64_t* __restrict__ ids, const __nv_bfloat16* __restrict__ embed,
                                __nv_bfloat16* __restrict__ out, int H, int hc, int vocab, int vocab_start,
                                int vocab_end, int* status) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const long long id = ids[t];
  const bool in_vocab = id >= 0 && id < vocab;
  if (!in_vocab && threadIdx.x == 0) set_status(status, kBadIndex, t);
  const bool mine = in_vocab && id >= vocab_start && id < vocab_end;
  const uint4* src = reinterpret_cast<const uint4*>(embed + (mine ? (id - vocab_start) : 0) * static_cast<long long>(H));
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(t) * hc * H);
  const int n16 = H / 8;
  for (int i = threadIdx.x; i < n16; i += blockDim.x) {
    uint4 v = mine ? src[i] : make_uint4(0, 0, 0, 0);
    for (int j = 0; j < hc; ++j) dst[j * n16 + i] = v;
  }
}

// One CTA per row; grid.y selects one of up to two independent (x, w, out) problems.
struct NormJob {
  const __nv_bfloat16* x; long long ldx;
  const __nv_bfloat16* w;            // may be null (weightless)
  __nv_bfloat16* out; long long ldo;
  int H;
  uint8_t* q_out; long long ldq;     // optional fp8 copy of the normed row
  float* q_scale; int q_scale_ld;    // [H/128, q_scale_ld] token-contiguous
};

__global__ void rmsnorm_kernel(NormJob j0, NormJob j1, float eps) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float sbuf[];     // H floats + 32
  const NormJob& j = blockIdx.y == 0 ? j0 : j1;
  const int t = blockIdx.x;
  float* row = sbuf;
  float* red = sbuf + j.H;
  const __nv_bfloat16* x = j.x + t * j.ldx;
  float ss = 0.f;
  for (int i = threadIdx.x; i < j.H; i += blockDim.x) {
    const float v = bf16_to_f(x[i]);
    row[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / j.H + eps);
  for (int i = threadIdx.x; i < j.H; i += blockDim.x) {
    float v = row[i] * r;
    if (j.w) v *= bf16_to_f(j.w[i]);
    const __nv_bfloat16 b = __float2bfloat16(v);
    if (j.out) j.out[t * j.ldo + i] = b;
    row[i] = bf16_to_f(b);
  }
  if (j.q_out) {
    __syncthreads();
    // one warp per 128-wide group
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int g = warp; g * 128 < j.H; g += nw) {
      float v[4];
      float amax = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int i = g * 128 + lane * 4 + k;
        v[k] = i < j.H ? row[i] : 0.f;
        amax = fmaxf(amax, fabsf(v[k]));
      }
      amax = warp_max(amax);
      const float scale = fmaxf(amax, 1e-10f) * (1.f / 448.f);
      const float inv = 1.f / scale;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int i = g * 128 + lane * 4 + k;
        if (i < j.H) j.q_out[t * j.ldq + i] = f_to_fp8(v[k] * inv);
      }
      if (lane == 0) j.q_scale[static_cast<long long>(g) * j.q_scale_ld + t] = scale;
    }
  }
}

// x bf16 [T, K] -> fp8 [T, K] + scales [K/128, ld] (scale = amax/448); one warp per group.
__global__ void quant_fp8_group_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q,
                                       long long ldq, float* __restrict__ scales, int scale_ld, int T, int K) {
  pdl_wait();
  pdl_trigger();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int groups = (K + 127) / 128;
  if (warp >= T * groups) return;
  const int t = warp / groups, g = warp % groups;
  float v[4];
  float amax = 0.f;
  const int i0 = g * 128 + lane * 4;
  // four values per lane: one 8-byte load and one 4-byte store when the rows allow it
  const bool vec = (i0 + 3 < K) && ((ldx & 3) == 0) && ((ldq & 3) == 0) &&
                   ((reinterpret_cast<uintptr_t>(x) & 7) == 0) && ((reinterpret_cast<uintptr_t>(q) & 3) == 0);
  if (vec) {
    const uint2 raw = *reinterpret_cast<const uint2*>(x + t * ldx + i0);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
#pragma unroll
    for (int k = 0; k < 4; ++k) amax = fmaxf(amax, fabsf(v[k]));
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i = i0 + k;
      v[k] = i < K ? bf16_to_f(x[t * ldx + i]) : 0.f;
      amax = fmaxf(amax, fabsf(v[k]));
    }
  }
  amax = warp_max(amax);
  const float scale = fmaxf(amax, 1e-10f) * (1.f / 448.f);
  const float inv = 1.f / scale;
  if (vec) {
    uint32_t packed = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) packed |= static_cast<uint32_t>(f_to_fp8(v[k] * inv)) << (8 * k);
    *reinterpret_cast<uint32_t*>(q + t * ldq + i0) = packed;
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i = i0 + k;
      if (i < K) q[t * ldq + i] = f_to_fp8(v[k] * inv);
    }
  }
  if (lane == 0) scales[static_cast<long long>(g) * scale_ld + t] = scale;
}

// gu [T, 2I] (gate | up) -> act [T, I] = silu(min(g, lim)) * clamp(u, -lim, lim); optional fp8 copy.
__global__ void swiglu_clamp_kernel(const __nv_bfloat16* __restrict__ gu, long long ldg, __nv_bfloat16* __restrict__ act,
                                    long long lda, int I, float limit, uint8_t* q_out, long long ldq, float* q_scale,
                                    int q_scale_ld) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int g = warp; g * 128 < I; g += nw) {
    float v[4];
    float amax = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i = g * 128 + lane * 4 + k;
      float r = 0.f;
      if (i < I) {
        float a = bf16_to_f(gu[t * ldg + i]);
        float u = bf16_to_f(gu[t * ldg + I + i]);
        if (limit > 0.f) {
          a = fminf(a, limit);
          u = fminf(fmaxf(u, -limit), limit);
        }
        r = a / (1.f + __expf(-a)) * u;
        const __nv_bfloat16 b = __float2bfloat16(r);
        if (act) act[t * lda + i] = b;
        r = bf16_to_f(b);
      }
      v[k] = r;
      amax = fmaxf(amax, fabsf(r));
    }
    if (q_out) {
      amax = warp_max(amax);
      const float scale = fmaxf(amax, 1e-10f) * (1.f / 448.f);
      const float inv = 1.f / scale;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int i = g * 128 + lane * 4 + k;
        if (i < I) q_out[t * ldq + i] = f_to_fp8(v[k] * inv);
      }
      if (lane == 0) q_scale[static_cast<long long>(g) * q_scale_ld + t] = scale;
    }
  }
}

// The same sum for large batches: eight features per thread (16-byte loads; the 4-byte version reads the permuted
// expert outputs at a quarter of the HBM rate).  Same order of additions, so the results are identical.
__global__ void __launch_bounds__(128)
moe_combine_vec_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ w, const int* __restrict__ pair_row,
                       const __nv_bfloat16* __restrict__ shared, __nv_bfloat16* __restrict__ out, int H, int topk) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (i >= H) return;
  constexpr int kMaxK = 16;
  uint4 v[kMaxK];
  float wt[kMaxK];
#pragma unroll
  for (int j = 0; j < kMaxK; ++j) {
    v[j] = make_uint4(0, 0, 0, 0);
    wt[j] = 0.f;
    if (j < topk) {
      const int row = pair_row ? pair_row[t * topk + j] : t * topk + j;
      wt[j] = w[t * topk + j];
      if (row >= 0) v[j] = *reinterpret_cast<const uint4*>(y + static_cast<long long>(row) * H + i);
    }
  }
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < kMaxK; ++j) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[j]);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      acc[2 * q] = fmaf(wt[j], __low2float(h[q]), acc[2 * q]);
      acc[2 * q + 1] = fmaf(wt[j], __high2float(h[q]), acc[2 * q + 1]);
    }
  }
  if (shared) {
    const uint4 sv = *reinterpret_cast<const uint4*>(shared + static_cast<long long>(t) * H + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&sv);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      acc[2 * q] += __low2float(h[q]);
      acc[2 * q + 1] += __high2float(h[q]);
    }
  }
  uint4 o;
  __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int q = 0; q < 4; ++q) oh[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
  *reinterpret_cast<uint4*>(out + static_cast<long long>(t) * H + i) = o;
}

// out[t, :] = sum_j w[t, j] * y[pair(t, j), :] (+ shared[t, :]); fixed j order => deterministic.
// use_ll: this rank's sum is a partial over the expert-parallel ranks; instead of `out` it goes into every rank's
// all-reduce slot (symm.cuh, LLAr) and the consumer kernel adds the ranks.
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ w,
                                   const int* __restrict__ pair_row, const __nv_bfloat16* __restrict__ shared,
                                   __nv_bfloat16* __restrict__ out, int H, int topk, int use_ll, const LLAr ll) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 2;
  uint32_t epoch = 0;
  if (use_ll) {
    epoch = ll_push_epoch(ll);
    if (threadIdx.x == 0) ll_push_done(ll, epoch);      // counters[1] is read by the next kernel only
  }
  if (i >= H) return;
  constexpr int kMaxK = 16;
  int rows[kMaxK];
  float wt[kMaxK];
#pragma unroll
  for (int j = 0; j < kMaxK; ++j) {
    rows[j] = -1;
    wt[j] = 0.f;
    if (j < topk) {
      rows[j] = pair_row ? pair_row[t * topk + j] : t * topk + j;
      wt[j] = w[t * topk + j];
    }
  }
  __nv_bfloat162 v[kMaxK];
#pragma unroll
  for (int j = 0; j < kMaxK; ++j) {
    v[j] = __floats2bfloat162_rn(0.f, 0.f);
    if (rows[j] >= 0) v[j] = *reinterpret_cast<const __nv_bfloat162*>(y + static_cast<long long>(rows[j]) * H + i);
  }
  float a0 = 0.f, a1 = 0.f;
#pragma unroll
  for (int j = 0; j < kMaxK; ++j) {
    a0 = fmaf(wt[j], __low2float(v[j]), a0);
    a1 = fmaf(wt[j], __high2float(v[j]), a1);
  }
  if (shared) {
    const __nv_bfloat162 s = *reinterpret_cast<const __nv_bfloat162*>(shared + static_cast<long long>(t) * H + i);
    a0 += __low2float(s);
    a1 += __high2float(s);
  }
  if (use_ll) {
    const uint32_t d = pack_bf16x2(a0, a1);
    const long long word = (static_cast<long long>(t) * H + i) >> 1;
    for (int p = 0; p < ll.world; ++p) ll_store(ll, epoch, (ll.rank + p) % ll.world, word, d);
    return;
  }
  *reinterpret_cast<__nv_bfloat162*>(out + static_cast<long long>(t) * H + i) = __floats2bfloat162_rn(a0, a1);
}

}  // namespace stk

using namespace stk;

// Programmatic dependent launch of the decode-chain kernels: on unless STK_PDL=0 in the environment or switched off by
// stk_set_pdl(0).
static int g_pdl = -1;
STK_API int stk_pdl_enabled() {
  if (g_pdl < 0) {
    const char* e = getenv("STK_PDL");
    g_pdl = e != nullptr ? atoi(e) : 0xffff;      // STK_PDL=0: off; STK_PDL=<mask>: only those files' kernels
    if (e != nullptr && g_pdl == 1) g_pdl = 0xffff;
  }
  return g_pdl;
}
STK_API int stk_pdl_eager() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("STK_PDL_EAGER");
    v = (e != nullptr && e[0] == '1') ? 1 : 0;
  }
  return v;
}
STK_API int stk_set_pdl_mask(int mask) {
  g_pdl = mask;
  return 0;
}
STK_API int stk_set_pdl(int on) {
  g_pdl = on ? 0xffff : 0;
  return 0;
}


STK_API int stk_embed_hc(const int64_t* ids, const void* embed, void* out, int T, int H, int hc, int vocab,
                         int vocab_start, int vocab_end, int* status, void* stream) {
  if (T <= 0) return 0;
  if (H % 8) return -1;
  launch_pdl(embed_hc_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream, ids, (const __nv_bfloat16*)embed, (__nv_bfloat16*)out, H, hc,
                                                       vocab, vocab_start, vocab_end, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Up to two independent RMSNorm problems in one launch (the q / kv pair).  Pass H1 = 0 for one.
STK_API int stk_rmsnorm(const void* x0, long long ldx0, const void* w0, void* out0, long long ldo0, int H0,
                        void* q0, long long ldq0, float* qs0, int qs_ld0,
                        const void* x1, long long ldx1, const void* w1, void* out1, long long ldo1, int H1,
                        int T, float eps, void* stream) {
  if (T <= 0) return 0;
  NormJob a{(const __nv_bfloat16*)x0, ldx0, (const __nv_bfloat16*)w0, (__nv_bfloat16*)out0, ldo0, H0,
            (uint8_t*)q0, ldq0, qs0, qs_ld0};
  NormJob b{(const __nv_bfloat16*)x1, ldx1, (const __nv_bfloat16*)w1, (__nv_bfloat16*)out1, ldo1, H1,
            nullptr, 0, nullptr, 0};
  const int hmax = H0 > H1 ? H0 : H1;
  const size_t smem = (hmax + 32) * sizeof(float);
  if (smem > 200 * 1024) return -2;
  static bool configured = false;
  if (!configured && smem > 48 * 1024) {
    cudaFuncSetAttribute(rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    configured = true;
  }
  dim3 grid(T, H1 > 0 ? 2 : 1);
  launch_pdl(rmsnorm_kernel, dim3(grid), dim3(256), smem, (cudaStream_t)stream, a, b, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// out[t * ldo] = sum_k x[t, k]^2 (fp32); one CTA per row.
__global__ void __launch_bounds__(256)
row_sumsq_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, float* __restrict__ out, long long ldo, int K) {
  __shared__ float red[32];
  const int t = blockIdx.x;
  const uint4* row = reinterpret_cast<const uint4*>(x + t * ldx);
  float ss = 0.f;
  for (int i = threadIdx.x; i < K / 8; i += blockDim.x) {
    const uint4 v = __ldg(row + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      ss = fmaf(f.x, f.x, fmaf(f.y, f.y, ss));
    }
  }
  ss = stk::block_sum(ss, red);
  if (threadIdx.x == 0) out[t * ldo] = ss;
}

STK_API int stk_row_sumsq(const void* x, long long ldx, float* out, long long ldo, int T, int K, void* stream) {
  if (T <= 0) return 0;
  if (K % 8 || ldx % 8 || (reinterpret_cast<uintptr_t>(x) & 15)) return -1;
  row_sumsq_kernel<<<T, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, out, ldo, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_quant_fp8_group128(const void* x, long long ldx, void* q, long long ldq, float* scales, int scale_ld,
                                   int T, int K, void* stream) {
  if (T <= 0) return 0;
  const long long warps = static_cast<long long>(T) * ((K + 127) / 128);
  const int blocks = static_cast<int>((warps + 7) / 8);
  launch_pdl(quant_fp8_group_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq,
                                                                   scales, scale_ld, T, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_swiglu_clamp(const void* gu, long long ldg, void* act, long long lda, int T, int I, float limit,
                             void* q_out, long long ldq, float* q_scale, int q_scale_ld, void* stream) {
  if (T <= 0) return 0;
  launch_pdl(swiglu_clamp_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)gu, ldg, (__nv_bfloat16*)act, lda, I,
                                                           limit, (uint8_t*)q_out, ldq, q_scale, q_scale_ld);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_moe_combine(const void* y, const float* w, const int* pair_row, const void* shared, void* out, int T,
                            int H, int topk, const void* ll_ctx, void* stream) {
  if (T <= 0) return 0;
  if (H % 2 || topk > 16) return -1;
  LLAr ll;
  memset(&ll, 0, sizeof(ll));
  if (ll_ctx != nullptr) {
    memcpy(&ll, ll_ctx, sizeof(ll));
    if (static_cast<long long>(T) * H / 2 > ll.words) return -2;
  }
  if (ll_ctx == nullptr && T >= 64 && H % 8 == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (shared == nullptr || (reinterpret_cast<uintptr_t>(shared) & 15) == 0)) {
    launch_pdl(moe_combine_vec_kernel, dim3(T, (H / 8 + 127) / 128), dim3(128), 0, (cudaStream_t)stream,
               (const __nv_bfloat16*)y, w, pair_row, (const __nv_bfloat16*)shared, (__nv_bfloat16*)out, H, topk);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  dim3 grid(T, (H / 2 + 127) / 128);
  launch_pdl(moe_combine_kernel, dim3(grid), dim3(128), 0, (cudaStream_t)stream, (const __nv_bfloat16*)y, w, pair_row,
                                                          (const __nv_bfloat16*)shared, (__nv_bfloat16*)out, H, topk,
                                                          ll_ctx != nullptr ? 1 : 0, ll);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
