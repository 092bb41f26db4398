// Manifold hyper-connection kernels (4 residual streams):
//   mhc_dots      partial products  x_flat[t, :] . fn[j, :]  and  sum x^2   (split over hc*H)
//   mhc_finalize  rms, sigmoid pre/post mixes, Sinkhorn-normalised hc x hc combine matrix,
//                 weighted stream sum, fused RMSNorm -> layer input
//   mhc_post      out[j] = post[j]*x + sum_k comb[j,k]*res[k]
//   hc_head       collapse the streams with sigmoid weights
//
// Same math as the reference's prenorm GEMM + "big fuse" (overlay/mhc_tilelang.py:206-325)
// and its post mix (overlay/nvidia_model.py:1779-1785).  For large token counts the dot
// products can instead come from the tcgen05 GEMM (fn kept as a bf16 copy); `mhc_finalize`
// then takes them as a single pre-reduced split.
#define STK_PDL_CLASS 4      // bit of this file's kernels in the PDL mask (STK_PDL, stk_set_pdl_mask)
#include "common.cuh"

namespace stk {

constexpr int kMaxMix = 24;
constexpr int kTokBlock = 4;      // tokens sharing one pass over an fn slice

// grid (ceil(T/4), n_splits); partial [n_splits, T, n_mix + 1] (last entry = sum of squares)
template <int NMIX>
__global__ void __launch_bounds__(256)
mhc_dots_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ fn, float* __restrict__ partial, int T,
                int HC, int slice) {
  __shared__ float red[8][kTokBlock][NMIX + 1];
  const int t0 = blockIdx.x * kTokBlock;
  const int sp = blockIdx.y;
  const int k0 = sp * slice;
  const int k1 = min(HC, k0 + slice);
  float acc[kTokBlock][NMIX];
  float ss[kTokBlock];
#pragma unroll
  for (int i = 0; i < kTokBlock; ++i) {
    ss[i] = 0.f;
#pragma unroll
    for (int j = 0; j < NMIX; ++j) acc[i][j] = 0.f;
  }
  for (int k = k0 + threadIdx.x * 2; k < k1; k += blockDim.x * 2) {
    float xa[kTokBlock], xb[kTokBlock];
#pragma unroll
    for (int i = 0; i < kTokBlock; ++i) {
      if (t0 + i < T) {
        const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(x + static_cast<long long>(t0 + i) * HC + k);
        xa[i] = __low2float(v);
        xb[i] = __high2float(v);
      } else {
        xa[i] = xb[i] = 0.f;
      }
      ss[i] = fmaf(xa[i], xa[i], fmaf(xb[i], xb[i], ss[i]));
    }
#pragma unroll
    for (int j = 0; j < NMIX; ++j) {
      const float2 f = *reinterpret_cast<const float2*>(fn + static_cast<long long>(j) * HC + k);
#pragma unroll
      for (int i = 0; i < kTokBlock; ++i) acc[i][j] = fmaf(xa[i], f.x, fmaf(xb[i], f.y, acc[i][j]));
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int i = 0; i < kTokBlock; ++i) {
#pragma unroll
    for (int j = 0; j < NMIX; ++j) {
      const float v = warp_sum(acc[i][j]);
      if (lane == 0) red[warp][i][j] = v;
    }
    const float v = warp_sum(ss[i]);
    if (lane == 0) red[warp][i][NMIX] = v;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < kTokBlock * (NMIX + 1); idx += blockDim.x) {
    const int i = idx / (NMIX + 1), j = idx % (NMIX + 1);
    if (t0 + i >= T) continue;
    float s = 0.f;
    for (int w = 0; w < 8; ++w) s += red[w][i][j];
    partial[(static_cast<long long>(sp) * T + (t0 + i)) * (NMIX + 1) + j] = s;
  }
}

// One CTA (256 threads) per token.  partial: [n_splits, T, n_mix+1] fp32 when sumsq_in_partial,
// else dots only [n_splits, T, n_mix] and the kernel computes sum x^2 itself.
// mode 0: mHC pre (writes post [T,hc], comb [T,hc*hc], y [T,H] normed by norm_w)
// mode 1: hc_head (writes y [T,H] = sum_j w_j x_j, no norm)
__global__ void __launch_bounds__(256)
mhc_finalize_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ partial, int n_splits,
                    int partial_ld, int sumsq_in_partial, const float* __restrict__ base,
                    const float* __restrict__ scale, const __nv_bfloat16* __restrict__ norm_w, float* __restrict__ post,
                    float* __restrict__ comb, __nv_bfloat16* __restrict__ y, int T, int H, int hc, float rms_eps,
                    float hc_eps, int sinkhorn_iters, float post_mult, int mode, uint8_t* q_out, float* q_scale,
                    int q_scale_ld) {
  extern __shared__ float sm[];          // H floats (stream sum) + 64
  float* ybuf = sm;
  float* mixes = sm + H;                 // kMaxMix
  float* pre = mixes + kMaxMix;          // up to 8
  float* red = pre + 8;                  // 32
  const int t = blockIdx.x;
  const int n_mix = mode == 0 ? (2 + hc) * hc : hc;
  const long long HC = static_cast<long long>(hc) * H;
  const __nv_bfloat16* xt = x + t * HC;

  float ssq = 0.f;
  if (!sumsq_in_partial) {
    for (int k = threadIdx.x * 2; k < HC; k += blockDim.x * 2) {
      const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(xt + k);
      ssq = fmaf(__low2float(v), __low2float(v), fmaf(__high2float(v), __high2float(v), ssq));
    }
    ssq = block_sum(ssq, red);
  }
  if (threadIdx.x < 32) {
    if (threadIdx.x < n_mix) {
      float m = 0.f;
      for (int s = 0; s < n_splits; ++s) m += partial[(static_cast<long long>(s) * T + t) * partial_ld + threadIdx.x];
      mixes[threadIdx.x] = m;
    }
    if (sumsq_in_partial && threadIdx.x == 31) {
      float q = 0.f;
      for (int s = 0; s < n_splits; ++s) q += partial[(static_cast<long long>(s) * T + t) * partial_ld + n_mix];
      red[0] = q;
    }
  }
  __syncthreads();
  if (sumsq_in_partial) ssq = red[0];
  const float rms = rsqrtf(ssq / static_cast<float>(HC) + rms_eps);
  __syncthreads();

  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    if (mode == 0) {
      if (lane < hc) {
        pre[lane] = 1.f / (1.f + __expf(-(mixes[lane] * rms * scale[0] + base[lane]))) + hc_eps;
        post[t * hc + lane] = post_mult / (1.f + __expf(-(mixes[hc + lane] * rms * scale[1] + base[hc + lane])));
      }
      // Sinkhorn on an hc x hc matrix: lane = j*hc + k (hc <= 5 fits one warp)
      const int j = lane / hc, k = lane % hc;
      const bool act = lane < hc * hc;
      float c = act ? mixes[2 * hc + lane] * rms * scale[2] + base[2 * hc + lane] : -INFINITY;
      // row softmax
      float rmax = c;
      for (int o = 1; o < hc; ++o) {
        const float other = __shfl_sync(0xffffffffu, c, j * hc + ((k + o) % hc));
        if (act) rmax = fmaxf(rmax, other);
      }
      float e = act ? __expf(c - rmax) : 0.f;
      float rs = e;
      for (int o = 1; o < hc; ++o) {
        const float other = __shfl_sync(0xffffffffu, e, j * hc + ((k + o) % hc));
        if (act) rs += other;
      }
      c = act ? e / rs + hc_eps : 0.f;
      auto col_norm = [&]() {
        float cs = c;
        for (int o = 1; o < hc; ++o) {
          const float other = __shfl_sync(0xffffffffu, c, ((j + o) % hc) * hc + k);
          if (act) cs += other;
        }
        if (act) c = c / (cs + hc_eps);
      };
      auto row_norm = [&]() {
        float s = c;
        for (int o = 1; o < hc; ++o) {
          const float other = __shfl_sync(0xffffffffu, c, j * hc + ((k + o) % hc));
          if (act) s += other;
        }
        if (act) c = c / (s + hc_eps);
      };
      col_norm();
      for (int it = 0; it < sinkhorn_iters - 1; ++it) {
        row_norm();
        col_norm();
      }
      if (act) comb[t * hc * hc + lane] = c;
    } else {
      if (lane < hc) pre[lane] = 1.f / (1.f + __expf(-(mixes[lane] * rms * scale[0] + base[lane]))) + hc_eps;
    }
  }
  __syncthreads();

  // weighted stream sum (rounded to bf16 like the layer input the norm sees)
  float ss = 0.f;
  for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
    float a0 = 0.f, a1 = 0.f;
    for (int j = 0; j < hc; ++j) {
      const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(xt + static_cast<long long>(j) * H + i);
      a0 = fmaf(pre[j], __low2float(v), a0);
      a1 = fmaf(pre[j], __high2float(v), a1);
    }
    if (mode == 0) {
      a0 = bf16_to_f(__float2bfloat16(a0));
      a1 = bf16_to_f(__float2bfloat16(a1));
    }
    ybuf[i] = a0;
    ybuf[i + 1] = a1;
    ss = fmaf(a0, a0, fmaf(a1, a1, ss));
  }
  float r = 1.f;
  if (mode == 0 && norm_w != nullptr) {
    ss = block_sum(ss, red);
    r = rsqrtf(ss / H + rms_eps);
  }
  for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
    float a0 = ybuf[i] * r, a1 = ybuf[i + 1] * r;
    if (mode == 0 && norm_w != nullptr) {
      a0 *= bf16_to_f(norm_w[i]);
      a1 *= bf16_to_f(norm_w[i + 1]);
    }
    const __nv_bfloat162 o = __floats2bfloat162_rn(a0, a1);
    *reinterpret_cast<__nv_bfloat162*>(y + static_cast<long long>(t) * H + i) = o;
    ybuf[i] = __low2float(o);
    ybuf[i + 1] = __high2float(o);
  }
  if (q_out != nullptr) {
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int g = warp; g * 128 < H; g += 8) {
      float v[4];
      float amax = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int i = g * 128 + lane * 4 + k;
        v[k] = i < H ? ybuf[i] : 0.f;
        amax = fmaxf(amax, fabsf(v[k]));
      }
      amax = warp_max(amax);
      const float sc = fmaxf(amax, 1e-10f) * (1.f / 448.f);
      const float inv = 1.f / sc;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int i = g * 128 + lane * 4 + k;
        if (i < H) q_out[static_cast<long long>(t) * H + i] = f_to_fp8(v[k] * inv);
      }
      if (lane == 0) q_scale[static_cast<long long>(g) * q_scale_ld + t] = sc;
    }
  }
}

// out[t, j, :] = post[t, j] * x[t, :] + sum_k comb[t, j, k] * res[t, k, :]   (in place on res allowed
// only when out != res; the engine ping-pongs two residual buffers).
template <int HCM>
__global__ void __launch_bounds__(256)
mhc_post_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                const float* __restrict__ post, const float* __restrict__ comb, __nv_bfloat16* __restrict__ out, int H) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  __shared__ float sp[HCM], sc[HCM * HCM];
  if (threadIdx.x < HCM) sp[threadIdx.x] = post[t * HCM + threadIdx.x];
  if (threadIdx.x < HCM * HCM) sc[threadIdx.x] = comb[t * HCM * HCM + threadIdx.x];
  __syncthreads();
  const long long base = static_cast<long long>(t) * HCM * H;
  for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 2; i < H; i += gridDim.y * blockDim.x * 2) {
    const __nv_bfloat162 xv = *reinterpret_cast<const __nv_bfloat162*>(x + static_cast<long long>(t) * H + i);
    const float x0 = __low2float(xv), x1 = __high2float(xv);
    float r0[HCM], r1[HCM];
#pragma unroll
    for (int k = 0; k < HCM; ++k) {
      const __nv_bfloat162 rv = *reinterpret_cast<const __nv_bfloat162*>(res + base + static_cast<long long>(k) * H + i);
      r0[k] = __low2float(rv);
      r1[k] = __high2float(rv);
    }
#pragma unroll
    for (int j = 0; j < HCM; ++j) {
      float a0 = sp[j] * x0, a1 = sp[j] * x1;
#pragma unroll
      for (int k = 0; k < HCM; ++k) {
        a0 = fmaf(sc[j * HCM + k], r0[k], a0);
        a1 = fmaf(sc[j * HCM + k], r1[k], a1);
      }
      *reinterpret_cast<__nv_bfloat162*>(out + base + static_cast<long long>(j) * H + i) = __floats2bfloat162_rn(a0, a1);
    }
  }
}

}  // namespace stk

using namespace stk;

STK_API int stk_mhc_pick_splits(int T, int HC) {
  // enough CTAs to fill the machine at decode sizes, one slice >= 1024 elements
  int s = 1;
  const int tok_blocks = (T + kTokBlock - 1) / kTokBlock;
  while (tok_blocks * s < 148 && HC / (s * 2) >= 1024) s *= 2;
  return s;
}

// partial must hold n_splits * T * (n_mix + 1) floats.
STK_API int stk_mhc_dots(const void* x, const float* fn, float* partial, int T, int H, int hc, int n_mix,
                         int n_splits, void* stream) {
  if (T <= 0) return 0;
  const int HC = H * hc;
  if (HC % 2) return -1;
  int slice = (HC + n_splits - 1) / n_splits;
  slice = (slice + 1) & ~1;
  dim3 grid((T + kTokBlock - 1) / kTokBlock, n_splits);
  cudaStream_t st = (cudaStream_t)stream;
  if (n_mix == 24) mhc_dots_kernel<24><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, fn, partial, T, HC, slice);
  else if (n_mix == 4) mhc_dots_kernel<4><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, fn, partial, T, HC, slice);
  else if (n_mix == 8) mhc_dots_kernel<8><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, fn, partial, T, HC, slice);
  else if (n_mix == 2) mhc_dots_kernel<2><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, fn, partial, T, HC, slice);
  else return -2;
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_mhc_finalize(const void* x, const float* partial, int n_splits, int partial_ld, int sumsq_in_partial,
                             const float* base, const float* scale, const void* norm_w, float* post, float* comb,
                             void* y, int T, int H, int hc, float rms_eps, float hc_eps, int sinkhorn_iters,
                             float post_mult, int mode, void* q_out, float* q_scale, int q_scale_ld, void* stream) {
  if (T <= 0) return 0;
  if (hc * hc > 32 || (2 + hc) * hc > kMaxMix || H % 2) return -1;
  const size_t smem = (H + kMaxMix + 8 + 32) * sizeof(float);
  if (smem > 200 * 1024) return -2;
  static bool configured = false;
  if (!configured && smem > 48 * 1024) {
    cudaFuncSetAttribute(mhc_finalize_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    configured = true;
  }
  mhc_finalize_kernel<<<T, 256, smem, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, partial, n_splits, partial_ld, sumsq_in_partial, base, scale,
      (const __nv_bfloat16*)norm_w, post, comb, (__nv_bfloat16*)y, T, H, hc, rms_eps, hc_eps, sinkhorn_iters, post_mult,
      mode, (uint8_t*)q_out, q_scale, q_scale_ld);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_mhc_post(const void* x, const void* res, const float* post, const float* comb, void* out, int T, int H,
                         int hc, void* stream) {
  if (T <= 0) return 0;
  if (H % 2 || out == res) return -1;
  int gy = (H / 2 + 255) / 256;
  if (gy > 8) gy = 8;
  dim3 grid(T, gy);
  cudaStream_t st = (cudaStream_t)stream;
  if (hc == 4) launch_pdl(mhc_post_kernel<4>, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, post, comb, (__nv_bfloat16*)out, H);
  else if (hc == 2) launch_pdl(mhc_post_kernel<2>, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, post, comb, (__nv_bfloat16*)out, H);
  else return -2;
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// ---------------------------------------------------------------------------------------------
// Decode-sized batches: the whole mHC pre step (or hc_head) in ONE launch.  A thread-block cluster of
// 8 CTAs serves one token; the split dot products and both sums of squares are exchanged through
// distributed shared memory, so there is no partial buffer in global memory and no second kernel.
// ---------------------------------------------------------------------------------------------
#include <cooperative_groups.h>

namespace stk {
namespace cg = cooperative_groups;

constexpr int kClusterSize = 8;

constexpr int kClusterThreads = 512;
constexpr int kClusterWarps = kClusterThreads / 32;

// Fused post->pre: the residual streams this step reads are themselves the post-mix of the previous sub-block,
//   X'[j] = post_old[j] * fa + sum_k comb_old[j, k] * res_old[k]        (rounded to bf16, written to x_out),
// computed on the fly instead of by a separate launch.  fa == nullptr: the streams are read from `x` as given.
struct MhcFuse {
  const __nv_bfloat16* fa;        // [T, H] output of the previous attention / MoE sub-block
  const __nv_bfloat16* res_old;   // [T, hc, H]
  const float* post_old;          // [T, hc]
  const float* comb_old;          // [T, hc*hc]
  __nv_bfloat16* x_out;           // [T, hc, H]
};

template <int NMIX>
__global__ void __launch_bounds__(kClusterThreads)
mhc_cluster_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ fn, const float* __restrict__ base,
                   const float* __restrict__ scale, const __nv_bfloat16* __restrict__ norm_w, float* __restrict__ post,
                   float* __restrict__ comb, __nv_bfloat16* __restrict__ y, int H, int hc, float rms_eps, float hc_eps,
                   int sinkhorn_iters, float post_mult, int mode, uint8_t* q_out, float* q_scale, int q_scale_ld,
                   const MhcFuse fz) {
  cg::cluster_group cluster = cg::this_cluster();
  const int crank = static_cast<int>(cluster.block_rank());
  const int t = blockIdx.x / kClusterSize;
  __shared__ float part[NMIX + 1];          // this CTA's partial dots + sum x^2 (read by the peers)
  __shared__ float part2[1];                // this CTA's partial sum y^2
  __shared__ float red[kClusterWarps][NMIX + 1];
  __shared__ float mixes[NMIX + 1];
  __shared__ float pre[8];
  __shared__ float gmax[8];
  __shared__ float s_po[4], s_co[16];
  const int HC = H * hc;
  const bool fused = fz.fa != nullptr;
  // ahead of the previous kernel's completion: this CTA's slice of the (immutable) mix weights goes towards L2
  {
    const int pslice = ((HC / kClusterSize) + 1) & ~1;
    const int pk0 = crank * pslice, pk1 = min(HC, pk0 + pslice);
    for (int idx = threadIdx.x; idx < NMIX * ((pk1 - pk0 + 31) / 32); idx += blockDim.x) {
      const int j = idx % NMIX, c = idx / NMIX;
      prefetch_l2(fn + static_cast<long long>(j) * HC + pk0 + c * 32);
    }
  }
  pdl_wait();
  pdl_trigger();
  if (fused) {
    if (threadIdx.x < hc) s_po[threadIdx.x] = fz.post_old[t * hc + threadIdx.x];
    if (threadIdx.x < hc * hc) s_co[threadIdx.x] = fz.comb_old[t * hc * hc + threadIdx.x];
    __syncthreads();
  }
  const __nv_bfloat16* xt = fused ? nullptr : x + static_cast<long long>(t) * HC;
  const __nv_bfloat16* fat = fused ? fz.fa + static_cast<long long>(t) * H : nullptr;
  const __nv_bfloat16* rot = fused ? fz.res_old + static_cast<long long>(t) * HC : nullptr;
  const int slice = ((HC / kClusterSize) + 1) & ~1;
  const int k0 = crank * slice, k1 = min(HC, k0 + slice);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- phase 1: partial dot products over this CTA's slice ----
  float acc[NMIX];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NMIX; ++j) acc[j] = 0.f;
  // Four consecutive elements per thread: with 8 x 512 threads the whole [NMIX, HC] matrix is requested in one
  // round of 16-byte loads (the step is bounded by the latency of that single round, not by a loop of them).
  const bool vec4 = ((k0 | k1 | HC) & 3) == 0;
  if (vec4) {
    for (int k = k0 + threadIdx.x * 4; k < k1; k += blockDim.x * 4) {
      uint2 raw;
      if (fused) {
        const int j = k / H, h = k - j * H;
        const uint2 av = *reinterpret_cast<const uint2*>(fat + h);
        const __nv_bfloat162 a01 = *reinterpret_cast<const __nv_bfloat162*>(&av.x);
        const __nv_bfloat162 a23 = *reinterpret_cast<const __nv_bfloat162*>(&av.y);
        float v0 = s_po[j] * __low2float(a01), v1 = s_po[j] * __high2float(a01);
        float v2 = s_po[j] * __low2float(a23), v3 = s_po[j] * __high2float(a23);
        for (int kk = 0; kk < hc; ++kk) {
          const uint2 rv = *reinterpret_cast<const uint2*>(rot + static_cast<long long>(kk) * H + h);
          const __nv_bfloat162 r01 = *reinterpret_cast<const __nv_bfloat162*>(&rv.x);
          const __nv_bfloat162 r23 = *reinterpret_cast<const __nv_bfloat162*>(&rv.y);
          const float c = s_co[j * hc + kk];
          v0 = fmaf(c, __low2float(r01), v0); v1 = fmaf(c, __high2float(r01), v1);
          v2 = fmaf(c, __low2float(r23), v2); v3 = fmaf(c, __high2float(r23), v3);
        }
        const __nv_bfloat162 o01 = __floats2bfloat162_rn(v0, v1), o23 = __floats2bfloat162_rn(v2, v3);
        raw.x = *reinterpret_cast<const uint32_t*>(&o01);
        raw.y = *reinterpret_cast<const uint32_t*>(&o23);
        *reinterpret_cast<uint2*>(fz.x_out + static_cast<long long>(t) * HC + k) = raw;
      } else {
        raw = *reinterpret_cast<const uint2*>(xt + k);
      }
      const __nv_bfloat162 v0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
      const __nv_bfloat162 v1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
      const float x0 = __low2float(v0), x1 = __high2float(v0), x2 = __low2float(v1), x3 = __high2float(v1);
      ss = fmaf(x0, x0, fmaf(x1, x1, fmaf(x2, x2, fmaf(x3, x3, ss))));
      float4 f[NMIX];
#pragma unroll
      for (int j = 0; j < NMIX; ++j) f[j] = __ldg(reinterpret_cast<const float4*>(fn + static_cast<long long>(j) * HC + k));
#pragma unroll
      for (int j = 0; j < NMIX; ++j) acc[j] = fmaf(x0, f[j].x, fmaf(x1, f[j].y, fmaf(x2, f[j].z, fmaf(x3, f[j].w, acc[j]))));
    }
  } else if (!fused) {
    for (int k = k0 + threadIdx.x * 2; k < k1; k += blockDim.x * 2) {
      const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(xt + k);
      const float xa = __low2float(v), xb = __high2float(v);
      ss = fmaf(xa, xa, fmaf(xb, xb, ss));
#pragma unroll
      for (int j = 0; j < NMIX; ++j) {
        const float2 f = __ldg(reinterpret_cast<const float2*>(fn + static_cast<long long>(j) * HC + k));
        acc[j] = fmaf(xa, f.x, fmaf(xb, f.y, acc[j]));
      }
    }
  }
#pragma unroll
  for (int j = 0; j < NMIX; ++j) {
    const float v = warp_sum(acc[j]);
    if (lane == 0) red[warp][j] = v;
  }
  {
    const float v = warp_sum(ss);
    if (lane == 0) red[warp][NMIX] = v;
  }
  __syncthreads();
  if (threadIdx.x <= NMIX) {
    float s = 0.f;
    for (int w = 0; w < kClusterWarps; ++w) s += red[w][threadIdx.x];
    part[threadIdx.x] = s;
  }
  cluster.sync();
  if (threadIdx.x <= NMIX) {
    float s = 0.f;
    for (int r = 0; r < kClusterSize; ++r) s += cluster.map_shared_rank(part, r)[threadIdx.x];
    mixes[threadIdx.x] = s;
  }
  __syncthreads();
  const float rms = rsqrtf(mixes[NMIX] / static_cast<float>(HC) + rms_eps);

  // ---- phase 2: mixes -> pre / post / Sinkhorn combine (every CTA computes them; rank 0 stores) ----
  if (threadIdx.x < 32) {
    if (mode == 0) {
      if (lane < hc) {
        pre[lane] = 1.f / (1.f + __expf(-(mixes[lane] * rms * scale[0] + base[lane]))) + hc_eps;
        if (crank == 0) post[t * hc + lane] = post_mult / (1.f + __expf(-(mixes[hc + lane] * rms * scale[1] + base[hc + lane])));
      }
      const int j = lane / hc, k = lane % hc;
      const bool act = lane < hc * hc;
      float c = act ? mixes[2 * hc + lane] * rms * scale[2] + base[2 * hc + lane] : -INFINITY;
      float rmax = c;
      for (int o = 1; o < hc; ++o) {
        const float other = __shfl_sync(0xffffffffu, c, j * hc + ((k + o) % hc));
        if (act) rmax = fmaxf(rmax, other);
      }
      const float e = act ? __expf(c - rmax) : 0.f;
      float rs = e;
      for (int o = 1; o < hc; ++o) {
        const float other = __shfl_sync(0xffffffffu, e, j * hc + ((k + o) % hc));
        if (act) rs += other;
      }
      c = act ? e / rs + hc_eps : 0.f;
      // neighbour lanes of this matrix entry along its row and its column (fixed for the whole loop)
      int row_src[4], col_src[4];
#pragma unroll
      for (int o = 1; o < 4; ++o) {
        row_src[o] = j * hc + ((k + o) % hc);
        col_src[o] = ((j + o) % hc) * hc + k;
      }
      for (int it = 0; it < 2 * sinkhorn_iters - 1; ++it) {
        // even steps normalise columns, odd steps rows
        const bool col = (it & 1) == 0;
        float s = c;
        if (hc == 4) {
          const float a1 = __shfl_sync(0xffffffffu, c, col ? col_src[1] : row_src[1]);
          const float a2 = __shfl_sync(0xffffffffu, c, col ? col_src[2] : row_src[2]);
          const float a3 = __shfl_sync(0xffffffffu, c, col ? col_src[3] : row_src[3]);
          s = (c + a1) + (a2 + a3);
        } else {
          for (int o = 1; o < hc; ++o) {
            const int src = col ? ((j + o) % hc) * hc + k : j * hc + ((k + o) % hc);
            const float other = __shfl_sync(0xffffffffu, c, src);
            s += other;
          }
        }
        if (act) c = __fdividef(c, s + hc_eps);
      }
      if (act && crank == 0) comb[t * hc * hc + lane] = c;
    } else {
      if (lane < hc) pre[lane] = 1.f / (1.f + __expf(-(mixes[lane] * rms * scale[0] + base[lane]))) + hc_eps;
    }
  }
  __syncthreads();

  // ---- phase 3: weighted stream sum over this CTA's columns, cluster-wide RMSNorm ----
  const int cols = ((H / kClusterSize) + 1) & ~1;
  const int c0 = crank * cols, c1 = min(H, c0 + cols);
  constexpr int kMaxPer = 2;                           // column pairs per thread (H <= 8 * 512 * 2 * 2)
  float ya[kMaxPer], yb[kMaxPer];
  float ss2 = 0.f;
#pragma unroll
  for (int u = 0; u < kMaxPer; ++u) {
    const int i = c0 + (u * kClusterThreads + threadIdx.x) * 2;
    ya[u] = yb[u] = 0.f;
    if (i < c1) {
      float a0 = 0.f, a1 = 0.f;
      if (fused) {
        // recompute the (bf16-rounded) streams of these two columns from the previous sub-block's operands
        const __nv_bfloat162 av = *reinterpret_cast<const __nv_bfloat162*>(fat + i);
        float r0[4], r1[4];
        for (int kk = 0; kk < hc; ++kk) {
          const __nv_bfloat162 rv = *reinterpret_cast<const __nv_bfloat162*>(rot + static_cast<long long>(kk) * H + i);
          r0[kk] = __low2float(rv);
          r1[kk] = __high2float(rv);
        }
        for (int j = 0; j < hc; ++j) {
          float v0 = s_po[j] * __low2float(av), v1 = s_po[j] * __high2float(av);
          for (int kk = 0; kk < hc; ++kk) {
            v0 = fmaf(s_co[j * hc + kk], r0[kk], v0);
            v1 = fmaf(s_co[j * hc + kk], r1[kk], v1);
          }
          const __nv_bfloat162 o = __floats2bfloat162_rn(v0, v1);
          a0 = fmaf(pre[j], __low2float(o), a0);
          a1 = fmaf(pre[j], __high2float(o), a1);
        }
      } else {
      for (int j = 0; j < hc; ++j) {
        const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(xt + static_cast<long long>(j) * H + i);
        a0 = fmaf(pre[j], __low2float(v), a0);
        a1 = fmaf(pre[j], __high2float(v), a1);
      }
      }
      if (mode == 0) {
        a0 = bf16_to_f(__float2bfloat16(a0));
        a1 = bf16_to_f(__float2bfloat16(a1));
      }
      ya[u] = a0;
      yb[u] = a1;
      ss2 = fmaf(a0, a0, fmaf(a1, a1, ss2));
    }
  }
  float r = 1.f;
  const bool do_norm = mode == 0 && norm_w != nullptr;
  if (do_norm) {
    const float v = warp_sum(ss2);
    if (lane == 0) red[warp][0] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.f;
      for (int w = 0; w < kClusterWarps; ++w) s += red[w][0];
      part2[0] = s;
    }
    cluster.sync();
    float tot = 0.f;
    for (int rr = 0; rr < kClusterSize; ++rr) tot += cluster.map_shared_rank(part2, rr)[0];
    r = rsqrtf(tot / H + rms_eps);
  }
#pragma unroll
  for (int u = 0; u < kMaxPer; ++u) {
    const int i = c0 + (u * kClusterThreads + threadIdx.x) * 2;
    if (i < c1) {
      float a0 = ya[u] * r, a1 = yb[u] * r;
      if (do_norm) {
        a0 *= bf16_to_f(norm_w[i]);
        a1 *= bf16_to_f(norm_w[i + 1]);
      }
      const __nv_bfloat162 o = __floats2bfloat162_rn(a0, a1);
      *reinterpret_cast<__nv_bfloat162*>(y + static_cast<long long>(t) * H + i) = o;
      ya[u] = __low2float(o);
      yb[u] = __high2float(o);
    }
  }
  // keep this CTA's shared memory alive until every peer has read it
  cluster.sync();
  (void)q_out; (void)q_scale; (void)q_scale_ld; (void)gmax;
}

}  // namespace stk

static int mhc_cluster_launch(const void* x, const float* fn, const float* base, const float* scale, const void* norm_w,
                              float* post, float* comb, void* y, int T, int H, int hc, int n_mix, float rms_eps,
                              float hc_eps, int sinkhorn_iters, float post_mult, int mode, const MhcFuse& fz, void* stream) {
  if (T <= 0) return 0;
  if (fz.fa != nullptr && (hc > 4 || H % 4 || ((H * hc / kClusterSize + 1) & ~1) % 4)) return -3;
  if (hc * hc > 32 || H % 2 || H > kClusterSize * kClusterThreads * 2 * 2 || (H * hc) % 2) return -1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(T * kClusterSize);
  cfg.blockDim = dim3(kClusterThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kClusterSize;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_use((cudaStream_t)stream, STK_PDL_CLASS) ? 2 : 1;
  const __nv_bfloat16* xp = (const __nv_bfloat16*)x;
  const __nv_bfloat16* nw = (const __nv_bfloat16*)norm_w;
  __nv_bfloat16* yp = (__nv_bfloat16*)y;
  uint8_t* qn = nullptr;
  float* qs = nullptr;
  int qld = 0;
  cudaError_t e;
  if (n_mix == 24)
    e = cudaLaunchKernelEx(&cfg, mhc_cluster_kernel<24>, xp, fn, base, scale, nw, post, comb, yp, H, hc, rms_eps, hc_eps,
                           sinkhorn_iters, post_mult, mode, qn, qs, qld, fz);
  else if (n_mix == 4)
    e = cudaLaunchKernelEx(&cfg, mhc_cluster_kernel<4>, xp, fn, base, scale, nw, post, comb, yp, H, hc, rms_eps, hc_eps,
                           sinkhorn_iters, post_mult, mode, qn, qs, qld, fz);
  else if (n_mix == 8)
    e = cudaLaunchKernelEx(&cfg, mhc_cluster_kernel<8>, xp, fn, base, scale, nw, post, comb, yp, H, hc, rms_eps, hc_eps,
                           sinkhorn_iters, post_mult, mode, qn, qs, qld, fz);
  else
    return -2;
  return e == cudaSuccess ? 0 : -4;
}

STK_API int stk_mhc_cluster(const void* x, const float* fn, const float* base, const float* scale, const void* norm_w,
                            float* post, float* comb, void* y, int T, int H, int hc, int n_mix, float rms_eps,
                            float hc_eps, int sinkhorn_iters, float post_mult, int mode, void* stream) {
  MhcFuse fz = {nullptr, nullptr, nullptr, nullptr, nullptr};
  return mhc_cluster_launch(x, fn, base, scale, norm_w, post, comb, y, T, H, hc, n_mix, rms_eps, hc_eps, sinkhorn_iters,
                            post_mult, mode, fz, stream);
}

// Post-mix of the previous sub-block fused into this pre step: reads fa [T, H], res_old [T, hc, H], post_old, comb_old;
// writes the new residual streams to x_out and the usual pre outputs.
STK_API int stk_mhc_post_pre(const void* fa, const void* res_old, const float* post_old, const float* comb_old, void* x_out,
                             const float* fn, const float* base, const float* scale, const void* norm_w, float* post,
                             float* comb, void* y, int T, int H, int hc, int n_mix, float rms_eps, float hc_eps,
                             int sinkhorn_iters, float post_mult, int mode, void* stream) {
  MhcFuse fz = {(const __nv_bfloat16*)fa, (const __nv_bfloat16*)res_old, post_old, comb_old, (__nv_bfloat16*)x_out};
  if (fa == nullptr || res_old == nullptr || x_out == nullptr || x_out == res_old) return -1;
  return mhc_cluster_launch(nullptr, fn, base, scale, norm_w, post, comb, y, T, H, hc, n_mix, rms_eps, hc_eps,
                            sinkhorn_iters, post_mult, mode, fz, stream);
}
