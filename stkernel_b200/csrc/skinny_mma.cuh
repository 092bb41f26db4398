// Weight-streaming projection for 5..8 tokens (speculative verification rows, small decode batches).
//
// At these sizes the op is still a stream over the weight matrix (a few MB, once), but the CUDA-core dot products of
// the 1..4-token kernel pay tokens x the shared-memory reads and multiplies, and a tcgen05 tile pays its fixed costs
// (tensor maps, TMEM allocation, mbarrier pipeline, split-K workspace and reduction: ~10 us measured for a 6 MB
// weight).  Here the eight tokens are exactly the N=8 of a warp-level `mma.sync.m16n8k32` (e4m3) / `m16n8k16`
// (bf16): a CTA owns 16 weight rows, its eight warps split K, and every lane loads its part of the A fragment
// straight from global memory as 16-byte chunks -- no shared-memory staging of weights, no conversion of fp8 codes.
//
// K order: an mma is invariant under a permutation of K applied to both operands.  Within each 64-byte block of a
// row, lane (g = lane / 4, c = lane % 4) loads bytes [16c, 16c + 16) of rows g and g + 8; the four 32-bit words of
// that chunk are used as {a0, a2} of two consecutive mma steps (a1, a3 come from row g + 8), and the activation
// fragment reads the same bytes of token g's row in shared memory.  So every global load is a full 16 bytes and a
// row's 64-byte block is one contiguous request of four lanes.
//
// fp8: activations are quantised per (token, 128 values) exactly like the tensor-core GEMM path (scale = amax / 448)
// by the CTA itself in its prologue (optionally after the fused RMSNorm), each 64-byte block is accumulated on its
// own and folded into the fp32 result with w_scale x x_scale (two-level accumulation).
//
// Shares `SkinnyExtra` (norm prologue, folded all-reduce push) and the SwiGLU / grouped modes with skinny.cu, which
// includes this file.
#pragma once

namespace stk {

constexpr int kSmTokens = 8;          // token slots (the mma's N); rows beyond the batch are zeros
constexpr int kSmRows = 16;           // weight rows per CTA (the mma's M)
constexpr int kSmWarps = 8;
constexpr int kSmBatch = 8;           // 64-byte blocks per warp whose loads are in flight together
constexpr int kSkinnyMmaMaxTokens = 64;
constexpr long long kSkinnyMmaNarrowBytes = 4ll << 20;

__device__ __forceinline__ void mma_e4m3_16x8x32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_bf16_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Shared-memory layout (dynamic): activation rows [8][row_bytes + 64] (the pad spreads the eight rows over the banks),
// then fp8 only: x scales [8][K / 128] floats, then the cross-warp reduction buffer [8 warps][16][8] floats, then the
// staging area of the prologue (fp8: the raw bf16 rows [T][2K]; with the fused norm: its weights [2K bytes]).
template <bool kFp8, bool kSwiglu>
__global__ void __launch_bounds__(kSmWarps * 32, 2)
skinny_mma_kernel(const uint8_t* __restrict__ W, long long ldw_bytes, const float* __restrict__ w_scale, int w_scale_ld,
                  const __nv_bfloat16* __restrict__ x, long long ldx, void* __restrict__ out, long long ldo, int N, int K,
                  int out_fp32, int group_rows, float limit, int T_all, const SkinnyExtra ex) {
  extern __shared__ __align__(16) uint8_t sm_raw[];
  const int row_bytes = kFp8 ? K : 2 * K;
  const int xstride = row_bytes + 64;
  const int kgroups = K >> 7;
  uint8_t* xs = sm_raw;
  float* xsc = reinterpret_cast<float*>(sm_raw + kSmTokens * xstride);
  float* red = xsc + (kFp8 ? kSmTokens * kgroups : 0);
  __shared__ float s_nr[kSmTokens];
  __shared__ float s_ss[kSmWarps][kSmTokens];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int n0 = blockIdx.x * kSmRows;
  const int nblk = row_bytes >> 6;
  const int grp = group_rows > 0 ? n0 / group_rows : 0;
  // more than eight tokens (narrow weights only, see the launcher): blockIdx.y picks a group of eight
  const int t_base = blockIdx.y * kSmTokens;
  const int T = min(kSmTokens, T_all - t_base);
  const __nv_bfloat16* xg = x + static_cast<long long>(grp) * K + static_cast<long long>(t_base) * ldx;

  uint4 a_lo[kSmBatch], a_hi[kSmBatch];
  float wsc[kSmBatch];
  auto load_batch = [&](int wn, int b0) {
    const uint8_t* r_lo = W + static_cast<long long>(wn + g) * ldw_bytes + c * 16;
    const uint8_t* r_hi = r_lo + 8 * ldw_bytes;
#pragma unroll
    for (int i = 0; i < kSmBatch; ++i) {
      const int b = b0 + i * kSmWarps;
      if (b < nblk) {
        a_lo[i] = __ldg(reinterpret_cast<const uint4*>(r_lo + static_cast<long long>(b) * 64));
        a_hi[i] = __ldg(reinterpret_cast<const uint4*>(r_hi + static_cast<long long>(b) * 64));
        if constexpr (kFp8) wsc[i] = __ldg(w_scale + static_cast<long long>(wn >> 7) * w_scale_ld + (b >> 1));
      }
    }
  };
  // weights are immutable: the first batch is in flight while the kernel that produces x finishes
  load_batch(n0, warp);
  pdl_wait();
  pdl_trigger();
  uint32_t ll_epoch = 0;
  if (ex.use_ll) ll_epoch = ll_push_epoch(ex.ll);

  // ---- prologue: x -> shared memory (RMSNorm, quantisation, zero rows beyond the batch) ----
  // Every global byte the prologue needs (the T activation rows and, with the fused norm, its weight vector) is
  // requested at once with 16-byte asynchronous copies into shared memory: one memory round trip, whatever T and K.
  // x is T x (K / 8) chunks of eight bf16; thread `tid` takes chunks tid, tid + 256, ...; sixteen consecutive chunks =
  // one 128-value quantisation group = one half-warp.
  const int cpt = K >> 3;                              // chunks per token
  const int n_chunks = T * cpt;
  uint8_t* stage = reinterpret_cast<uint8_t*>(red + kSmWarps * kSmRows * kSmTokens);     // fp8: raw bf16 rows [T][2K]
  uint8_t* raw = kFp8 ? stage : xs;
  const int raw_stride = kFp8 ? 2 * K : xstride;
  uint8_t* nw_s = stage + (kFp8 ? T * 2 * K : 0);                                         // norm weights [2K bytes]
  for (int q = threadIdx.x; q < n_chunks; q += blockDim.x) {
    const int t = q / cpt, kc = q - t * cpt;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(raw + t * raw_stride + kc * 16)),
                 "l"(xg + t * ldx + kc * 8) : "memory");
  }
  if (ex.norm_w != nullptr)
    for (int kc = threadIdx.x; kc < cpt; kc += blockDim.x)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(nw_s + kc * 16)), "l"(ex.norm_w + kc * 8)
                   : "memory");
  asm volatile("cp.async.commit_group;" ::: "memory");
  // token slots beyond the batch: zeros (their results are never stored)
  {
    const int row16 = row_bytes >> 4;
    for (int idx = threadIdx.x; idx < (kSmTokens - T) * row16; idx += blockDim.x) {
      const int t = T + idx / row16, k16 = idx % row16;
      *reinterpret_cast<uint4*>(xs + t * xstride + k16 * 16) = make_uint4(0, 0, 0, 0);
    }
    if constexpr (kFp8)
      for (int idx = threadIdx.x; idx < (kSmTokens - T) * kgroups; idx += blockDim.x) xsc[T * kgroups + idx] = 0.f;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  if (ex.norm_w != nullptr) {
    float ss[kSmTokens];
#pragma unroll
    for (int t = 0; t < kSmTokens; ++t) ss[t] = 0.f;
    for (int q = threadIdx.x; q < n_chunks; q += blockDim.x) {
      const int t = q / cpt, kc = q - t * cpt;
      const uint4 v4 = *reinterpret_cast<const uint4*>(raw + t * raw_stride + kc * 16);
      const uint32_t* rp = reinterpret_cast<const uint32_t*>(&v4);
      float part = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 v = unpack_bf16x2(rp[j]);
        part = fmaf(v.x, v.x, fmaf(v.y, v.y, part));
      }
#pragma unroll
      for (int tt = 0; tt < kSmTokens; ++tt) ss[tt] += (tt == t) ? part : 0.f;
    }
#pragma unroll
    for (int t = 0; t < kSmTokens; ++t) {
      const float v = warp_sum(ss[t]);
      if (lane == 0) s_ss[warp][t] = v;
    }
    __syncthreads();
    if (threadIdx.x < kSmTokens) {
      float sum = 0.f;
      for (int w = 0; w < kSmWarps; ++w) sum += s_ss[w][threadIdx.x];
      s_nr[threadIdx.x] = rsqrtf(sum / static_cast<float>(K) + ex.norm_eps);
    }
    __syncthreads();
  }
  if (kFp8 || ex.norm_w != nullptr) {
    // n_chunks is a multiple of 16: a half-warp is either all inside or all outside
    for (int q0 = warp * 32; q0 < n_chunks; q0 += blockDim.x) {        // whole warps: the shuffles below are full-warp
      const int q = q0 + lane;
      const bool ok = q < n_chunks;
      const int t = ok ? q / cpt : 0, kc = ok ? q - t * cpt : 0;
      uint4 v4 = *reinterpret_cast<const uint4*>(raw + t * raw_stride + kc * 16);
      uint32_t* rp = reinterpret_cast<uint32_t*>(&v4);
      if (ex.norm_w != nullptr) {
        const uint4 w4 = *reinterpret_cast<const uint4*>(nw_s + kc * 16);
        const uint32_t* wp = reinterpret_cast<const uint32_t*>(&w4);
        const float nr = s_nr[t];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 a = unpack_bf16x2(rp[j]), w = unpack_bf16x2(wp[j]);
          rp[j] = pack_bf16x2(a.x * nr * w.x, a.y * nr * w.y);
        }
      }
      if constexpr (kFp8) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 a = unpack_bf16x2(rp[j]);
          v[2 * j] = a.x;
          v[2 * j + 1] = a.y;
        }
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
        // the sixteen lanes of a half-warp hold one group; the other half reduces its own
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float scale = fmaxf(amax, 1e-10f) * (1.f / 448.f);
        const float inv = 1.f / scale;
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          lo |= static_cast<uint32_t>(f_to_fp8(v[j] * inv)) << (8 * j);
          hi |= static_cast<uint32_t>(f_to_fp8(v[4 + j] * inv)) << (8 * j);
        }
        if (ok) {
          *reinterpret_cast<uint2*>(xs + t * xstride + kc * 8) = make_uint2(lo, hi);
          if ((lane & 15) == 0) xsc[t * kgroups + (kc >> 4)] = scale;
        }
      } else {
        if (ok) *reinterpret_cast<uint4*>(xs + t * xstride + kc * 16) = v4;
      }
    }
  }
  __syncthreads();

  // ---- the stream over this CTA's rows ----
  float res[kSwiglu ? 2 : 1] = {};
  const int r_out = threadIdx.x >> 3, t_out = threadIdx.x & 7;       // reduction mapping of threads 0..127
#pragma unroll
  for (int pass = 0; pass < (kSwiglu ? 2 : 1); ++pass) {
    const int wn = n0 + pass * N;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int b0 = warp; b0 < nblk; b0 += kSmBatch * kSmWarps) {
      if (!(pass == 0 && b0 == warp)) load_batch(wn, b0);
#pragma unroll
      for (int i = 0; i < kSmBatch; ++i) {
        const int b = b0 + i * kSmWarps;
        if (b < nblk) {
          const uint4 bx = *reinterpret_cast<const uint4*>(xs + g * xstride + b * 64 + c * 16);
          if constexpr (kFp8) {
            float tmp[4] = {0.f, 0.f, 0.f, 0.f};
            mma_e4m3_16x8x32(tmp, a_lo[i].x, a_hi[i].x, a_lo[i].y, a_hi[i].y, bx.x, bx.y);
            mma_e4m3_16x8x32(tmp, a_lo[i].z, a_hi[i].z, a_lo[i].w, a_hi[i].w, bx.z, bx.w);
            const int kg = b >> 1;
            const float ws = wsc[i];
            const float s0 = ws * xsc[(2 * c) * kgroups + kg], s1 = ws * xsc[(2 * c + 1) * kgroups + kg];
            acc[0] = fmaf(tmp[0], s0, acc[0]);
            acc[1] = fmaf(tmp[1], s1, acc[1]);
            acc[2] = fmaf(tmp[2], s0, acc[2]);
            acc[3] = fmaf(tmp[3], s1, acc[3]);
          } else {
            mma_bf16_16x8x16(acc, a_lo[i].x, a_hi[i].x, a_lo[i].y, a_hi[i].y, bx.x, bx.y);
            mma_bf16_16x8x16(acc, a_lo[i].z, a_hi[i].z, a_lo[i].w, a_hi[i].w, bx.z, bx.w);
          }
        }
      }
    }
    // rows g / g + 8, tokens 2c / 2c + 1 of this warp's K slice
    float* rw = red + warp * (kSmRows * kSmTokens);
    rw[g * kSmTokens + 2 * c] = acc[0];
    rw[g * kSmTokens + 2 * c + 1] = acc[1];
    rw[(g + 8) * kSmTokens + 2 * c] = acc[2];
    rw[(g + 8) * kSmTokens + 2 * c + 1] = acc[3];
    __syncthreads();
    if (threadIdx.x < kSmRows * kSmTokens) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kSmWarps; ++w) s += red[w * (kSmRows * kSmTokens) + threadIdx.x];
      res[pass] = s;
    }
    __syncthreads();
  }
  float v = res[0];
  if constexpr (kSwiglu) {
    float gt = v, up = res[1];
    if (limit > 0.f) {
      gt = fminf(gt, limit);
      up = fminf(fmaxf(up, -limit), limit);
    }
    v = gt / (1.f + __expf(-gt)) * up;
  }
  const int n = n0 + r_out;
  if (ex.use_ll) {
    // rows n and n + 1 share a word: the values meet in shared memory, then one thread per (row pair, token) stores
    // the word to every rank
    if (threadIdx.x < kSmRows * kSmTokens) red[threadIdx.x] = v;
    __syncthreads();
    if (threadIdx.x < (kSmRows / 2) * kSmTokens) {
      const int rp = threadIdx.x >> 3, t = threadIdx.x & 7;
      const int ne = n0 + 2 * rp;
      if (t < T && ne + 1 < N) {
        const uint32_t d = pack_bf16x2(red[(2 * rp) * kSmTokens + t], red[(2 * rp + 1) * kSmTokens + t]);
        const long long word = (static_cast<long long>(t_base + t) * N + ne) >> 1;
        for (int p = 0; p < ex.ll.world; ++p) ll_store(ex.ll, ll_epoch, (ex.ll.rank + p) % ex.ll.world, word, d);
      }
    }
    if (threadIdx.x == 0) ll_push_done(ex.ll, ll_epoch);
  } else if (threadIdx.x < kSmRows * kSmTokens && t_out < T && n < N) {
    const long long o = static_cast<long long>(t_base + t_out) * ldo + n;
    if (out_fp32) reinterpret_cast<float*>(out)[o] = v;
    else reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16(v);
  }
}

// Host side: called by skinny_launch for 5..8 tokens.  Returns -20.. for shapes outside this kernel.
static int skinny_mma_launch(const void* W, long long ldw_bytes, int is_fp8, const float* w_scale, int w_scale_ld,
                             const void* x, long long ldx, void* out, long long ldo, int T, int N, int K, int out_fp32,
                             int groups, int swiglu, float limit, const SkinnyExtra& ex, cudaStream_t st) {
  // up to 8 tokens for any weight; up to 64 for narrow bf16 weights (<= 4 MB: the router gate), where the matrix stays
  // in L2 while each group of eight tokens streams it again and a tensor-core tile would be mostly padding.  Not for
  // fp8 weights (every CTA would re-quantise the activations: measured slower than the tcgen05 tile) and not for
  // wider ones: their rows x token-groups grid fills every SM and, on the side stream, held back the persistent GEMMs
  // of the main chain (measured on one GPU at 64 tokens: +12 us on each of 37 fp8 projections per step)
  const long long w_bytes = static_cast<long long>(N) * (swiglu ? 2 : 1) * K * (is_fp8 ? 1 : 2);
  if (T < 1 || N % kSmRows || K % 128) return -20;
  if (T > kSmTokens && (is_fp8 || T > kSkinnyMmaMaxTokens || w_bytes > kSkinnyMmaNarrowBytes)) return -20;
  if ((ldx & 7) || (reinterpret_cast<uintptr_t>(x) & 15)) return -21;       // 16-byte loads of the activation rows
  if (ex.route || ex.k_split > 1) return -22;
  if (ex.norm_w != nullptr && (reinterpret_cast<uintptr_t>(ex.norm_w) & 15)) return -21;
  int group_rows = 0;
  if (groups > 1) {
    group_rows = N / groups;
    if (group_rows % kSmRows) return -23;
  }
  if (is_fp8 && (N % 128) && !swiglu) {
    // a CTA's 16 rows always share one 128-row scale block (16 divides 128); nothing to check
  }
  const int row_bytes = is_fp8 ? K : 2 * K;
  // activation rows + x scales + reduction buffer + staging (raw bf16 rows for the fp8 path, norm weights)
  const size_t smem = static_cast<size_t>(kSmTokens) * (row_bytes + 64) + (is_fp8 ? kSmTokens * (K / 128) * 4 : 0) +
                      kSmWarps * kSmRows * kSmTokens * 4 + (is_fp8 ? static_cast<size_t>(T < kSmTokens ? T : kSmTokens) * 2 * K : 0) +
                      (ex.norm_w != nullptr ? 2 * K : 0);
  if (smem > 200 * 1024) return -24;
  const dim3 grid(N / kSmRows, (T + kSmTokens - 1) / kSmTokens);
#define STK_SMMA(F_, S_)                                                                                              \
  {                                                                                                                   \
    static bool configured = false;                                                                                   \
    if (!configured) {                                                                                                \
      cudaFuncSetAttribute(skinny_mma_kernel<F_, S_>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);       \
      configured = true;                                                                                              \
    }                                                                                                                 \
    launch_pdl(skinny_mma_kernel<F_, S_>, grid, dim3(kSmWarps * 32), smem, st, (const uint8_t*)W, ldw_bytes,    \
               w_scale, w_scale_ld, (const __nv_bfloat16*)x, ldx, out, ldo, N, K, out_fp32, group_rows, limit, T, ex); \
  }
  if (is_fp8) {
    if (swiglu) STK_SMMA(true, true) else STK_SMMA(true, false)
  } else {
    if (swiglu) STK_SMMA(false, true) else STK_SMMA(false, false)
  }
#undef STK_SMMA
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace stk
