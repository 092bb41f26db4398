// Grouped expert GEMM on the 5th-generation tensor cores, NVFP4 weights x fp16 activations (W4A16).
//
// Tokens arrive sorted by expert (`offsets[e]` .. `offsets[e+1]` are the rows of local expert e in the
// permuted activation matrix).  A persistent grid walks (expert, 128-row weight tile) pairs and, for
// each, the expert's token tiles:
//
//   TMA warp         activation tile [BT tokens x 64 k] fp16, 128-byte swizzle
//   dequant warps    sixteen warps, one thread per half weight row: 16 bytes of e2m1 codes + 2 e4m3
//                    group scales -> 32 fp16 values written straight into the swizzled K-major
//                    operand tile (a ring of six K blocks per thread is in flight in registers)
//   MMA warp         tcgen05.mma kind::f16 into TMEM (double-buffered accumulators)
//   epilogue warps   FC1: gate and up tiles sit side by side in TMEM, so one thread holds both values
//                    of an output and applies SwiGLU with clamp before storing fp16;
//                    FC2: scaled bf16 store.  Rows past the expert's last token are masked.
//
// e2m1 x e4m3 is exact in fp16, the per-matrix fp32 scale is applied in the epilogue.
// This is the engine's counterpart of the reference's fused W4A16 MoE kernel and, for the
// expert-parallel layout, of its mega-MoE grouped GEMM (overlay/nvidia_model.py:227-559).
#include <cuda_fp4.h>

#include "common.cuh"

namespace stk {

int make_tmap_2d(CUtensorMap* tm, const void* base, int elem_bytes, long long rows, long long cols, long long ld,
                 int box_rows);

struct MoeGArgs {
  const uint8_t* w;        // [E_l, rows, K/2]
  const uint8_t* s;        // [E_l, rows, K/16]
  const float* gscale;     // [E_l]
  const int* offsets;      // [E_l + 1]
  int e_local;
  int rows;                // weight rows per expert (2I for FC1, H for FC2)
  int n_out;               // output features per token (I for FC1, H for FC2)
  int K;
  void* out;               // FC1: fp16 [P, I]; FC2: bf16 [P, H]
  float limit;
  int* status;
  // Expert-parallel mode: rows of expert e are pushed into the activation matrix by peers (and by this
  // GPU's own dispatch); `arrived[e]` counts the rows that have landed.  nullptr = rows are already there.
  const uint32_t* arrived;
  uint32_t spin_budget;
};

template <int BT, bool kFc1>
struct MoeGCfg {
  static constexpr int kATiles = kFc1 ? 2 : 1;
  static constexpr int kStageBytes = kATiles * 128 * 128 + BT * 128;
  static constexpr int kStagesRaw = (200 * 1024) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 6 ? 6 : kStagesRaw;
  static constexpr int kAccCols = kATiles * BT;
  static constexpr int kTmemCols = (2 * kAccCols <= 32) ? 32 : (2 * kAccCols <= 64) ? 64 : (2 * kAccCols <= 128) ? 128
                                   : (2 * kAccCols <= 256) ? 256 : 512;
};

struct alignas(8) MoeGBars {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
};

// Half of a weight row's K block: 32 e2m1 codes (16 bytes) and their two e4m3 group scales.
struct RawRow {
  uint4 w;
  uint32_t sc;
};

__device__ __forceinline__ void load_raw(RawRow& r, const uint8_t* wrow, const uint8_t* srow, int kb, int half) {
  r.w = __ldg(reinterpret_cast<const uint4*>(wrow + kb * 32 + half * 16));
  r.sc = __ldg(reinterpret_cast<const uint16_t*>(srow + kb * 4 + half * 2));
}

// 32 values of one weight row -> 64 bytes of fp16 (chunks 4*half .. 4*half+3) in the swizzled tile row.
__device__ __forceinline__ void dequant_store(const RawRow& r, uint8_t* tile, int row, int half) {
  uint8_t* dst = tile + row * 128;
  const int sw = row & 7;
  const uint32_t words[4] = {r.w.x, r.w.y, r.w.z, r.w.w};
#pragma unroll
  for (int cc = 0; cc < 4; ++cc) {                  // 16-byte chunk = 8 values = one code word
    const int c = half * 4 + cc;
    const int g = cc >> 1;                          // 16-value scale group inside this half
    const __half_raw sraw = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>((r.sc >> (8 * g)) & 0xff), __NV_E4M3);
    const __half2 sc2 = __half2half2(*reinterpret_cast<const __half*>(&sraw));
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const __half2_raw hr = __nv_cvt_fp4x2_to_halfraw2(static_cast<__nv_fp4x2_storage_t>((words[cc] >> (8 * b)) & 0xff), __NV_E2M1);
      oh[b] = __hmul2(*reinterpret_cast<const __half2*>(&hr), sc2);
    }
    *reinterpret_cast<uint4*>(dst + ((c ^ sw) << 4)) = o;
  }
}

template <int BT, bool kFc1>
__global__ void __launch_bounds__(704, 1)
moe_grouped_kernel(const __grid_constant__ CUtensorMap tmX, const MoeGArgs a) {
  using Cfg = MoeGCfg<BT, kFc1>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kATiles = Cfg::kATiles;
  constexpr int CW = BT >= 32 ? 32 : 16;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;                                        // kStages x kATiles x 16 KB
  uint8_t* smem_b = smem + kStages * kATiles * 128 * 128;        // kStages x BT*128
  MoeGBars* bars = reinterpret_cast<MoeGBars*>(smem_b + kStages * BT * 128);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->full[s], 1 + 16);          // TMA arrive (+tx bytes) and sixteen dequant warps
      mbar_init(&bars->empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->tmem_full[i], 1);
      mbar_init(&bars->tmem_empty[i], 4);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, Cfg::kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) tma_prefetch_desc(&tmX);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  const int tiles_n = a.rows / (128 * kATiles);     // FC1: tiles over I; FC2: tiles over H
  const int pairs = a.e_local * tiles_n;
  const int k_blocks = a.K / 64;
  constexpr uint32_t kIdesc = umma_idesc(0u, 0u, 128, BT);       // fp16 x fp16 -> fp32

  if (warp == 0) {
    // ------------------------------ TMA producer (activations) ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int v = blockIdx.x; v < pairs && ok; v += gridDim.x) {
        const int e = v / tiles_n;
        const int r0 = a.offsets[e], cnt = a.offsets[e + 1] - r0;
        if (a.arrived != nullptr && cnt > 0) {
          // rows of this expert come over NVLink: start as soon as they are all here (bounded wait)
          bool here = false;
          for (uint32_t i = 0; i < a.spin_budget; ++i) {
            uint32_t got;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(got) : "l"(a.arrived + e) : "memory");
            if (got >= static_cast<uint32_t>(cnt)) { here = true; break; }
            if (i > 64) __nanosleep(64);
          }
          if (!here) { set_status(a.status, kTimeoutPeerFlag, 760); ok = false; break; }
          asm volatile("fence.proxy.async.global;" ::: "memory");      // peer stores (generic proxy) -> TMA reads
        }
        for (int tt = 0; tt * BT < cnt && ok; ++tt) {
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(&bars->empty[stage], phase ^ 1, a.status, 700 + stage)) { ok = false; break; }
            mbar_expect_tx(&bars->full[stage], BT * 128);
            tma_load_2d(smem_b + stage * BT * 128, &tmX, &bars->full[stage], kb * 64, r0 + tt * BT);
            if (++stage == kStages) { stage = 0; phase ^= 1; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int ab = 0;
      uint32_t aphase = 0;
      bool ok = true;
      for (int v = blockIdx.x; v < pairs && ok; v += gridDim.x) {
        const int e = v / tiles_n;
        const int cnt = a.offsets[e + 1] - a.offsets[e];
        for (int tt = 0; tt * BT < cnt && ok; ++tt) {
          if (!mbar_wait(&bars->tmem_empty[ab], aphase ^ 1, a.status, 710 + ab)) { ok = false; break; }
          tc_fence_after();
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(&bars->full[stage], phase, a.status, 720 + stage)) { ok = false; break; }
            tc_fence_after();
            const uint64_t bdesc = umma_desc_sw128(smem_u32(smem_b + stage * BT * 128));
#pragma unroll
            for (int at = 0; at < kATiles; ++at) {
              const uint64_t adesc = umma_desc_sw128(smem_u32(smem_a + (stage * kATiles + at) * 128 * 128));
              const uint32_t d = tmem_base + ab * Cfg::kAccCols + at * BT;
#pragma unroll
              for (int k = 0; k < 4; ++k) umma_f16(d, adesc + 2 * k, bdesc + 2 * k, kIdesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(&bars->empty[stage]);
            if (++stage == kStages) { stage = 0; phase ^= 1; }
          }
          if (ok) {
            umma_commit(&bars->tmem_full[ab]);
            if (++ab == 2) { ab = 0; aphase ^= 1; }
          }
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    int ab = 0;
    uint32_t aphase = 0;
    bool ok = true;
    for (int v = blockIdx.x; v < pairs && ok; v += gridDim.x) {
      const int e = v / tiles_n, tn = v % tiles_n;
      const int r0 = a.offsets[e], cnt = a.offsets[e + 1] - r0;
      const float gs = a.gscale[e];
      const int n = tn * 128 + row;                       // output feature of this thread
      for (int tt = 0; tt * BT < cnt && ok; ++tt) {
        if (!mbar_wait(&bars->tmem_full[ab], aphase, a.status, 730 + ab)) { ok = false; break; }
        tc_fence_after();
        const int valid = min(BT, cnt - tt * BT);
        const long long orow0 = static_cast<long long>(r0) + tt * BT;
#pragma unroll
        for (int c = 0; c < BT / CW; ++c) {
          uint32_t rg[32], ru[32];
          const uint32_t base = tmem_base + ab * Cfg::kAccCols + c * CW + lane_addr;
          if constexpr (CW == 32) {
            tmem_ld_32x32(base, rg);
            if constexpr (kFc1) tmem_ld_32x32(base + BT, ru);
          } else {
            uint32_t t16[16];
            tmem_ld_32x16(base, t16);
#pragma unroll
            for (int i = 0; i < 16; ++i) rg[i] = t16[i];
            if constexpr (kFc1) {
              tmem_ld_32x16(base + BT, t16);
#pragma unroll
              for (int i = 0; i < 16; ++i) ru[i] = t16[i];
            }
          }
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < CW; ++j) {
            const int col = c * CW + j;
            if (col < valid) {
              if constexpr (kFc1) {
                float g = __uint_as_float(rg[j]) * gs, u = __uint_as_float(ru[j]) * gs;
                if (a.limit > 0.f) {
                  g = fminf(g, a.limit);
                  u = fminf(fmaxf(u, -a.limit), a.limit);
                }
                reinterpret_cast<__half*>(a.out)[(orow0 + col) * a.n_out + n] = __float2half(g / (1.f + __expf(-g)) * u);
              } else {
                reinterpret_cast<__nv_bfloat16*>(a.out)[(orow0 + col) * a.n_out + n] = __float2bfloat16(__uint_as_float(rg[j]) * gs);
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->tmem_empty[ab]);
        if (++ab == 2) { ab = 0; aphase ^= 1; }
      }
    }
  } else {
    // ------------------------------ dequant producers (weights) ------------------------------
    // 512 threads: each owns half a row (32 values) of one or two operand tiles.  FC1 (two tiles):
    // thread -> (tile = pt / 256, row, half); FC2 (one tile): 256 threads per (row, half), the other
    // 256 take every second K block.
    const int pt = threadIdx.x - 192;                     // 0..511
    const int half = pt & 1;
    const int row = (pt >> 1) & 127;
    const int sel = pt >> 8;                              // FC1: which tile; FC2: which K-block parity
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    const long long wstride = a.K / 2, sstride = a.K / 16;
    for (int v = blockIdx.x; v < pairs && ok; v += gridDim.x) {
      const int e = v / tiles_n, tn = v % tiles_n;
      const int cnt = a.offsets[e + 1] - a.offsets[e];
      if (cnt <= 0) continue;
      const uint8_t* wexp = a.w + static_cast<long long>(e) * a.rows * wstride;
      const uint8_t* sexp = a.s + static_cast<long long>(e) * a.rows * sstride;
      const int at = kFc1 ? sel : 0;
      const long long rr = static_cast<long long>(at) * (a.rows / kATiles) + tn * 128 + row;
      const uint8_t* wrow = wexp + rr * wstride;
      const uint8_t* srow = sexp + rr * sstride;
      // K blocks this thread converts: FC1 all of them; FC2 those with kb % 2 == sel
      const int kb_first = kFc1 ? 0 : sel;
      const int kb_step = kFc1 ? 1 : 2;
      for (int tt = 0; tt * BT < cnt && ok; ++tt) {
        // a ring of kDepth raw K blocks is in flight in registers; a slot is refilled right after use
        constexpr int kDepth = 6;
        RawRow ring[kDepth];
#pragma unroll
        for (int d = 0; d < kDepth; ++d) {
          const int kb = kb_first + d * kb_step;
          if (kb < k_blocks) load_raw(ring[d], wrow, srow, kb, half);
        }
        for (int kb0 = 0; kb0 < k_blocks && ok; kb0 += kDepth * kb_step) {
#pragma unroll
          for (int d = 0; d < kDepth; ++d) {
#pragma unroll
            for (int sub = 0; sub < (kFc1 ? 1 : 2); ++sub) {
              // every thread visits every K block (to arrive on its barrier); it converts only its own
              const int kb = kb0 + d * kb_step + sub;
              if (kb < k_blocks && ok) {
                const bool mine = kFc1 || ((kb & 1) == sel);
                if (!mbar_wait(&bars->empty[stage], phase ^ 1, a.status, 740 + stage)) {
                  ok = false;
                } else {
                  if (mine) dequant_store(ring[d], smem_a + (stage * kATiles + at) * 128 * 128, row, half);
                  fence_proxy_async();
                  __syncwarp();
                  if (lane == 0) mbar_arrive(&bars->full[stage]);
                  if (mine && kb + kDepth * kb_step < k_blocks) load_raw(ring[d], wrow, srow, kb + kDepth * kb_step, half);
                  if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
              }
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// sorted row q <- activations of token sorted[q] / topk, converted to fp16.
__global__ void moe_permute_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ sorted,
                                   const int* __restrict__ offsets, int e_local, int topk, __half* __restrict__ xs, int H) {
  const int q = blockIdx.x;
  if (q >= offsets[e_local]) return;
  const int t = sorted[q] / topk;
  const uint4* src = reinterpret_cast<const uint4*>(x + t * ldx);
  uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<long long>(q) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    const uint4 v = __ldg(src + i);
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) oh[j] = __float22half2_rn(__bfloat1622float2(b[j]));
    dst[i] = o;
  }
}

template <int BT, bool kFc1>
static int launch_moe_grouped(const CUtensorMap& tx, const MoeGArgs& a, int grid, cudaStream_t st) {
  using Cfg = MoeGCfg<BT, kFc1>;
  const int smem = Cfg::kStages * Cfg::kStageBytes + static_cast<int>(sizeof(MoeGBars)) + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(moe_grouped_kernel<BT, kFc1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return -3;
    configured = true;
  }
  moe_grouped_kernel<BT, kFc1><<<grid, 704, smem, st>>>(tx, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace stk

using namespace stk;

STK_API int stk_moe_permute(const void* x, long long ldx, const int* sorted, const int* offsets, int e_local, int topk,
                            void* xs, int max_rows, int H, void* stream) {
  if (max_rows <= 0) return 0;
  if (H % 8 || (ldx % 8)) return -1;
  moe_permute_kernel<<<max_rows, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, sorted, offsets, e_local, topk,
                                                               (__half*)xs, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// xs: fp16 [xs_rows, K] sorted activations (xs_rows >= total rows + bt, tail readable).
// fc1 = 1: w rows = 2*n_out (gate rows then up rows), out fp16 [P, n_out] = swiglu;  fc1 = 0: w rows = n_out, out bf16.
static int moe_grouped_launch(const void* xs, long long xs_rows, const void* w, const void* s, const float* gscale,
                              const int* offsets, int e_local, int n_out, int K, void* out, int fc1, float limit, int bt,
                              int* status, int sm_count, const uint32_t* arrived, uint32_t spin_budget, void* stream) {
  if (e_local <= 0) return 0;
  if (K % 64 || n_out % 128 || (bt != 16 && bt != 32 && bt != 64 && bt != 128)) return -1;
  CUtensorMap tx;
  if (make_tmap_2d(&tx, xs, 2, xs_rows, K, K, bt) != 0) return -2;
  MoeGArgs a;
  a.w = (const uint8_t*)w; a.s = (const uint8_t*)s; a.gscale = gscale; a.offsets = offsets; a.e_local = e_local;
  a.rows = fc1 ? 2 * n_out : n_out; a.n_out = n_out; a.K = K; a.out = out; a.limit = limit; a.status = status;
  a.arrived = arrived; a.spin_budget = spin_budget;
  const int pairs = e_local * (n_out / 128);
  const int grid = pairs < sm_count ? pairs : sm_count;
  cudaStream_t st = (cudaStream_t)stream;
#define STK_MG(BT_) (fc1 ? launch_moe_grouped<BT_, true>(tx, a, grid, st) : launch_moe_grouped<BT_, false>(tx, a, grid, st))
  switch (bt) {
    case 16: return STK_MG(16);
    case 32: return STK_MG(32);
    case 64: return STK_MG(64);
    default: return STK_MG(128);
  }
#undef STK_MG
}

STK_API int stk_moe_grouped(const void* xs, long long xs_rows, const void* w, const void* s, const float* gscale,
                            const int* offsets, int e_local, int n_out, int K, void* out, int fc1, float limit, int bt,
                            int* status, int sm_count, void* stream) {
  return moe_grouped_launch(xs, xs_rows, w, s, gscale, offsets, e_local, n_out, K, out, fc1, limit, bt, status, sm_count,
                            nullptr, 0u, stream);
}

// Expert-parallel FC1: the activation rows of local expert e are complete once arrived[e] reaches the expert's row
// count; the producer warp waits for that per expert, so tiles of early experts run while later rows are in flight.
STK_API int stk_moe_grouped_ep(const void* xs, long long xs_rows, const void* w, const void* s, const float* gscale,
                               const int* offsets, int e_local, int n_out, int K, void* out, int fc1, float limit, int bt,
                               int* status, int sm_count, const void* arrived, int spin_budget, void* stream) {
  return moe_grouped_launch(xs, xs_rows, w, s, gscale, offsets, e_local, n_out, K, out, fc1, limit, bt, status, sm_count,
                            (const uint32_t*)arrived, static_cast<uint32_t>(spin_budget), stream);
}
