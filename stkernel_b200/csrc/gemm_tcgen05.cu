// Dense linear layer on the 5th-generation tensor cores:  out[T, N] = X[T, K] * W[N, K]^T
//
// * Operands arrive by TMA (128-byte swizzle) into a multi-stage shared-memory ring.
// * One elected thread issues tcgen05.mma; the accumulator lives in TMEM (double buffered).
// * The weight tile is the 128-row "M" operand and the token tile is the "N" operand
//   (16..256 tokens), so decode-sized batches still use full-height MMAs and each epilogue
//   thread owns one output feature, which makes the global stores contiguous across a warp.
// * bf16 operands: one accumulation over all of K, epilogue once per tile.
// * fp8 e4m3 operands with 128x128 weight scales and 1x128 activation scales: one TMEM
//   accumulation per 128-wide K block; the epilogue warps fold `w_scale * x_scale` into
//   fp32 register accumulators while the next block's MMAs run (two-level accumulation).
// * Split-K for skinny problems: partial tiles go to an fp32 workspace, the last CTA to
//   finish a tile sums the partials in split order (deterministic) and writes the output.
// * Persistent grid: one CTA per SM walks the (split, token-tile, feature-tile) list.
//
// Covers the reference's DeepGEMM fp8_gemm_nt call sites (overlay/dspark_v2.py:92-107,
// probes/oproj_prof.py:65-71) and its bf16 cuBLAS projections.
#include <string.h>

#define STK_PDL_CLASS 8      // bit of this file's kernels in the PDL mask (STK_PDL, stk_set_pdl_mask)
#include <stdlib.h>

#include "common.cuh"
#include "stk_c_api.h"
#include "symm.cuh"

namespace stk {

struct GemmArgs {
  int T, N;
  int k_blocks;          // K extent in 128-byte blocks
  int splits;            // split-K factor (>= 1)
  int tiles_n, tiles_t;
  void* out;             // [T, ldo]
  long long ldo;
  int out_fp32;
  const float* w_scale;  // fp8 only: [ceil(N/128), w_scale_ld]
  int w_scale_ld;
  const float* x_scale;  // fp8 only: [k_blocks, x_scale_ld]  (token index contiguous)
  int x_scale_ld;
  float* workspace;      // split-K partials [splits, T, N]
  int* counters;         // one per output tile; zero on entry, zero again on exit
  int* status;
  // Grouped mode (block-diagonal weights, e.g. the per-o-group low-rank projection): feature tile
  // `tn` belongs to group tn / group_tiles and reads X columns starting at group * group_k_elems.
  int group_tiles;       // 0 = plain GEMM
  int group_k_elems;
  // Fused all-reduce (row-parallel layers): every rank pushes its partial output tile into all
  // peers' slots as soon as the tile's accumulation ends, then sums the tiles it received in
  // rank order.  The transfer of tile i overlaps the MMAs of tile i+1 of the same CTA and of
  // all other CTAs.
  int ar_enabled;
  SymmCtx ar;
  // Arrival-gated activations (all-gather -> GEMM): X is the gathered matrix in this rank's symmetric region,
  // rows [s * gate_rows, (s+1) * gate_rows) are pushed by rank s and are complete once flag (kAgKind, 0, s)
  // carries the current epoch.  Token tiles are visited starting with this rank's own shard.
  int gate_enabled;
  int gate_rows;
  // Token-major mode (fp8, T >= 128): the operands swap roles -- TMEM lanes are tokens, columns are weight rows -- so
  // the activation scale of a K block is one value per thread and the weight scale one value per tile: the per-block
  // rescale is a single multiplier per thread instead of one per accumulator column.  T/N/tiles_* then describe the
  // swapped problem (a.N = tokens, a.T = weight rows); out is still [tokens, ldo].
  int token_major;
  // Whether the split-K reduction may write `out` with 16-byte (fp32) / 4-byte (bf16) vector stores: the host sets
  // it from the alignment of `out` and `ldo`; otherwise the reduction writes element by element.
  int out_vec_ok;
};

constexpr int kArKind = 3;
constexpr int kGateKind = 4;      // flags written by the all-gather push kernel (symm.cu)

template <int BT>
struct GemmCfg {
  static constexpr int kStageBytes = 128 * 128 + BT * 128;
  // bf16 staging tile [BT][128] for the fused all-reduce epilogue (token tiles up to 128)
  static constexpr int kArTileBytes = BT <= 128 ? BT * 256 : 0;
  static constexpr int kStagesRaw = (196 * 1024) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kTmemCols = (2 * BT <= 32) ? 32 : (2 * BT <= 64) ? 64 : (2 * BT <= 128) ? 128 : (2 * BT <= 256) ? 256 : 512;
  static constexpr int kChunk = BT >= 32 ? 32 : 16;
};

struct alignas(8) GemmBarriers {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int last_flag;
};

template <int CW>
__device__ __forceinline__ void tmem_ld_chunk(uint32_t taddr, uint32_t (&r)[32]) {
  if constexpr (CW == 32) {
    tmem_ld_32x32(taddr, r);
  } else {
    uint32_t t[16];
    tmem_ld_32x16(taddr, t);
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = t[i];
  }
}

__device__ __forceinline__ void epi_bar_sync(int nthreads) {
  asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}

template <int BT, bool kFp8>
__global__ void __launch_bounds__(kFp8 ? 320 : 192, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const GemmArgs a) {
  using Cfg = GemmCfg<BT>;
  constexpr int kStages = Cfg::kStages;
  constexpr int CW = Cfg::kChunk;
  // epilogue warps: fp8 with wide tiles splits the columns over two warps per lane quarter
  constexpr int kEpiWarps = (kFp8 && BT >= 64) ? 8 : 4;
  constexpr int kColsPerWarp = (kEpiWarps == 8) ? BT / 2 : BT;
  constexpr int kChunksPerWarp = kColsPerWarp / CW;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;                                  // kStages x 16 KB
  uint8_t* smem_b = smem + kStages * 128 * 128;            // kStages x BT*128
  GemmBarriers* bars = reinterpret_cast<GemmBarriers*>(smem_b + kStages * BT * 128);
  __nv_bfloat16* ar_tile = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uint8_t*>(bars) + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->tmem_full[i], 1);
      mbar_init(&bars->tmem_empty[i], kEpiWarps);
    }
    bars->last_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, Cfg::kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  // Launched with programmatic serialization (plain GEMMs only): barriers, TMEM and descriptors are set up and the
  // first weight tiles of this CTA are on their way to L2 while the previous kernel finishes; activations, split-K
  // counters and epochs are touched only after the wait.
  if (warp == 0 && lane == 0 && !a.token_major && static_cast<int>(blockIdx.x) < a.splits * a.tiles_t * a.tiles_n) {
    const int u = blockIdx.x;
    const int tn = u % a.tiles_n;
    const int sp = u / (a.tiles_n * a.tiles_t);
    const int kbs = (a.k_blocks + a.splits - 1) / a.splits;
    const int kb0 = sp * kbs;
    const int kb1 = min(a.k_blocks, min(kb0 + kbs, kb0 + 8));
    for (int kb = kb0; kb < kb1; ++kb) tma_prefetch_2d(&tmW, kb * (kFp8 ? 128 : 64), tn * 128);
  }
  pdl_wait();
  pdl_trigger();
  uint32_t ar_epoch = 0;
  if (a.ar_enabled) ar_epoch = *epoch_ptr(a.ar, kArKind, 0) + 1;   // bumped only after every CTA has finished

  uint32_t gate_epoch = 0;
  int tt_rot = 0;
  if (a.gate_enabled) {
    gate_epoch = *epoch_ptr(a.ar, kGateKind, 0);                   // the push of this call has already run on this rank
    tt_rot = (a.ar.rank * a.gate_rows) / BT;
  }
  const int units = a.splits * a.tiles_t * a.tiles_n;
  const int kb_per_split = (a.k_blocks + a.splits - 1) / a.splits;
  constexpr uint32_t kIdesc = umma_idesc(kFp8 ? 0u : 1u, kFp8 ? 0u : 1u, 128, BT);
  constexpr uint32_t kTxBytes = 128 * 128 + BT * 128;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int issued = 0;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
        const int tn = u % a.tiles_n;
        const int tt = ((u / a.tiles_n) % a.tiles_t + tt_rot) % a.tiles_t;
        const int sp = u / (a.tiles_n * a.tiles_t);
        const int kb0 = sp * kb_per_split;
        const int kb1 = min(a.k_blocks, kb0 + kb_per_split);
        if (a.gate_enabled) {
          // the rows of this token tile come from one or two source ranks: wait (bounded) for their pushes
          const int s0 = (tt * BT) / a.gate_rows;
          const int s1 = min(a.ar.world - 1, (min(a.T, (tt + 1) * BT) - 1) / a.gate_rows);
          for (int sr = s0; sr <= s1 && ok; ++sr) {
            if (sr == a.ar.rank) continue;
            if (!wait_flag(flag_ptr(a.ar, a.ar.rank, kGateKind, 0, sr), gate_epoch, a.ar.spin_budget, a.status, 600 + sr))
              ok = false;
          }
          if (!ok) break;
          asm volatile("fence.proxy.async.global;" ::: "memory");    // peer stores (generic proxy) -> TMA reads
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, a.status, 100 + stage)) { ok = false; break; }
          mbar_expect_tx(&bars->full[stage], kTxBytes);
          const int kx = kb * (kFp8 ? 128 : 64);
          const int gx = a.group_tiles ? (tn / a.group_tiles) * a.group_k_elems : 0;
          tma_load_2d(smem_a + stage * 128 * 128, &tmW, &bars->full[stage], kx, tn * 128);
          tma_load_2d(smem_b + stage * BT * 128, &tmX, &bars->full[stage], gx + kx, tt * BT);
          ++issued;
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Drain: wait (bounded) until every load issued to the ring has landed.
        const int pending = issued < kStages ? issued : kStages;
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < pending; ++i) {
          if (--s < 0) { s = kStages - 1; ph ^= 1; }
          mbar_wait(&bars->full[s], ph, nullptr, 0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int ab = 0;
      uint32_t aphase = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
        const int sp = u / (a.tiles_n * a.tiles_t);
        const int kb0 = sp * kb_per_split;
        const int kb1 = min(a.k_blocks, kb0 + kb_per_split);
        if constexpr (!kFp8) {
          if (!mbar_wait(&bars->tmem_empty[ab], aphase ^ 1, a.status, 200 + ab)) { ok = false; break; }
          tc_fence_after();
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if constexpr (kFp8) {
            if (!mbar_wait(&bars->tmem_empty[ab], aphase ^ 1, a.status, 200 + ab)) { ok = false; break; }
          }
          if (!mbar_wait(&bars->full[stage], phase, a.status, 300 + stage)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d = tmem_base + ab * BT;
          const uint64_t adesc = umma_desc_sw128(smem_u32(smem_a + stage * 128 * 128));
          const uint64_t bdesc = umma_desc_sw128(smem_u32(smem_b + stage * BT * 128));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // advance 32 bytes along K inside the swizzled 128-byte row (encoded >> 4)
            const uint32_t acc = kFp8 ? (k > 0) : (kb > kb0 || k > 0);
            if constexpr (kFp8) umma_f8(d, adesc + 2 * k, bdesc + 2 * k, kIdesc, acc);
            else umma_f16(d, adesc + 2 * k, bdesc + 2 * k, kIdesc, acc);
          }
          umma_commit(&bars->empty[stage]);
          if constexpr (kFp8) {
            umma_commit(&bars->tmem_full[ab]);
            if (++ab == 2) { ab = 0; aphase ^= 1; }
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if constexpr (!kFp8) {
          if (ok) {
            umma_commit(&bars->tmem_full[ab]);
            if (++ab == 2) { ab = 0; aphase ^= 1; }
          }
        }
      }
    }
  } else if (warp - 2 < kEpiWarps) {
    // ------------------------------ epilogue -----------------------------------
    const int e = warp - 2;
    const int q = warp & 3;                         // TMEM lane quarter this warp may read
    const int col_base = (kEpiWarps == 8) ? (e >> 2) * kColsPerWarp : 0;
    const int row = q * 32 + lane;
    int ab = 0;
    uint32_t aphase = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
      const int tn = u % a.tiles_n;
      const int tt = ((u / a.tiles_n) % a.tiles_t + tt_rot) % a.tiles_t;
      const int sp = u / (a.tiles_n * a.tiles_t);
      const int kb0 = sp * kb_per_split;
      const int kb1 = min(a.k_blocks, kb0 + kb_per_split);
      const int n = tn * 128 + row;
      const int t0 = tt * BT + col_base;
      const bool n_ok = n < a.N;

      const int ar_par = ar_epoch & 1;
      const long long ar_slot = a.ar.gemm_bytes / 2;      // bf16 elements per (parity, source) slot
      auto ar_push = [&](int t, float v) {
        if constexpr (Cfg::kArTileBytes > 0) ar_tile[(t - tt * BT) * 128 + row] = __float2bfloat16(v);
      };
      // copy the staged tile to every rank with 16-byte stores, signal it, wait (bounded) for every
      // rank's tile, and sum the tiles in rank order
      auto ar_finish = [&]() -> bool {
        const int tile = (tt * a.tiles_n + tn) & 4095;
        const int et = threadIdx.x - 64;
        const int nthr = kEpiWarps * 32;
        const int rows_valid = min(BT, a.T - tt * BT);
        const int nvec = rows_valid * 16;
        epi_bar_sync(nthr);
        for (int p = 0; p < a.ar.world; ++p) {
          const int peer = (a.ar.rank + p) % a.ar.world;
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.ar.base[peer] + a.ar.off_gemm) +
                               (static_cast<long long>(ar_par) * a.ar.world + a.ar.rank) * ar_slot;
          for (int v = et; v < nvec; v += nthr) {
            const int r = v >> 4, cvec = v & 15;
            const uint4 val = *reinterpret_cast<const uint4*>(ar_tile + r * 128 + cvec * 8);
            *reinterpret_cast<uint4*>(dst + static_cast<long long>(tt * BT + r) * a.N + tn * 128 + cvec * 8) = val;
          }
        }
        epi_bar_sync(nthr);
        if (et < a.ar.world) {
          __threadfence_system();      // cumulative with the barrier: orders every thread's pushes before the flag
          st_release_sys(flag_ptr(a.ar, et, kArKind, tile, a.ar.rank), ar_epoch);
        }
        if (et == 0) bars->last_flag = 1;
        epi_bar_sync(nthr);
        if (et < a.ar.world) {
          if (!wait_flag(flag_ptr(a.ar, a.ar.rank, kArKind, tile, et), ar_epoch, a.ar.spin_budget, a.status, 500 + et))
            bars->last_flag = 0;
        }
        epi_bar_sync(nthr);
        const bool got = bars->last_flag != 0;
        if (got) {
          const __nv_bfloat16* slots = reinterpret_cast<const __nv_bfloat16*>(a.ar.base[a.ar.rank] + a.ar.off_gemm) +
                                       static_cast<long long>(ar_par) * a.ar.world * ar_slot;
          for (int v = et; v < nvec; v += nthr) {
            const int r = v >> 4, cvec = v & 15;
            const long long off = static_cast<long long>(tt * BT + r) * a.N + tn * 128 + cvec * 8;
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int rk = 0; rk < a.ar.world; ++rk) {
              const uint4 val = __ldcg(reinterpret_cast<const uint4*>(slots + rk * ar_slot + off));
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&val);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                acc[2 * i] += __low2float(h[i]);
                acc[2 * i + 1] += __high2float(h[i]);
              }
            }
            if (a.out_fp32) {
              float* o = reinterpret_cast<float*>(a.out) + static_cast<long long>(tt * BT + r) * a.ldo + tn * 128 + cvec * 8;
#pragma unroll
              for (int i = 0; i < 8; ++i) o[i] = acc[i];
            } else {
              uint4 ov;
              __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
              for (int i = 0; i < 4; ++i) oh[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.out) + static_cast<long long>(tt * BT + r) * a.ldo +
                                        tn * 128 + cvec * 8) = ov;
            }
          }
        }
        epi_bar_sync(nthr);
        return got;
      };
      auto store = [&](int t, float v) {
        if (n_ok && t < a.T) {
          if (a.splits > 1) {
            a.workspace[(static_cast<long long>(sp) * a.T + t) * a.N + n] = v;
          } else if (a.ar_enabled) {
            ar_push(t, v);
          } else if (a.out_fp32) {
            reinterpret_cast<float*>(a.out)[t * a.ldo + n] = v;
          } else {
            reinterpret_cast<__nv_bfloat16*>(a.out)[t * a.ldo + n] = __float2bfloat16(v);
          }
        }
      };

      if constexpr (kFp8) {
        float acc[kColsPerWarp];
#pragma unroll
        for (int j = 0; j < kColsPerWarp; ++j) acc[j] = 0.f;
        if (a.token_major) {
          // lane = token n, columns = weight rows t0 .. t0 + kColsPerWarp of row block tt (BT == 128)
          for (int kb = kb0; kb < kb1 && ok; ++kb) {
            const float s = a.w_scale[tt * a.w_scale_ld + kb] *
                            (n_ok ? a.x_scale[static_cast<long long>(kb) * a.x_scale_ld + n] : 0.f);
            if (!mbar_wait(&bars->tmem_full[ab], aphase, a.status, 400 + ab)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < kChunksPerWarp; ++c) {
              uint32_t r[32];
              tmem_ld_chunk<CW>(tmem_base + ab * BT + col_base + c * CW + (static_cast<uint32_t>(q * 32) << 16), r);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < CW; ++j) acc[c * CW + j] = fmaf(__uint_as_float(r[j]), s, acc[c * CW + j]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->tmem_empty[ab]);
            if (++ab == 2) { ab = 0; aphase ^= 1; }
          }
          if (ok && n_ok) {
            // a thread owns kColsPerWarp consecutive outputs of its token row
            const long long o0 = static_cast<long long>(n) * a.ldo + t0;
            const bool vec = !a.out_fp32 && (a.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(a.out) & 15) == 0) &&
                             t0 + kColsPerWarp <= a.T;
            if (vec) {
#pragma unroll
              for (int j = 0; j < kColsPerWarp; j += 8) {
                uint4 ov;
                __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
                for (int i = 0; i < 4; ++i) oh[i] = __floats2bfloat162_rn(acc[j + 2 * i], acc[j + 2 * i + 1]);
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.out) + o0 + j) = ov;
              }
            } else {
#pragma unroll
              for (int j = 0; j < kColsPerWarp; ++j) {
                if (t0 + j < a.T) {
                  if (a.out_fp32) reinterpret_cast<float*>(a.out)[o0 + j] = acc[j];
                  else reinterpret_cast<__nv_bfloat16*>(a.out)[o0 + j] = __float2bfloat16(acc[j]);
                }
              }
            }
          }
        } else {
        for (int kb = kb0; kb < kb1 && ok; ++kb) {
          const float sw = a.w_scale[tn * a.w_scale_ld + kb];
          const int gkb = a.group_tiles ? (tn / a.group_tiles) * a.k_blocks : 0;
          const float* xs = a.x_scale + static_cast<long long>(gkb + kb) * a.x_scale_ld;
          if (!mbar_wait(&bars->tmem_full[ab], aphase, a.status, 400 + ab)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < kChunksPerWarp; ++c) {
            uint32_t r[32];
            tmem_ld_chunk<CW>(tmem_base + ab * BT + col_base + c * CW + (static_cast<uint32_t>(q * 32) << 16), r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < CW; j += 4) {
              const int t = t0 + c * CW + j;
              float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
              if (t + 4 <= a.x_scale_ld) s4 = __ldg(reinterpret_cast<const float4*>(xs + t));
              acc[c * CW + j + 0] = fmaf(__uint_as_float(r[j + 0]), sw * s4.x, acc[c * CW + j + 0]);
              acc[c * CW + j + 1] = fmaf(__uint_as_float(r[j + 1]), sw * s4.y, acc[c * CW + j + 1]);
              acc[c * CW + j + 2] = fmaf(__uint_as_float(r[j + 2]), sw * s4.z, acc[c * CW + j + 2]);
              acc[c * CW + j + 3] = fmaf(__uint_as_float(r[j + 3]), sw * s4.w, acc[c * CW + j + 3]);
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->tmem_empty[ab]);
          if (++ab == 2) { ab = 0; aphase ^= 1; }
        }
        if (ok) {
#pragma unroll
          for (int j = 0; j < kColsPerWarp; ++j) store(t0 + j, acc[j]);
        }
        }
      } else {
        if (!mbar_wait(&bars->tmem_full[ab], aphase, a.status, 400 + ab)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < kChunksPerWarp; ++c) {
          uint32_t r[32];
          tmem_ld_chunk<CW>(tmem_base + ab * BT + col_base + c * CW + (static_cast<uint32_t>(q * 32) << 16), r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < CW; ++j) store(t0 + c * CW + j, __uint_as_float(r[j]));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->tmem_empty[ab]);
        if (++ab == 2) { ab = 0; aphase ^= 1; }
      }

      if (a.ar_enabled && a.splits == 1 && ok) ok = ar_finish();
      if (a.splits > 1 && ok) {
        // Publish this split's partial; the CTA that completes the tile reduces it.
        __threadfence();
        epi_bar_sync(kEpiWarps * 32);
        if (threadIdx.x == 64) {
          const int prev = atomicAdd(&a.counters[tt * a.tiles_n + tn], 1);
          bars->last_flag = (prev == a.splits - 1);
          if (prev == a.splits - 1) a.counters[tt * a.tiles_n + tn] = 0;
        }
        epi_bar_sync(kEpiWarps * 32);
        const bool last = bars->last_flag != 0;
        epi_bar_sync(kEpiWarps * 32);
        if (last) {
          __threadfence();
          // Cooperative reduction: the tile's partials are [split][token][128 features] fp32 rows of
          // 512 contiguous bytes; every epilogue thread sums float4 vectors (all loads independent).
          {
            const int et2 = threadIdx.x - 64;
            const int nthr2 = kEpiWarps * 32;
            const int rows_valid = min(BT, a.T - tt * BT);
            const int cols_valid = min(128, a.N - tn * 128);
            const bool vec_ok = (cols_valid == 128) && ((a.N & 3) == 0) && (a.out_vec_ok || a.ar_enabled);
            if (vec_ok) {
              // four output vectors per thread at a time, so that 4 x (unrolled splits) loads are in flight: one vector
              // at a time left a reducing CTA at a few dozen GB/s
              const int total = rows_valid * 32;
              for (int v0 = et2; v0 < total; v0 += nthr2 * 4) {
                float4 s4[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) s4[u] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
                for (int p = 0; p < a.splits; ++p) {
#pragma unroll
                  for (int u = 0; u < 4; ++u) {
                    const int v = v0 + u * nthr2;
                    if (v < total) {
                      const int r = v >> 5, c4 = (v & 31) * 4;
                      const float4 x = __ldcg(reinterpret_cast<const float4*>(
                          &a.workspace[(static_cast<long long>(p) * a.T + tt * BT + r) * a.N + tn * 128 + c4]));
                      s4[u].x += x.x; s4[u].y += x.y; s4[u].z += x.z; s4[u].w += x.w;
                    }
                  }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  const int v = v0 + u * nthr2;
                  if (v >= total) break;
                  const int r = v >> 5, c4 = (v & 31) * 4;
                  const int t = tt * BT + r;
                  if (a.ar_enabled) {
                    if constexpr (Cfg::kArTileBytes > 0) {
                      __nv_bfloat162* d = reinterpret_cast<__nv_bfloat162*>(ar_tile + r * 128 + c4);
                      d[0] = __floats2bfloat162_rn(s4[u].x, s4[u].y);
                      d[1] = __floats2bfloat162_rn(s4[u].z, s4[u].w);
                    }
                  } else if (a.out_fp32) {
                    *reinterpret_cast<float4*>(reinterpret_cast<float*>(a.out) + t * a.ldo + tn * 128 + c4) = s4[u];
                  } else {
                    __nv_bfloat162* d = reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(a.out) + t * a.ldo + tn * 128 + c4);
                    d[0] = __floats2bfloat162_rn(s4[u].x, s4[u].y);
                    d[1] = __floats2bfloat162_rn(s4[u].z, s4[u].w);
                  }
                }
              }
            } else {
              for (int v = et2; v < rows_valid * cols_valid; v += nthr2) {
                const int r = v / cols_valid, cc = v % cols_valid;
                const int t = tt * BT + r, nn = tn * 128 + cc;
                float sacc = 0.f;
                for (int p = 0; p < a.splits; ++p) sacc += __ldcg(&a.workspace[(static_cast<long long>(p) * a.T + t) * a.N + nn]);
                if (a.ar_enabled) {
                  if constexpr (Cfg::kArTileBytes > 0) ar_tile[r * 128 + cc] = __float2bfloat16(sacc);
                } else if (a.out_fp32) {
                  reinterpret_cast<float*>(a.out)[t * a.ldo + nn] = sacc;
                } else {
                  reinterpret_cast<__nv_bfloat16*>(a.out)[t * a.ldo + nn] = __float2bfloat16(sacc);
                }
              }
            }
          }
          if (a.ar_enabled) ok = ar_finish();
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
  if (a.ar_enabled && threadIdx.x == 0) {
    // the last CTA to leave advances the epoch for the next call
    __threadfence();
    uint32_t* done = epoch_ptr(a.ar, kArKind, 1);
    if (atomicAdd(done, 1u) == gridDim.x - 1) {
      *done = 0;
      *epoch_ptr(a.ar, kArKind, 0) = ar_epoch;
      __threadfence();
    }
  }
}

// ---------------------------------------------------------------------------------
// Wide tile for large bf16 problems: one CTA owns 256 tokens x 256 weight rows (token-major: TMEM lanes are tokens,
// so an epilogue thread writes 64 contiguous bytes of its token's output row per chunk).
//
// Measured on the 128 x 256 tile above (4096 x 4096 x 8192, ncu): tensor pipe 31 % active, no unit saturated; the
// kernel is paced by operand delivery (48 KB per 512 tensor-core cycles per SM, 7.9 TB/s out of L2 over all SMs), and
// adding L2 prefetch requests made it slower -- it is the L2 -> SM path that is short, not DRAM.  Two 128-token MMAs that
// share one 256-row weight stage need 64 KB per 1024 cycles: two thirds of the traffic per FLOP, and the three-stage
// ring covers 3072 tensor-core cycles instead of 2048.  The two accumulators take all 512 TMEM columns, so the
// epilogue of a tile is not overlapped with the next tile's MMAs; eight epilogue warps with 16-byte stores keep it short.
// ---------------------------------------------------------------------------------
struct WideArgs {
  int T, N, k_blocks, tiles_n, tiles_t;
  void* out;
  long long ldo;
  int out_fp32;
  int* status;
};

constexpr int kWideStages = 3;
constexpr int kWideStageBytes = 2 * 128 * 128 + 256 * 128;       // two weight tiles + one token tile = 64 KB

__global__ void __launch_bounds__(320, 1)
gemm_wide_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const WideArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  GemmBarriers* bars = reinterpret_cast<GemmBarriers*>(smem + kWideStages * kWideStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kWideStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->tmem_full[0], 1);
    mbar_init(&bars->tmem_empty[0], 8);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  pdl_wait();
  pdl_trigger();
  const int units = a.tiles_n * a.tiles_t;
  constexpr uint32_t kIdesc = umma_idesc(1u, 1u, 128, 256);

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0, issued = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
        const int tn = u % a.tiles_n, tt = u / a.tiles_n;
        for (int kb = 0; kb < a.k_blocks; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, a.status, 100 + stage)) { ok = false; break; }
          mbar_expect_tx(&bars->full[stage], kWideStageBytes);
          uint8_t* st = smem + stage * kWideStageBytes;
          // token-major: the two A operands are 128-token tiles (TMEM lanes = tokens), B is the 256-row weight tile
          tma_load_2d(st, &tmX, &bars->full[stage], kb * 64, tt * 256);
          tma_load_2d(st + 128 * 128, &tmX, &bars->full[stage], kb * 64, tt * 256 + 128);
          tma_load_2d(st + 2 * 128 * 128, &tmW, &bars->full[stage], kb * 64, tn * 256);
          ++issued;
          if (++stage == kWideStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // drain: wait (bounded) until every load issued to the ring has landed
        const int pending = issued < kWideStages ? issued : kWideStages;
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < pending; ++i) {
          if (--s < 0) { s = kWideStages - 1; ph ^= 1; }
          mbar_wait(&bars->full[s], ph, nullptr, 0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, aphase = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
        if (!mbar_wait(&bars->tmem_empty[0], aphase ^ 1, a.status, 200)) { ok = false; break; }
        tc_fence_after();
        for (int kb = 0; kb < a.k_blocks; ++kb) {
          if (!mbar_wait(&bars->full[stage], phase, a.status, 300 + stage)) { ok = false; break; }
          tc_fence_after();
          const uint8_t* st = smem + stage * kWideStageBytes;
          const uint64_t a0 = umma_desc_sw128(smem_u32(st));
          const uint64_t a1 = umma_desc_sw128(smem_u32(st + 128 * 128));
          const uint64_t bd = umma_desc_sw128(smem_u32(st + 2 * 128 * 128));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
            umma_f16(tmem_base, a0 + 2 * k, bd + 2 * k, kIdesc, acc);
            umma_f16(tmem_base + 256, a1 + 2 * k, bd + 2 * k, kIdesc, acc);
          }
          umma_commit(&bars->empty[stage]);
          if (++stage == kWideStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&bars->tmem_full[0]);
        aphase ^= 1;
      }
    }
  } else {
    // eight epilogue warps: lane quarter q = warp % 4 (the TMEM lanes a warp may read), column half h
    const int e = warp - 2;
    const int q = warp & 3, h = e >> 2;
    uint32_t aphase = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
      const int tn = u % a.tiles_n, tt = u / a.tiles_n;
      if (!mbar_wait(&bars->tmem_full[0], aphase, a.status, 400)) { ok = false; break; }
      tc_fence_after();
      // a thread owns one token row and, per chunk, 32 consecutive output features: 64 contiguous bytes of bf16
      const bool vec_ok = !a.out_fp32 && (a.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(a.out) & 15) == 0);
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        const int t = tt * 256 + m * 128 + q * 32 + lane;
        const bool t_ok = t < a.T;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          const int col = h * 128 + c * 32;
          tmem_ld_32x32(tmem_base + m * 256 + col + (static_cast<uint32_t>(q * 32) << 16), r);
          tmem_ld_wait();
          const int n0 = tn * 256 + col;
          if (t_ok) {
            if (vec_ok && n0 + 32 <= a.N) {
              __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(a.out) + static_cast<long long>(t) * a.ldo + n0;
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 ov;
                __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  oh[i] = __floats2bfloat162_rn(__uint_as_float(r[j + 2 * i]), __uint_as_float(r[j + 2 * i + 1]));
                *reinterpret_cast<uint4*>(o + j) = ov;
              }
            } else if (a.out_fp32) {
              float* o = reinterpret_cast<float*>(a.out) + static_cast<long long>(t) * a.ldo + n0;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < a.N) o[j] = __uint_as_float(r[j]);
            } else {
              __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(a.out) + static_cast<long long>(t) * a.ldo + n0;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < a.N) o[j] = __float2bfloat16(__uint_as_float(r[j]));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->tmem_empty[0]);
      aphase ^= 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

// 2-D row-major [rows, cols] tensor with `ld` elements between rows; box = [box_rows, 128 bytes].
int make_tmap_2d(CUtensorMap* tm, const void* base, int elem_bytes, long long rows, long long cols, long long ld,
                 int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return -1;
  CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                         : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                           : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * elem_bytes};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / elem_bytes), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

// Paged uint8 tensor [pages][rows_per_page][128 B] with `page_stride` bytes between pages; box = one page's rows.
int make_tmap_pages(CUtensorMap* tm, const void* base, long long pages, int rows_per_page, long long page_stride) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return -1;
  cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(rows_per_page), static_cast<cuuint64_t>(pages)};
  cuuint64_t strides[2] = {128, static_cast<cuuint64_t>(page_stride)};
  cuuint32_t box[3] = {128, static_cast<cuuint32_t>(rows_per_page), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

template <int BT, bool kFp8>
static int launch_gemm(const CUtensorMap& tw, const CUtensorMap& tx, const GemmArgs& a, int grid, cudaStream_t st) {
  using Cfg = GemmCfg<BT>;
  const int smem = Cfg::kStages * Cfg::kStageBytes + 256 + Cfg::kArTileBytes + 1024;
  static_assert(sizeof(GemmBarriers) <= 256, "barrier block");
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_kernel<BT, kFp8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return -3;
    configured = true;
  }
  if (a.ar_enabled || a.gate_enabled) {
    gemm_kernel<BT, kFp8><<<grid, kFp8 ? 320 : 192, smem, st>>>(tw, tx, a);      // waits on peers: plain launch
  } else {
    launch_pdl(gemm_kernel<BT, kFp8>, dim3(grid), dim3(kFp8 ? 320 : 192), smem, st, tw, tx, a);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace stk

using namespace stk;

STK_API int stk_gemm_pick_bt(int T, int is_fp8) {
  const int cap = is_fp8 ? 128 : 256;
  int bt = 16;
  while (bt < T && bt < cap) bt *= 2;
  return bt;
}

// Suggested split-K factor so that a skinny problem still fills the SMs.
STK_API int stk_gemm_pick_splits(int T, int N, int K, int is_fp8, int sm_count) {
  const int bt = stk_gemm_pick_bt(T, is_fp8);
  const int tiles = ((N + 127) / 128) * ((T + bt - 1) / bt);
  const int kb = (K * (is_fp8 ? 1 : 2) + 127) / 128;
  if (tiles >= sm_count || T > 128) return 1;
  int s = sm_count / tiles;
  if (s > kb / 4) s = kb / 4;      // keep at least four K blocks per split
  if (s > 16) s = 16;
  return s < 1 ? 1 : s;
}

STK_API long long stk_gemm_workspace_bytes(int T, int N, int splits) {
  return splits > 1 ? static_cast<long long>(splits) * T * N * 4 : 0;
}

// STK_GEMM_WIDE=0 keeps large bf16 problems on the 128 x 256 tile (A/B runs)
static bool gemm_wide_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("STK_GEMM_WIDE");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

static int gemm_launch(const void* W, long long ldw, const void* X, long long ldx, void* out, long long ldo, int T, int N,
                       int K, int is_fp8, int out_fp32, const float* w_scale, int w_scale_ld, const float* x_scale,
                       int x_scale_ld, int splits, float* workspace, int* counters, int* status, int sm_count,
                       int groups, const void* ar_ctx, const void* gate_ctx, int gate_rows, void* stream, int bt_override = 0) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  const int es = is_fp8 ? 1 : 2;
  if ((ldw * es) % 16 || (ldx * es) % 16 || (reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(X) & 15))
    return -10;
  if (is_fp8 && (w_scale == nullptr || x_scale == nullptr || (x_scale_ld & 3))) return -11;
  if (splits > 1 && (workspace == nullptr || counters == nullptr)) return -12;
  if (groups < 1) groups = 1;
  // fp8 with at least a full tile of tokens: token-major orientation (see GemmArgs::token_major)
  const bool token_major = is_fp8 && T >= 128 && groups == 1 && ar_ctx == nullptr && gate_ctx == nullptr && splits <= 1 &&
                           (reinterpret_cast<uintptr_t>(X) & 15) == 0;
  if (token_major) {
    CUtensorMap ta, tb;
    if (make_tmap_2d(&ta, X, 1, T, K, ldx, 128) != 0) return -13;        // lanes: tokens
    if (make_tmap_2d(&tb, W, 1, N, K, ldw, 128) != 0) return -14;        // columns: weight rows
    GemmArgs a;
    memset(&a, 0, sizeof(a));
    a.T = N; a.N = T;
    a.k_blocks = (K + 127) / 128;
    a.splits = 1;
    a.tiles_n = (T + 127) / 128;
    a.tiles_t = (N + 127) / 128;
    a.out = out; a.ldo = ldo; a.out_fp32 = out_fp32;
    a.w_scale = w_scale; a.w_scale_ld = w_scale_ld;
    a.x_scale = x_scale; a.x_scale_ld = x_scale_ld;
    a.status = status;
    a.token_major = 1;
    const int units = a.tiles_n * a.tiles_t;
    const int grid = units < sm_count ? units : sm_count;
    return launch_gemm<128, true>(ta, tb, a, grid, reinterpret_cast<cudaStream_t>(stream));
  }
  if (!is_fp8 && groups == 1 && ar_ctx == nullptr && gate_ctx == nullptr && splits <= 1 && bt_override == 0 && T >= 512 &&
      N >= 512 && gemm_wide_enabled()) {
    CUtensorMap tw2, tx2;
    if (make_tmap_2d(&tw2, W, 2, N, K, ldw, 256) != 0) return -13;       // B operand: 256 weight rows
    if (make_tmap_2d(&tx2, X, 2, T, K, ldx, 128) != 0) return -14;       // A operands: 128 tokens each
    WideArgs wa;
    wa.T = T; wa.N = N;
    wa.k_blocks = (K * 2 + 127) / 128;
    wa.tiles_n = (N + 255) / 256;
    wa.tiles_t = (T + 255) / 256;
    wa.out = out; wa.ldo = ldo; wa.out_fp32 = out_fp32; wa.status = status;
    const int wunits = wa.tiles_n * wa.tiles_t;
    const int wgrid = wunits < sm_count ? wunits : sm_count;
    const int wsmem = kWideStages * kWideStageBytes + 256 + 1024;
    static bool wide_configured = false;
    if (!wide_configured) {
      if (cudaFuncSetAttribute(gemm_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, wsmem) != cudaSuccess) return -3;
      wide_configured = true;
    }
    launch_pdl(gemm_wide_kernel, dim3(wgrid), dim3(320), wsmem, reinterpret_cast<cudaStream_t>(stream), tw2, tx2, wa);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  int bt = stk_gemm_pick_bt(T, is_fp8);
  if (!is_fp8 && T > 128 && groups == 1) {
    // mid-size bf16 problems: split-K through the fp32 workspace costs more than it gains above 128 tokens
    // (measured), so parallelism comes from narrower token tiles until about 0.7 x the SMs have a tile
    const int wt = (N + 127) / 128;
    while (bt > 64 && wt * ((T + bt - 1) / bt) * 10 < sm_count * 7) bt /= 2;
  }
  if (bt_override == 16 || bt_override == 32 || bt_override == 64 || bt_override == 128) bt = bt_override;
  CUtensorMap tw, tx;
  if (make_tmap_2d(&tw, W, es, N, K, ldw, 128) != 0) return -13;
  if (groups > 1 && ((K * es) % 128 || N % (128 * groups))) return -17;   // groups must split on tile boundaries
  if (make_tmap_2d(&tx, X, es, T, static_cast<long long>(K) * groups, ldx, bt) != 0) return -14;
  GemmArgs a;
  a.T = T; a.N = N;
  a.k_blocks = (K * es + 127) / 128;
  a.splits = splits < 1 ? 1 : splits;
  if (a.splits > a.k_blocks) a.splits = a.k_blocks;
  {  // no split may own an empty K range: its accumulator would never be written
    const int per = (a.k_blocks + a.splits - 1) / a.splits;
    a.splits = (a.k_blocks + per - 1) / per;
  }
  a.tiles_n = (N + 127) / 128;
  a.tiles_t = (T + bt - 1) / bt;
  a.out = out; a.ldo = ldo; a.out_fp32 = out_fp32;
  a.w_scale = w_scale; a.w_scale_ld = w_scale_ld;
  a.x_scale = x_scale; a.x_scale_ld = x_scale_ld;
  a.workspace = workspace; a.counters = counters; a.status = status;
  a.group_tiles = groups > 1 ? (N / groups) / 128 : 0;
  a.group_k_elems = K;
  {
    const uintptr_t o = reinterpret_cast<uintptr_t>(out);
    a.out_vec_ok = out_fp32 ? ((o & 15) == 0 && (ldo & 3) == 0) : ((o & 3) == 0 && (ldo & 1) == 0);
  }
  a.ar_enabled = 0;
  memset(&a.ar, 0, sizeof(a.ar));
  if (ar_ctx != nullptr) {
    memcpy(&a.ar, ar_ctx, sizeof(a.ar));
    if (static_cast<long long>(T) * N * 2 > a.ar.gemm_bytes || ldo % 8 || N % 128 || bt > 128 ||
        (reinterpret_cast<uintptr_t>(out) & 15))
      return -18;
    a.ar_enabled = 1;
  }
  a.gate_enabled = 0;
  a.gate_rows = 0;
  a.token_major = 0;
  if (gate_ctx != nullptr) {
    if (ar_ctx != nullptr || gate_rows <= 0 || a.splits != 1) return -19;
    memcpy(&a.ar, gate_ctx, sizeof(a.ar));
    a.gate_enabled = 1;
    a.gate_rows = gate_rows;
  }
  const int units = a.splits * a.tiles_n * a.tiles_t;
  const int grid = units < sm_count ? units : sm_count;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define STK_LAUNCH(BT_) (is_fp8 ? launch_gemm<BT_, true>(tw, tx, a, grid, st) : launch_gemm<BT_, false>(tw, tx, a, grid, st))
  switch (bt) {
    case 16: return STK_LAUNCH(16);
    case 32: return STK_LAUNCH(32);
    case 64: return STK_LAUNCH(64);
    case 128: return STK_LAUNCH(128);
    case 256: return is_fp8 ? -15 : launch_gemm<256, false>(tw, tx, a, grid, st);
  }
#undef STK_LAUNCH
  return -16;
}

STK_API int stk_gemm(const void* W, long long ldw, const void* X, long long ldx, void* out, long long ldo, int T, int N,
                     int K, int is_fp8, int out_fp32, const float* w_scale, int w_scale_ld, const float* x_scale,
                     int x_scale_ld, int splits, float* workspace, int* counters, int* status, int sm_count,
                     int groups, const void* ar_ctx, void* stream) {
  return gemm_launch(W, ldw, X, ldx, out, ldo, T, N, K, is_fp8, out_fp32, w_scale, w_scale_ld, x_scale, x_scale_ld, splits,
                     workspace, counters, status, sm_count, groups, ar_ctx, nullptr, 0, stream);
}

// Plain GEMM with an explicit token-tile width (16/32/64/128): narrow weights with many tokens get their parallelism
// from token tiles instead of split-K (e.g. the 24-row hyper-connection mix projection over [T, 16384]).
STK_API int stk_gemm_tile(const void* W, long long ldw, const void* X, long long ldx, void* out, long long ldo, int T, int N,
                          int K, int out_fp32, int bt, int splits, float* workspace, int* counters, int* status,
                          int sm_count, void* stream) {
  return gemm_launch(W, ldw, X, ldx, out, ldo, T, N, K, 0, out_fp32, nullptr, 0, nullptr, 0, splits < 1 ? 1 : splits,
                     workspace, counters, status, sm_count, 1, nullptr, nullptr, 0, stream, bt);
}

// All-gather -> GEMM: X is the gathered [T, K] matrix inside this rank's symmetric region (filled by
// stk_symm_ag_push on every rank, `gate_rows` rows per source rank); tiles wait only for the shards they read.
STK_API int stk_gemm_gated(const void* W, long long ldw, const void* X, long long ldx, void* out, long long ldo, int T,
                           int N, int K, int is_fp8, int out_fp32, const float* w_scale, int w_scale_ld,
                           const float* x_scale, int x_scale_ld, int* status, int sm_count, const void* gate_ctx,
                           int gate_rows, void* stream) {
  return gemm_launch(W, ldw, X, ldx, out, ldo, T, N, K, is_fp8, out_fp32, w_scale, w_scale_ld, x_scale, x_scale_ld, 1,
                     nullptr, nullptr, status, sm_count, 1, nullptr, gate_ctx, gate_rows, stream);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free entry point (declared in stk_no_alloc.h).
// ---------------------------------------------------------------------------------------------
namespace {
constexpr long long kNoAllocWorkspaceBytes = 8ll << 20;      // split-K partials: splits * T * N * 4 bytes
constexpr int kNoAllocCounters = 4096;                        // one per output tile
constexpr long long kNoAllocBytes = kNoAllocWorkspaceBytes + kNoAllocCounters * 4;
// Lives in every context that loads the library until the process exits.  Zero-initialised by the
// loader; the GEMM leaves its tile counters at zero when it finishes.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];
constexpr int kMaxDevices = 64;
static void* g_noalloc_ptr[kMaxDevices] = {};
}  // namespace

STK_API long long stk_gemm_noalloc_max_workspace_bytes() { return kNoAllocWorkspaceBytes; }

static int noalloc_resolve(unsigned char** base) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -30;
  if (g_noalloc_ptr[dev] == nullptr) {
    // First call on this device: resolve the device address of the static array.  In host code the
    // array's name is only a handle for this query, never a pointer a kernel may be given.
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) return -31;
    g_noalloc_ptr[dev] = p;
  }
  *base = static_cast<unsigned char*>(g_noalloc_ptr[dev]);
  return 0;
}

// Zeroes the built-in tile counters on `stream` (a memset node, no allocation).  Needed only after a call whose
// status word came back non-zero: a split that gave up a wait never counted itself in, so its tile's counter is
// left between 1 and splits-1 and the next split-K call on that tile would reduce too early.
STK_API int stk_gemm_noalloc_reset(void* stream) {
  unsigned char* base = nullptr;
  const int rc = noalloc_resolve(&base);
  if (rc != 0) return rc;
  return cudaMemsetAsync(base + kNoAllocWorkspaceBytes, 0, kNoAllocCounters * 4, reinterpret_cast<cudaStream_t>(stream)) ==
                 cudaSuccess ? 0 : -34;
}

STK_API int stk_gemm_noalloc(const void* W, long long ldw, const void* X, long long ldx, void* out, long long ldo,
                             int T, int N, int K, int is_fp8, int out_fp32, const float* w_scale, int w_scale_ld,
                             const float* x_scale, int x_scale_ld, int splits, int* status, int sm_count, void* stream) {
  unsigned char* base = nullptr;
  const int rc = noalloc_resolve(&base);
  if (rc != 0) return rc;
  if (splits < 1) splits = 1;
  const int bt = stk_gemm_pick_bt(T, is_fp8);
  const long long tiles = static_cast<long long>((N + 127) / 128) * ((T + bt - 1) / bt);
  if (splits > 1) {
    if (static_cast<long long>(splits) * T * N * 4 > kNoAllocWorkspaceBytes) return -32;   // beyond the built-in scratch
    if (tiles > kNoAllocCounters) return -33;
  }
  float* workspace = reinterpret_cast<float*>(base);
  int* counters = reinterpret_cast<int*>(base + kNoAllocWorkspaceBytes);
  return stk_gemm(W, ldw, X, ldx, out, ldo, T, N, K, is_fp8, out_fp32, w_scale, w_scale_ld, x_scale, x_scale_ld, splits,
                  workspace, counters, status, sm_count, 1, nullptr, stream);
}
