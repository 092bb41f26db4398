// Lightning-indexer scoring on the 5th-generation tensor cores (fp8 q, fp8 indexer-K cache, head dim 128).
//
//   score[t, s] = k_scale[s] * sum_h w[t, h] * relu(q[t, h, :] . k[s, :])            s < n_valid[t]
//
// One CTA owns a block of 128 cache rows of one request and a chunk of tokens.  The block's K rows (two 64-row pages,
// each a contiguous [64 x 128 B] region of the paged cache) are brought into shared memory once by TMA as the
// M = 128 operand (a 3-D tensor map [page][row][128 B] over the cache, one box per page); the q rows of one or two tokens ([64 heads x 128 B] each, contiguous) stream through a two-stage
// ring as the N operand.  tcgen05.mma kind::f8f6f4 writes D[row, (token, head)] into a double-buffered TMEM
// accumulator, so each epilogue thread owns one cache row and finds all heads of a token in its own TMEM lane:
// ReLU, the head weights and the sum over heads are thread-local, and a warp stores 32 consecutive scores of a
// token.  (The reference reaches the same scores through DeepGEMM's fp8 paged MQA logits kernel:
// probes/sai_probe.py:2316-2337.)
//
// Tokens are walked as tiles of up to TPT consecutive tokens of the same request; when the request changes inside a
// chunk the K block is reloaded (the MMA thread signals when the old block is no longer read).  Every wait is bounded.
#define STK_PDL_CLASS 16      // bit of this file's kernels in the PDL mask (STK_PDL, stk_set_pdl_mask)
#include "common.cuh"

namespace stk {

int make_tmap_2d(CUtensorMap* tm, const void* base, int elem_bytes, long long rows, long long cols, long long ld,
                 int box_rows);
int make_tmap_pages(CUtensorMap* tm, const void* base, long long pages, int rows_per_page, long long page_stride);

struct IdxTcArgs {
  const float* w;              // [T, 64] folded head weights
  const uint8_t* kbase;        // paged cache base (for the per-row scales)
  long long page_stride;
  int n_pages;
  const int* block_table; int bt_stride;
  const int* tok_req;          // [T]
  const int* n_valid;          // [T]
  float* scores; long long ld_scores;
  int T, tokens_per_cta;
  int* status;
};

struct IdxTcBarriers {
  uint64_t a_full, a_free;
  uint64_t q_full[2], q_empty[2];
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int any;
};

constexpr int kIdxHeads = 64;
constexpr int kIdxRowBytes = 128;          // 128 fp8 values
constexpr int kIdxPageRows = 64;

__device__ __forceinline__ int idx_page(const IdxTcArgs& a, int req, int page_idx) {
  int p = page_idx < a.bt_stride ? a.block_table[static_cast<long long>(req) * a.bt_stride + page_idx] : 0;
  if (p < 0 || p >= a.n_pages) p = 0;      // rows of such a page are beyond n_valid and never stored
  return p;
}

// Tile walk shared by the three roles: tokens [t, t + n) of request `req`; returns false at the end of the chunk.
template <int TPT>
__device__ __forceinline__ bool idx_next_tile(const IdxTcArgs& a, int& t, int t1, int& n, int& req) {
  if (t >= t1) return false;
  req = a.tok_req[t];
  n = 1;
  if (TPT == 2 && t + 1 < t1 && a.tok_req[t + 1] == req) n = 2;
  return true;
}

// grid (row blocks, token chunks); 192 threads: warp 0 TMA producer, warp 1 MMA issuer, warps 2..5 epilogue.
template <int TPT>
__global__ void __launch_bounds__(192)
indexer_scores_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmQ,
                         const IdxTcArgs a) {
  constexpr int N = kIdxHeads * TPT;                 // MMA N: (token, head) columns
  constexpr int kQBytes = N * kIdxRowBytes;
  constexpr int kABytes = 128 * kIdxRowBytes;
  constexpr uint32_t kIdesc = umma_idesc(0u, 0u, 128, N);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_q = smem + kABytes;
  IdxTcBarriers* bars = reinterpret_cast<IdxTcBarriers*>(smem_q + 2 * kQBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rb = blockIdx.x;
  const int r0 = rb * 128;
  const int t0 = blockIdx.y * a.tokens_per_cta;
  const int t1 = min(a.T, t0 + a.tokens_per_cta);

  if (threadIdx.x == 0) {
    mbar_init(&bars->a_full, 1);
    mbar_init(&bars->a_free, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->q_full[i], 1);
      mbar_init(&bars->q_empty[i], 1);
      mbar_init(&bars->acc_full[i], 1);
      mbar_init(&bars->acc_empty[i], 4);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmQ);
  }
  pdl_wait();
  pdl_trigger();
  // nothing to do when no token of the chunk sees this row block (causal prefill: early tokens, late rows)
  int mine = 0;
  for (int t = t0 + threadIdx.x; t < t1; t += blockDim.x) mine |= (a.tok_req[t] >= 0 && a.n_valid[t] > r0) ? 1 : 0;
  if (!__syncthreads_or(mine)) return;
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 2 * N);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  auto live_tile = [&](int t, int n, int req) -> bool {
    if (req < 0) return false;
    int nv = a.n_valid[t];
    if (n == 2) nv = max(nv, a.n_valid[t + 1]);
    return nv > r0;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0, cur = -2, nchg = 0, t = t0, n = 0, req = 0;
      uint32_t qphase = 0;
      bool ok = true, a_pending = false;
      int q_issued = 0;
      while (ok && idx_next_tile<TPT>(a, t, t1, n, req)) {
        if (live_tile(t, n, req)) {
          if (req != cur) {
            if (cur != -2) {
              // the MMA thread commits a_free once every MMA that reads the old block has completed
              if (!mbar_wait(&bars->a_free, static_cast<uint32_t>(nchg & 1), a.status, 700)) { ok = false; break; }
              ++nchg;
            }
            mbar_expect_tx(&bars->a_full, kABytes);
            tma_load_3d(smem_a, &tmK, &bars->a_full, 0, 0, idx_page(a, req, 2 * rb));
            tma_load_3d(smem_a + kABytes / 2, &tmK, &bars->a_full, 0, 0, idx_page(a, req, 2 * rb + 1));
            a_pending = true;
            cur = req;
          }
          if (!mbar_wait(&bars->q_empty[stage], qphase ^ 1, a.status, 701 + stage)) { ok = false; break; }
          mbar_expect_tx(&bars->q_full[stage], kQBytes);
          tma_load_2d(smem_q + stage * kQBytes, &tmQ, &bars->q_full[stage], 0, t * kIdxHeads);
          ++q_issued;
          if (++stage == 2) { stage = 0; qphase ^= 1; }
        }
        t += n;
      }
      if (!ok) {
        // drain (bounded, silent): loads that were issued must land before the CTA leaves
        if (a_pending) mbar_wait(&bars->a_full, static_cast<uint32_t>(nchg & 1), nullptr, 0);
        int s = stage;
        uint32_t ph = qphase;
        for (int i = 0; i < (q_issued < 2 ? q_issued : 2); ++i) {
          if (--s < 0) { s = 1; ph ^= 1; }
          mbar_wait(&bars->q_full[s], ph, nullptr, 0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      int stage = 0, ab = 0, cur = -2, seg = 0, t = t0, n = 0, req = 0;
      uint32_t qphase = 0, aphase = 0;
      bool ok = true;
      while (ok && idx_next_tile<TPT>(a, t, t1, n, req)) {
        if (live_tile(t, n, req)) {
          if (req != cur) {
            if (cur != -2) umma_commit(&bars->a_free);
            if (!mbar_wait(&bars->a_full, static_cast<uint32_t>(seg & 1), a.status, 710)) { ok = false; break; }
            ++seg;
            cur = req;
          }
          if (!mbar_wait(&bars->acc_empty[ab], aphase ^ 1, a.status, 711 + ab)) { ok = false; break; }
          if (!mbar_wait(&bars->q_full[stage], qphase, a.status, 713 + stage)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d = tmem_base + ab * N;
          const uint64_t adesc = umma_desc_sw128(smem_u32(smem_a));
          const uint64_t bdesc = umma_desc_sw128(smem_u32(smem_q + stage * kQBytes));
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f8(d, adesc + 2 * k, bdesc + 2 * k, kIdesc, k > 0);
          umma_commit(&bars->q_empty[stage]);
          umma_commit(&bars->acc_full[ab]);
          if (++stage == 2) { stage = 0; qphase ^= 1; }
          if (++ab == 2) { ab = 0; aphase ^= 1; }
        }
        t += n;
      }
    }
  } else {
    // ------------------------------ epilogue (4 warps, one cache row per thread) ------------------------------
    const int q4 = warp & 3;                              // TMEM lane quarter this warp may read
    const int L = q4 * 32 + lane;                         // row of the block = TMEM lane
    const int r = r0 + L;
    const uint32_t lane_addr = static_cast<uint32_t>(q4 * 32) << 16;
    int ab = 0, cur = -2, t = t0, n = 0, req = 0;
    uint32_t aphase = 0;
    float kscale = 0.f;
    bool ok = true;
    while (ok && idx_next_tile<TPT>(a, t, t1, n, req)) {
      if (live_tile(t, n, req)) {
        if (req != cur) {
          const int page = idx_page(a, req, 2 * rb + (L >> 6));
          kscale = *reinterpret_cast<const float*>(a.kbase + static_cast<long long>(page) * a.page_stride +
                                                   kIdxPageRows * kIdxRowBytes + (L & 63) * 4);
          cur = req;
        }
        if (!mbar_wait(&bars->acc_full[ab], aphase, a.status, 720 + ab)) { ok = false; break; }
        tc_fence_after();
        for (int j = 0; j < n; ++j) {
          const int tj = t + j;
          const float4* wj = reinterpret_cast<const float4*>(a.w + static_cast<long long>(tj) * kIdxHeads);
          float acc = 0.f;
          // all 64 head columns of this token are requested before the single wait
          uint32_t v0[32], v1[32];
          tmem_ld_32x32(tmem_base + lane_addr + ab * N + j * kIdxHeads, v0);
          tmem_ld_32x32(tmem_base + lane_addr + ab * N + j * kIdxHeads + 32, v1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 w4 = __ldg(wj + (i >> 2));
            acc = fmaf(w4.x, fmaxf(__uint_as_float(v0[i]), 0.f), acc);
            acc = fmaf(w4.y, fmaxf(__uint_as_float(v0[i + 1]), 0.f), acc);
            acc = fmaf(w4.z, fmaxf(__uint_as_float(v0[i + 2]), 0.f), acc);
            acc = fmaf(w4.w, fmaxf(__uint_as_float(v0[i + 3]), 0.f), acc);
          }
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 w4 = __ldg(wj + 8 + (i >> 2));
            acc = fmaf(w4.x, fmaxf(__uint_as_float(v1[i]), 0.f), acc);
            acc = fmaf(w4.y, fmaxf(__uint_as_float(v1[i + 1]), 0.f), acc);
            acc = fmaf(w4.z, fmaxf(__uint_as_float(v1[i + 2]), 0.f), acc);
            acc = fmaf(w4.w, fmaxf(__uint_as_float(v1[i + 3]), 0.f), acc);
          }
          if (r < a.n_valid[tj]) a.scores[static_cast<long long>(tj) * a.ld_scores + r] = acc * kscale;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->acc_empty[ab]);
        if (++ab == 2) { ab = 0; aphase ^= 1; }
      }
      t += n;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * N);
  }
}

}  // namespace stk

using namespace stk;

// q: fp8 e4m3 [T, 64, 128] contiguous; kcache: fp8 pages of [64 x 128 B rows][64 fp32 scales]; w: folded weights
// [T, 64]; scores fp32 [T, ld] (entries >= n_valid[t] are left untouched).  Returns -20 for layouts it does not cover
// (the caller then uses the CUDA-core scorer).
STK_API int stk_indexer_scores_tc(const void* q, const float* w, const void* kcache, long long page_stride, int n_pages,
                                  const int* block_table, int bt_stride, const int* tok_req, const int* n_valid,
                                  float* scores, long long ld_scores, int T, int max_rows, int ih, int di, int* status,
                                  void* stream) {
  if (T <= 0 || max_rows <= 0) return 0;
  if (ih != kIdxHeads || di != kIdxRowBytes) return -20;
  if (page_stride < kIdxPageRows * (kIdxRowBytes + 4) || page_stride % 16 || n_pages <= 0) return -20;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(kcache) & 15) ||
      (reinterpret_cast<uintptr_t>(w) & 15))
    return -21;
  const int tpt = T >= 128 ? 2 : 1;
  CUtensorMap tk, tq;
  if (make_tmap_pages(&tk, kcache, n_pages, kIdxPageRows, page_stride) != 0) return -13;
  if (make_tmap_2d(&tq, q, 1, static_cast<long long>(T) * kIdxHeads, kIdxRowBytes, kIdxRowBytes, kIdxHeads * tpt) != 0)
    return -14;
  IdxTcArgs a;
  a.w = w; a.kbase = (const uint8_t*)kcache; a.page_stride = page_stride; a.n_pages = n_pages;
  a.block_table = block_table; a.bt_stride = bt_stride; a.tok_req = tok_req; a.n_valid = n_valid;
  a.scores = scores; a.ld_scores = ld_scores; a.T = T; a.status = status;
  // decode-sized steps: one token per CTA (every token its own request); large steps: chunks of 128 tokens, so that a
  // K block is loaded once per 64 tiles while the grid still covers the GPU several times
  a.tokens_per_cta = T >= 128 ? 128 : 1;
  dim3 grid((max_rows + 127) / 128, (T + a.tokens_per_cta - 1) / a.tokens_per_cta);
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  if (tpt == 2) {
    constexpr int smem = 128 * 128 + 2 * 128 * 128 + 256 + 1024;
    static bool configured = false;
    if (!configured) {
      if (cudaFuncSetAttribute(indexer_scores_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return -3;
      configured = true;
    }
    e = launch_pdl(indexer_scores_tc_kernel<2>, grid, dim3(192), smem, st, tk, tq, a);
  } else {
    constexpr int smem = 128 * 128 + 2 * 64 * 128 + 256 + 1024;
    e = launch_pdl(indexer_scores_tc_kernel<1>, grid, dim3(192), smem, st, tk, tq, a);
  }
  return e == cudaSuccess ? 0 : -4;
}
