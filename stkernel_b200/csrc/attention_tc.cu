// Sparse multi-head latent attention on the 5th-generation tensor cores (fp8_ds_mla rows, D = 512).
//
// One CTA per (query token, row split).  The row list (SWA window rows, then top-k compressed rows)
// is walked in blocks of 128 rows:
//
//   producer warps   gather the 584-byte rows by slot id, dequantise fp8 x UE8M0 -> bf16 and write them
//                    into shared memory as 8 panels of [128 rows x 64 dims], 128-byte swizzled
//   MMA warp         S^T[row, head] = K_block . Q^T      (K panels as the K-major A operand)
//                    O^T[dim, head] += V^T . P           (the same panels as the MN-major A operand:
//                                                         K = V = the latent row, stored once)
//   softmax warps    read S^T from TMEM (one row per thread), online softmax with a per-head running
//                    maximum (cross-row maximum by warp shuffles), write P as the K-major B operand,
//                    rescale O in TMEM only when a head's maximum moved
//
// Accumulators live in TMEM: S (NH columns) and four O^T tiles of [128 dims x NH heads].
// The CTA writes an un-normalised partial (o, m, l) that `sparse_mla_combine` merges with the sink.
// Every mbarrier wait is bounded; on expiry the status word is set and the CTA drains and exits.
//
// Replaces the reference's FlashInfer sparse-MLA decode/prefill kernels
// (overlay/flashinfer_sparse.py:323-541).
#define STK_PDL_CLASS 128      // bit of this file's kernels in the PDL mask (STK_PDL, stk_set_pdl_mask)
#include "common.cuh"

namespace stk {

struct MlaTcArgs {
  const __nv_bfloat16* q;      // [T, nh, 512]
  long long ldt;
  const uint8_t* swa_base; long long swa_stride;
  const uint8_t* comp_base; long long comp_stride;
  const int* swa_slots; int swa_ld; const int* swa_lens;
  const int* topk_slots; int topk_ld; const int* topk_lens;   // may be null
  float* partial;              // [T, n_splits, nh, 514]
  // Direct output (n_splits == 1 only, out != nullptr): the CTA merges the sink, normalises, applies the inverse
  // RoPE to the rope dims and writes bf16 [T, nh, 512] itself; no partial is written and no combine pass runs.
  __nv_bfloat16* out; long long ldo;
  const float* sink;           // [nh] or null
  const int64_t* positions;    // [T] or null (no inverse RoPE)
  const float* inv_freq;       // [32]
  int T, nh, n_splits, rows_per_split;
  float scale;
  int* status;
  unsigned long long* trace;   // optional [8] stage timestamps (ns) of CTA (0,0): a device-side stage trace
};

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define STK_TRACE(slot) do { if (a.trace && blockIdx.x == 0 && blockIdx.y == 0) a.trace[slot] = global_ns(); } while (0)

constexpr int kD = 512, kR = 64, kNope = 448, kDataBytes = 576, kPanels = 8, kRows = 128;
constexpr int kPanelBytes = kRows * 128;                 // 16 KB
constexpr int kProducerWarps = 8, kSoftmaxWarps = 4;
constexpr int kThreads = 32 * (1 + kSoftmaxWarps + kProducerWarps);

struct alignas(8) MlaBars {
  uint64_t k_full, s_full, p_full, pv_done;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
      "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
      "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// MN-major operand, 128-byte swizzle: 128-byte column blocks are `lbo` bytes apart along M/N,
// 8-row groups are 1024 bytes apart along K.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(lbo_bytes >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void named_bar_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

// fp8 e4m3 x4 (one 32-bit word) times a power-of-two scale -> four bf16 (two packed words)
__device__ __forceinline__ void fp8x4_to_bf16x4(uint32_t w, float sc, uint32_t& lo, uint32_t& hi) {
  const __half2_raw h01 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w & 0xffff), __NV_E4M3);
  const __half2_raw h23 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w >> 16), __NV_E4M3);
  const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
  const float2 f23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
  const __nv_bfloat162 b01 = __floats2bfloat162_rn(f01.x * sc, f01.y * sc);
  const __nv_bfloat162 b23 = __floats2bfloat162_rn(f23.x * sc, f23.y * sc);
  lo = *reinterpret_cast<const uint32_t*>(&b01);
  hi = *reinterpret_cast<const uint32_t*>(&b23);
}

// One level of a butterfly all-lane reduction over CNT values per lane: lanes exchange the half they
// give up, so 32 lanes x CNT values reduce with CNT-ish shuffles instead of 5 x CNT.
template <int CNT, bool kMax>
__device__ __forceinline__ void bfly_level(float* v, int off, bool bit) {
  if constexpr (CNT > 1) {
    constexpr int H = CNT / 2;
#pragma unroll
    for (int i = 0; i < H; ++i) {
      const float mine = bit ? v[H + i] : v[i];
      const float send = bit ? v[i] : v[H + i];
      const float recv = __shfl_xor_sync(0xffffffffu, send, off);
      v[i] = kMax ? fmaxf(mine, recv) : mine + recv;
    }
  } else {
    const float recv = __shfl_xor_sync(0xffffffffu, v[0], off);
    v[0] = kMax ? fmaxf(v[0], recv) : v[0] + recv;
  }
}
// Reduce v[h] over the 32 lanes for every h < NH; lane l ends with heads (l*NH/32) .. +max(NH/32,1)
// in v[0..]; they are written to out[h].
template <int NH, bool kMax>
__device__ __forceinline__ void bfly_reduce_store(float (&v)[NH], float* out, int lane) {
  constexpr int C1 = NH / 2 > 0 ? NH / 2 : 1, C2 = C1 / 2 > 0 ? C1 / 2 : 1, C3 = C2 / 2 > 0 ? C2 / 2 : 1,
                C4 = C3 / 2 > 0 ? C3 / 2 : 1, C5 = C4 / 2 > 0 ? C4 / 2 : 1;
  bfly_level<NH, kMax>(v, 16, (lane & 16) != 0);
  bfly_level<C1, kMax>(v, 8, (lane & 8) != 0);
  bfly_level<C2, kMax>(v, 4, (lane & 4) != 0);
  bfly_level<C3, kMax>(v, 2, (lane & 2) != 0);
  bfly_level<C4, kMax>(v, 1, (lane & 1) != 0);
  const int base = (lane * NH) >> 5;
#pragma unroll
  for (int i = 0; i < C5; ++i) out[base + i] = v[i];
}

template <int NH>
__global__ void __launch_bounds__(kThreads, 1)
sparse_mla_tc_kernel(const MlaTcArgs a) {
  pdl_wait();
  pdl_trigger();
  constexpr int kTmemCols = (5 * NH <= 128) ? 128 : (5 * NH <= 256) ? 256 : 512;
  constexpr int kQBytes = kPanels * NH * 128;
  constexpr int kPBytes = 2 * NH * 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_s = smem;                                   // 8 panels x 16 KB
  uint8_t* q_s = k_s + kPanels * kPanelBytes;            // 8 panels x NH x 128 B
  uint8_t* p_s = q_s + kQBytes;                          // 2 panels x NH x 128 B
  MlaBars* bars = reinterpret_cast<MlaBars*>(p_s + kPBytes);
  float* smax = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 64);   // [4][NH]
  float* m_run = smax + 4 * NH;                          // [NH]
  float* alpha_s = m_run + NH;                           // [NH]
  float* lsum = alpha_s + NH;                            // [4][NH]
  float* l_run = lsum + 4 * NH;                          // [NH]
  int* flags = reinterpret_cast<int*>(l_run + NH);       // [0] any head rescaled in this block

  const int t = blockIdx.x, sp = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_swa = a.swa_lens[t];
  const int n_top = a.topk_slots ? a.topk_lens[t] : 0;
  const int L = n_swa + n_top;
  const int r_begin = sp * a.rows_per_split;
  const int r_end = min(L, r_begin + a.rows_per_split);
  const int n_blocks = r_end > r_begin ? (r_end - r_begin + kRows - 1) / kRows : 0;
  float* prow = a.partial + (static_cast<long long>(t) * a.n_splits + sp) * a.nh * (kD + 2);

  if (threadIdx.x == 0) STK_TRACE(0);
  if (n_blocks == 0 && a.out != nullptr) {
    // no keys at all: only the sink takes probability mass, the output is zero
    __nv_bfloat16* orow = a.out + static_cast<long long>(t) * a.ldo;
    for (int i = threadIdx.x; i < a.nh * kD; i += blockDim.x) orow[i] = __float2bfloat16(0.f);
    return;
  }
  if (n_blocks == 0) {
    for (int i = threadIdx.x; i < a.nh * (kD + 2); i += blockDim.x) {
      const int d = i % (kD + 2);
      prow[i] = d == kD ? -INFINITY : 0.f;
    }
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(&bars->k_full, kProducerWarps);
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->p_full, kSoftmaxWarps);
    mbar_init(&bars->pv_done, 1);
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  // Q -> shared memory, K-major panels [NH x 64 dims], 128-byte swizzle; heads >= nh are zero.
  // All global loads of a thread are issued before its stores.
  {
    constexpr int kChunks = NH * (kD / 8);
    constexpr int kPer = (kChunks + kThreads - 1) / kThreads;
    uint4 qv[kPer];
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int i = threadIdx.x + j * kThreads;
      qv[j] = make_uint4(0, 0, 0, 0);
      if (i < kChunks) {
        const int h = i / (kD / 8), c8 = i % (kD / 8);
        if (h < a.nh) qv[j] = __ldg(reinterpret_cast<const uint4*>(a.q + t * a.ldt + static_cast<long long>(h) * kD + c8 * 8));
      }
    }
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int i = threadIdx.x + j * kThreads;
      if (i < kChunks) {
        const int h = i / (kD / 8), c8 = i % (kD / 8);
        const int panel = c8 >> 3, c = c8 & 7;
        *reinterpret_cast<uint4*>(q_s + panel * (NH * 128) + h * 128 + ((c ^ (h & 7)) << 4)) = qv[j];
      }
    }
  }
  if (threadIdx.x < NH) { m_run[threadIdx.x] = -INFINITY; l_run[threadIdx.x] = 0.f; }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x == 0) STK_TRACE(1);
  const uint32_t tmem_base = bars->tmem_base;
  const uint32_t tmem_s = tmem_base;                     // S^T: NH columns
  const uint32_t tmem_o = tmem_base + NH;                // 4 x NH columns

  if (warp == 0) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      constexpr uint32_t kIdescQK = umma_idesc(1u, 1u, 128, NH);
      constexpr uint32_t kIdescPV = umma_idesc(1u, 1u, 128, NH) | (1u << 15);     // A is MN-major
      bool ok = true;
      for (int b = 0; b < n_blocks && ok; ++b) {
        const uint32_t ph = b & 1;
        if (!mbar_wait(&bars->k_full, ph, a.status, 600)) { ok = false; break; }
        if (b == 0) STK_TRACE(2);
        tc_fence_after();
#pragma unroll
        for (int p = 0; p < kPanels; ++p) {
          const uint64_t ad = umma_desc_sw128(smem_u32(k_s + p * kPanelBytes));
          const uint64_t bd = umma_desc_sw128(smem_u32(q_s + p * (NH * 128)));
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f16(tmem_s, ad + 2 * k, bd + 2 * k, kIdescQK, (p | k) != 0);
        }
        umma_commit(&bars->s_full);
        if (!mbar_wait(&bars->p_full, ph, a.status, 601)) { ok = false; break; }
        if (b == 0) STK_TRACE(4);
        tc_fence_after();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t ad = umma_desc_mn_sw128(smem_u32(k_s + (2 * j) * kPanelBytes + kk * 2048), kPanelBytes);
            const uint64_t bd = umma_desc_sw128(smem_u32(p_s + (kk >> 2) * (NH * 128))) + 2 * (kk & 3);
            umma_f16(tmem_o + j * NH, ad, bd, kIdescPV, (b > 0 || kk > 0) ? 1u : 0u);
          }
        }
        umma_commit(&bars->pv_done);
      }
      if (!ok) bars->abort_flag = 1;
    }
  } else if (warp <= kSoftmaxWarps) {
    // ------------------------------- softmax / epilogue -------------------------------
    const int q4 = warp & 3;                              // TMEM lane quarter
    const int row = q4 * 32 + lane;                       // row of the block owned by this thread
    const int sw = warp - 1;                              // 0..3
    const uint32_t lane_addr = static_cast<uint32_t>(q4 * 32) << 16;
    const float sl2 = a.scale * 1.4426950408889634f;
    const int own = threadIdx.x - 32;                     // owner thread of head `own` when < NH
    bool ok = true;
    for (int b = 0; b < n_blocks && ok; ++b) {
      const uint32_t ph = b & 1;
      const int li = r_begin + b * kRows + row;
      bool valid = li < r_end;
      if (valid) {
        const int slot = li < n_swa ? a.swa_slots[static_cast<long long>(t) * a.swa_ld + li]
                                    : a.topk_slots[static_cast<long long>(t) * a.topk_ld + (li - n_swa)];
        valid = slot >= 0;
      }
      if (!mbar_wait(&bars->s_full, ph, a.status, 610)) { ok = false; break; }
      if (b == 0 && threadIdx.x == 32) STK_TRACE(3);
      tc_fence_after();
      float s[NH];
#pragma unroll
      for (int c = 0; c < NH; c += 16) {
        uint32_t r16[16];
        tmem_ld_32x16(tmem_s + lane_addr + c, r16);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) s[c + i] = valid ? __uint_as_float(r16[i]) * sl2 : -INFINITY;
      }
      if (b == 0 && threadIdx.x == 32) STK_TRACE(8);
      // block maximum per head over the 128 rows (destroys s; it is re-read from TMEM below)
      bfly_reduce_store<NH, true>(s, smax + sw * NH, lane);
      if (b == 0 && threadIdx.x == 32) STK_TRACE(9);
      named_bar_sync(2, kSoftmaxWarps * 32);
      if (own < NH) {
        const float bm = fmaxf(fmaxf(smax[own], smax[NH + own]), fmaxf(smax[2 * NH + own], smax[3 * NH + own]));
        const float mo = m_run[own];
        const float mn = fmaxf(mo, bm);
        const float al = (mo == -INFINITY || mn == -INFINITY) ? 1.f : exp2f(mo - mn);     // mo == mn -> 1
        alpha_s[own] = al;
        m_run[own] = mn;
        l_run[own] *= al;
      }
      if (threadIdx.x == 32) flags[0] = 0;
      named_bar_sync(2, kSoftmaxWarps * 32);
      if (own < NH && b > 0 && alpha_s[own] != 1.f) flags[0] = 1;
      if (b == 0 && threadIdx.x == 32) STK_TRACE(11);
      // P = exp2(s - m), bf16, written as the K-major B operand [head][row]
      const int ppanel = row >> 6, prow_in = row & 63;
      uint8_t* pdst = p_s + ppanel * (NH * 128) + (prow_in & 7) * 2;
#pragma unroll
      for (int c = 0; c < NH; c += 16) {
        uint32_t r16[16];
        tmem_ld_32x16(tmem_s + lane_addr + c, r16);
        float mloc[16];
#pragma unroll
        for (int i = 0; i < 16; i += 4) {
          const float4 m4 = *reinterpret_cast<const float4*>(m_run + c + i);
          mloc[i] = m4.x; mloc[i + 1] = m4.y; mloc[i + 2] = m4.z; mloc[i + 3] = m4.w;
        }
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int h = c + i;
          const float p = (!valid || mloc[i] == -INFINITY) ? 0.f : ex2_approx(__uint_as_float(r16[i]) * sl2 - mloc[i]);
          const __nv_bfloat16 pb = __float2bfloat16(p);
          s[h] = __bfloat162float(pb);
          *reinterpret_cast<__nv_bfloat16*>(pdst + h * 128 + (((prow_in >> 3) ^ (h & 7)) << 4)) = pb;
        }
      }
      // row sums of P per head (the same rounded values the tensor core multiplies)
      bfly_reduce_store<NH, false>(s, lsum + sw * NH, lane);
      if (b == 0 && threadIdx.x == 32) STK_TRACE(12);
      named_bar_sync(2, kSoftmaxWarps * 32);
      if (b == 0 && threadIdx.x == 32) STK_TRACE(13);
      if (own < NH) l_run[own] += lsum[own] + lsum[NH + own] + lsum[2 * NH + own] + lsum[3 * NH + own];
      if (flags[0]) {
        // some head's maximum moved: scale the O^T columns (the previous block's PV has completed,
        // because this block's rows could only be loaded after it)
#pragma unroll
        for (int c = 0; c < NH; c += 16) {
          float al[16];
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            const float4 a4 = *reinterpret_cast<const float4*>(alpha_s + c + i);
            al[i] = a4.x; al[i + 1] = a4.y; al[i + 2] = a4.z; al[i + 3] = a4.w;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t r16[16];
            tmem_ld_32x16(tmem_o + j * NH + c + lane_addr, r16);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) r16[i] = __float_as_uint(__uint_as_float(r16[i]) * al[i]);
            tmem_st_32x16(tmem_o + j * NH + c + lane_addr, r16);
          }
        }
        tmem_st_wait();
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full);
    }
    // ---- epilogue: wait for the last PV, write the partial ----
    if (ok) ok = mbar_wait(&bars->pv_done, (n_blocks - 1) & 1, a.status, 611);
    if (threadIdx.x == 32) STK_TRACE(5);
    tc_fence_after();
    if (ok && a.out != nullptr) {
      // direct output: per-head factor exp(m - M) / (exp(sink - M) + l * exp(m - M)) with M = max(sink, m)
      named_bar_sync(2, kSoftmaxWarps * 32);
      if (own < NH) {
        const float m_nat = m_run[own] * 0.6931471805599453f;
        const float sk = (a.sink != nullptr && own < a.nh) ? a.sink[own] : -INFINITY;
        const float M = fmaxf(sk, m_nat);
        float f = 0.f;
        if (m_nat != -INFINITY) {
          const float w = __expf(m_nat - M);
          const float denom = (sk != -INFINITY ? __expf(sk - M) : 0.f) + l_run[own] * w;
          f = denom > 0.f ? w / denom : 0.f;
        }
        alpha_s[own] = f;
      }
      named_bar_sync(2, kSoftmaxWarps * 32);
      __nv_bfloat16* orow = a.out + static_cast<long long>(t) * a.ldo;
      const float pos = a.positions != nullptr ? static_cast<float>(a.positions[t]) : 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int d = j * 128 + row;
        const bool rot = a.positions != nullptr && j == 3 && q4 >= 2;      // d >= 448: warp-uniform
        float sn = 0.f, cs = 1.f;
        if (rot) sincosf(pos * a.inv_freq[(d - kNope) >> 1], &sn, &cs);
#pragma unroll
        for (int c = 0; c < NH; c += 16) {
          uint32_t r16[16];
          tmem_ld_32x16(tmem_o + j * NH + c + lane_addr, r16);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if (c + i < a.nh) {
              float v = __uint_as_float(r16[i]) * alpha_s[c + i];
              if (rot) {
                // the pair (even d, d + 1) sits in neighbouring lanes; values are rounded to bf16 before the rotation,
                // as the separate combine pass does
                v = __bfloat162float(__float2bfloat16(v));
                const float p = __shfl_xor_sync(0xffffffffu, v, 1);
                v = (d & 1) ? (-p * sn + v * cs) : (v * cs + p * sn);
              }
              orow[static_cast<long long>(c + i) * kD + d] = __float2bfloat16(v);
            }
          }
        }
      }
    } else if (ok) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int c = 0; c < NH; c += 16) {
          uint32_t r16[16];
          tmem_ld_32x16(tmem_o + j * NH + c + lane_addr, r16);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if (c + i < a.nh) prow[(c + i) * (kD + 2) + j * 128 + row] = __uint_as_float(r16[i]);
          }
        }
      }
      named_bar_sync(2, kSoftmaxWarps * 32);
      if (own < a.nh) {
        prow[own * (kD + 2) + kD] = m_run[own] * 0.6931471805599453f;      // back to natural-log units
        prow[own * (kD + 2) + kD + 1] = l_run[own];
      }
    }
  } else {
    // ------------------------------- producers -------------------------------
    const int pt = threadIdx.x - 32 * (1 + kSoftmaxWarps);     // 0..255
    const int row = pt >> 1, half = pt & 1;
    bool ok = true;
    for (int b = 0; b < n_blocks && ok; ++b) {
      if (b > 0) {
        if (!mbar_wait(&bars->pv_done, (b - 1) & 1, a.status, 620)) { ok = false; break; }
      }
      const int li = r_begin + b * kRows + row;
      int slot = -1;
      const uint8_t* cbase = a.swa_base;
      long long cstride = a.swa_stride;
      if (li < r_end) {
        if (li < n_swa) slot = a.swa_slots[static_cast<long long>(t) * a.swa_ld + li];
        else { slot = a.topk_slots[static_cast<long long>(t) * a.topk_ld + (li - n_swa)]; cbase = a.comp_base; cstride = a.comp_stride; }
      }
      const int sw7 = row & 7;
      if (slot < 0) {
        const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int pp = 0; pp < 4; ++pp) {
          uint8_t* dst = k_s + (half * 4 + pp) * kPanelBytes + row * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(dst + (c << 4)) = z;
        }
      } else {
        const uint8_t* pbase = cbase + static_cast<long long>(slot >> 6) * cstride;
        const int rr = slot & 63;
        const uint8_t* drow = pbase + static_cast<long long>(rr) * kDataBytes;
        const uint8_t* srow = pbase + 64LL * kDataBytes + rr * 8;
        const uint2 sc8 = *reinterpret_cast<const uint2*>(srow);
        // two fp8 panels at a time: issue the eight 16-byte loads, then convert and store
        auto fp8_panels2 = [&](int first_panel, int n_panels) {
          uint4 w[8];
#pragma unroll
          for (int v = 0; v < 8; ++v)
            if (v < n_panels * 4) w[v] = __ldg(reinterpret_cast<const uint4*>(drow + first_panel * 64) + v);
#pragma unroll
          for (int pp = 0; pp < 2; ++pp) {
            if (pp < n_panels) {
              const int panel = first_panel + pp;
              const uint32_t sbyte = ((panel < 4 ? sc8.x : sc8.y) >> (8 * (panel & 3))) & 0xff;
              const float sc = __uint_as_float(sbyte << 23);               // 2^(byte - 127)
              uint8_t* dst = k_s + panel * kPanelBytes + row * 128;
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                const uint4 x = w[pp * 4 + v];
                uint4 o0, o1;
                fp8x4_to_bf16x4(x.x, sc, o0.x, o0.y);
                fp8x4_to_bf16x4(x.y, sc, o0.z, o0.w);
                fp8x4_to_bf16x4(x.z, sc, o1.x, o1.y);
                fp8x4_to_bf16x4(x.w, sc, o1.z, o1.w);
                *reinterpret_cast<uint4*>(dst + (((2 * v) ^ sw7) << 4)) = o0;
                *reinterpret_cast<uint4*>(dst + (((2 * v + 1) ^ sw7) << 4)) = o1;
              }
            }
          }
        };
        if (half == 0) {
          fp8_panels2(0, 2);
          fp8_panels2(2, 2);
        } else {
          uint4 rp[8];
#pragma unroll
          for (int c = 0; c < 8; ++c) rp[c] = __ldg(reinterpret_cast<const uint4*>(drow + kNope) + c);   // 64 bf16 rope dims
          fp8_panels2(4, 2);
          fp8_panels2(6, 1);
          uint8_t* dst = k_s + 7 * kPanelBytes + row * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(dst + ((c ^ sw7) << 4)) = rp[c];
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->k_full);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) STK_TRACE(6);
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int NH>
static int launch_mla_tc(const MlaTcArgs& a, cudaStream_t st) {
  const int smem = kPanels * kPanelBytes + kPanels * NH * 128 + 2 * NH * 128 + 64 + (4 * NH + NH + NH + 4 * NH + NH) * 4 + 64 + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(sparse_mla_tc_kernel<NH>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return -3;
    configured = true;
  }
  dim3 grid(a.T, a.n_splits);
  launch_pdl(sparse_mla_tc_kernel<NH>, dim3(grid), dim3(kThreads), smem, st, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace stk

using namespace stk;

static int mla_tc_run(const void* q, long long ldt, const void* swa_cache, long long swa_stride, const void* comp_cache,
                      long long comp_stride, const int* swa_slots, int swa_ld, const int* swa_lens, const int* topk_slots,
                      int topk_ld, const int* topk_lens, float* workspace, int n_splits, int T, int nh, int D, int R,
                      int max_rows, float scale, void* out, long long ldo, const float* sink, const int64_t* positions,
                      const float* inv_freq, int* status, void* trace, void* stream) {
  if (T <= 0) return 0;
  if (D != kD || R != kR || nh > 64 || nh < 1) return -20;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (ldt % 8)) return -21;
  if (out != nullptr && n_splits != 1) return -22;
  MlaTcArgs a;
  a.q = (const __nv_bfloat16*)q; a.ldt = ldt;
  a.swa_base = (const uint8_t*)swa_cache; a.swa_stride = swa_stride;
  a.comp_base = (const uint8_t*)comp_cache; a.comp_stride = comp_stride;
  a.swa_slots = swa_slots; a.swa_ld = swa_ld; a.swa_lens = swa_lens;
  a.topk_slots = topk_slots; a.topk_ld = topk_ld; a.topk_lens = topk_lens;
  a.partial = workspace; a.T = T; a.nh = nh; a.n_splits = n_splits;
  a.out = (__nv_bfloat16*)out; a.ldo = ldo; a.sink = sink; a.positions = positions; a.inv_freq = inv_freq;
  const int rps = (max_rows + n_splits - 1) / n_splits;
  a.rows_per_split = ((rps + kRows - 1) / kRows) * kRows;
  a.scale = scale; a.status = status; a.trace = (unsigned long long*)trace;
  cudaStream_t st = (cudaStream_t)stream;
  if (nh <= 16) return launch_mla_tc<16>(a, st);
  if (nh <= 32) return launch_mla_tc<32>(a, st);
  return launch_mla_tc<64>(a, st);
}

// Same contract as stk_sparse_mla (partials + combine), restricted to fp8_ds_mla rows with D = 512,
// R = 64 and at most 64 local heads.  Returns -20 for shapes it does not cover.
STK_API int stk_sparse_mla_tc(const void* q, long long ldt, const void* swa_cache, long long swa_stride,
                              const void* comp_cache, long long comp_stride, const int* swa_slots, int swa_ld,
                              const int* swa_lens, const int* topk_slots, int topk_ld, const int* topk_lens,
                              float* workspace, int n_splits, int T, int nh, int D, int R, int max_rows, float scale,
                              int* status, void* trace, void* stream) {
  return mla_tc_run(q, ldt, swa_cache, swa_stride, comp_cache, comp_stride, swa_slots, swa_ld, swa_lens, topk_slots,
                    topk_ld, topk_lens, workspace, n_splits, T, nh, D, R, max_rows, scale, nullptr, 0, nullptr, nullptr,
                    nullptr, status, trace, stream);
}

// One CTA per token over its whole row list, final output written by the kernel (sink merged, normalised, inverse
// RoPE on the rope dims when positions != null): for steps with enough tokens to fill the GPU without row splits.
STK_API int stk_sparse_mla_tc_out(const void* q, long long ldt, const void* swa_cache, long long swa_stride,
                                  const void* comp_cache, long long comp_stride, const int* swa_slots, int swa_ld,
                                  const int* swa_lens, const int* topk_slots, int topk_ld, const int* topk_lens, int T,
                                  int nh, int D, int R, int max_rows, float scale, void* out, long long ldo,
                                  const float* sink, const int64_t* positions, const float* inv_freq, int* status,
                                  void* stream) {
  if (out == nullptr) return -23;
  return mla_tc_run(q, ldt, swa_cache, swa_stride, comp_cache, comp_stride, swa_slots, swa_ld, swa_lens, topk_slots,
                    topk_ld, topk_lens, nullptr, 1, T, nh, D, R, max_rows, scale, out, ldo, sink, positions, inv_freq,
                    status, nullptr, stream);
}
