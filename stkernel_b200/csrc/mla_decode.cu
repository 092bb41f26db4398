// Sparse multi-head latent attention for decode-sized steps (a handful of tokens, 8-64 query heads).
//
// At these sizes the op is a few megabytes and a few million multiply-adds per token: neither bytes nor flops but
// the length of the dependent chain sets its time, and a tensor-core tile pipeline (gather -> dequantise to shared
// memory -> MMA -> softmax -> MMA) is the longest chain there is.  This kernel keeps everything in registers:
//
//   * grid (splits, tokens, head blocks of 8): a CTA takes a contiguous share of the token's row list (sliding-window
//     rows, then top-k rows of the compressed cache) for 8 heads; its 8 warps are 4 row groups x 2 head groups of 4.
//   * a warp reads a cached fp8_ds_mla row as it lies in memory: lane l < 28 takes the 16 e4m3 codes of dims
//     [16 l, 16 l + 16) with their UE8M0 scale byte, every lane takes one bf16 pair of the 64 rope dims; K = V, so the
//     same registers serve q.k (packed half2, one block scale per lane) and the p.v accumulation (fp32).
//   * the per-head RMSNorm and RoPE of q happen here, on load (no separate launch rewrites q in place);
//   * scores of 4 heads are reduced across the warp with a transposing butterfly (6 shuffles for 4 sums), the softmax
//     is updated once per batch of 4 rows;
//   * the row groups merge through shared memory, the CTA writes one un-normalised partial (o, m, l) per head, and a
//     second small kernel merges the splits in one round of independent loads, adds the sink to the denominator,
//     applies the inverse RoPE the output projection expects and writes bf16.
//
// Same contract as the tensor-core kernel (attention_tc.cu), which serves prefill and large decode batches.  Takes the
// place of the reference's flashinfer_trtllm_batch_decode_sparse_mla_dsv4 decode call
// (overlay/flashinfer_sparse.py:323-400) and of the q half of its fused qnorm/rope/insert op
// (overlay/attention.py:704-729).
#define STK_PDL_CLASS 128
#include <string.h>

#include "common.cuh"

namespace stk {

constexpr int kMdD = 512, kMdR = 64, kMdNope = kMdD - kMdR;   // row geometry (fp8_ds_mla)
constexpr int kMdRowData = kMdNope + 2 * kMdR;                // 576 data bytes per row
constexpr int kMdHeads = 8;                                   // heads per CTA
constexpr int kMdBatch = 4;                                   // rows per softmax update
constexpr int kMdP = 516;                                     // floats per partial: 512 o, m, l, 2 pad (16-byte rows)

struct MdCache {
  const uint8_t* base;
  long long page_stride;
};

struct MdArgs {
  const __nv_bfloat16* q;      // [T, nh, 512]
  long long ldt;
  MdCache swa, comp;
  const int* swa_slots; int swa_ld; const int* swa_lens;
  const int* topk_slots; int topk_ld; const int* topk_lens;   // may be null
  int swa_ld_rows, topk_rows;  // widths of the two lists (the static split runs over their concatenation)
  const int64_t* positions;    // [T]   (q RoPE)
  const float* inv_freq;       // [32]
  float* partial;              // [T, S, nh, kMdP]
  int nh, S;
  float scale, eps;
  int prep_q;                  // 1: q arrives raw: per-head weightless RMSNorm + RoPE here
  long long swa_slots_n, comp_slots_n;   // extents for the index guard
  int* status;
  // Insert of the step's own latent rows (pure decode: every request contributes one token, so no token of the step
  // attends to another token's new row): the warp that meets the token's own slot in the window list builds the cached
  // row from the raw kv projection itself -- RMSNorm, RoPE, UE8M0 block quantisation, exactly as the stand-alone insert
  // -- writes it to the cache and attends to it from registers.  No insert launch in front of the attention.
  const __nv_bfloat16* kv_new;     // [T, 512] raw kv rows, or nullptr
  long long kv_ld;
  const __nv_bfloat16* kv_norm_w;  // [512]
  const int64_t* cur_slot;         // [T] slot of each token's own row in the window cache (-1: none)
  uint8_t* swa_write;              // the window cache, writable
};

__device__ __forceinline__ __half2 h2_from_raw(__half2_raw r) { return *reinterpret_cast<__half2*>(&r); }
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// grid (S, T, nh / 8), 512 threads = 8 row groups x 2 head groups.  The split of the row list is static: CTA s owns
// the virtual rows [32 s, 32 s + 32), where virtual row v < W is entry v of the window list and v >= W entry v - W of
// the top-k list (entries past the lists' lengths are masked).  Nothing about the split depends on loaded data, so a
// warp requests q, the list lengths and its four slots together, then its four rows together: two round trips.
__global__ void __launch_bounds__(512)
mla_decode_split_kernel(const MdArgs a) {
  extern __shared__ __align__(16) float sm[];   // [16 warps][4 heads][kMdP] for the cross-row-group merge
  const int s = blockIdx.x, t = blockIdx.y, hb = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hg = warp & 1, rg = warp >> 1;            // head group (4 heads), row group (4 rows)
  const int head0 = hb * kMdHeads + hg * 4;
  const int W = a.swa_ld_rows;
  const int v0 = s * 32 + rg * kMdBatch;
  pdl_wait();
  pdl_trigger();

  // ---- round trip 1: list lengths, this warp's four slots, q of this warp's four heads ----
  const int n_swa = __ldg(a.swa_lens + t);
  const int n_top = a.topk_slots != nullptr ? __ldg(a.topk_lens + t) : 0;
  int slot[kMdBatch];
  bool in_swa[kMdBatch];
#pragma unroll
  for (int j = 0; j < kMdBatch; ++j) {
    const int v = v0 + j;
    in_swa[j] = v < W;
    slot[j] = -1;
    if (in_swa[j]) slot[j] = __ldg(a.swa_slots + t * a.swa_ld + v);
    else if (a.topk_slots != nullptr && v - W < a.topk_rows) slot[j] = __ldg(a.topk_slots + t * a.topk_ld + (v - W));
  }
  __half2 qn[4][8];
  __half2 qr[4];
  {
    uint4 qv[4][2];
    uint32_t qrp[4];
#pragma unroll
    for (int hh = 0; hh < 4; ++hh) {
      const __nv_bfloat16* qrow = a.q + t * a.ldt + static_cast<long long>(head0 + hh) * kMdD;
      qv[hh][0] = qv[hh][1] = make_uint4(0, 0, 0, 0);
      if (lane < 28) {
        qv[hh][0] = *reinterpret_cast<const uint4*>(qrow + lane * 16);
        qv[hh][1] = *reinterpret_cast<const uint4*>(qrow + lane * 16 + 8);
      }
      qrp[hh] = *reinterpret_cast<const uint32_t*>(qrow + kMdNope + 2 * lane);
    }
    const float pos = a.prep_q ? static_cast<float>(__ldg(a.positions + t)) : 0.f;
    float sn = 0.f, cs = 1.f;
    if (a.prep_q) sincosf(pos * __ldg(a.inv_freq + lane), &sn, &cs);
#pragma unroll
    for (int hh = 0; hh < 4; ++hh) {
      float f[16];
      const uint32_t w[8] = {qv[hh][0].x, qv[hh][0].y, qv[hh][0].z, qv[hh][0].w, qv[hh][1].x, qv[hh][1].y, qv[hh][1].z, qv[hh][1].w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 p = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
        f[2 * i] = p.x; f[2 * i + 1] = p.y;
      }
      float2 rp = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qrp[hh]));
      if (a.prep_q) {
        float ss = fmaf(rp.x, rp.x, rp.y * rp.y);
#pragma unroll
        for (int i = 0; i < 16; ++i) ss = fmaf(f[i], f[i], ss);
        const float r = rsqrtf(warp_sum(ss) / static_cast<float>(kMdD) + a.eps);
#pragma unroll
        for (int i = 0; i < 16; ++i) f[i] *= r;
        const float x = rp.x * r, y = rp.y * r;
        rp.x = x * cs - y * sn;
        rp.y = x * sn + y * cs;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) qn[hh][i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      qr[hh] = __floats2half2_rn(rp.x, rp.y);
    }
  }

  // ---- round trip 2: the four rows ----
  uint4 kraw[kMdBatch];
  uint32_t rraw[kMdBatch];
  uint32_t sbyte[kMdBatch];
  bool valid[kMdBatch];
  const long long own_slot = a.kv_new != nullptr ? __ldg(a.cur_slot + t) : -1;
  int own_j = -1;
#pragma unroll
  for (int j = 0; j < kMdBatch; ++j) {
    const int v = v0 + j;
    const int idx = in_swa[j] ? v : v - W;
    valid[j] = slot[j] >= 0 && idx < (in_swa[j] ? n_swa : n_top);
    const long long lim = in_swa[j] ? a.swa_slots_n : a.comp_slots_n;
    if (valid[j] && slot[j] >= lim) {
      set_status(a.status, kBadIndex, t);
      valid[j] = false;
    }
    kraw[j] = make_uint4(0, 0, 0, 0);
    rraw[j] = 0;
    sbyte[j] = 127;
    if (valid[j] && in_swa[j] && own_slot >= 0 && static_cast<long long>(slot[j]) == own_slot) {
      own_j = j;                          // built below, once, outside this unrolled loop
    } else if (valid[j]) {
      const MdCache& c = in_swa[j] ? a.swa : a.comp;
      const uint8_t* page = c.base + static_cast<long long>(slot[j] >> 6) * c.page_stride;
      const uint8_t* drow = page + static_cast<long long>(slot[j] & 63) * kMdRowData;
      if (lane < 28) {
        kraw[j] = __ldg(reinterpret_cast<const uint4*>(drow + lane * 16));
        sbyte[j] = __ldg(page + 64LL * kMdRowData + (slot[j] & 63) * 8 + (lane >> 2));
      }
      rraw[j] = __ldg(reinterpret_cast<const uint32_t*>(drow + kMdNope + lane * 4));
    }
  }
  if (own_j >= 0) {
    uint4 own_k;
    uint32_t own_r, own_sb = 127;
      // ---- this token's own row: built here, stored, used from registers ----
      const __nv_bfloat16* src = a.kv_new + t * a.kv_ld;
      float f[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) f[i] = 0.f;
      float wn[16];
      if (lane < 28) {
        const uint4 x0 = *reinterpret_cast<const uint4*>(src + lane * 16), x1 = *reinterpret_cast<const uint4*>(src + lane * 16 + 8);
        const uint4 w0 = __ldg(reinterpret_cast<const uint4*>(a.kv_norm_w + lane * 16));
        const uint4 w1 = __ldg(reinterpret_cast<const uint4*>(a.kv_norm_w + lane * 16 + 8));
        const uint32_t xw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
        const uint32_t ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float2 p = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xw[i]));
          const float2 q2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ww[i]));
          f[2 * i] = p.x; f[2 * i + 1] = p.y;
          wn[2 * i] = q2.x; wn[2 * i + 1] = q2.y;
        }
      }
      float2 rp = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + kMdNope + 2 * lane));
      const float2 rw = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a.kv_norm_w + kMdNope + 2 * lane));
      float ss = fmaf(rp.x, rp.x, rp.y * rp.y);
#pragma unroll
      for (int i = 0; i < 16; ++i) ss = fmaf(f[i], f[i], ss);
      const float nr = rsqrtf(warp_sum(ss) / static_cast<float>(kMdD) + a.eps);
      float amax = 0.f;
      if (lane < 28) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          f[i] = bf16_to_f(__float2bfloat16(f[i] * nr * wn[i]));
          amax = fmaxf(amax, fabsf(f[i]));
        }
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));       // a quantisation block = 64 dims = 4 lanes
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      uint8_t sb;
      const float sc = ue8m0_scale(amax, &sb);
      const float inv_sc = 1.f / sc;
      uint32_t codes[4] = {0, 0, 0, 0};
      if (lane < 28) {
#pragma unroll
        for (int i = 0; i < 16; ++i) codes[i >> 2] |= static_cast<uint32_t>(f_to_fp8(f[i] * inv_sc)) << (8 * (i & 3));
        own_sb = sb;
      }
      own_k = make_uint4(codes[0], codes[1], codes[2], codes[3]);
      {
        // RoPE of the pair at the token's position (rounded to bf16 after the norm and again after the rotation, as the
        // separate norm and insert kernels store them)
        const float x = bf16_to_f(__float2bfloat16(rp.x * nr * rw.x)), y = bf16_to_f(__float2bfloat16(rp.y * nr * rw.y));
        float sn2, cs2;
        sincosf(static_cast<float>(__ldg(a.positions + t)) * __ldg(a.inv_freq + lane), &sn2, &cs2);
        own_r = pack2(x * cs2 - y * sn2, x * sn2 + y * cs2);
      }
      // one CTA per token stores the row (every head block and split that meets the slot computes the same bytes)
      if (hb == 0) {
        uint8_t* page = a.swa_write + static_cast<long long>(own_slot >> 6) * a.swa.page_stride;
        uint8_t* drow = page + static_cast<long long>(own_slot & 63) * kMdRowData;
        uint8_t* srow = page + 64LL * kMdRowData + (own_slot & 63) * 8;
        if (lane < 28) {
          *reinterpret_cast<uint4*>(drow + lane * 16) = own_k;
          if ((lane & 3) == 0) srow[lane >> 2] = sb;
        } else if (lane == 28) {
          srow[7] = 0;
        }
        *reinterpret_cast<uint32_t*>(drow + kMdNope + lane * 4) = own_r;
      }
#pragma unroll
    for (int j = 0; j < kMdBatch; ++j)
      if (j == own_j) { kraw[j] = own_k; rraw[j] = own_r; sbyte[j] = own_sb; }
  }
  // a CTA none of whose 32 rows exists only marks its partials empty
  const bool cta_any = (s * 32 < n_swa) || (s * 32 + 32 > W && s * 32 < W + n_top);
  if (!cta_any) {
    if (threadIdx.x < kMdHeads)
      a.partial[((static_cast<long long>(t) * a.S + s) * a.nh + hb * kMdHeads + threadIdx.x) * kMdP + 512] = -INFINITY;
    return;
  }

  float acc[4][18];
  float m_run = -INFINITY, l_run = 0.f;      // of head (lane >> 3) -- replicated over 8 lanes
  {
    float sc_row[kMdBatch];
    float score[kMdBatch];
    __half2 kh[kMdBatch][9];
#pragma unroll
    for (int j = 0; j < kMdBatch; ++j) {
      const uint32_t w[4] = {kraw[j].x, kraw[j].y, kraw[j].z, kraw[j].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        kh[j][2 * i] = h2_from_raw(__nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] & 0xffff), __NV_E4M3));
        kh[j][2 * i + 1] = h2_from_raw(__nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] >> 16), __NV_E4M3));
      }
      kh[j][8] = __float22half2_rn(__bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rraw[j])));
      sc_row[j] = exp2f(static_cast<float>(sbyte[j]) - 127.f);
      // four heads' partial dot products of this lane
      float d[4];
#pragma unroll
      for (int hh = 0; hh < 4; ++hh) {
        __half2 p = __hmul2(qn[hh][0], kh[j][0]);
#pragma unroll
        for (int i = 1; i < 8; ++i) p = __hfma2(qn[hh][i], kh[j][i], p);
        const float2 pf = __half22float2(p);
        const float2 rf = __half22float2(__hmul2(qr[hh], kh[j][8]));
        d[hh] = (pf.x + pf.y) * sc_row[j] + (rf.x + rf.y);
      }
      // transposing butterfly: after two exchange steps lane group (lane >> 3) holds the sum of head (lane >> 3)
      const bool up = lane & 16;
      const float send0 = up ? d[0] : d[2], send1 = up ? d[1] : d[3];
      const float keep0 = up ? d[2] : d[0], keep1 = up ? d[3] : d[1];
      const float g0 = keep0 + __shfl_xor_sync(0xffffffffu, send0, 16);
      const float g1 = keep1 + __shfl_xor_sync(0xffffffffu, send1, 16);
      const bool up2 = lane & 8;
      const float sendb = up2 ? g0 : g1, keepb = up2 ? g1 : g0;
      float v = keepb + __shfl_xor_sync(0xffffffffu, sendb, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 4);
      v += __shfl_xor_sync(0xffffffffu, v, 2);
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      score[j] = valid[j] ? v * a.scale : -INFINITY;
    }
    // ---- softmax over the batch (head lane >> 3 in this lane) ----
    float bm = score[0];
#pragma unroll
    for (int j = 1; j < kMdBatch; ++j) bm = fmaxf(bm, score[j]);
    float p[kMdBatch];
#pragma unroll
    for (int j = 0; j < kMdBatch; ++j) p[j] = 0.f;
    if (bm != -INFINITY) {
      m_run = bm;
#pragma unroll
      for (int j = 0; j < kMdBatch; ++j) {
        p[j] = __expf(score[j] - bm);
        l_run += p[j];
      }
    }
    // ---- p.v: every lane needs p of all four heads.  The four rows of the batch accumulate in packed fp16 (p <= 1
    // times the row's block scale, times an e4m3 code: four terms stay far inside the format), widened once. ----
#pragma unroll
    for (int hh = 0; hh < 4; ++hh) {
      __half2 an[8], ar;
#pragma unroll
      for (int j = 0; j < kMdBatch; ++j) {
        const float ph = __shfl_sync(0xffffffffu, p[j], hh * 8);
        const __half2 pn = __float2half2_rn(ph * sc_row[j]), pr = __float2half2_rn(ph);
        if (j == 0) {
#pragma unroll
          for (int i = 0; i < 8; ++i) an[i] = __hmul2(pn, kh[j][i]);
          ar = __hmul2(pr, kh[j][8]);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) an[i] = __hfma2(pn, kh[j][i], an[i]);
          ar = __hfma2(pr, kh[j][8], ar);
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 v = __half22float2(an[i]);
        acc[hh][2 * i] = v.x;
        acc[hh][2 * i + 1] = v.y;
      }
      const float2 v = __half22float2(ar);
      acc[hh][16] = v.x;
      acc[hh][17] = v.y;
    }
  }

  // ---- merge the eight row groups of each head group through shared memory ----
  float* mine = sm + static_cast<long long>(warp) * 4 * kMdP;
#pragma unroll
  for (int hh = 0; hh < 4; ++hh) {
    float* o = mine + hh * kMdP;
    if (lane < 28) {
#pragma unroll
      for (int i = 0; i < 16; i += 4)
        *reinterpret_cast<float4*>(o + lane * 16 + i) = make_float4(acc[hh][i], acc[hh][i + 1], acc[hh][i + 2], acc[hh][i + 3]);
    }
    *reinterpret_cast<float2*>(o + kMdNope + 2 * lane) = make_float2(acc[hh][16], acc[hh][17]);
    const float mh = __shfl_sync(0xffffffffu, m_run, hh * 8), lh = __shfl_sync(0xffffffffu, l_run, hh * 8);
    if (lane == 0) { o[512] = mh; o[513] = lh; }
  }
  __syncthreads();
  // 64 threads per head: the eight row groups' weights exp(m_r - M) once per thread, then 8 elements each
  float* dst = a.partial + ((static_cast<long long>(t) * a.S + s) * a.nh + hb * kMdHeads) * kMdP;
  {
    const int h = threadIdx.x >> 6, e0 = threadIdx.x & 63;
    const int g = h >> 2, hh = h & 3;
    float wr[8], M = -INFINITY;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      wr[r] = sm[((r * 2 + g) * 4 + hh) * kMdP + 512];
      M = fmaxf(M, wr[r]);
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) wr[r] = (wr[r] == -INFINITY) ? 0.f : __expf(wr[r] - M);
    for (int e = e0; e < 514; e += 64) {
      float v = 0.f;
      if (e == 512) {
        v = M;
      } else {
#pragma unroll
        for (int r = 0; r < 8; ++r) v = fmaf(sm[((r * 2 + g) * 4 + hh) * kMdP + e], wr[r], v);
      }
      dst[h * kMdP + e] = v;
    }
  }
}

constexpr int kMdMaxS = 128;

// grid (T * nh), 512 threads = 4 split groups x 128 threads of 4 dims.  Two round trips: (m, l) of every split, then
// the o rows of the non-empty splits, all requested together.
__global__ void __launch_bounds__(512)
mla_decode_merge_kernel(const float* __restrict__ partial, const float* __restrict__ sink, __nv_bfloat16* __restrict__ out,
                        long long ldo, int nh, int S, const int64_t* __restrict__ positions,
                        const float* __restrict__ inv_freq) {
  __shared__ float s_m[kMdMaxS], s_l[kMdMaxS], s_den[4];
  __shared__ __align__(16) float s_o[4][512];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x / nh, h = blockIdx.x % nh;
  const float* base = partial + (static_cast<long long>(t) * S * nh + h) * kMdP;
  const long long sstride = static_cast<long long>(nh) * kMdP;
  float pos = 0.f, ifr0 = 0.f, ifr1 = 0.f;
  const int sg = threadIdx.x >> 7, d = (threadIdx.x & 127) * 4;
  if (positions != nullptr && d >= kMdNope && sg == 0) {
    pos = static_cast<float>(__ldg(positions + t));
    ifr0 = __ldg(inv_freq + (d - kMdNope) / 2);
    ifr1 = __ldg(inv_freq + (d - kMdNope) / 2 + 1);
  }
  const float sk = sink != nullptr ? __ldg(sink + h) : -INFINITY;
  if (threadIdx.x < S) {
    const float m = base[threadIdx.x * sstride + 512];
    s_m[threadIdx.x] = m;
    s_l[threadIdx.x] = m == -INFINITY ? 0.f : base[threadIdx.x * sstride + 513];
  }
  __syncthreads();
  float M = sk;
  for (int s = 0; s < S; ++s) M = fmaxf(M, s_m[s]);
  float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
  float den = 0.f;
  // this thread's splits are sg, sg + 4, ...: eight rows are requested before the first is used
  for (int s0 = sg; s0 < S; s0 += 32) {
    float w[8];
    float4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int s = s0 + 4 * u;
      const float m = s < S ? s_m[s] : -INFINITY;
      w[u] = (m == -INFINITY) ? 0.f : __expf(m - M);
      v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (w[u] != 0.f) v[u] = *reinterpret_cast<const float4*>(base + s * sstride + d);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int s = s0 + 4 * u;
      if (w[u] != 0.f) den = fmaf(w[u], s_l[s], den);
      o.x = fmaf(v[u].x, w[u], o.x); o.y = fmaf(v[u].y, w[u], o.y); o.z = fmaf(v[u].z, w[u], o.z); o.w = fmaf(v[u].w, w[u], o.w);
    }
  }
  *reinterpret_cast<float4*>(&s_o[sg][d]) = o;
  if ((threadIdx.x & 127) == 0) s_den[sg] = den;
  __syncthreads();
  if (sg != 0) return;
  float dtot = (s_den[0] + s_den[1]) + (s_den[2] + s_den[3]);
  if (sink != nullptr && M != -INFINITY) dtot += __expf(sk - M);
  const float inv = dtot > 0.f ? 1.f / dtot : 0.f;
  float r[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) r[c] = ((s_o[0][d + c] + s_o[1][d + c]) + (s_o[2][d + c] + s_o[3][d + c])) * inv;
  if (positions != nullptr && d >= kMdNope) {
    const float ifr[2] = {ifr0, ifr1};
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      // round to bf16 first: a separate rotation pass would read the stored attention output
      const float x0 = bf16_to_f(__float2bfloat16(r[2 * p])), x1 = bf16_to_f(__float2bfloat16(r[2 * p + 1]));
      float sn, cs;
      sincosf(pos * ifr[p], &sn, &cs);
      r[2 * p] = x0 * cs + x1 * sn;
      r[2 * p + 1] = -x0 * sn + x1 * cs;
    }
  }
  *reinterpret_cast<uint2*>(out + t * ldo + static_cast<long long>(h) * kMdD + d) =
      make_uint2(pack2(r[0], r[1]), pack2(r[2], r[3]));
}

}  // namespace stk

using namespace stk;

// Splits of the (window + top-k) row list: 32 rows per CTA; 0 when the lists are too long for this kernel.
STK_API int stk_mla_decode_splits(int T, int nh, int max_rows, int sm_count) {
  (void)T; (void)nh; (void)sm_count;
  const int s = (max_rows + 31) / 32;
  return s <= kMdMaxS ? (s < 1 ? 1 : s) : 0;
}

// q [T, nh, 512] bf16 (ldt elements between tokens), fp8_ds_mla caches, nh a multiple of 8.
// prep_q: q is the raw projection output; its per-head weightless RMSNorm (eps) and RoPE (positions, inv_freq) happen
// on load.  positions/inv_freq also drive the inverse RoPE of the output (always applied when positions != nullptr).
// workspace: T * S * nh * 516 floats, 16-byte aligned; S = stk_mla_decode_splits(..., swa_rows + topk_rows, ...).
STK_API int stk_sparse_mla_decode(const void* q, long long ldt, const void* swa_cache, long long swa_stride,
                                  long long swa_slots_n, const void* comp_cache, long long comp_stride,
                                  long long comp_slots_n, const int* swa_slots, int swa_ld, int swa_rows, const int* swa_lens,
                                  const int* topk_slots, int topk_ld, int topk_rows, const int* topk_lens, const float* sink, void* out,
                                  long long ldo, float* workspace, int S, int T, int nh, float scale, int prep_q,
                                  float eps, const int64_t* positions, const float* inv_freq, int out_inv_rope,
                                  const void* kv_new, long long kv_ld, const void* kv_norm_w, const int64_t* cur_slot,
                                  int* status, void* stream) {
  // kv_new != nullptr (pure decode steps only): the kernel also builds and inserts each token's own latent row from
  // the raw kv projection (RMSNorm with kv_norm_w and eps, RoPE, UE8M0 quantisation) at cur_slot[t] of the window cache.
  if (T <= 0) return 0;
  if (nh % kMdHeads || S != (swa_rows + (topk_slots ? topk_rows : 0) + 31) / 32 || S > kMdMaxS || (ldt % 8) || (reinterpret_cast<uintptr_t>(q) & 15) || (ldo % 4) ||
      (reinterpret_cast<uintptr_t>(workspace) & 15) || (reinterpret_cast<uintptr_t>(out) & 7))
    return -1;
  if (prep_q && (positions == nullptr || inv_freq == nullptr)) return -2;
  MdArgs a;
  memset(&a, 0, sizeof(a));
  a.q = (const __nv_bfloat16*)q; a.ldt = ldt;
  a.swa = MdCache{(const uint8_t*)swa_cache, swa_stride};
  a.comp = MdCache{(const uint8_t*)(comp_cache ? comp_cache : swa_cache), comp_cache ? comp_stride : swa_stride};
  a.swa_slots = swa_slots; a.swa_ld = swa_ld; a.swa_lens = swa_lens;
  a.topk_slots = topk_slots; a.topk_ld = topk_ld; a.topk_lens = topk_lens;
  a.swa_ld_rows = swa_rows; a.topk_rows = topk_slots ? topk_rows : 0;
  a.positions = positions; a.inv_freq = inv_freq;
  a.partial = workspace; a.nh = nh; a.S = S; a.scale = scale; a.eps = eps; a.prep_q = prep_q;
  a.swa_slots_n = swa_slots_n; a.comp_slots_n = comp_cache ? comp_slots_n : swa_slots_n;
  a.status = status;
  if (kv_new != nullptr) {
    if (kv_norm_w == nullptr || cur_slot == nullptr || positions == nullptr || inv_freq == nullptr || (kv_ld % 8) ||
        (reinterpret_cast<uintptr_t>(kv_new) & 15) || (reinterpret_cast<uintptr_t>(kv_norm_w) & 15))
      return -5;
    a.kv_new = (const __nv_bfloat16*)kv_new; a.kv_ld = kv_ld; a.kv_norm_w = (const __nv_bfloat16*)kv_norm_w;
    a.cur_slot = cur_slot;
    a.swa_write = (uint8_t*)const_cast<void*>(swa_cache);
  }
  const size_t smem = 16 * 4 * kMdP * sizeof(float);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(mla_decode_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -3;
    configured = true;
  }
  cudaStream_t st = (cudaStream_t)stream;
  launch_pdl(mla_decode_split_kernel, dim3(S, T, nh / kMdHeads), dim3(512), smem, st, a);
  launch_pdl(mla_decode_merge_kernel, dim3(T * nh), dim3(512), 0, st, (const float*)workspace, sink, (__nv_bfloat16*)out, ldo,
             nh, S, out_inv_rope ? positions : (const int64_t*)nullptr, inv_freq);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
