// Paged KV-cache producers and readers.
//
//   q_norm_rope            per-head weightless RMSNorm + interleaved RoPE on the last R dims of Q
//   kv_rope_quant_insert   RoPE + UE8M0 fp8 quantise (64-wide blocks) + paged write of the latent row
//   kv_gather_dequant      paged rows -> dense bf16
//   compress_windows       gated pooling of completed ratio-sized windows (+ overlap), RMSNorm, RoPE,
//                          quantise, paged write into the compressed cache or the indexer-K cache
//   compress_save_state    keep the raw (value, gate) rows that future windows still need
//   indexer_q_prep         RoPE + bf16 round + per-(token, head) ue8m0 fp8 quantise, scale folded
//                          into the head weights
//
// Row format "fp8_ds_mla" (overlay/ops_cache_utils.py:29-152): per token nope fp8 bytes, then
// rope bf16, and 8 scale bytes stored after the 64 data rows of the page:
//   page = [64 x data_bytes][64 x 8 scale bytes][padding to page_stride].
// Offsets use 64-bit arithmetic (caches exceed 2^31 bytes).
#define STK_PDL_CLASS 32      // bit of this file's kernels in the PDL mask (STK_PDL, stk_set_pdl_mask)
#include "common.cuh"

namespace stk {

struct RopeTab {
  const float* inv_freq;   // [R/2]
};

__device__ __forceinline__ void rope_pair(float& a, float& b, float pos, float inv, bool inverse) {
  float s, c;
  sincosf(pos * inv, &s, &c);
  if (inverse) s = -s;
  const float x = a * c - b * s;
  const float y = a * s + b * c;
  a = x;
  b = y;
}

// q [T, nh, D] in place.  One warp per (token, head).
__device__ __forceinline__ void q_norm_rope_body(int block, __nv_bfloat16* __restrict__ q, long long ldt,
                                                 const int64_t* __restrict__ positions, const float* __restrict__ inv_freq,
                                                 int T, int nh, int D, int R, float eps, int do_norm, int inverse) {
  const int w = (block * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= T * nh) return;
  const int t = w / nh, h = w % nh;
  __nv_bfloat16* row = q + t * ldt + static_cast<long long>(h) * D;
  const float pos = static_cast<float>(positions[t]);
  float ss = 0.f;
  if (do_norm) {
    for (int i = lane * 2; i < D; i += 64) {
      const __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(row + i);
      ss = fmaf(__low2float(v), __low2float(v), fmaf(__high2float(v), __high2float(v), ss));
    }
    ss = warp_sum(ss);
  }
  const float r = do_norm ? rsqrtf(ss / D + eps) : 1.f;
  const int nope = D - R;
  for (int i = lane * 2; i < D; i += 64) {
    const __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(row + i);
    float a = __low2float(v) * r, b = __high2float(v) * r;
    if (i >= nope) rope_pair(a, b, pos, inv_freq[(i - nope) >> 1], inverse != 0);
    *reinterpret_cast<__nv_bfloat162*>(row + i) = __floats2bfloat162_rn(a, b);
  }
}

__global__ void q_norm_rope_kernel(__nv_bfloat16* __restrict__ q, long long ldt, const int64_t* __restrict__ positions,
                                   const float* __restrict__ inv_freq, int T, int nh, int D, int R, float eps,
                                   int do_norm, int inverse) {
  pdl_wait();
  pdl_trigger();
  q_norm_rope_body(blockIdx.x, q, ldt, positions, inv_freq, T, nh, D, R, eps, do_norm, inverse);
}

struct CacheGeom {
  uint8_t* base;
  long long page_stride;   // bytes
  int data_bytes;          // per row (fp8: nope + 2R; bf16: 2D)
  int fp8;                 // 1: fp8_ds_mla rows, 0: bf16 rows
};

__device__ __forceinline__ void write_latent_row(const CacheGeom& c, long long slot, const float* vals /*smem D*/,
                                                 int D, int R, int lane) {
  const long long page = slot >> 6;
  const int r = static_cast<int>(slot & 63);
  uint8_t* pbase = c.base + page * c.page_stride;
  if (!c.fp8) {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(pbase + static_cast<long long>(r) * c.data_bytes);
    for (int i = lane * 2; i < D; i += 64)
      *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(vals[i], vals[i + 1]);
    return;
  }
  const int nope = D - R;
  uint8_t* drow = pbase + static_cast<long long>(r) * c.data_bytes;
  uint8_t* srow = pbase + 64LL * c.data_bytes + r * 8;
  const int nb = nope / 64;
  for (int b = 0; b < nb; ++b) {
    const float a = vals[b * 64 + lane * 2], bb = vals[b * 64 + lane * 2 + 1];
    const float amax = warp_max(fmaxf(fabsf(a), fabsf(bb)));
    uint8_t byte;
    const float sc = ue8m0_scale(amax, &byte);
    const float inv = 1.f / sc;
    const uint16_t packed = static_cast<uint16_t>(f_to_fp8(a * inv)) | (static_cast<uint16_t>(f_to_fp8(bb * inv)) << 8);
    *reinterpret_cast<uint16_t*>(drow + b * 64 + lane * 2) = packed;
    if (lane == 0) srow[b] = byte;
  }
  if (lane < 8 - nb) srow[nb + lane] = 0;
  __nv_bfloat16* rdst = reinterpret_cast<__nv_bfloat16*>(drow + nope);
  for (int i = lane * 2; i < R; i += 64)
    *reinterpret_cast<__nv_bfloat162*>(rdst + i) = __floats2bfloat162_rn(vals[nope + i], vals[nope + i + 1]);
}

// kv [T, D] bf16.  One warp per token; slot -1 = padding (skipped).  With norm_w the row is RMS-normalised here
// (weight norm_w, rounded to bf16 as a separate norm kernel would store it) instead of arriving normalised.
__device__ __forceinline__ void kv_rope_quant_insert_body(int block, float* sm, const __nv_bfloat16* __restrict__ kv,
                                                          long long ldk, const int64_t* __restrict__ positions,
                                                          const int64_t* __restrict__ slots,
                                                          const float* __restrict__ inv_freq, const CacheGeom& cache,
                                                          int T, int D, int R, long long num_slots, int* status,
                                                          const __nv_bfloat16* __restrict__ norm_w = nullptr,
                                                          float norm_eps = 0.f) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = block * (blockDim.x >> 5) + warp;
  if (t >= T) return;
  const long long slot = slots[t];
  if (slot < 0) return;
  if (slot >= num_slots) {
    if (lane == 0) set_status(status, kBadIndex, t);
    return;
  }
  float* vals = sm + warp * D;
  const float pos = static_cast<float>(positions[t]);
  const int nope = D - R;
  float nr = 1.f;
  if (norm_w != nullptr) {
    float ss = 0.f;
    for (int i = lane * 2; i < D; i += 64) {
      const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(kv + t * ldk + i);
      ss = fmaf(__low2float(v), __low2float(v), fmaf(__high2float(v), __high2float(v), ss));
    }
    nr = rsqrtf(warp_sum(ss) / D + norm_eps);
  }
  for (int i = lane * 2; i < D; i += 64) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(kv + t * ldk + i);
    float a = __low2float(v), b = __high2float(v);
    if (norm_w != nullptr) {
      const __nv_bfloat162 w = *reinterpret_cast<const __nv_bfloat162*>(norm_w + i);
      a = bf16_to_f(__float2bfloat16(a * nr * __low2float(w)));
      b = bf16_to_f(__float2bfloat16(b * nr * __high2float(w)));
    }
    if (i >= nope) {
      rope_pair(a, b, pos, inv_freq[(i - nope) >> 1], false);
      a = bf16_to_f(__float2bfloat16(a));
      b = bf16_to_f(__float2bfloat16(b));
    }
    vals[i] = a;
    vals[i + 1] = b;
  }
  __syncwarp();
  write_latent_row(cache, slot, vals, D, R, lane);
}

__global__ void kv_rope_quant_insert_kernel(const __nv_bfloat16* __restrict__ kv, long long ldk,
                                            const int64_t* __restrict__ positions, const int64_t* __restrict__ slots,
                                            const float* __restrict__ inv_freq, CacheGeom cache, int T, int D, int R,
                                            long long num_slots, int* status) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float sm[];
  kv_rope_quant_insert_body(blockIdx.x, sm, kv, ldk, positions, slots, inv_freq, cache, T, D, R, num_slots, status);
}

// One launch for both halves of the step's "write" work: blocks [0, q_blocks) norm + rotate Q in place,
// the rest rotate, quantise and insert the latent rows.  (The reference's horizontally fused
// qnorm/rope/kv-insert custom op: overlay/attention.py:704-729.)
__global__ void __launch_bounds__(256)
q_rope_kv_insert_kernel(__nv_bfloat16* __restrict__ q, long long ldt, int nh, float eps, int q_blocks,
                        const __nv_bfloat16* __restrict__ kv, long long ldk, const int64_t* __restrict__ positions,
                        const int64_t* __restrict__ slots, const float* __restrict__ inv_freq, CacheGeom cache, int T,
                        int D, int R, long long num_slots, int* status, const __nv_bfloat16* __restrict__ kv_norm_w) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float sm[];
  if (static_cast<int>(blockIdx.x) < q_blocks) {
    q_norm_rope_body(blockIdx.x, q, ldt, positions, inv_freq, T, nh, D, R, eps, 1, 0);
  } else {
    kv_rope_quant_insert_body(blockIdx.x - q_blocks, sm, kv, ldk, positions, slots, inv_freq, cache, T, D, R, num_slots,
                              status, kv_norm_w, eps);
  }
}

// rows[i, :] = dequant(cache row slots[i]); slot < 0 -> zeros.  One warp per row.
__global__ void kv_gather_dequant_kernel(CacheGeom cache, const int64_t* __restrict__ slots,
                                         __nv_bfloat16* __restrict__ out, int n, int D, int R) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= n) return;
  const long long slot = slots[w];
  __nv_bfloat16* dst = out + static_cast<long long>(w) * D;
  if (slot < 0) {
    for (int i = lane * 2; i < D; i += 64) *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(0.f, 0.f);
    return;
  }
  const uint8_t* pbase = cache.base + (slot >> 6) * cache.page_stride;
  const int r = static_cast<int>(slot & 63);
  if (!cache.fp8) {
    const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(pbase + static_cast<long long>(r) * cache.data_bytes);
    for (int i = lane * 2; i < D; i += 64)
      *reinterpret_cast<__nv_bfloat162*>(dst + i) = *reinterpret_cast<const __nv_bfloat162*>(src + i);
    return;
  }
  const int nope = D - R;
  const uint8_t* drow = pbase + static_cast<long long>(r) * cache.data_bytes;
  const uint8_t* srow = pbase + 64LL * cache.data_bytes + r * 8;
  for (int i = lane * 2; i < nope; i += 64) {
    const float sc = exp2f(static_cast<float>(srow[i >> 6]) - 127.f);
    const uint16_t p = *reinterpret_cast<const uint16_t*>(drow + i);
    *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(fp8_to_f(p & 0xff) * sc, fp8_to_f(p >> 8) * sc);
  }
  const __nv_bfloat16* rsrc = reinterpret_cast<const __nv_bfloat16*>(drow + nope);
  for (int i = lane * 2; i < R; i += 64)
    *reinterpret_cast<__nv_bfloat162*>(dst + nope + i) = *reinterpret_cast<const __nv_bfloat162*>(rsrc + i);
}

// ---- KV compressor ----------------------------------------------------------------
struct CompressArgs {
  const float* kvs;            // [T, kvs_ld]: value slots (c*D) then gate slots (c*D)
  long long kvs_ld;
  const float* ape;            // [ratio, c*D]
  const __nv_bfloat16* norm_w; // [D]
  const float* inv_freq;
  const int64_t* positions;    // [T]
  const int* tok_req;          // [T] request row (block table / state row)
  const int* tok_first_pos;    // [T] position of the request's first token in this step
  float* state;                // [num_req_rows, ring, 2*c*D]
  const int* block_table;      // [num_req_rows, bt_stride] pages of the destination cache
  int bt_stride;
  CacheGeom cache;
  int idx_format;              // 1: indexer-K rows (fp8 D bytes + fp32 scale), 0: latent rows
  int T, D, R, ratio, c, ring;
  long long num_slots;
  float eps;
  int* status;
};

__device__ __forceinline__ const float* compress_src_row(const CompressArgs& a, int t, long long pos_t, long long p) {
  const int first = a.tok_first_pos[t];
  if (p >= first) return a.kvs + static_cast<long long>(t - (pos_t - p)) * a.kvs_ld;
  return a.state + (static_cast<long long>(a.tok_req[t]) * a.ring + (p % a.ring)) * (2LL * a.c * a.D);
}

// One CTA per token; only the token that closes a window does work.
__global__ void __launch_bounds__(128)
compress_windows_kernel(CompressArgs a) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float sm[];    // D floats + 32
  const int t = blockIdx.x;
  const long long pos = a.positions[t];
  if (pos < 0 || (pos + 1) % a.ratio != 0) return;
  const long long j = (pos + 1) / a.ratio - 1;
  const long long p0 = j * a.ratio;
  float* pooled = sm;
  float* red = sm + a.D;
  const int cD = a.c * a.D;
  const bool has_prev = (a.c == 2) && (j >= 1);
  for (int d = threadIdx.x; d < a.D; d += blockDim.x) {
    float m = -INFINITY, l = 0.f, acc = 0.f;
    for (int i = 0; i < a.ratio; ++i) {
      const float* row = compress_src_row(a, t, pos, p0 + i);
      const float v = row[d];
      const float g = row[cD + d] + a.ape[i * cD + d];
      const float mn = fmaxf(m, g);
      const float corr = __expf(m - mn), e = __expf(g - mn);
      l = l * corr + e;
      acc = acc * corr + e * v;
      m = mn;
    }
    if (has_prev) {
      for (int i = 0; i < a.ratio; ++i) {
        const float* row = compress_src_row(a, t, pos, p0 - a.ratio + i);
        const float v = row[a.D + d];
        const float g = row[cD + a.D + d] + a.ape[i * cD + a.D + d];
        const float mn = fmaxf(m, g);
        const float corr = __expf(m - mn), e = __expf(g - mn);
        l = l * corr + e;
        acc = acc * corr + e * v;
        m = mn;
      }
    }
    pooled[d] = acc / l;
  }
  __syncthreads();
  float ss = 0.f;
  for (int d = threadIdx.x; d < a.D; d += blockDim.x) ss = fmaf(pooled[d], pooled[d], ss);
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / a.D + a.eps);
  const int nope = a.D - a.R;
  __syncthreads();
  for (int d = threadIdx.x * 2; d < a.D; d += blockDim.x * 2) {
    float x = pooled[d] * r * bf16_to_f(a.norm_w[d]);
    float y = pooled[d + 1] * r * bf16_to_f(a.norm_w[d + 1]);
    if (d >= nope) rope_pair(x, y, static_cast<float>(p0), a.inv_freq[(d - nope) >> 1], false);
    pooled[d] = x;
    pooled[d + 1] = y;
  }
  __syncthreads();
  // destination slot in the compressed cache
  const int page = a.block_table[static_cast<long long>(a.tok_req[t]) * a.bt_stride + (j >> 6)];
  const long long slot = static_cast<long long>(page) * 64 + (j & 63);
  if (page < 0 || slot >= a.num_slots) {
    if (threadIdx.x == 0) set_status(a.status, kBadIndex, t);
    return;
  }
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    if (!a.idx_format) {
      if (a.cache.fp8) {
        // rope dims are stored as bf16: round them first like the SWA path does
        for (int d = nope + lane; d < a.D; d += 32) pooled[d] = bf16_to_f(__float2bfloat16(pooled[d]));
        __syncwarp();
      }
      write_latent_row(a.cache, slot, pooled, a.D, a.R, lane);
    } else {
      uint8_t* pbase = a.cache.base + (slot >> 6) * a.cache.page_stride;
      const int rr = static_cast<int>(slot & 63);
      if (a.cache.fp8) {
        float amax = 0.f;
        for (int d = lane; d < a.D; d += 32) amax = fmaxf(amax, fabsf(pooled[d]));
        amax = warp_max(amax);
        const float sc = ue8m0_scale(amax, nullptr);
        const float inv = 1.f / sc;
        uint8_t* drow = pbase + static_cast<long long>(rr) * a.D;
        for (int d = lane; d < a.D; d += 32) drow[d] = f_to_fp8(pooled[d] * inv);
        if (lane == 0) *reinterpret_cast<float*>(pbase + 64LL * a.D + rr * 4) = sc;
      } else {
        __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(pbase + static_cast<long long>(rr) * a.D * 2);
        for (int d = lane; d < a.D; d += 32) drow[d] = __float2bfloat16(pooled[d]);
      }
    }
  }
}

// Keep the raw rows of the last `ring` positions of each request (runs after compress_windows).
__global__ void compress_save_state_kernel(CompressArgs a, const int* __restrict__ tok_last_pos) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const long long pos = a.positions[t];
  if (pos < 0 || pos + a.ring <= tok_last_pos[t]) return;
  const long long w = 2LL * a.c * a.D;
  const float* src = a.kvs + static_cast<long long>(t) * a.kvs_ld;
  float* dst = a.state + (static_cast<long long>(a.tok_req[t]) * a.ring + (pos % a.ring)) * w;
  for (int i = threadIdx.x; i < w; i += blockDim.x) dst[i] = src[i];
}

// ---- indexer Q ---------------------------------------------------------------------
// q [T, ih, d] bf16, w [T, ih] fp32 -> q_out (fp8 or bf16), w_out fp32.  One warp per (t, head).
__global__ void indexer_q_prep_kernel(const __nv_bfloat16* __restrict__ q, long long ldq, const float* __restrict__ w, long long ldw,
                                      const int64_t* __restrict__ positions, const float* __restrict__ inv_freq,
                                      void* __restrict__ q_out, float* __restrict__ w_out, int T, int ih, int d, int R,
                                      int quantize) {
  pdl_wait();
  pdl_trigger();
  const int wp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wp >= T * ih) return;
  const int t = wp / ih, h = wp % ih;
  const __nv_bfloat16* row = q + t * ldq + static_cast<long long>(h) * d;
  const float pos = static_cast<float>(positions[t]);
  const int nope = d - R;
  const float fold = rsqrtf(static_cast<float>(d)) * rsqrtf(static_cast<float>(ih));
  float amax = 0.f;
  // each lane owns pairs (i, i+1) for i = lane*2 + 64*k; d <= 256 => at most 4 pairs
  float va[4], vb[4];
  int np = 0;
  for (int i = lane * 2; i < d; i += 64, ++np) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(row + i);
    float a = __low2float(v), b = __high2float(v);
    if (i >= nope) rope_pair(a, b, pos, inv_freq[(i - nope) >> 1], false);
    a = bf16_to_f(__float2bfloat16(a));
    b = bf16_to_f(__float2bfloat16(b));
    va[np] = a;
    vb[np] = b;
    amax = fmaxf(amax, fmaxf(fabsf(a), fabsf(b)));
  }
  amax = warp_max(amax);
  if (quantize) {
    const float sc = ue8m0_scale(amax, nullptr);
    const float inv = 1.f / sc;
    uint8_t* dst = reinterpret_cast<uint8_t*>(q_out) + (static_cast<long long>(t) * ih + h) * d;
    np = 0;
    for (int i = lane * 2; i < d; i += 64, ++np)
      *reinterpret_cast<uint16_t*>(dst + i) =
          static_cast<uint16_t>(f_to_fp8(va[np] * inv)) | (static_cast<uint16_t>(f_to_fp8(vb[np] * inv)) << 8);
    if (lane == 0) w_out[t * ih + h] = w[t * ldw + h] * sc * fold;
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(q_out) + (static_cast<long long>(t) * ih + h) * d;
    np = 0;
    for (int i = lane * 2; i < d; i += 64, ++np)
      *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(va[np], vb[np]);
    if (lane == 0) w_out[t * ih + h] = w[t * ldw + h] * fold;
  }
}

}  // namespace stk

using namespace stk;

STK_API int stk_q_norm_rope(void* q, long long ldt, const int64_t* positions, const float* inv_freq, int T, int nh,
                            int D, int R, float eps, int do_norm, int inverse, void* stream) {
  if (T <= 0) return 0;
  if (D % 2 || R % 2) return -1;
  const long long warps = static_cast<long long>(T) * nh;
  launch_pdl(q_norm_rope_kernel, dim3(static_cast<int>((warps + 7) / 8)), dim3(256), 0, (cudaStream_t)stream, 
      (__nv_bfloat16*)q, ldt, positions, inv_freq, T, nh, D, R, eps, do_norm, inverse);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_kv_rope_quant_insert(const void* kv, long long ldk, const int64_t* positions, const int64_t* slots,
                                     const float* inv_freq, void* cache, long long page_stride, int data_bytes,
                                     int fp8, long long num_slots, int T, int D, int R, int* status, void* stream) {
  if (T <= 0) return 0;
  if (D % 2 || (fp8 && ((D - R) % 64 || (D - R) / 64 > 8))) return -1;
  CacheGeom g{(uint8_t*)cache, page_stride, data_bytes, fp8};
  const int wpb = 4;
  launch_pdl(kv_rope_quant_insert_kernel, dim3((T + wpb - 1) / wpb), dim3(wpb * 32), wpb * D * sizeof(float), (cudaStream_t)stream, 
      (const __nv_bfloat16*)kv, ldk, positions, slots, inv_freq, g, T, D, R, num_slots, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_q_rope_kv_insert(void* q, long long ldt, int nh, float eps, const void* kv, long long ldk,
                                 const int64_t* positions, const int64_t* slots, const float* inv_freq, void* cache,
                                 long long page_stride, int data_bytes, int fp8, long long num_slots, int T, int D, int R,
                                 const void* kv_norm_w, int* status, void* stream) {
  // kv_norm_w != nullptr: kv arrives un-normalised and is RMS-normalised (same eps) inside the insert.
  // q == nullptr (nh = 0): only the latent rows are written (the attention kernel norms and rotates q itself).
  if (T <= 0) return 0;
  if (D % 2 || R % 2 || (fp8 && ((D - R) % 64 || (D - R) / 64 > 8))) return -1;
  CacheGeom g{(uint8_t*)cache, page_stride, data_bytes, fp8};
  if (q == nullptr) nh = 0;
  const int q_blocks = static_cast<int>((static_cast<long long>(T) * nh + 7) / 8);
  const int kv_blocks = (T + 7) / 8;
  launch_pdl(q_rope_kv_insert_kernel, dim3(q_blocks + kv_blocks), dim3(256), 8 * D * sizeof(float), (cudaStream_t)stream, 
      (__nv_bfloat16*)q, ldt, nh, eps, q_blocks, (const __nv_bfloat16*)kv, ldk, positions, slots, inv_freq, g, T, D, R,
      num_slots, status, (const __nv_bfloat16*)kv_norm_w);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_kv_gather_dequant(const void* cache, long long page_stride, int data_bytes, int fp8,
                                  const int64_t* slots, void* out, int n, int D, int R, void* stream) {
  if (n <= 0) return 0;
  CacheGeom g{(uint8_t*)const_cast<void*>(cache), page_stride, data_bytes, fp8};
  kv_gather_dequant_kernel<<<(n + 7) / 8, 256, 0, (cudaStream_t)stream>>>(g, slots, (__nv_bfloat16*)out, n, D, R);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_compress_windows(const float* kvs, long long kvs_ld, const float* ape, const void* norm_w, const float* inv_freq,
                                 const int64_t* positions, const int* tok_req, const int* tok_first_pos,
                                 const int* tok_last_pos, float* state, const int* block_table, int bt_stride,
                                 void* cache, long long page_stride, int data_bytes, int fp8, int idx_format,
                                 long long num_slots, int T, int D, int R, int ratio, int c, int ring, float eps,
                                 int* status, void* stream) {
  if (T <= 0) return 0;
  if (D % 2 || c < 1 || c > 2) return -1;
  CompressArgs a;
  a.kvs = kvs; a.kvs_ld = kvs_ld; a.ape = ape; a.norm_w = (const __nv_bfloat16*)norm_w; a.inv_freq = inv_freq; a.positions = positions;
  a.tok_req = tok_req; a.tok_first_pos = tok_first_pos; a.state = state; a.block_table = block_table;
  a.bt_stride = bt_stride; a.cache = CacheGeom{(uint8_t*)cache, page_stride, data_bytes, fp8};
  a.idx_format = idx_format; a.T = T; a.D = D; a.R = R; a.ratio = ratio; a.c = c; a.ring = ring;
  a.num_slots = num_slots; a.eps = eps; a.status = status;
  cudaStream_t st = (cudaStream_t)stream;
  launch_pdl(compress_windows_kernel, dim3(T), dim3(128), (D + 32) * sizeof(float), st, a);
  launch_pdl(compress_save_state_kernel, dim3(T), dim3(128), 0, st, a, tok_last_pos);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_indexer_q_prep(const void* q, long long ldq, const float* w, long long ldw, const int64_t* positions,
                               const float* inv_freq, void* q_out, float* w_out, int T, int ih, int d, int R,
                               int quantize, void* stream) {
  if (T <= 0) return 0;
  if (d % 2 || d > 256) return -1;
  const long long warps = static_cast<long long>(T) * ih;
  launch_pdl(indexer_q_prep_kernel, dim3(static_cast<int>((warps + 7) / 8)), dim3(256), 0, (cudaStream_t)stream, 
      (const __nv_bfloat16*)q, ldq, w, ldw, positions, inv_freq, q_out, w_out, T, ih, d, R, quantize);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
