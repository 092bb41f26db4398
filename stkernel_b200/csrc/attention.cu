// Sparse multi-head latent attention over paged rows (K = V = the latent row).
//
// Each query token attends to the rows named by two index lists — its sliding-window rows in the
// SWA cache and its top-k rows in the compressed cache — plus a per-head sink logit that only
// enters the softmax denominator.  Rows are fp8_ds_mla (dequantised on load) or bf16.
//
// This is the split-row formulation: grid (token, split); every CTA walks its share of the row
// list in 32-row blocks with an online softmax and writes an un-normalised partial
// (o, m, l) to a workspace; `sparse_mla_combine` merges the splits and applies the sink.
// It serves decode batches and is the numerics check of the tensor-core kernel.
//
// Takes the place of the reference's flashinfer_trtllm_batch_decode_sparse_mla_dsv4 call
// (overlay/flashinfer_sparse.py:387-400,528-541).
#define STK_PDL_CLASS 128      // bit of this file's kernels in the PDL mask (STK_PDL, stk_set_pdl_mask)
#include "common.cuh"

namespace stk {

struct MlaCache {
  const uint8_t* base;
  long long page_stride;
  int data_bytes;
  int fp8;
};

struct MlaArgs {
  const __nv_bfloat16* q;      // [T, nh, D]
  long long ldt;
  MlaCache swa, comp;
  const int* swa_slots; int swa_ld; const int* swa_lens;
  const int* topk_slots; int topk_ld; const int* topk_lens;   // may be null
  float* partial;              // [T, n_splits, nh, D + 2]
  int T, nh, D, R, n_splits, rows_per_split;
  float scale;
};

constexpr int kRB = 32;        // rows per block

__device__ __forceinline__ void load_row_bf16(const MlaCache& c, int slot, __nv_bfloat16* dst, int D, int R, int lane) {
  if (slot < 0) {
    for (int i = lane * 2; i < D; i += 64) *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(0.f, 0.f);
    return;
  }
  const uint8_t* pbase = c.base + static_cast<long long>(slot >> 6) * c.page_stride;
  const int r = slot & 63;
  if (!c.fp8) {
    const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(pbase + static_cast<long long>(r) * c.data_bytes);
    for (int i = lane * 2; i < D; i += 64)
      *reinterpret_cast<__nv_bfloat162*>(dst + i) = *reinterpret_cast<const __nv_bfloat162*>(src + i);
    return;
  }
  const int nope = D - R;
  const uint8_t* drow = pbase + static_cast<long long>(r) * c.data_bytes;
  const uint8_t* srow = pbase + 64LL * c.data_bytes + r * 8;
  for (int i = lane * 2; i < nope; i += 64) {
    const float sc = exp2f(static_cast<float>(srow[i >> 6]) - 127.f);
    const uint16_t p = *reinterpret_cast<const uint16_t*>(drow + i);
    *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(fp8_to_f(p & 0xff) * sc, fp8_to_f(p >> 8) * sc);
  }
  const __nv_bfloat16* rsrc = reinterpret_cast<const __nv_bfloat16*>(drow + nope);
  for (int i = lane * 2; i < R; i += 64)
    *reinterpret_cast<__nv_bfloat162*>(dst + nope + i) = *reinterpret_cast<const __nv_bfloat162*>(rsrc + i);
}

template <int NH>
__global__ void __launch_bounds__(256)
sparse_mla_split_kernel(MlaArgs a) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ uint8_t smraw[];
  const int D = a.D;
  const int DP = D + 2;                       // padded row (bank-conflict-free column reads)
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smraw);            // [NH][D]
  __nv_bfloat16* Ks = Qs + NH * D;                                         // [kRB][DP]
  float* S = reinterpret_cast<float*>(Ks + kRB * DP + (((kRB * DP) & 1) ? 1 : 0));   // [NH][kRB]
  float* m_s = S + NH * kRB;                                               // [NH]
  float* l_s = m_s + NH;
  float* alpha_s = l_s + NH;

  const int t = blockIdx.x, sp = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_swa = a.swa_lens[t];
  const int n_top = a.topk_slots ? a.topk_lens[t] : 0;
  const int L = n_swa + n_top;
  const int r_begin = sp * a.rows_per_split;
  const int r_end = min(L, r_begin + a.rows_per_split);

  for (int i = tid; i < NH * D / 2; i += 256) {
    const int h = (i * 2) / D, d = (i * 2) % D;
    __nv_bfloat162 v = __floats2bfloat162_rn(0.f, 0.f);
    if (h < a.nh) v = *reinterpret_cast<const __nv_bfloat162*>(a.q + t * a.ldt + static_cast<long long>(h) * D + d);
    *reinterpret_cast<__nv_bfloat162*>(Qs + h * D + d) = v;
  }
  if (tid < NH) {
    m_s[tid] = -INFINITY;
    l_s[tid] = 0.f;
  }
  float acc[NH][2];
#pragma unroll
  for (int h = 0; h < NH; ++h) acc[h][0] = acc[h][1] = 0.f;
  const int d0 = tid * 2;                      // this thread's output dims (D <= 512)
  __syncthreads();

  for (int rb = r_begin; rb < r_end; rb += kRB) {
    // ---- load + dequantise up to 32 rows ----
    for (int rr = warp; rr < kRB; rr += 8) {
      const int li = rb + rr;
      int slot = -1;
      const MlaCache* c = &a.swa;
      if (li < r_end) {
        if (li < n_swa) slot = a.swa_slots[static_cast<long long>(t) * a.swa_ld + li];
        else { slot = a.topk_slots[static_cast<long long>(t) * a.topk_ld + (li - n_swa)]; c = &a.comp; }
      }
      load_row_bf16(*c, slot, Ks + rr * DP, D, a.R, lane);
    }
    __syncthreads();
    // ---- S = scale * Q K^T ----
    for (int idx = tid; idx < NH * kRB; idx += 256) {
      const int h = idx / kRB, r = idx % kRB;
      const __nv_bfloat16* qrow = Qs + h * D;
      const __nv_bfloat16* krow = Ks + r * DP;
      float s0 = 0.f, s1 = 0.f;
      for (int d = 0; d < D; d += 2) {
        const __nv_bfloat162 qv = *reinterpret_cast<const __nv_bfloat162*>(qrow + d);
        const __nv_bfloat162 kv = *reinterpret_cast<const __nv_bfloat162*>(krow + d);
        s0 = fmaf(__low2float(qv), __low2float(kv), s0);
        s1 = fmaf(__high2float(qv), __high2float(kv), s1);
      }
      // rows past the list end or with a padding slot are masked
      const int li = rb + r;
      bool valid = li < r_end;
      if (valid) {
        const int slot = li < n_swa ? a.swa_slots[static_cast<long long>(t) * a.swa_ld + li]
                                    : a.topk_slots[static_cast<long long>(t) * a.topk_ld + (li - n_swa)];
        valid = slot >= 0;
      }
      S[h * kRB + r] = valid ? (s0 + s1) * a.scale : -INFINITY;
    }
    __syncthreads();
    // ---- online softmax bookkeeping: one warp per head, lane = row ----
    for (int h = warp; h < NH; h += 8) {
      const float s = S[h * kRB + lane];
      const float bm = warp_max(s);
      const float mo = m_s[h];
      const float mn = fmaxf(mo, bm);
      const float p = (mn == -INFINITY) ? 0.f : __expf(s - mn);
      const float ps = warp_sum(p);
      S[h * kRB + lane] = p;
      if (lane == 0) {
        const float al = (mn == -INFINITY) ? 1.f : __expf(mo - mn);
        alpha_s[h] = al;
        l_s[h] = l_s[h] * al + ps;
        m_s[h] = mn;
      }
    }
    __syncthreads();
    // ---- O = O * alpha + P V ----
    if (d0 < D) {
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        const float al = alpha_s[h];
        acc[h][0] *= al;
        acc[h][1] *= al;
      }
      for (int r = 0; r < kRB; ++r) {
        const __nv_bfloat162 kv = *reinterpret_cast<const __nv_bfloat162*>(Ks + r * DP + d0);
        const float v0 = __low2float(kv), v1 = __high2float(kv);
#pragma unroll
        for (int h = 0; h < NH; ++h) {
          const float p = S[h * kRB + r];
          acc[h][0] = fmaf(p, v0, acc[h][0]);
          acc[h][1] = fmaf(p, v1, acc[h][1]);
        }
      }
    }
    __syncthreads();
  }
  // ---- write the partial ----
  float* prow = a.partial + (static_cast<long long>(t) * a.n_splits + sp) * a.nh * (D + 2);
  if (d0 < D) {
#pragma unroll
    for (int h = 0; h < NH; ++h) {
      if (h < a.nh) {
        prow[h * (D + 2) + d0] = acc[h][0];
        prow[h * (D + 2) + d0 + 1] = acc[h][1];
      }
    }
  }
  if (tid < a.nh) {
    prow[tid * (D + 2) + D] = m_s[tid];
    prow[tid * (D + 2) + D + 1] = l_s[tid];
  }
}

// grid (T, nh); merges splits, adds the sink to the denominator, optionally applies the inverse
// RoPE on the last R dims (the rotation the output projection expects), writes bf16.
__global__ void sparse_mla_combine_kernel(const float* __restrict__ partial, const float* __restrict__ sink,
                                          __nv_bfloat16* __restrict__ out, long long ldo, int nh, int D, int n_splits,
                                          const int64_t* __restrict__ positions, const float* __restrict__ inv_freq,
                                          int R) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, h = blockIdx.y;
  const float* base = partial + (static_cast<long long>(t) * n_splits * nh + h) * (D + 2);
  const long long sstride = static_cast<long long>(nh) * (D + 2);
  float M = sink ? sink[h] : -INFINITY;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, base[s * sstride + D]);
  float denom = sink ? __expf(sink[h] - M) : 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = base[s * sstride + D];
    if (ms != -INFINITY) denom += base[s * sstride + D + 1] * __expf(ms - M);
  }
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  const int nope = D - R;
  const float pos = positions ? static_cast<float>(positions[t]) : 0.f;
  for (int d = threadIdx.x * 2; d < D; d += blockDim.x * 2) {
    float o0 = 0.f, o1 = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = base[s * sstride + D];
      if (ms != -INFINITY) {
        const float w = __expf(ms - M);
        o0 = fmaf(base[s * sstride + d], w, o0);
        o1 = fmaf(base[s * sstride + d + 1], w, o1);
      }
    }
    o0 *= inv;
    o1 *= inv;
    if (positions != nullptr && d >= nope) {
      // round to bf16 first: the un-fused path stores the attention output before rotating it
      o0 = __bfloat162float(__float2bfloat16(o0));
      o1 = __bfloat162float(__float2bfloat16(o1));
      float sn, cs;
      sincosf(pos * inv_freq[(d - nope) >> 1], &sn, &cs);
      const float x = o0 * cs + o1 * sn;
      const float y = -o0 * sn + o1 * cs;
      o0 = x;
      o1 = y;
    }
    *reinterpret_cast<__nv_bfloat162*>(out + t * ldo + static_cast<long long>(h) * D + d) = __floats2bfloat162_rn(o0, o1);
  }
}

}  // namespace stk

using namespace stk;

STK_API long long stk_sparse_mla_workspace_bytes(int T, int nh, int D, int n_splits) {
  return static_cast<long long>(T) * n_splits * nh * (D + 2) * 4;
}

STK_API int stk_sparse_mla_pick_splits(int T, int max_rows) {
  // fill ~2 waves of 148 SMs, at least 64 rows per split
  int s = (296 + T - 1) / (T > 0 ? T : 1);
  const int cap = (max_rows + 63) / 64;
  if (s > cap) s = cap;
  return s < 1 ? 1 : s;
}

STK_API int stk_sparse_mla(const void* q, long long ldt, const void* swa_cache, long long swa_stride, int swa_data_bytes,
                           const void* comp_cache, long long comp_stride, int comp_data_bytes, int fp8,
                           const int* swa_slots, int swa_ld, const int* swa_lens, const int* topk_slots, int topk_ld,
                           const int* topk_lens, const float* sink, void* out, long long ldo, float* workspace,
                           int n_splits, int T, int nh, int D, int R, int max_rows, float scale, void* stream) {
  if (T <= 0) return 0;
  if (D > 512 || D % 2 || nh > 64) return -1;
  MlaArgs a;
  a.q = (const __nv_bfloat16*)q; a.ldt = ldt;
  a.swa = MlaCache{(const uint8_t*)swa_cache, swa_stride, swa_data_bytes, fp8};
  a.comp = MlaCache{(const uint8_t*)comp_cache, comp_stride, comp_data_bytes, fp8};
  a.swa_slots = swa_slots; a.swa_ld = swa_ld; a.swa_lens = swa_lens;
  a.topk_slots = topk_slots; a.topk_ld = topk_ld; a.topk_lens = topk_lens;
  a.partial = workspace; a.T = T; a.nh = nh; a.D = D; a.R = R; a.n_splits = n_splits;
  int rps = (max_rows + n_splits - 1) / n_splits;
  a.rows_per_split = ((rps + kRB - 1) / kRB) * kRB;
  a.scale = scale;
  int NH = 4;
  while (NH < nh) NH *= 2;
  const size_t smem = static_cast<size_t>(NH) * D * 2 + static_cast<size_t>(kRB) * (D + 2) * 2 + 4 +
                      (static_cast<size_t>(NH) * kRB + 3 * NH) * 4;
  dim3 grid(T, n_splits);
  cudaStream_t st = (cudaStream_t)stream;
#define STK_MLA(NH_)                                                                                              \
  {                                                                                                               \
    static bool configured = false;                                                                               \
    if (!configured) {                                                                                            \
      cudaFuncSetAttribute(sparse_mla_split_kernel<NH_>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
      configured = true;                                                                                          \
    }                                                                                                             \
    launch_pdl(sparse_mla_split_kernel<NH_>, dim3(grid), dim3(256), smem, st, a);                                                      \
  }
  switch (NH) {
    case 4: STK_MLA(4) break;
    case 8: STK_MLA(8) break;
    case 16: STK_MLA(16) break;
    case 32: STK_MLA(32) break;
    case 64: STK_MLA(64) break;
    default: return -2;
  }
#undef STK_MLA
  dim3 g2(T, nh);
  launch_pdl(sparse_mla_combine_kernel, dim3(g2), dim3(128), 0, st, workspace, sink, (__nv_bfloat16*)out, ldo, nh, D, n_splits, nullptr, nullptr, 0);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_sparse_mla_combine(const float* workspace, const float* sink, void* out, long long ldo, int T, int nh,
                                   int D, int n_splits, const int64_t* positions, const float* inv_freq, int R,
                                   void* stream) {
  if (T <= 0) return 0;
  if (D % 2) return -1;
  dim3 g2(T, nh);
  launch_pdl(sparse_mla_combine_kernel, dim3(g2), dim3(128), 0, (cudaStream_t)stream, workspace, sink, (__nv_bfloat16*)out, ldo, nh, D, n_splits,
                                                                  positions, inv_freq, R);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
