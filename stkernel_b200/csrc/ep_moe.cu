// Expert-parallel MoE over NVLink peer memory: route exchange, dispatch, return and combine.
//
// Every rank holds T of its own tokens and E/world experts.  One step:
//
//   ep_route      each rank counts its (token, expert) pairs per expert, stores the histogram into every
//                 peer's table and raises an epoch flag there; after the (bounded) wait for all flags
//                 every rank knows the full [world, E] matrix and derives, with no further messages,
//                 (a) the row offsets of its local experts and (b) for each of its own pairs the exact
//                 row it occupies in the destination rank's expert-sorted activation matrix.
//   ep_dispatch   one warp per pair: the token row is converted to fp16 and stored straight into that
//                 row of the owner's matrix (16-byte peer stores), then the owner's per-expert arrival
//                 counter is incremented with a release.  No receive-side permutation, no barrier.
//   FC1 / FC2     the grouped tcgen05 GEMM (moe_grouped.cu) consumes the matrix; its producer warp waits
//                 per expert on the arrival counter, so early experts compute while later rows travel.
//   ep_return     one warp per sorted row: the bf16 result row goes back to the pair's slot on the token's
//                 home rank, followed by a release increment of that rank's return counter.
//   ep_combine    waits (bounded) until all T*topk rows are back, then sums them with the router weights.
//
// All cross-rank waits are bounded and report through the status word; counters are reset by the next
// ep_route, which no peer can overtake (a peer dispatches only after it has seen this rank's new flag).
// Takes the place of the reference's all2all dispatch/combine managers (overlay/cuda_communicator.py:490-548)
// and of its mega-MoE symmetric buffers (overlay/nvidia_model.py:373-450).
#include "common.cuh"
#include "symm.cuh"

namespace stk {

struct EpCtx {
  uint8_t* base[kMaxRanks];
  int rank, world;
  int E, e_local, topk, H;
  long long off_counts;    // int      [world][E]     histogram of every source rank
  long long off_flags;     // uint32   [world]        route epoch of every source rank
  long long off_epoch;     // uint32   [1]            this rank's route epoch (device resident)
  long long off_arrived;   // uint32   [e_local]      rows landed per local expert
  long long off_retcnt;    // uint32   [1]            result rows landed for this rank's tokens
  long long off_meta;      // int      [cap_rows]     (source rank << 24) | pair index
  long long off_xs;        // half     [cap_rows + 256][H]
  long long off_ret;       // bf16     [max_pairs][H]
  long long cap_rows, max_pairs;
  uint32_t spin_budget;
};

template <typename T>
__device__ __forceinline__ T* ep_ptr(const EpCtx& c, int on_rank, long long off) {
  return reinterpret_cast<T*>(c.base[on_rank] + off);
}

__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// One CTA of 1024 threads.  offsets_local [e_local + 1], dest_base [E], cursor [E] are plain local arrays.
__global__ void __launch_bounds__(1024)
ep_route_kernel(const EpCtx c, const int* __restrict__ ids, int n_pairs, int* __restrict__ offsets_local,
                int* __restrict__ dest_base, int* __restrict__ cursor, int* status) {
  __shared__ int hist[1024];
  __shared__ int tot[1024];
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  const int E = c.E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  if (threadIdx.x == 0) {
    uint32_t* ep = ep_ptr<uint32_t>(c, c.rank, c.off_epoch);
    s_epoch = *ep + 1;
    *ep = s_epoch;
    s_ok = 1;
    *ep_ptr<uint32_t>(c, c.rank, c.off_retcnt) = 0;
  }
  for (int e = threadIdx.x; e < c.e_local; e += blockDim.x) ep_ptr<uint32_t>(c, c.rank, c.off_arrived)[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  // publish: histogram into every rank's table (own included), then the flag
  for (int i = threadIdx.x; i < c.world * E; i += blockDim.x) {
    const int r = i / E, e = i % E;
    ep_ptr<int>(c, r, c.off_counts)[c.rank * E + e] = hist[e];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < c.world) st_release_sys(ep_ptr<uint32_t>(c, threadIdx.x, c.off_flags) + c.rank, s_epoch);
  if (threadIdx.x < c.world) {
    if (!wait_flag(ep_ptr<uint32_t>(c, c.rank, c.off_flags) + threadIdx.x, s_epoch, c.spin_budget, status, 800 + threadIdx.x))
      s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) {
    // leave a consistent (empty) plan behind: nothing is dispatched, nothing is expected
    for (int e = threadIdx.x; e <= c.e_local; e += blockDim.x) offsets_local[e] = 0;
    for (int e = threadIdx.x; e < E; e += blockDim.x) { dest_base[e] = -1; cursor[e] = 0; }
    return;
  }
  const int* counts = ep_ptr<int>(c, c.rank, c.off_counts);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0;
    for (int s = 0; s < c.world; ++s) t += counts[s * E + e];
    tot[e] = t;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int owner = e / c.e_local;
    int base = 0;
    for (int j = owner * c.e_local; j < e; ++j) base += tot[j];           // experts before e on its owner
    for (int s = 0; s < c.rank; ++s) base += counts[s * E + e];           // sources before this rank
    dest_base[e] = base;
    cursor[e] = 0;
  }
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int j = 0; j < c.e_local; ++j) {
      offsets_local[j] = acc;
      acc += tot[c.rank * c.e_local + j];
    }
    offsets_local[c.e_local] = acc;
    if (acc > c.cap_rows) set_status(status, kBadIndex, 810);
  }
}

// One warp per (token, k) pair.
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const EpCtx c, const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ ids,
                   int n_pairs, const int* __restrict__ dest_base, int* __restrict__ cursor, int* status) {
  const int lane = threadIdx.x & 31;
  const int p = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (p >= n_pairs) return;
  const int e = ids[p];
  if (e < 0 || e >= c.E) return;
  const int base = dest_base[e];
  if (base < 0) return;
  int slot = 0;
  if (lane == 0) slot = base + atomicAdd(&cursor[e], 1);
  slot = __shfl_sync(0xffffffffu, slot, 0);
  if (slot >= c.cap_rows) {
    if (lane == 0) set_status(status, kBadIndex, 820);
    return;
  }
  const int owner = e / c.e_local;
  const int t = p / c.topk;
  const uint4* src = reinterpret_cast<const uint4*>(x + t * ldx);
  uint4* dst = reinterpret_cast<uint4*>(ep_ptr<__half>(c, owner, c.off_xs) + static_cast<long long>(slot) * c.H);
  for (int i = lane; i < c.H / 8; i += 32) {
    const uint4 v = __ldg(src + i);
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) oh[j] = __float22half2_rn(__bfloat1622float2(b[j]));
    dst[i] = o;
  }
  if (lane == 0) ep_ptr<int>(c, owner, c.off_meta)[slot] = (c.rank << 24) | p;
  __threadfence_system();
  __syncwarp();
  if (lane == 0) red_release_sys_add(ep_ptr<uint32_t>(c, owner, c.off_arrived) + (e % c.e_local), 1u);
}

// One warp per sorted row of this rank's expert output y [rows, H] bf16.
__global__ void __launch_bounds__(256)
ep_return_kernel(const EpCtx c, const __nv_bfloat16* __restrict__ y, const int* __restrict__ offsets_local, int max_rows,
                 int* status) {
  const int lane = threadIdx.x & 31;
  const int q = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (q >= max_rows || q >= offsets_local[c.e_local]) return;
  const int m = ep_ptr<int>(c, c.rank, c.off_meta)[q];
  const int src = (m >> 24) & 0xff, pair = m & 0xffffff;
  if (src >= c.world || pair >= c.max_pairs) {
    if (lane == 0) set_status(status, kBadIndex, 830);
    return;
  }
  const uint4* from = reinterpret_cast<const uint4*>(y + static_cast<long long>(q) * c.H);
  uint4* to = reinterpret_cast<uint4*>(ep_ptr<__nv_bfloat16>(c, src, c.off_ret) + static_cast<long long>(pair) * c.H);
  for (int i = lane; i < c.H / 8; i += 32) to[i] = from[i];
  __threadfence_system();
  __syncwarp();
  if (lane == 0) red_release_sys_add(ep_ptr<uint32_t>(c, src, c.off_retcnt), 1u);
}

// out[t] = sum_k w[t,k] * ret[t*topk + k] (+ shared[t]); one CTA per token.
__global__ void __launch_bounds__(256)
ep_combine_kernel(const EpCtx c, const float* __restrict__ w, const int* __restrict__ ids,
                  const __nv_bfloat16* __restrict__ shared, long long lds, __nv_bfloat16* __restrict__ out, long long ldo,
                  int T, int* status) {
  __shared__ int s_ok;
  const int t = blockIdx.x;
  if (threadIdx.x == 0) {
    // pairs with an out-of-range expert id were never dispatched: the route kernel's plan is the count to expect
    const uint32_t expect = static_cast<uint32_t>(T) * c.topk;
    const uint32_t* cnt = ep_ptr<uint32_t>(c, c.rank, c.off_retcnt);
    int ok = 0;
    for (uint32_t i = 0; i < c.spin_budget; ++i) {
      if (ld_acquire_sys(cnt) >= expect) { ok = 1; break; }
      if (i > 64) __nanosleep(64);
    }
    if (!ok) set_status(status, kTimeoutPeerFlag, 840);
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;
  const __nv_bfloat16* ret = ep_ptr<__nv_bfloat16>(c, c.rank, c.off_ret);
  for (int i = threadIdx.x; i < c.H / 8; i += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (shared != nullptr) add_bf16x8(acc, *reinterpret_cast<const uint4*>(shared + t * lds + i * 8));
    for (int k = 0; k < c.topk; ++k) {
      const int e = ids[t * c.topk + k];
      if (e < 0 || e >= c.E) continue;
      const float wk = w[t * c.topk + k];
      const uint4 v = *reinterpret_cast<const uint4*>(ret + (static_cast<long long>(t) * c.topk + k) * c.H + i * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] = fmaf(wk, f.x, acc[2 * j]);
        acc[2 * j + 1] = fmaf(wk, f.y, acc[2 * j + 1]);
      }
    }
    *reinterpret_cast<uint4*>(out + t * ldo + i * 8) = pack_bf16x8(acc);
  }
}

}  // namespace stk

using namespace stk;

STK_API int stk_ep_ctx_size() { return static_cast<int>(sizeof(EpCtx)); }

STK_API long long stk_ep_region_bytes(int world, int E, int e_local, int H, long long cap_rows, long long max_pairs) {
  long long off = 0;
  off += static_cast<long long>(world) * E * 4;            // counts
  off = (off + 255) / 256 * 256 + 256;                      // flags
  off += 256;                                               // epoch
  off += (static_cast<long long>(e_local) * 4 + 255) / 256 * 256;
  off += 256;                                               // retcnt
  off += (cap_rows * 4 + 255) / 256 * 256;                  // meta
  off += (cap_rows + 256) * H * 2;                          // xs
  off += max_pairs * H * 2;                                 // ret
  return off + 4096;
}

STK_API int stk_ep_ctx_fill(void* ctx, const long long* bases, int rank, int world, int E, int topk, int H,
                            long long cap_rows, long long max_pairs, int spin_budget) {
  if (world < 1 || world > kMaxRanks || E % world || E > 1024 || H % 8 || max_pairs >= (1 << 24)) return -1;
  EpCtx* c = static_cast<EpCtx*>(ctx);
  for (int r = 0; r < kMaxRanks; ++r) c->base[r] = r < world ? reinterpret_cast<uint8_t*>(bases[r]) : nullptr;
  c->rank = rank; c->world = world; c->E = E; c->e_local = E / world; c->topk = topk; c->H = H;
  long long off = 0;
  c->off_counts = off; off += static_cast<long long>(world) * E * 4; off = (off + 255) / 256 * 256;
  c->off_flags = off; off += 256;
  c->off_epoch = off; off += 256;
  c->off_arrived = off; off += (static_cast<long long>(c->e_local) * 4 + 255) / 256 * 256;
  c->off_retcnt = off; off += 256;
  c->off_meta = off; off += (cap_rows * 4 + 255) / 256 * 256;
  c->off_xs = off; off += (cap_rows + 256) * H * 2;
  c->off_ret = off; off += max_pairs * H * 2;
  c->cap_rows = cap_rows; c->max_pairs = max_pairs;
  c->spin_budget = static_cast<uint32_t>(spin_budget);
  return 0;
}

STK_API long long stk_ep_ctx_offset(const void* ctx, int which) {
  const EpCtx* c = static_cast<const EpCtx*>(ctx);
  switch (which) {
    case 0: return c->off_xs;
    case 1: return c->off_arrived;
    case 2: return c->off_ret;
    case 3: return c->off_meta;
    default: return -1;
  }
}

STK_API int stk_ep_route(const void* ctx, const int* ids, int n_pairs, int* offsets_local, int* dest_base, int* cursor,
                         int* status, void* stream) {
  const EpCtx* c = static_cast<const EpCtx*>(ctx);
  if (n_pairs > c->max_pairs) return -1;
  ep_route_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(*c, ids, n_pairs, offsets_local, dest_base, cursor, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_ep_dispatch(const void* ctx, const void* x, long long ldx, const int* ids, int n_pairs, const int* dest_base,
                            int* cursor, int* status, void* stream) {
  const EpCtx* c = static_cast<const EpCtx*>(ctx);
  if (n_pairs <= 0) return 0;
  if (ldx % 8) return -1;
  ep_dispatch_kernel<<<(n_pairs + 7) / 8, 256, 0, (cudaStream_t)stream>>>(*c, (const __nv_bfloat16*)x, ldx, ids, n_pairs,
                                                                        dest_base, cursor, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_ep_return(const void* ctx, const void* y, const int* offsets_local, int max_rows, int* status, void* stream) {
  const EpCtx* c = static_cast<const EpCtx*>(ctx);
  if (max_rows <= 0) return 0;
  ep_return_kernel<<<(max_rows + 7) / 8, 256, 0, (cudaStream_t)stream>>>(*c, (const __nv_bfloat16*)y, offsets_local, max_rows,
                                                                       status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_ep_combine(const void* ctx, const float* w, const int* ids, const void* shared, long long lds, void* out,
                           long long ldo, int T, int* status, void* stream) {
  const EpCtx* c = static_cast<const EpCtx*>(ctx);
  if (T <= 0) return 0;
  ep_combine_kernel<<<T, 256, 0, (cudaStream_t)stream>>>(*c, w, ids, (const __nv_bfloat16*)shared, lds, (__nv_bfloat16*)out,
                                                         ldo, T, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
