// Symmetric peer memory over NVLink and the all-reduce kernels built on it.
//
// Every rank allocates one region with cudaMalloc, exports it as a CUDA IPC handle, and maps
// every peer's region into its own address space.  Kernels then store straight into peer
// memory (plain st.global over NVLink through NVSwitch) and signal with release-stores of a
// monotonically increasing epoch; readers acquire-load the flags with a bounded spin and, on
// expiry, record {code, detail} in a status word and skip the dependent work.  No proxy
// thread, no host bounce, no multicast loads.
//
//   one-shot  (small messages): every rank pushes its whole buffer into slot [parity][rank] of
//             every peer, then sums the `world` slots it received in rank order in fp32
//             (deterministic, like the reference's k_reduce: overlay/dsv4_oneshot_ar.cu:104-115).
//   two-shot  (large messages): push chunk p to its owner p (reduce-scatter), the owner sums
//             and pushes the result to every peer (all-gather).
//
// Epochs live in device memory and are advanced by the kernels themselves, so a captured CUDA
// graph can replay a collective any number of times.  Slots are double-buffered by epoch
// parity: a rank can start call e+2 only after every peer has started e+1, i.e. finished e.
#include <string.h>

#include "common.cuh"
#include "symm.cuh"

namespace stk {

// ---- one-shot ---------------------------------------------------------------------
// grid = nblocks (<= kMaxArBlocks); block b owns 16-byte vectors [b*per, (b+1)*per).
__global__ void __launch_bounds__(512)
oneshot_ar_kernel(SymmCtx c, const uint4* __restrict__ in, uint4* __restrict__ out, long long n_vec, int kind,
                  int* status) {
  __shared__ int ok_s;
  const int b = blockIdx.x;
  const long long per = (n_vec + gridDim.x - 1) / gridDim.x;
  const long long v0 = b * per, v1 = min(n_vec, v0 + per);
  uint32_t* ep = epoch_ptr(c, kind, b);
  const uint32_t epoch = *ep + 1;
  const int par = epoch & 1;
  const long long slot_vecs = c.oneshot_bytes / 16;
  // push my chunk into slot [par][rank] of every rank (own included)
  for (int p = 0; p < c.world; ++p) {
    const int peer = (c.rank + p) % c.world;
    uint4* dst = reinterpret_cast<uint4*>(c.base[peer] + c.off_oneshot) + (static_cast<long long>(par) * c.world + c.rank) * slot_vecs;
    for (long long i = v0 + threadIdx.x; i < v1; i += blockDim.x) dst[i] = in[i];
  }
  __syncthreads();
  if (threadIdx.x < c.world) {
    __threadfence_system();      // cumulative with the barrier: every thread's pushes precede the flag
    st_release_sys(flag_ptr(c, threadIdx.x, kind, b, c.rank), epoch);
  }
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < c.world) {
    if (!wait_flag(flag_ptr(c, c.rank, kind, b, threadIdx.x), epoch, c.spin_budget, status, threadIdx.x)) ok_s = 0;
  }
  __syncthreads();
  if (ok_s) {
    const uint4* slots = reinterpret_cast<const uint4*>(c.base[c.rank] + c.off_oneshot) + static_cast<long long>(par) * c.world * slot_vecs;
    for (long long i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < c.world; ++r) add_bf16x8(acc, __ldcg(slots + r * slot_vecs + i));
      out[i] = pack_bf16x8(acc);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *ep = epoch;
}

// ---- two-shot ------------------------------------------------------------------------
// The message is cut into world chunks; grid blocks are spread over (chunk, sub-block).
__global__ void __launch_bounds__(512)
twoshot_ar_kernel(SymmCtx c, const uint4* __restrict__ in, uint4* __restrict__ out, long long n_vec, int kind,
                  int* status) {
  __shared__ int ok_s;
  const int b = blockIdx.x;
  const int nb = gridDim.x;
  uint32_t* ep = epoch_ptr(c, kind, b);
  const uint32_t epoch = *ep + 1;
  const int par = epoch & 1;
  const long long chunk = (n_vec + c.world - 1) / c.world;          // vectors per owner
  const long long per = (chunk + nb - 1) / nb;                      // this block's share of every chunk
  const long long o0 = b * per, o1 = min(chunk, o0 + per);
  // phase 1: push my piece of chunk p to owner p
  for (int p = 0; p < c.world; ++p) {
    const int peer = (c.rank + p) % c.world;
    uint4* dst = reinterpret_cast<uint4*>(c.base[peer] + c.off_rs) + (static_cast<long long>(par) * c.world + c.rank) * chunk;
    const long long g0 = peer * chunk;
    for (long long i = o0 + threadIdx.x; i < o1; i += blockDim.x) {
      if (g0 + i < n_vec) dst[i] = in[g0 + i];
    }
  }
  __syncthreads();
  if (threadIdx.x < c.world) {
    __threadfence_system();      // cumulative with the barrier: every thread's pushes precede the flag
    st_release_sys(flag_ptr(c, threadIdx.x, kind, b, c.rank), epoch);
  }
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < c.world) {
    if (!wait_flag(flag_ptr(c, c.rank, kind, b, threadIdx.x), epoch, c.spin_budget, status, 100 + threadIdx.x)) ok_s = 0;
  }
  __syncthreads();
  // phase 2: reduce my chunk, push the result to every rank's all-gather buffer
  if (ok_s) {
    const uint4* slots = reinterpret_cast<const uint4*>(c.base[c.rank] + c.off_rs) + static_cast<long long>(par) * c.world * chunk;
    const long long g0 = c.rank * chunk;
    for (long long i = o0 + threadIdx.x; i < o1; i += blockDim.x) {
      if (g0 + i >= n_vec) break;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < c.world; ++r) add_bf16x8(acc, __ldcg(slots + r * chunk + i));
      const uint4 v = pack_bf16x8(acc);
      for (int p = 0; p < c.world; ++p) {
        const int peer = (c.rank + p) % c.world;
        reinterpret_cast<uint4*>(c.base[peer] + c.off_ag + static_cast<long long>(par) * c.twoshot_bytes)[g0 + i] = v;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x < c.world) {
    __threadfence_system();
    st_release_sys(flag_ptr(c, threadIdx.x, kind + 1, b, c.rank), epoch);
  }
  __syncthreads();
  if (threadIdx.x < c.world) {
    if (!wait_flag(flag_ptr(c, c.rank, kind + 1, b, threadIdx.x), epoch, c.spin_budget, status, 200 + threadIdx.x)) ok_s = 0;
  }
  __syncthreads();
  // phase 3: copy this block's share of every chunk out of the all-gather buffer
  if (ok_s) {
    const uint4* ag = reinterpret_cast<const uint4*>(c.base[c.rank] + c.off_ag + static_cast<long long>(par) * c.twoshot_bytes);
    for (int p = 0; p < c.world; ++p) {
      const long long g0 = p * chunk;
      for (long long i = o0 + threadIdx.x; i < o1; i += blockDim.x) {
        if (g0 + i < n_vec) out[g0 + i] = __ldcg(ag + g0 + i);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *ep = epoch;
}

// ---- reduce-scatter and all-gather along dim 0 (sequence-parallel prefill) ---------------------------------------
// The two halves of the two-shot all-reduce as kernels of their own, over the same staging regions.  Because they
// share those regions with the all-reduce (whose parity scheme assumes a pure sequence of all-reduces), each closes
// the one window a neighbouring collective could reach: the reduce-scatter ends with a barrier (a rank reads its
// staging area after the last flag exchange, so a faster rank's next push must wait), the all-gather starts with one
// (a rank may still be copying a previous result out of the gather area).  A barrier is one flag exchange, about 5 us;
// these kernels move tens of megabytes.
constexpr int kRsKind = 5, kAgCollKind = 6, kBarKind = 7;
constexpr int kAgBarBlock0 = 1024;            // barrier flags of the all-gather live beside those of the reduce-scatter

__device__ __forceinline__ bool block_flag_exchange(const SymmCtx& c, int kind, int block, uint32_t epoch, int* ok_s,
                                                    int* status, int detail) {
  __syncthreads();
  if (threadIdx.x < c.world) {
    __threadfence_system();      // cumulative with the barrier: every thread's stores precede the flag
    st_release_sys(flag_ptr(c, threadIdx.x, kind, block, c.rank), epoch);
  }
  __syncthreads();
  if (threadIdx.x < c.world) {
    if (!wait_flag(flag_ptr(c, c.rank, kind, block, threadIdx.x), epoch, c.spin_budget, status, detail + threadIdx.x)) *ok_s = 0;
  }
  __syncthreads();
  return *ok_s != 0;
}

// in: [world * chunk_vecs] (chunk p is meant for rank p); out: [chunk_vecs] = sum over ranks of their chunk `rank`.
__global__ void __launch_bounds__(512)
symm_reduce_scatter_kernel(SymmCtx c, const uint4* __restrict__ in, uint4* __restrict__ out, long long chunk_vecs,
                           int* status) {
  __shared__ int ok_s;
  const int b = blockIdx.x, nb = gridDim.x;
  uint32_t* ep = epoch_ptr(c, kRsKind, b);
  const uint32_t epoch = *ep + 1;
  const int par = epoch & 1;
  const long long per = (chunk_vecs + nb - 1) / nb;
  const long long o0 = b * per, o1 = min(chunk_vecs, o0 + per);
  if (threadIdx.x == 0) ok_s = 1;
  for (int p = 0; p < c.world; ++p) {
    const int peer = (c.rank + p) % c.world;
    uint4* dst = reinterpret_cast<uint4*>(c.base[peer] + c.off_rs) + (static_cast<long long>(par) * c.world + c.rank) * chunk_vecs;
    const uint4* src = in + static_cast<long long>(peer) * chunk_vecs;
    for (long long i = o0 + threadIdx.x; i < o1; i += blockDim.x) dst[i] = __ldg(src + i);
  }
  if (block_flag_exchange(c, kRsKind, b, epoch, &ok_s, status, 700)) {
    const uint4* slots = reinterpret_cast<const uint4*>(c.base[c.rank] + c.off_rs) + static_cast<long long>(par) * c.world * chunk_vecs;
    for (long long i = o0 + threadIdx.x; i < o1; i += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < c.world; ++r) add_bf16x8(acc, __ldcg(slots + r * chunk_vecs + i));
      out[i] = pack_bf16x8(acc);
    }
  }
  block_flag_exchange(c, kBarKind, b, epoch, &ok_s, status, 720);      // nobody pushes again before everybody has read
  if (threadIdx.x == 0) *ep = epoch;
}

// shard: [shard_vecs]; out: [world * shard_vecs], rank-major.
__global__ void __launch_bounds__(512)
symm_all_gather_kernel(SymmCtx c, const uint4* __restrict__ shard, uint4* __restrict__ out, long long shard_vecs,
                       int* status) {
  __shared__ int ok_s;
  const int b = blockIdx.x, nb = gridDim.x;
  uint32_t* ep = epoch_ptr(c, kAgCollKind, b);
  const uint32_t epoch = *ep + 1;
  const int par = epoch & 1;
  const long long per = (shard_vecs + nb - 1) / nb;
  const long long o0 = b * per, o1 = min(shard_vecs, o0 + per);
  if (threadIdx.x == 0) ok_s = 1;
  if (block_flag_exchange(c, kBarKind, kAgBarBlock0 + b, epoch, &ok_s, status, 740)) {      // everybody has left the previous collective
    for (int p = 0; p < c.world; ++p) {
      const int peer = (c.rank + p) % c.world;
      uint4* dst = reinterpret_cast<uint4*>(c.base[peer] + c.off_ag + static_cast<long long>(par) * c.twoshot_bytes) +
                   static_cast<long long>(c.rank) * shard_vecs;
      for (long long i = o0 + threadIdx.x; i < o1; i += blockDim.x) dst[i] = __ldg(shard + i);
    }
    if (block_flag_exchange(c, kAgCollKind, b, epoch, &ok_s, status, 760)) {
      const uint4* ag = reinterpret_cast<const uint4*>(c.base[c.rank] + c.off_ag + static_cast<long long>(par) * c.twoshot_bytes);
      for (int r = 0; r < c.world; ++r)
        for (long long i = o0 + threadIdx.x; i < o1; i += blockDim.x) out[r * shard_vecs + i] = __ldcg(ag + r * shard_vecs + i);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *ep = epoch;
}

// A wait that nothing satisfies, on a local flag: exercises the timeout path without any peer.
__global__ void flag_timeout_probe_kernel(const uint32_t* flag, uint32_t epoch, uint32_t budget, int* status) {
  if (threadIdx.x == 0) {
    for (uint32_t i = 0; i < budget; ++i) {
      if (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) >= 0) return;
    }
    set_status(status, kTimeoutLocalFlag, 7);
  }
}

}  // namespace stk

using namespace stk;

STK_API int stk_symm_alloc(long long bytes, void** out) {
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return -1;
  if (cudaMemset(p, 0, bytes) != cudaSuccess) return -2;
  *out = p;
  return 0;
}
STK_API int stk_symm_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : -1; }
STK_API int stk_symm_export(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return -1;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
STK_API int stk_symm_import(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return -1;
  *out = p;
  return 0;
}
STK_API int stk_symm_close(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : -1; }

// ctx: pointer to a host copy of SymmCtx (filled by the Python side through stk_symm_ctx_fill).
STK_API int stk_symm_ctx_size() { return static_cast<int>(sizeof(SymmCtx)); }
STK_API int stk_symm_ctx_fill(void* ctx, const long long* bases, int rank, int world, long long off_flags,
                              long long off_epochs, long long off_oneshot, long long oneshot_bytes, long long off_rs,
                              long long off_ag, long long twoshot_bytes, long long off_gemm, long long gemm_bytes,
                              int spin_budget) {
  if (world > kMaxRanks) return -1;
  SymmCtx c;
  memset(&c, 0, sizeof(c));
  for (int i = 0; i < world; ++i) c.base[i] = reinterpret_cast<uint8_t*>(bases[i]);
  c.rank = rank; c.world = world; c.off_flags = off_flags; c.off_epochs = off_epochs; c.off_oneshot = off_oneshot;
  c.oneshot_bytes = oneshot_bytes; c.off_rs = off_rs; c.off_ag = off_ag; c.twoshot_bytes = twoshot_bytes;
  c.off_gemm = off_gemm; c.gemm_bytes = gemm_bytes;
  c.spin_budget = static_cast<uint32_t>(spin_budget);
  memcpy(ctx, &c, sizeof(c));
  return 0;
}

// In-place capable (out may equal in).  n_bytes must be a multiple of 16.
STK_API int stk_oneshot_allreduce(const void* ctx, const void* in, void* out, long long n_bytes, int nblocks,
                                  int* status, void* stream) {
  const SymmCtx* c = reinterpret_cast<const SymmCtx*>(ctx);
  if (n_bytes % 16 || n_bytes > c->oneshot_bytes || nblocks < 1 || nblocks > kMaxArBlocks) return -1;
  oneshot_ar_kernel<<<nblocks, 512, 0, (cudaStream_t)stream>>>(*c, (const uint4*)in, (uint4*)out, n_bytes / 16, 0, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_twoshot_allreduce(const void* ctx, const void* in, void* out, long long n_bytes, int nblocks,
                                  int* status, void* stream) {
  const SymmCtx* c = reinterpret_cast<const SymmCtx*>(ctx);
  if (n_bytes % 16 || n_bytes > c->twoshot_bytes || nblocks < 1 || nblocks > kMaxArBlocks) return -1;
  twoshot_ar_kernel<<<nblocks, 512, 0, (cudaStream_t)stream>>>(*c, (const uint4*)in, (uint4*)out, n_bytes / 16, 1, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// out[chunk] = sum over ranks of in[rank * chunk ..]; total_bytes = world * chunk bytes <= the two-shot capacity.
STK_API int stk_symm_reduce_scatter(const void* ctx, const void* in, void* out, long long total_bytes, int nblocks,
                                    int* status, void* stream) {
  const SymmCtx* c = reinterpret_cast<const SymmCtx*>(ctx);
  if (total_bytes <= 0 || total_bytes % (16ll * c->world) || total_bytes > c->twoshot_bytes || nblocks < 1 ||
      nblocks > kMaxArBlocks)
    return -1;
  symm_reduce_scatter_kernel<<<nblocks, 512, 0, (cudaStream_t)stream>>>(*c, (const uint4*)in, (uint4*)out,
                                                                         total_bytes / c->world / 16, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// out[rank-major] = every rank's shard; world * shard_bytes <= the two-shot capacity.
STK_API int stk_symm_all_gather(const void* ctx, const void* shard, void* out, long long shard_bytes, int nblocks,
                                int* status, void* stream) {
  const SymmCtx* c = reinterpret_cast<const SymmCtx*>(ctx);
  if (shard_bytes <= 0 || shard_bytes % 16 || shard_bytes * c->world > c->twoshot_bytes || nblocks < 1 ||
      nblocks > kMaxArBlocks)
    return -1;
  symm_all_gather_kernel<<<nblocks, 512, 0, (cudaStream_t)stream>>>(*c, (const uint4*)shard, (uint4*)out, shard_bytes / 16,
                                                                     status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// ---- all-gather push (feeds the arrival-gated GEMM) ----------------------------------------------
// Every rank copies its shard into slot `rank` of the gathered matrix at byte offset `dst_off` of EVERY
// rank's region (its own included) with 16-byte stores; the last CTA to finish raises flag (kAgKind, 0, rank)
// on every peer with the call's epoch and advances the local epoch.
constexpr int kAgKind = 4;

__global__ void __launch_bounds__(512)
ag_push_kernel(SymmCtx c, const uint4* __restrict__ shard, long long shard_vecs, long long dst_off, int* status) {
  __shared__ uint32_t s_last;
  const uint32_t epoch = *epoch_ptr(c, kAgKind, 0) + 1;
  for (int r = 0; r < c.world; ++r) {
    const int peer = (c.rank + r) % c.world;                       // start with the local copy, then spread over the links
    uint4* dst = reinterpret_cast<uint4*>(c.base[peer] + dst_off) + static_cast<long long>(c.rank) * shard_vecs;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < shard_vecs;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
      dst[i] = __ldg(shard + i);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* done = epoch_ptr(c, kAgKind, 1);
    s_last = atomicAdd(done, 1u) == gridDim.x - 1 ? 1u : 0u;
    if (s_last) *done = 0;
  }
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (threadIdx.x < c.world) st_release_sys(flag_ptr(c, threadIdx.x, kAgKind, 0, c.rank), epoch);
    if (threadIdx.x == 0) *epoch_ptr(c, kAgKind, 0) = epoch;
  }
  (void)status;
}

STK_API int stk_symm_ag_push(const void* ctx, const void* shard, long long shard_bytes, long long dst_off, int nblocks,
                             int* status, void* stream) {
  const SymmCtx* c = reinterpret_cast<const SymmCtx*>(ctx);
  if (shard_bytes <= 0 || shard_bytes % 16 || dst_off % 16 || nblocks < 1 || nblocks > kMaxArBlocks) return -1;
  ag_push_kernel<<<nblocks, 512, 0, (cudaStream_t)stream>>>(*c, (const uint4*)shard, shard_bytes / 16, dst_off, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// ---- peer-memory datapath probe -----------------------------------------------------------------------------------
// What the link rooflines divide by is measured, not assumed (the counterpart of the reference's probes/uma_datapath.cu:
// "which buffer types work, at what bandwidth, at what small-message latency").
//   peer_copy_kernel   16-byte loads from `src`, 16-byte stores to `dst`; either side may be a peer's region.  Block
//                      b of a multi-peer launch serves peer b % n_peers, so one launch drives all links at once.
//   peer_pingpong      `rounds` flag round trips between ranks `a` and `b` inside one kernel on each side (bounded
//                      waits): device time / rounds = the 8-byte store -> remote poll -> store back -> poll latency.
namespace stk {
struct PeerCopyJob {
  uint4* dst[kMaxRanks];
  const uint4* src[kMaxRanks];
  int n_peers;
  long long n_vec;          // per peer
};

__global__ void __launch_bounds__(512)
peer_copy_kernel(PeerCopyJob j) {
  const int p = blockIdx.x % j.n_peers;
  const int bpp = gridDim.x / j.n_peers;                 // blocks per peer
  const int bi = blockIdx.x / j.n_peers;
  if (bi >= bpp) return;
  uint4* dst = j.dst[p];
  const uint4* src = j.src[p];
  for (long long i = static_cast<long long>(bi) * blockDim.x + threadIdx.x; i < j.n_vec; i += static_cast<long long>(bpp) * blockDim.x)
    dst[i] = src[i];
}

__global__ void peer_pingpong_kernel(uint32_t* my_flag, uint32_t* peer_flag, int initiator, int rounds, uint32_t base,
                                     uint32_t budget, int* status) {
  if (threadIdx.x != 0) return;
  for (int r = 1; r <= rounds; ++r) {
    const uint32_t e = base + static_cast<uint32_t>(r);
    if (initiator) {
      st_release_sys(peer_flag, e);
      if (!wait_flag(my_flag, e, budget, status, 900)) return;
    } else {
      if (!wait_flag(my_flag, e, budget, status, 901)) return;
      st_release_sys(peer_flag, e);
    }
  }
}

}  // namespace stk
using namespace stk;

// dsts/srcs: n_peers device addresses each (this process's mappings); bytes per peer, a multiple of 16.
STK_API int stk_peer_copy(const long long* dsts, const long long* srcs, int n_peers, long long bytes, int blocks_per_peer,
                          void* stream) {
  if (n_peers < 1 || n_peers > kMaxRanks || bytes <= 0 || bytes % 16 || blocks_per_peer < 1) return -1;
  PeerCopyJob j;
  memset(&j, 0, sizeof(j));
  for (int i = 0; i < n_peers; ++i) {
    if ((dsts[i] & 15) || (srcs[i] & 15)) return -2;
    j.dst[i] = reinterpret_cast<uint4*>(dsts[i]);
    j.src[i] = reinterpret_cast<const uint4*>(srcs[i]);
  }
  j.n_peers = n_peers;
  j.n_vec = bytes / 16;
  peer_copy_kernel<<<blocks_per_peer * n_peers, 512, 0, (cudaStream_t)stream>>>(j);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_peer_pingpong(void* my_flag, void* peer_flag, int initiator, int rounds, int base, int budget, int* status,
                              void* stream) {
  if (rounds < 1 || my_flag == nullptr || peer_flag == nullptr) return -1;
  peer_pingpong_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((uint32_t*)my_flag, (uint32_t*)peer_flag, initiator, rounds,
                                                         (uint32_t)base, (uint32_t)budget, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_flag_timeout_probe(const void* flag, int epoch, int budget, int* status, void* stream) {
  flag_timeout_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((const uint32_t*)flag, (uint32_t)epoch, (uint32_t)budget,
                                                                status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
