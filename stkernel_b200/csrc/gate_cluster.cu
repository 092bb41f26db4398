// Router gate projection + top-k expert selection for decode-sized batches as ONE thread-block cluster.
//
// The gate is a [E, K] bf16 matrix (E = 256 experts, K = 4096): 2 MB, far too little work to fill the GPU, so its
// time is the chain of dependent round trips, not bytes.  A grid of independent CTAs needs global memory to bring
// the E logits together (atomics or stores, a fence, an arrival counter, reading the logits back: four or five L2
// round trips after the dot products).  Here the CTAs of a 16-wide cluster own E/16 experts each, one warp per
// expert row:
//   * before `griddepcontrol.wait` every warp pulls its whole weight row into registers (weights are immutable, so
//     the loads overlap the tail of the kernel that produces the activations);
//   * after it: one load of the token(s), the dot products, a warp sum, ONE store per logit into the shared memory of
//     the cluster's first CTA through distributed shared memory, one cluster barrier;
//   * the first CTA routes: one warp per token runs the selection of router.cuh on the logits in its shared memory.
// Counterpart of the fused small-M gate of overlay/nvidia_model.py:565-670 (split-K Triton partials + a torch sum +
// the separate top-k kernel).
#include <cooperative_groups.h>

#include "common.cuh"
#include "router.cuh"

#define STK_PDL_CLASS 2      // bit of this file's kernels in the PDL mask (STK_PDL, stk_set_pdl_mask)

namespace cg = cooperative_groups;
using namespace stk;

namespace {

constexpr int kGcCluster = 16;      // CTAs per cluster (above the portable 8: the kernel opts in)
constexpr int kGcWarps = 16;        // warps per CTA
constexpr int kGcIters = 16;        // 16-byte chunks per lane per row: K <= 16 * 32 * 8 = 4096
constexpr int kGcMaxT = 8;
constexpr int kGcMaxE = 512;

struct GateClusterArgs {
  const __nv_bfloat16* W;
  long long ldw;                    // elements
  const __nv_bfloat16* x;
  long long ldx;
  int T, E, K;
  RouterArgs router;
};

__device__ __forceinline__ void gc_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void gc_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

__global__ void __launch_bounds__(kGcWarps * 32, 1) gate_route_cluster_kernel(GateClusterArgs a) {
  cg::cluster_group cluster = cg::this_cluster();
  const int crank = static_cast<int>(cluster.block_rank());
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_chunks = a.K >> 3;
  const int rows_per_cta = (a.E + kGcCluster - 1) / kGcCluster;        // host: rows_per_cta <= 2 * kGcWarps
  __shared__ __align__(16) float s_logits[kGcMaxT][kGcMaxE];            // used in the cluster's first CTA only

  // first row of this warp, into registers ahead of the previous kernel's completion
  uint4 wv[kGcIters];
  const int e0 = crank * rows_per_cta + warp;
  const bool have0 = warp < rows_per_cta && e0 < a.E;
  {
    const uint4* wrow = reinterpret_cast<const uint4*>(a.W + static_cast<long long>(have0 ? e0 : 0) * a.ldw);
#pragma unroll
    for (int it = 0; it < kGcIters; ++it) {
      const int c = it * 32 + lane;
      wv[it] = (have0 && c < n_chunks) ? __ldg(wrow + c) : make_uint4(0, 0, 0, 0);
    }
  }
  pdl_trigger();
  pdl_wait();
  // the tokens: one burst of 16-byte asynchronous copies into shared memory (one memory round trip for any T)
  extern __shared__ __align__(16) uint8_t s_x[];                        // [T][K] bf16
  for (int q = threadIdx.x; q < a.T * n_chunks; q += blockDim.x) {
    const int t = q / n_chunks, kc = q - t * n_chunks;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(s_x + (static_cast<size_t>(t) * n_chunks + kc) * 16)),
                 "l"(a.x + static_cast<long long>(t) * a.ldx + kc * 8) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  float* dst = cluster.map_shared_rank(&s_logits[0][0], 0);
  for (int e = e0, first = 1; e < min(a.E, (crank + 1) * rows_per_cta); e += kGcWarps, first = 0) {
    if (!first) {
      const uint4* wrow = reinterpret_cast<const uint4*>(a.W + static_cast<long long>(e) * a.ldw);
#pragma unroll
      for (int it = 0; it < kGcIters; ++it) {
        const int c = it * 32 + lane;
        wv[it] = c < n_chunks ? __ldg(wrow + c) : make_uint4(0, 0, 0, 0);
      }
    }
    for (int t = 0; t < a.T; ++t) {
      const uint4* xrow = reinterpret_cast<const uint4*>(s_x) + static_cast<size_t>(t) * n_chunks;
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int it = 0; it < kGcIters; ++it) {
        const int c = it * 32 + lane;
        if (c < n_chunks) {
          const uint4 xv = xrow[c];
          const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv[it]);
          const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 wf = __bfloat1622float2(wp[j]), xf = __bfloat1622float2(xp[j]);
            acc0 = fmaf(wf.x, xf.x, acc0);
            acc1 = fmaf(wf.y, xf.y, acc1);
          }
        }
      }
      const float v = warp_sum(acc0 + acc1);
      if (lane == 0) dst[t * kGcMaxE + e] = v;
    }
  }
  // the stores above are released by the arrive, acquired by the wait; every CTA stays until the first one has them
  gc_cluster_arrive();
  gc_cluster_wait();
  if (crank == 0) {
    for (int t = warp; t < a.T; t += kGcWarps) route_token<false>(a.router, &s_logits[t][0], t, lane);
  }
}

// Whether a 16-CTA cluster of this kernel can be resident on the current device (asked once per process).
bool gate_cluster_launchable() {
  static int state = 0;          // 0 unknown, 1 yes, -1 no
  if (state != 0) return state > 0;
  state = -1;
  if (cudaFuncSetAttribute(gate_route_cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  if (cudaFuncSetAttribute(gate_route_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kGcMaxT * kGcIters * 32 * 16) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kGcCluster);
  cfg.blockDim = dim3(kGcWarps * 32);
  cfg.dynamicSmemBytes = kGcMaxT * kGcIters * 32 * 16;       // the largest case: 8 tokens x 4096 values
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kGcCluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gate_route_cluster_kernel, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  if (n >= 1) state = 1;
  return state > 0;
}

}  // namespace

STK_API int stk_gate_route_cluster_ok() { return gate_cluster_launchable() ? 1 : 0; }

// x [T, K] bf16 (row stride ldx elements, 16-byte aligned rows), W [E, K] bf16; writes ids [T, topk] and weights [T, topk].
// Returns -1 when the shape is outside this kernel (T > 8, K > 4096 or not a multiple of 8, E > 512, topk > 32, rows not
// 16-byte aligned); the caller then uses the grid-wide path.
STK_API int stk_gate_route_cluster(const void* W, long long ldw, const void* x, long long ldx, int T, int E, int K,
                                   const float* bias, const int* tid2eid, const int64_t* token_ids, int vocab, int* ids,
                                   float* weights, int topk, int scoring, int renorm, float scaling, int* status,
                                   void* stream) {
  if (T < 1 || T > kGcMaxT || K % 8 || K > kGcIters * 32 * 8 || E < 1 || E > kGcMaxE || topk < 1 || topk > 32) return -1;
  if ((ldw % 8) || (ldx % 8) || (reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(x) & 15)) return -1;
  if ((E + kGcCluster - 1) / kGcCluster > 2 * kGcWarps) return -1;
  if (!gate_cluster_launchable()) return -1;
  GateClusterArgs a;
  a.W = static_cast<const __nv_bfloat16*>(W);
  a.ldw = ldw;
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.ldx = ldx;
  a.T = T; a.E = E; a.K = K;
  a.router = RouterArgs{bias, tid2eid, token_ids, vocab, ids, weights, E, topk, scoring, renorm, scaling, status};
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kGcCluster);
  cfg.blockDim = dim3(kGcWarps * 32);
  cfg.dynamicSmemBytes = static_cast<size_t>(T) * K * 2;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kGcCluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_use((cudaStream_t)stream, STK_PDL_CLASS) ? 2 : 1;
  if (cudaLaunchKernelEx(&cfg, gate_route_cluster_kernel, a) != cudaSuccess) {
    cudaGetLastError();
    return -4;
  }
  return 0;
}
