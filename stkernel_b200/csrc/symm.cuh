// Symmetric-region descriptor and flag primitives shared by the collective kernels and by the
// kernels that fuse a collective into their epilogue.
#pragma once
#include "common.cuh"

namespace stk {

constexpr int kMaxRanks = 8;
constexpr int kMaxArBlocks = 256;

struct SymmCtx {
  uint8_t* base[kMaxRanks];   // each rank's region as mapped in this process (base[rank] = own)
  int rank, world;
  long long off_flags;        // uint32 flags
  long long off_epochs;       // uint32 local epoch counters (only the owner reads/writes)
  long long off_oneshot;      // [2][world][oneshot_bytes]
  long long oneshot_bytes;
  long long off_rs;           // [2][world][chunk_bytes]   reduce-scatter receive slots
  long long off_ag;           // [2][total_bytes]          all-gather result
  long long twoshot_bytes;    // capacity of one all-gather buffer
  long long off_gemm;         // [2][world][gemm_bytes]    slots of the GEMM-fused all-reduce
  long long gemm_bytes;
  uint32_t spin_budget;
};

// flag layout (uint32 index): kind * kMaxArBlocks*kMaxRanks*... kept simple: [kind][block][src]
__device__ __forceinline__ uint32_t* flag_ptr(const SymmCtx& c, int on_rank, int kind, int block, int src) {
  return reinterpret_cast<uint32_t*>(c.base[on_rank] + c.off_flags) +
         (static_cast<long long>(kind) * 4096 + block) * kMaxRanks + src;
}
__device__ __forceinline__ uint32_t* epoch_ptr(const SymmCtx& c, int kind, int block) {
  return reinterpret_cast<uint32_t*>(c.base[c.rank] + c.off_epochs) + kind * 4096 + block;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Bounded wait for flag >= epoch (wrap-safe).  Returns false on expiry.
__device__ __forceinline__ bool wait_flag(const uint32_t* p, uint32_t epoch, uint32_t budget, int* status, int detail) {
  for (uint32_t i = 0; i < budget; ++i) {
    if (static_cast<int32_t>(ld_acquire_sys(p) - epoch) >= 0) return true;
    if (i > 64) __nanosleep(40);
  }
  set_status(status, kTimeoutPeerFlag, detail);
  return false;
}

__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4& v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[2 * i] += __low2float(h[i]);
    acc[2 * i + 1] += __high2float(h[i]);
  }
}
__device__ __forceinline__ uint4 pack_bf16x8(const float (&acc)[8]) {
  uint4 o;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
  return o;
}

}  // namespace stk
