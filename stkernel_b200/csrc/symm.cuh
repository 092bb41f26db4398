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

// ---- all-reduce folded into its producer and its consumer ------------------------------------------------
// For decode-sized activations the sum over ranks needs no kernel of its own.  The kernel that produces a
// row-parallel partial result stores it straight into every rank's receive slot, and the kernel that consumes the
// sum reads the `world` slots and adds them in a fixed order.  Each 8-byte word carries two bf16 values and the
// 32-bit epoch of the exchange, written with one store, so the payload is its own flag: no fence, no separate flag
// store, no wait kernel.  Slots are double-buffered by epoch parity; a word whose epoch is not the expected one has
// simply not arrived yet (the previous use of the slot left epoch - 2).
//
// Epochs are device-resident so that captured graphs replay: the producer reads counters[0] (the epoch the last
// consumer finished) and stamps counters[0] + 1; before it exits it writes that value to counters[1], which the
// consumer reads; before the consumer exits it writes the value back to counters[0].  Every CTA writes the same
// value, so no CTA has to be elected; a kernel never writes the word it reads.  Producer and consumer must be
// ordered on one stream (with programmatic dependent launch: read the counter after pdl_wait()).
//
// Safety of slot reuse: a rank starts exchange e + 2 only after its own consumer of e + 1 finished, which needed
// every peer's words of e + 1, which every peer wrote only after its consumer of e had finished reading.
struct LLAr {
  uint2* slots[kMaxRanks];   // each rank's receive region as mapped here: [2 parities][world sources][words]
  uint32_t* counters;        // local, two words (see above)
  long long words;           // capacity per (parity, source) in 8-byte words
  int rank, world;
  uint32_t spin_budget;      // polls before a consumer gives up on a word
};

__device__ __forceinline__ uint32_t ll_push_epoch(const LLAr& l) { return __ldcg(l.counters) + 1; }
__device__ __forceinline__ void ll_push_done(const LLAr& l, uint32_t e) { l.counters[1] = e; }
__device__ __forceinline__ uint32_t ll_read_epoch(const LLAr& l) { return __ldcg(l.counters + 1); }
__device__ __forceinline__ void ll_read_done(const LLAr& l, uint32_t e) { l.counters[0] = e; }

// Store one word (two bf16 values packed in `data`) into slot [parity(e)][my rank] of rank `peer`.
__device__ __forceinline__ void ll_store(const LLAr& l, uint32_t e, int peer, long long word, uint32_t data) {
  uint2* dst = l.slots[peer] + (static_cast<long long>(e & 1) * l.world + l.rank) * l.words + word;
  // one 64-bit scalar store: single-copy atomic, so a reader sees the payload and its epoch together
  const unsigned long long v = static_cast<unsigned long long>(data) | (static_cast<unsigned long long>(e) << 32);
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(v) : "memory");
}
__device__ __forceinline__ uint2 ll_load(const uint2* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return make_uint2(static_cast<uint32_t>(v), static_cast<uint32_t>(v >> 32));
}
// Word `word` of source rank `src` for exchange e, polled until its epoch matches.  On expiry records a status and
// returns false with data = 0 (the caller carries on with zeros: wrong numbers, no hang).
__device__ __forceinline__ bool ll_wait_word(const LLAr& l, uint32_t e, int src, long long word, uint32_t& data,
                                             int* status) {
  const uint2* p = l.slots[l.rank] + (static_cast<long long>(e & 1) * l.world + src) * l.words + word;
  for (uint32_t i = 0; i < l.spin_budget; ++i) {
    const uint2 v = ll_load(p);
    if (v.y == e) { data = v.x; return true; }
    if (i > 128) __nanosleep(20);
  }
  data = 0;
  set_status(status, kTimeoutPeerFlag, 300 + src);
  return false;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t v) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v));
}

}  // namespace stk
