// stk_gemm_noalloc — the split-K tensor-core GEMM for callers that must not allocate.
//
// This entry point has no counterpart in the reference; it exists for hosts that embed the library
// where device allocation is off limits: a plug-in running inside another runtime's stream callback
// or captured region, a real-time loop that may not take the allocator's lock, or a process whose
// memory budget was fixed at start-up and whose cudaMalloc would therefore fail or stall.
//
// What it does: out[T, N] = X[T, K] * W[N, K]^T, exactly like stk_gemm, except that the split-K
// workspace (fp32 partial tiles) and the per-tile arrival counters are not supplied by the caller.
// They live in one array built into the library image (8 MiB + 16 KiB of device memory per GPU that
// loads the library, held until the process exits).  The caller still passes the inputs and `out`.
//
// Limits and rules:
//   * splits * T * N * 4 bytes must not exceed stk_gemm_noalloc_max_workspace_bytes() (8 MiB) and the
//     output may have at most 4096 tiles of 128 x tile_T; larger problems are rejected with -32 / -33
//     before anything is launched.  With splits == 1 no scratch is used and any size is accepted.
//   * Neither this function nor anything it calls invokes cudaMalloc, cudaFree or an allocating
//     library routine.
//   * The first call on each device looks up the device address of the built-in array (one
//     cudaGetSymbolAddress, with that device current).  Make that first call outside of any stream
//     capture; later calls do no set-up.
//   * All calls on a device share the one array.  Two calls whose kernels can overlap on the GPU
//     (different streams, no dependency between them) race on it; order them with an event or keep
//     them on one stream.  The counters are zero between calls: the kernel resets each one as its
//     tile completes; the workspace keeps the previous call's partials and is fully overwritten
//     before it is read.
//   * After a call that left a non-zero code in `status` (a wait inside the kernel ran out), the
//     counters may be left non-zero and nothing outside the library can reach them: enqueue
//     stk_gemm_noalloc_reset(stream) before the next split-K call.
//   * `out` may have any alignment and row stride: the split-K reduction uses vector stores only when
//     `out` is 16-byte aligned with ldo % 4 == 0 (fp32) or 4-byte aligned with an even ldo (bf16), and
//     element stores otherwise.
//   * The array's device address is cached per device ordinal for the primary context (the one the
//     CUDA runtime uses); a host that drives several contexts on one device must make the primary
//     context current for these calls.
//   * Return value: 0 on launch, negative on rejected arguments (same codes as stk_gemm, plus
//     -30 no current device, -31 symbol lookup failed, -32 workspace too small, -33 too many tiles,
//     -34 reset could not be enqueued).
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

long long stk_gemm_noalloc_max_workspace_bytes(void);

int stk_gemm_noalloc(const void* W, long long ldw, const void* X, long long ldx, void* out, long long ldo, int T, int N,
                     int K, int is_fp8, int out_fp32, const float* w_scale, int w_scale_ld, const float* x_scale,
                     int x_scale_ld, int splits, int* status, int sm_count, void* stream);

// Zeroes the built-in tile counters on `stream`; allocates nothing.  See the rule on non-zero status above.
int stk_gemm_noalloc_reset(void* stream);

#ifdef __cplusplus
}
#endif
