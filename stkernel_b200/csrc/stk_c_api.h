// C entry points of libstk_b200.so.  Every function takes raw device pointers and a
// CUDA stream (as void*), allocates nothing unless its comment says so, and returns 0
// on a successful launch or a negative code for rejected arguments.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

// ---- dense GEMM (gemm_tcgen05.cu) ----
int stk_gemm_pick_bt(int T, int is_fp8);
int stk_gemm_pick_splits(int T, int N, int K, int is_fp8, int sm_count);
long long stk_gemm_workspace_bytes(int T, int N, int splits);
int stk_gemm(const void* W, long long ldw, const void* X, long long ldx, void* out, long long ldo, int T, int N,
             int K, int is_fp8, int out_fp32, const float* w_scale, int w_scale_ld, const float* x_scale,
             int x_scale_ld, int splits, float* workspace, int* counters, int* status, int sm_count, int groups,
             const void* ar_ctx, void* stream);

#ifdef __cplusplus
}
#endif
