// Per-step attention metadata built on the device (fixed-address outputs, no host sync):
//
//   swa_indices            per token: physical SWA-cache slots of [pos-W+1, pos] (-1 padded) + length
//                          (overlay/sparse_swa_dsv4.py:748-804)
//   swa_indices_noncausal  DSpark draft block: every query of a request sees [prefix-W, seq_len),
//                          block tokens included (overlay/sparse_swa_dsv4.py:808-870)
//   compressed_valid       n_valid[t] = (pos+1) / ratio   (causal bound of overlay/indexer.py:948-1020)
//   c128_indices           the most recent `cap` complete ratio-128 windows as slots
//   token_maps             tok_req / first / last positions from per-request query ranges
#define STK_PDL_CLASS 512      // bit of this file's kernels in the PDL mask (STK_PDL, stk_set_pdl_mask)
#include "common.cuh"

namespace stk {

__global__ void swa_indices_kernel(const int64_t* __restrict__ positions, const int* __restrict__ tok_req,
                                   const int* __restrict__ block_table, int bt_stride, int* __restrict__ slots,
                                   int ld, int* __restrict__ lens, int window) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const long long pos = positions[t];
  const int req = tok_req[t];
  int n = 0;
  long long lo = 0;
  if (pos >= 0 && req >= 0) {
    lo = pos - window + 1;
    if (lo < 0) lo = 0;
    n = static_cast<int>(pos - lo + 1);
  }
  for (int i = threadIdx.x; i < ld; i += blockDim.x) {
    int slot = -1;
    if (i < n) {
      const long long p = lo + i;
      const int page = block_table[static_cast<long long>(req) * bt_stride + (p >> 6)];
      if (page >= 0) slot = page * 64 + static_cast<int>(p & 63);
    }
    slots[static_cast<long long>(t) * ld + i] = slot;
  }
  if (threadIdx.x == 0) lens[t] = n;
}

// prefix_len[req]: tokens before the draft block; seq_len[req]: prefix + block tokens.
__global__ void swa_indices_noncausal_kernel(const int* __restrict__ tok_req, const int* __restrict__ prefix_len,
                                             const int* __restrict__ seq_len, const int* __restrict__ block_table,
                                             int bt_stride, int* __restrict__ slots, int ld, int* __restrict__ lens,
                                             int window) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int req = tok_req[t];
  int n = 0;
  long long lo = 0;
  if (req >= 0) {
    lo = static_cast<long long>(prefix_len[req]) - window;
    if (lo < 0) lo = 0;
    n = static_cast<int>(seq_len[req] - lo);
    if (n > ld) { lo += n - ld; n = ld; }
  }
  for (int i = threadIdx.x; i < ld; i += blockDim.x) {
    int slot = -1;
    if (i < n) {
      const long long p = lo + i;
      const int page = block_table[static_cast<long long>(req) * bt_stride + (p >> 6)];
      if (page >= 0) slot = page * 64 + static_cast<int>(p & 63);
    }
    slots[static_cast<long long>(t) * ld + i] = slot;
  }
  if (threadIdx.x == 0) lens[t] = n;
}

__global__ void compressed_valid_kernel(const int64_t* __restrict__ positions, int* __restrict__ n_valid, int T,
                                        int ratio) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const long long pos = positions[t];
  n_valid[t] = pos >= 0 ? static_cast<int>((pos + 1) / ratio) : 0;
}

__global__ void c128_indices_kernel(const int64_t* __restrict__ positions, const int* __restrict__ tok_req,
                                    const int* __restrict__ block_table, int bt_stride, int* __restrict__ slots,
                                    int ld, int* __restrict__ lens, int ratio, int cap) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const long long pos = positions[t];
  const int req = tok_req[t];
  int nv = (pos >= 0 && req >= 0) ? static_cast<int>((pos + 1) / ratio) : 0;
  const int lo = nv > cap ? nv - cap : 0;
  const int n = nv - lo;
  for (int i = threadIdx.x; i < ld; i += blockDim.x) {
    int slot = -1;
    if (i < n) {
      const int j = lo + i;
      const int page = block_table[static_cast<long long>(req) * bt_stride + (j >> 6)];
      if (page >= 0) slot = page * 64 + (j & 63);
    }
    slots[static_cast<long long>(t) * ld + i] = slot;
  }
  if (threadIdx.x == 0) lens[t] = n;
}

// query_start [n_req + 1] (token offsets), req_rows [n_req] (block-table row), start_pos [n_req]
// -> per token: request row, position, first/last position of its request in this step.
__global__ void token_maps_kernel(const int* __restrict__ query_start, const int* __restrict__ req_rows,
                                  const int* __restrict__ start_pos, int n_req, int* __restrict__ tok_req,
                                  int64_t* __restrict__ positions, int* __restrict__ first_pos,
                                  int* __restrict__ last_pos, const int* __restrict__ block_table, int bt_stride,
                                  int64_t* __restrict__ slot_mapping, int T_padded) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T_padded) return;
  int r = -1;
  for (int i = 0; i < n_req; ++i) {
    if (t >= query_start[i] && t < query_start[i + 1]) { r = i; break; }
  }
  if (r < 0) {
    tok_req[t] = -1;
    positions[t] = -1;
    first_pos[t] = 0;
    last_pos[t] = -1;
    if (slot_mapping) slot_mapping[t] = -1;
    return;
  }
  tok_req[t] = req_rows[r];
  positions[t] = start_pos[r] + (t - query_start[r]);
  first_pos[t] = start_pos[r];
  last_pos[t] = start_pos[r] + (query_start[r + 1] - query_start[r]) - 1;
  if (slot_mapping) {
    const long long p = start_pos[r] + (t - query_start[r]);
    const int page = block_table[static_cast<long long>(req_rows[r]) * bt_stride + (p >> 6)];
    slot_mapping[t] = page >= 0 ? static_cast<long long>(page) * 64 + (p & 63) : -1;
  }
}

}  // namespace stk

using namespace stk;

STK_API int stk_swa_indices(const int64_t* positions, const int* tok_req, const int* block_table, int bt_stride,
                            int* slots, int ld, int* lens, int T, int window, void* stream) {
  if (T <= 0) return 0;
  launch_pdl(swa_indices_kernel, dim3(T), dim3(128), 0, (cudaStream_t)stream, positions, tok_req, block_table, bt_stride, slots, ld, lens,
                                                          window);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_swa_indices_noncausal(const int* tok_req, const int* prefix_len, const int* seq_len,
                                      const int* block_table, int bt_stride, int* slots, int ld, int* lens, int T,
                                      int window, void* stream) {
  if (T <= 0) return 0;
  launch_pdl(swa_indices_noncausal_kernel, dim3(T), dim3(128), 0, (cudaStream_t)stream, tok_req, prefix_len, seq_len, block_table,
                                                                    bt_stride, slots, ld, lens, window);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_compressed_valid(const int64_t* positions, int* n_valid, int T, int ratio, void* stream) {
  if (T <= 0) return 0;
  launch_pdl(compressed_valid_kernel, dim3((T + 127) / 128), dim3(128), 0, (cudaStream_t)stream, positions, n_valid, T, ratio);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_c128_indices(const int64_t* positions, const int* tok_req, const int* block_table, int bt_stride,
                             int* slots, int ld, int* lens, int T, int ratio, int cap, void* stream) {
  if (T <= 0) return 0;
  launch_pdl(c128_indices_kernel, dim3(T), dim3(128), 0, (cudaStream_t)stream, positions, tok_req, block_table, bt_stride, slots, ld, lens,
                                                           ratio, cap);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_token_maps(const int* query_start, const int* req_rows, const int* start_pos, int n_req, int* tok_req,
                           int64_t* positions, int* first_pos, int* last_pos, const int* block_table, int bt_stride,
                           int64_t* slot_mapping, int T_padded, void* stream) {
  if (T_padded <= 0) return 0;
  launch_pdl(token_maps_kernel, dim3((T_padded + 127) / 128), dim3(128), 0, (cudaStream_t)stream, query_start, req_rows, start_pos, n_req,
                                                                              tok_req, positions, first_pos, last_pos,
                                                                              block_table, bt_stride, slot_mapping,
                                                                              T_padded);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
