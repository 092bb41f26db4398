// Sampling and speculative-decoding kernels.
//
//   gumbel_argmax     token = argmax(logits/T + g(seed, pos, v)); g from a counter-based hash so the
//                     noise is a pure function of (seed, position, vocab id): the drafter, the
//                     verifier and every tensor-parallel rank draw identical noise.
//   coupled_accept    accept draft i iff all earlier drafts were accepted and it equals the
//                     verifier's token at that offset; the emitted token is always the verifier's
//                     (overlay/dspark_speculator_v2.py:32-38,282-294).
//   markov_topk_bias  DSpark first-order Markov head on the base-logit top-k:
//                     out[idx] = base[idx] + W2[idx] . embed, -inf elsewhere
//                     (overlay/dspark_v2.py:184-236).
//   sample_threshold  per-row logit threshold of top-k and/or top-p (nucleus) truncation; the arg-max kernel then
//                     skips logits below it, so truncated sampling keeps the same (seed, position, vocab id) noise
//                     and drafts stay coupled with their verification.
//   argmax_exchange   tensor-parallel LM head without gathering logits: every rank takes the noisy arg-max of its own
//                     vocabulary shard (noise keyed by the global vocab id), pushes (value, id, status) to all ranks
//                     and picks the winner of the `world` candidates -- 24 bytes per row and rank over NVLink.
#define STK_PDL_CLASS 256      // bit of this file's kernels in the PDL mask (STK_PDL, stk_set_pdl_mask)
#include <string.h>

#include "common.cuh"
#include "symm.cuh"

namespace stk {

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x = (x ^ (x >> 16)) * 0x7FEB352Du;
  x = (x ^ (x >> 15)) * 0x846CA68Bu;
  x = x ^ (x >> 16);
  return x;
}

__device__ __forceinline__ uint32_t gumbel_key(long long seed, long long pos) {
  uint32_t h = mix32(static_cast<uint32_t>(seed & 0xffffffffLL) ^ 0x9E3779B9u);
  h = mix32(h ^ mix32(static_cast<uint32_t>((seed >> 32) & 0xffffffffLL) + 0x85EBCA6Bu));
  h = mix32(h ^ mix32(static_cast<uint32_t>(pos & 0xffffffffLL) + 0xC2B2AE35u));
  return h;
}

__device__ __forceinline__ float gumbel_from_key(uint32_t key, uint32_t v) {
  const uint32_t h = mix32(key ^ mix32(v + 0x27D4EB2Fu));
  const float u = (static_cast<float>(h >> 8) + 0.5f) * (1.0f / 16777216.0f);
  return -logf(-logf(u));
}

__device__ __forceinline__ uint32_t ordered_key_f(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

template <typename T> __device__ __forceinline__ float ld_logit(const T* p, long long i);
template <> __device__ __forceinline__ float ld_logit<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ld_logit<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}

// grid (rows, chunks).  part_val/part_idx: [rows, chunks].
template <typename T>
__global__ void __launch_bounds__(256)
gumbel_argmax_partial_kernel(const T* __restrict__ logits, long long ld, const float* __restrict__ temperature,
                             const int64_t* __restrict__ seed, const int64_t* __restrict__ pos,
                             const int* __restrict__ row_group, int pos_stride, float* __restrict__ part_val,
                             int* __restrict__ part_idx, float* __restrict__ processed, long long ldp, int V,
                             int v_offset, const uint32_t* __restrict__ thr_keys) {
  // v_offset: global vocabulary id of column 0 (vocabulary-sharded logits): noise and the reported id use global ids.
  // thr_keys: per-row ordered key below which a logit is outside the top-k / top-p set (nullptr: no truncation).
  pdl_wait();
  pdl_trigger();
  __shared__ float sv[8];
  __shared__ int si[8];
  const int row = blockIdx.x;
  const int g = row_group ? row_group[row] : row;          // request that owns seed/temperature
  const float temp = temperature[g];
  const bool greedy = temp <= 0.f;
  const float inv_t = greedy ? 1.f : 1.f / temp;
  // position of this row: pos[g] + (row offset inside the group) when pos_stride > 0
  const long long p = pos[g] + (pos_stride > 0 ? (row % pos_stride) : 0);
  const uint32_t key = gumbel_key(seed[g], p);
  const int chunk = (V + gridDim.y - 1) / gridDim.y;
  const int v0 = blockIdx.y * chunk, v1 = min(V, v0 + chunk);
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  const uint32_t thr = thr_keys ? thr_keys[row] : 0u;
  for (int v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
    const float raw = ld_logit<T>(logits, row * ld + v);
    float l = raw * inv_t;
    if (thr_keys != nullptr && ordered_key_f(raw) < thr) l = -INFINITY;
    if (processed) processed[row * ldp + v] = l;
    const int gv = v + v_offset;
    const float x = greedy ? l : l + gumbel_from_key(key, static_cast<uint32_t>(gv));
    if (x > best || (x == best && gv < best_i)) { best = x; best_i = gv; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; }
  }
  if (lane == 0) { sv[warp] = best; si[warp] = best_i; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < best_i)) { best = sv[w]; best_i = si[w]; }
    part_val[row * gridDim.y + blockIdx.y] = best;
    part_idx[row * gridDim.y + blockIdx.y] = best_i;
  }
}

__global__ void gumbel_argmax_final_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx,
                                           int chunks, int64_t* __restrict__ out, int rows) {
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int c = 0; c < chunks; ++c) {
    const float v = part_val[row * chunks + c];
    const int i = part_idx[row * chunks + c];
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  }
  out[row] = best_i == 0x7fffffff ? 0 : best_i;
}

// ---- top-k / top-p threshold ------------------------------------------------------------------------------------
// One CTA of 1024 threads per row.  Works on the ordered keys of the raw logits (truncation does not depend on the
// temperature's sign, and the mass of top-p is taken at the row's temperature as the samplers of the reference's engine
// do: softmax(logits / T)).  Radix select, 8 bits per pass:
//   top-k: walk the histogram of counts from the top until k entries are covered -> key of the k-th largest logit;
//   top-p: among the survivors of top-k, walk the histogram of probability mass until p of the total is covered.
// Ties at the threshold are kept (the set may be slightly larger than k / the minimal nucleus, never smaller).
// thr_out[row] = max(key_k, key_p): a logit is inside the set iff its key >= thr_out[row].
template <typename T>
__global__ void __launch_bounds__(1024)
sample_threshold_kernel(const T* __restrict__ logits, long long ld, const float* __restrict__ temperature,
                        const int* __restrict__ row_group, const int* __restrict__ top_k,
                        const float* __restrict__ top_p, uint32_t* __restrict__ thr_out, int V) {
  __shared__ int hist[256];
  __shared__ float mass[256];
  __shared__ uint32_t s_prefix;
  __shared__ int s_rem;
  __shared__ float s_mrem;
  __shared__ float s_red[32];
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  const int g = row_group ? row_group[row] : row;
  const T* lrow = logits + row * ld;
  const int k = top_k ? top_k[g] : 0;
  const float p = top_p ? top_p[g] : 1.f;
  const float temp = temperature[g];
  uint32_t key_k = 0u;
  if (k > 0 && k < V) {
    if (threadIdx.x == 0) { s_prefix = 0; s_rem = k; }
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      for (int v = threadIdx.x; v < V; v += blockDim.x) {
        const uint32_t key = ordered_key_f(ld_logit<T>(lrow, v));
        if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        int rem = s_rem, b = 255;
        for (; b > 0; --b) {
          if (hist[b] >= rem) break;
          rem -= hist[b];
        }
        s_prefix = prefix | (static_cast<uint32_t>(b) << shift);
        s_rem = rem;
      }
      __syncthreads();
    }
    key_k = s_prefix;
  }
  uint32_t key_p = 0u;
  if (p < 1.f && temp > 0.f) {
    const float inv_t = 1.f / temp;
    // row maximum and the total mass of the top-k survivors
    float mx = -INFINITY;
    for (int v = threadIdx.x; v < V; v += blockDim.x) mx = fmaxf(mx, ld_logit<T>(lrow, v));
    mx = block_max(mx, s_red);
    __syncthreads();
    float z = 0.f;
    for (int v = threadIdx.x; v < V; v += blockDim.x) {
      const float l = ld_logit<T>(lrow, v);
      if (ordered_key_f(l) >= key_k) z += __expf((l - mx) * inv_t);
    }
    z = block_sum(z, s_red);
    __syncthreads();
    if (threadIdx.x == 0) { s_prefix = 0; s_mrem = p * z; }
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      for (int i = threadIdx.x; i < 256; i += blockDim.x) mass[i] = 0.f;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      for (int v = threadIdx.x; v < V; v += blockDim.x) {
        const float l = ld_logit<T>(lrow, v);
        const uint32_t key = ordered_key_f(l);
        if (key >= key_k && (key & mask) == prefix) atomicAdd(&mass[(key >> shift) & 0xff], __expf((l - mx) * inv_t));
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        float rem = s_mrem;
        int b = 255;
        for (; b > 0; --b) {
          if (mass[b] >= rem) break;
          rem -= mass[b];
        }
        s_prefix = prefix | (static_cast<uint32_t>(b) << shift);
        s_mrem = rem;
      }
      __syncthreads();
    }
    key_p = s_prefix;
  }
  if (threadIdx.x == 0) thr_out[row] = key_k > key_p ? key_k : key_p;
}

// ---- arg-max across vocabulary shards ---------------------------------------------------------------------------
// One CTA, thread = row.  Reduces this rank's chunk candidates, pushes (value, global id, status word) into every
// rank's slot of the folded all-reduce exchange (three words per row), waits (bounded) for all ranks and keeps the
// largest value (ties: lowest id) -- the same token on every rank.  agreed_status = the largest status code any rank
// reported, so that every rank learns of a failed wait or a bad index on any of them with the step's tokens.
__global__ void __launch_bounds__(256)
argmax_exchange_kernel(const LLAr ll, const float* __restrict__ part_val, const int* __restrict__ part_idx, int chunks,
                       int64_t* __restrict__ out, int rows, const int* __restrict__ status_in, int* __restrict__ agreed_status,
                       int* status) {
  pdl_wait();
  pdl_trigger();
  const uint32_t e = ll_push_epoch(ll);
  const int row = threadIdx.x;
  if (row < rows) {
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int c = 0; c < chunks; ++c) {
      const float v = part_val[row * chunks + c];
      const int i = part_idx[row * chunks + c];
      if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
    const uint32_t st = status_in ? static_cast<uint32_t>(status_in[0]) : 0u;
    for (int p = 0; p < ll.world; ++p) {
      const int peer = (ll.rank + p) % ll.world;
      ll_store(ll, e, peer, 3LL * row, __float_as_uint(best));
      ll_store(ll, e, peer, 3LL * row + 1, static_cast<uint32_t>(best_i));
      ll_store(ll, e, peer, 3LL * row + 2, st);
    }
    float win = -INFINITY;
    int win_i = 0x7fffffff;
    uint32_t worst = 0;
    for (int r = 0; r < ll.world; ++r) {
      uint32_t dv, di, ds;
      ll_wait_word(ll, e, r, 3LL * row, dv, status);
      ll_wait_word(ll, e, r, 3LL * row + 1, di, status);
      ll_wait_word(ll, e, r, 3LL * row + 2, ds, status);
      const float v = __uint_as_float(dv);
      const int i = static_cast<int>(di);
      if (v > win || (v == win && i < win_i)) { win = v; win_i = i; }
      worst = ds > worst ? ds : worst;
    }
    out[row] = win_i == 0x7fffffff ? 0 : win_i;
    if (row == 0 && agreed_status != nullptr) agreed_status[0] = static_cast<int>(worst);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    ll_push_done(ll, e);
    ll_read_done(ll, e);
  }
}

// verifier [B, N+1], draft [B, N] -> n_acc [B], emitted [B, N+1] (-1 past the first mismatch)
__global__ void coupled_accept_kernel(const int64_t* __restrict__ verifier, const int64_t* __restrict__ draft,
                                      int64_t* __restrict__ n_acc, int64_t* __restrict__ emitted, int B, int N) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  bool ok = true;
  int acc = 0;
  for (int i = 0; i <= N; ++i) {
    const int64_t tok = verifier[b * (N + 1) + i];
    emitted[b * (N + 1) + i] = ok ? tok : -1;
    if (i < N) {
      ok = ok && (tok == draft[b * N + i]);
      acc += ok ? 1 : 0;
    }
  }
  n_acc[b] = acc;
}

// ---- Markov head -----------------------------------------------------------------------
__device__ __forceinline__ uint32_t fkey(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One CTA (1024 threads) per row: threshold of the k largest logits by radix select, then
// out[v] = (selected) ? base[v] + W2[v] . embed : -inf.   Ties at the threshold: lowest ids.
template <typename T>
__global__ void __launch_bounds__(1024)
markov_topk_bias_kernel(const T* __restrict__ base, long long ld, const __nv_bfloat16* __restrict__ w2,
                        const __nv_bfloat16* __restrict__ embed, long long lde, float* __restrict__ out,
                        long long ldo, int V, int R, int k) {
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining;
  __shared__ int warp_eq[32];
  __shared__ int base_eq;
  extern __shared__ float emb[];       // R floats
  const int row = blockIdx.x;
  const T* brow = base + row * ld;
  for (int i = threadIdx.x; i < R; i += blockDim.x) emb[i] = __bfloat162float(embed[row * lde + i]);
  if (threadIdx.x == 0) { s_prefix = 0; s_remaining = k; base_eq = 0; }
  const bool dense = k <= 0 || k >= V;
  uint32_t thr = 0;
  int need_eq = 0x7fffffff;
  if (!dense) {
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      for (int v = threadIdx.x; v < V; v += blockDim.x) {
        const uint32_t key = fkey(ld_logit<T>(brow, v));
        if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        int rem = s_remaining;
        int b = 255;
        for (; b > 0; --b) {
          if (hist[b] >= rem) break;
          rem -= hist[b];
        }
        s_prefix = prefix | (static_cast<uint32_t>(b) << shift);
        s_remaining = rem;
      }
      __syncthreads();
    }
    thr = s_prefix;
    need_eq = s_remaining;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int v0 = 0; v0 < V; v0 += blockDim.x) {
    const int v = v0 + threadIdx.x;
    const bool in = v < V;
    float l = 0.f;
    uint32_t key = 0;
    if (in) { l = ld_logit<T>(brow, v); key = fkey(l); }
    const bool gt = dense ? in : (in && key > thr);
    const bool eq = !dense && in && key == thr;
    const uint32_t be = __ballot_sync(0xffffffffu, eq);
    if (lane == 0) warp_eq[warp] = __popc(be);
    __syncthreads();
    int oe = base_eq;
    for (int w = 0; w < warp; ++w) oe += warp_eq[w];
    oe += __popc(be & ((1u << lane) - 1));
    const bool take = gt || (eq && oe < need_eq);
    if (in) {
      float o = -INFINITY;
      if (take) {
        const __nv_bfloat162* wr = reinterpret_cast<const __nv_bfloat162*>(w2 + static_cast<long long>(v) * R);
        float d0 = 0.f, d1 = 0.f;
        for (int i = 0; i < R / 2; ++i) {
          const __nv_bfloat162 wv = wr[i];
          d0 = fmaf(__low2float(wv), emb[2 * i], d0);
          d1 = fmaf(__high2float(wv), emb[2 * i + 1], d1);
        }
        o = l + d0 + d1;
      }
      out[row * ldo + v] = o;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int te = 0;
      for (int w = 0; w < 32; ++w) te += warp_eq[w];
      base_eq += te;
    }
    __syncthreads();
  }
}


// Sequential Markov sampling over pre-selected candidates, all N positions of a request in one launch.
// cand_idx/cand_val [B, N, K]: the base-logit top-K of every draft position (index -1 = unused slot).
// For i = 0..N-1:  e = W1[prev];  logit_c = cand_val[i, c] + W2[cand_idx[i, c]] . e;
//                  token_i = argmax_c(logit_c / T + g(seed, pos + i, vocab id))   (T <= 0: greedy; ties -> lowest id)
//                  prev = token_i.
// One CTA of 1024 threads per request; two threads per candidate, each streaming half of its W2 row with eight
// 16-byte loads in flight, so a position costs about two memory round trips.  This is the drafter's whole sampling loop: the proposals depend on each other, the candidate sets do not.
__global__ void __launch_bounds__(1024)
markov_chain_kernel(const int* __restrict__ cand_idx, const float* __restrict__ cand_val, const int64_t* __restrict__ anchors,
                    const __nv_bfloat16* __restrict__ w1, const __nv_bfloat16* __restrict__ w2,
                    const float* __restrict__ temperature, const int64_t* __restrict__ seed, const int64_t* __restrict__ pos,
                    int64_t* __restrict__ out, int N, int K, int R, int V) {
  extern __shared__ float emb[];                 // R floats
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ int s_prev;
  const int b = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half = threadIdx.x & 1;              // two threads per candidate, half a W2 row each
  const int hv = R / 16;                         // 16-byte vectors per half row
  const float temp = temperature[b];
  const bool greedy = temp <= 0.f;
  const float inv_t = greedy ? 1.f : 1.f / temp;
  if (threadIdx.x == 0) {
    const long long a = anchors[b];
    s_prev = (a >= 0 && a < V) ? static_cast<int>(a) : 0;
  }
  __syncthreads();
  for (int i = 0; i < N; ++i) {
    const int prev = s_prev;
    for (int r = threadIdx.x; r < R; r += blockDim.x) emb[r] = __bfloat162float(w1[static_cast<long long>(prev) * R + r]);
    __syncthreads();
    const uint32_t key = gumbel_key(seed[b], pos[b] + i);
    const int* ci = cand_idx + (static_cast<long long>(b) * N + i) * K;
    const float* cv = cand_val + (static_cast<long long>(b) * N + i) * K;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int c0 = 0; c0 < K; c0 += 512) {
      const int c = c0 + (threadIdx.x >> 1);
      const int v = c < K ? ci[c] : -1;
      const bool valid = v >= 0 && v < V;
      float d = 0.f;
      if (valid) {
        const uint4* row = reinterpret_cast<const uint4*>(w2 + static_cast<long long>(v) * R) + half * hv;
        const float* e = emb + half * (R / 2);
        for (int j0 = 0; j0 < hv; j0 += 8) {
          uint4 q[8];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (j0 + j < hv) q[j] = __ldg(row + j0 + j);        // eight loads in flight before the first multiply
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (j0 + j < hv) {
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q[j]);
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const float2 f = __bfloat1622float2(h[u]);
                d = fmaf(f.x, e[8 * (j0 + j) + 2 * u], fmaf(f.y, e[8 * (j0 + j) + 2 * u + 1], d));
              }
            }
          }
        }
      }
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      if (valid && half == 0) {
        const float l = (cv[c] + d) * inv_t;
        const float x = greedy ? l : l + gumbel_from_key(key, static_cast<uint32_t>(v));
        if (x > best || (x == best && v < best_i)) { best = x; best_i = v; }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; }
    }
    if (lane == 0) { sv[warp] = best; si[warp] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float bb = sv[0];
      int bi = si[0];
      for (int w = 1; w < 32; ++w)
        if (sv[w] > bb || (sv[w] == bb && si[w] < bi)) { bb = sv[w]; bi = si[w]; }
      if (bi == 0x7fffffff) bi = 0;              // no candidate at all: emit token 0 rather than an invalid id
      s_prev = bi;
      out[static_cast<long long>(b) * N + i] = bi;
    }
    __syncthreads();
  }
}

}  // namespace stk

using namespace stk;

// part_val/part_idx: scratch of rows*chunks entries each.  row_group may be null (row == request).
// top_k (int per request, <= 0: off) / top_p (float per request, >= 1: off) / thr_scratch (uint32 per row): all three
// nullptr for untruncated sampling.  v_offset: global vocabulary id of logits column 0.  ll_ctx != nullptr: the logits
// are one rank's vocabulary shard; the winner is agreed on across the ranks of the exchange (at most 256 rows, no
// truncation) and agreed_status receives the largest status code of any rank (status_in = this rank's status word).
STK_API int stk_gumbel_argmax(const void* logits, long long ld, int logits_bf16, const float* temperature,
                              const int64_t* seed, const int64_t* pos, const int* row_group, int pos_stride,
                              float* part_val, int* part_idx, int chunks, int64_t* out, float* processed,
                              long long ldp, int rows, int V, const int* top_k, const float* top_p,
                              void* thr_scratch, int v_offset, const void* ll_ctx, const int* status_in,
                              int* agreed_status, int* status, void* stream) {
  if (rows <= 0) return 0;
  dim3 grid(rows, chunks);
  cudaStream_t st = (cudaStream_t)stream;
  uint32_t* thr = nullptr;
  if (top_k != nullptr || top_p != nullptr) {
    if (thr_scratch == nullptr || ll_ctx != nullptr) return -1;
    thr = reinterpret_cast<uint32_t*>(thr_scratch);
    if (logits_bf16)
      launch_pdl(sample_threshold_kernel<__nv_bfloat16>, dim3(rows), dim3(1024), 0, st, (const __nv_bfloat16*)logits, ld,
                 temperature, row_group, top_k, top_p, thr, V);
    else
      launch_pdl(sample_threshold_kernel<float>, dim3(rows), dim3(1024), 0, st, (const float*)logits, ld, temperature,
                 row_group, top_k, top_p, thr, V);
  }
  if (logits_bf16)
    launch_pdl(gumbel_argmax_partial_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16*)logits, ld, temperature,
                                                                      seed, pos, row_group, pos_stride, part_val,
                                                                      part_idx, processed, ldp, V, v_offset, (const uint32_t*)thr);
  else
    launch_pdl(gumbel_argmax_partial_kernel<float>, dim3(grid), dim3(256), 0, st, (const float*)logits, ld, temperature, seed, pos,
                                                              row_group, pos_stride, part_val, part_idx, processed,
                                                              ldp, V, v_offset, (const uint32_t*)thr);
  if (ll_ctx != nullptr) {
    LLAr ll;
    memcpy(&ll, ll_ctx, sizeof(ll));
    if (rows > 256 || 3LL * rows > ll.words) return -2;
    launch_pdl(argmax_exchange_kernel, dim3(1), dim3(256), 0, st, ll, (const float*)part_val, (const int*)part_idx, chunks, out,
               rows, status_in, agreed_status, status);
  } else {
    launch_pdl(gumbel_argmax_final_kernel, dim3((rows + 127) / 128), dim3(128), 0, st, part_val, part_idx, chunks, out, rows);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_coupled_accept(const int64_t* verifier, const int64_t* draft, int64_t* n_acc, int64_t* emitted, int B,
                               int N, void* stream) {
  if (B <= 0) return 0;
  coupled_accept_kernel<<<(B + 127) / 128, 128, 0, (cudaStream_t)stream>>>(verifier, draft, n_acc, emitted, B, N);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_markov_topk_bias(const void* base, long long ld, int base_bf16, const void* w2, const void* embed,
                                 long long lde, float* out, long long ldo, int rows, int V, int R, int k,
                                 void* stream) {
  if (rows <= 0) return 0;
  if (R % 2) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  if (base_bf16)
    markov_topk_bias_kernel<__nv_bfloat16><<<rows, 1024, R * sizeof(float), st>>>(
        (const __nv_bfloat16*)base, ld, (const __nv_bfloat16*)w2, (const __nv_bfloat16*)embed, lde, out, ldo, V, R, k);
  else
    markov_topk_bias_kernel<float><<<rows, 1024, R * sizeof(float), st>>>(
        (const float*)base, ld, (const __nv_bfloat16*)w2, (const __nv_bfloat16*)embed, lde, out, ldo, V, R, k);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

STK_API int stk_markov_chain(const int* cand_idx, const float* cand_val, const int64_t* anchors, const void* w1,
                             const void* w2, const float* temperature, const int64_t* seed, const int64_t* pos,
                             int64_t* out, int B, int N, int K, int R, int V, void* stream) {
  if (B <= 0 || N <= 0) return 0;
  if (R % 16 || K <= 0) return -1;
  markov_chain_kernel<<<B, 1024, R * sizeof(float), (cudaStream_t)stream>>>(
      cand_idx, cand_val, anchors, (const __nv_bfloat16*)w1, (const __nv_bfloat16*)w2, temperature, seed, pos, out, N, K, R, V);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
