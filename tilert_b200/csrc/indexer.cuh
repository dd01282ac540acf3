// DSA lightning indexer: scores every cached key for each query token, then selects the top-k
// key positions with a radix select.
//
//   logit[s, t] = sum_h w[s, h] * relu(q[s, h, :] . k[t, :])        t <= position of token s
//
// Scoring is HBM-bound on the key scan (256 bytes per key, read once); the dot products run on
// bf16 tensor-core MMAs (keys are the M dimension, heads the N dimension).  Selection works on
// the order-preserving unsigned image of the f32 logits, so it is exact: the k largest values,
// equal values by lower index first.
#pragma once

#include "common.cuh"

namespace tb {

constexpr int kIdxWarps = 4;
constexpr int kIdxKeysPerWarp = 16;
constexpr int kIdxPitch = 136;  // bf16 elements per smem row (128 + 8 pad: conflict-free ldmatrix)

// grid = (ceil(T / 64), tokens); block = 128 threads; dynamic smem = (H + 64) * kIdxPitch * 2 bytes
template <int H>
__global__ void __launch_bounds__(kIdxWarps * 32) indexer_logits_kernel(
    const __nv_bfloat16* __restrict__ q,       // [tokens, H, 128]
    const __nv_bfloat16* __restrict__ kcache,  // [T, 128]
    const __nv_bfloat16* __restrict__ w,       // [tokens, H]
    float* __restrict__ logits,                // [tokens, logits_stride]
    long long logits_stride, int n_keys,       // keys scored: t in [0, n_keys)
    const int* __restrict__ pos, int pos_offset  // token s may see keys t <= *pos + pos_offset + s
) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [H][pitch]
  __nv_bfloat16* sk = sq + H * kIdxPitch;                          // [64][pitch]
  __shared__ float sw[H];
  const int tok = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int key0 = blockIdx.x * (kIdxWarps * kIdxKeysPerWarp);

  // stage q (H x 128) and this CTA's 64 keys with 16-byte loads: all loads of a thread are requested
  // before the first is stored (a load-store loop would pay one memory round trip per iteration)
  constexpr int kThreads = kIdxWarps * 32;
  constexpr int kQIters = H * 16 / kThreads, kKIters = 64 * 16 / kThreads;
  uint4 qv[kQIters], kv[kKIters];
#pragma unroll
  for (int it = 0; it < kKIters; ++it) {
    const int i = it * kThreads + threadIdx.x;
    const int r = i >> 4, c = i & 15;
    kv[it] = make_uint4(0, 0, 0, 0);
    if (key0 + r < n_keys) {
      asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(kv[it].x), "=r"(kv[it].y), "=r"(kv[it].z), "=r"(kv[it].w)
                   : "l"(kcache + static_cast<long long>(key0 + r) * 128 + c * 8));
    }
  }
#pragma unroll
  for (int it = 0; it < kQIters; ++it) {
    const int i = it * kThreads + threadIdx.x;
    qv[it] = *reinterpret_cast<const uint4*>(q + (static_cast<long long>(tok) * H + (i >> 4)) * 128 + (i & 15) * 8);
  }
#pragma unroll
  for (int it = 0; it < kKIters; ++it) {
    const int i = it * kThreads + threadIdx.x;
    *reinterpret_cast<uint4*>(sk + (i >> 4) * kIdxPitch + (i & 15) * 8) = kv[it];
  }
#pragma unroll
  for (int it = 0; it < kQIters; ++it) {
    const int i = it * kThreads + threadIdx.x;
    *reinterpret_cast<uint4*>(sq + (i >> 4) * kIdxPitch + (i & 15) * 8) = qv[it];
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x) sw[i] = bf2f(w[tok * H + i]);
  __syncthreads();

  float acc[H / 8][4];
#pragma unroll
  for (int n = 0; n < H / 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;

  const __nv_bfloat16* wk = sk + warp * kIdxKeysPerWarp * kIdxPitch;
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    uint32_t a[4];
    // A (16 keys x 16 dims): matrices (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
    ldmatrix_x4(a, wk + (lane & 15) * kIdxPitch + ks * 16 + (lane >> 4) * 8);
#pragma unroll
    for (int n2 = 0; n2 < H / 16; ++n2) {
      uint32_t b[4];
      // B for two n-tiles: (heads 0-7, k 0-7), (heads 0-7, k 8-15), (heads 8-15, k 0-7), (heads 8-15, k 8-15)
      ldmatrix_x4(b, sq + (n2 * 16 + (lane & 7) + ((lane >> 4) << 3)) * kIdxPitch + ks * 16 + ((lane >> 3) & 1) * 8);
      const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
      mma_bf16_16816(acc[2 * n2], a, b0);
      mma_bf16_16816(acc[2 * n2 + 1], a, b1);
    }
  }
  // relu, weight, sum over heads: thread holds keys (g, g+8) x heads (8n + 2q, 8n + 2q + 1)
  const int g = lane >> 2, qd = lane & 3;
  float lo = 0.f, hi = 0.f;
#pragma unroll
  for (int n = 0; n < H / 8; ++n) {
    const float w0 = sw[n * 8 + 2 * qd], w1 = sw[n * 8 + 2 * qd + 1];
    lo += fmaxf(acc[n][0], 0.f) * w0 + fmaxf(acc[n][1], 0.f) * w1;
    hi += fmaxf(acc[n][2], 0.f) * w0 + fmaxf(acc[n][3], 0.f) * w1;
  }
  lo += __shfl_xor_sync(0xffffffffu, lo, 1);
  lo += __shfl_xor_sync(0xffffffffu, lo, 2);
  hi += __shfl_xor_sync(0xffffffffu, hi, 1);
  hi += __shfl_xor_sync(0xffffffffu, hi, 2);
  if (qd == 0) {
    const int last = *pos + pos_offset + tok;
    const int k_lo = key0 + warp * kIdxKeysPerWarp + g, k_hi = k_lo + 8;
    if (k_lo < n_keys) logits[tok * logits_stride + k_lo] = k_lo <= last ? lo : -INFINITY;
    if (k_hi < n_keys) logits[tok * logits_stride + k_hi] = k_hi <= last ? hi : -INFINITY;
  }
}

// ------------------------------------------------------------------ radix top-k
__device__ __forceinline__ uint32_t f32_order_key(float v) {
  uint32_t u = __float_as_uint(v);
  if (u == 0x80000000u) u = 0u;  // -0.0 compares equal to +0.0
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
constexpr uint32_t kNegInfKey = 0x007fffffu;  // order key of -inf: never selected

constexpr int kTopkThreads = 1024;
constexpr int kTopkItems = 8;  // consecutive elements per thread in the ordered compaction

// One CTA per row.  Selects the k largest logits among [0, n) (entries equal to -inf are skipped),
// ties by lower index, and writes their indices in ascending order; unused slots get -1.
// The selection for one row by one CTA of kTopkThreads threads; `dst` may be shared or global memory.
template <int THREADS>
__device__ __forceinline__ void topk_radix_row(const float* row, int n, int k, int* dst) {
  constexpr int kTopkThreads = THREADS;  // shadows the launch constant: the strides below follow the caller's block
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining;
  __shared__ int s_warp_gt[32], s_warp_eq[32];
  __shared__ int s_base_sel, s_base_eq;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // count eligible entries
  int cnt = 0;
  for (int i = tid; i < n; i += kTopkThreads) cnt += f32_order_key(__ldcg(row + i)) > kNegInfKey;
  if (tid < 256) hist[tid] = 0;
  if (tid == 0) { s_prefix = 0; s_remaining = 0; }
  __syncthreads();
  {
    int wsum = cnt;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, o);
    if (lane == 0) atomicAdd(&s_remaining, wsum);
  }
  __syncthreads();
  const int n_eligible = s_remaining;
  __syncthreads();

  uint32_t thr = kNegInfKey + 1;  // select everything eligible
  int need_eq = 0x7fffffff;       // how many entries equal to thr to take
  bool take_all = n_eligible <= k;
  if (!take_all) {
    if (tid == 0) s_remaining = k;
    __syncthreads();
    uint32_t prefix = 0, mask = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
      if (tid < 256) hist[tid] = 0;
      __syncthreads();
      for (int i = tid; i < n; i += kTopkThreads) {
        const uint32_t key = f32_order_key(__ldcg(row + i));
        if (key > kNegInfKey && (key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1);
      }
      __syncthreads();
      if (warp == 0) {
        // find the digit where the count of larger-or-equal digits reaches the remaining quota:
        // lane l owns bins 8l .. 8l+7; suffix sums across lanes, then a short scan inside one lane
        const int rem = s_remaining;
        int b[8], ssum = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          b[j] = hist[lane * 8 + j];
          ssum += b[j];
        }
        int suf = ssum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int v = __shfl_down_sync(0xffffffffu, suf, o);
          if (lane + o < 32) suf += v;
        }
        int suf_next = __shfl_down_sync(0xffffffffu, suf, 1);
        if (lane == 31) suf_next = 0;
        if (suf >= rem && suf_next < rem) {
          int r = rem - suf_next, d = 0;
          bool found = false;
#pragma unroll
          for (int j = 7; j >= 0; --j) {
            if (!found) {
              if (b[j] >= r || j == 0) {
                d = j;
                found = true;
              } else {
                r -= b[j];
              }
            }
          }
          s_remaining = r;
          s_prefix = prefix | (static_cast<uint32_t>(lane * 8 + d) << shift);
        }
      }
      __syncthreads();
      prefix = s_prefix;
      mask |= 0xffu << shift;
      __syncthreads();
    }
    thr = prefix;
    need_eq = s_remaining;
  }

  // ordered compaction: chunk of kTopkThreads * kTopkItems consecutive elements per pass
  if (tid == 0) { s_base_sel = 0; s_base_eq = 0; }
  __syncthreads();
  for (int base = 0; base < n; base += kTopkThreads * kTopkItems) {
    const int i0 = base + tid * kTopkItems;
    uint32_t gt_mask = 0, eq_mask = 0;
#pragma unroll
    for (int j = 0; j < kTopkItems; ++j) {
      const int i = i0 + j;
      if (i < n) {
        const uint32_t key = f32_order_key(__ldcg(row + i));
        if (key > kNegInfKey) {
          if (take_all || key > thr) gt_mask |= 1u << j;
          else if (key == thr) eq_mask |= 1u << j;
        }
      }
    }
    const int my_gt = __popc(gt_mask), my_eq = __popc(eq_mask);
    // exclusive scans of (gt, eq) over the CTA in thread order
    int sc_gt = my_gt, sc_eq = my_eq;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, sc_gt, o), b = __shfl_up_sync(0xffffffffu, sc_eq, o);
      if (lane >= o) { sc_gt += a; sc_eq += b; }
    }
    if (lane == 31) { s_warp_gt[warp] = sc_gt; s_warp_eq[warp] = sc_eq; }
    __syncthreads();
    int pre_gt = 0, pre_eq = 0, tot_gt = 0, tot_eq = 0;
    for (int w2 = 0; w2 < kTopkThreads / 32; ++w2) {
      const int a = s_warp_gt[w2], b = s_warp_eq[w2];
      if (w2 < warp) { pre_gt += a; pre_eq += b; }
      tot_gt += a; tot_eq += b;
    }
    const int base_sel = s_base_sel, base_eq = s_base_eq;
    // ties consumed before this thread (in index order) and how many of them were taken
    int eq_before = base_eq + pre_eq + sc_eq - my_eq;
    int gt_before = pre_gt + sc_gt - my_gt;
    // selected-so-far = base_sel (all earlier chunks) + gt in this chunk before me + ties taken in this chunk before me
    const int eq_taken_before_chunk = min(base_eq, need_eq);
    int eq_taken_before_me = min(eq_before, need_eq) - eq_taken_before_chunk;
    int w = base_sel + gt_before + eq_taken_before_me;
#pragma unroll
    for (int j = 0; j < kTopkItems; ++j) {
      if (gt_mask & (1u << j)) {
        if (w < k) dst[w] = i0 + j;
        ++w;
      } else if (eq_mask & (1u << j)) {
        if (eq_before < need_eq) {
          if (w < k) dst[w] = i0 + j;
          ++w;
        }
        ++eq_before;
      }
    }
    __syncthreads();
    if (tid == 0) {
      const int eq_taken_chunk = min(base_eq + tot_eq, need_eq) - eq_taken_before_chunk;
      s_base_sel = base_sel + tot_gt + eq_taken_chunk;
      s_base_eq = base_eq + tot_eq;
    }
    __syncthreads();
  }
  const int n_sel = s_base_sel;
  for (int i = n_sel + tid; i < k; i += kTopkThreads) dst[i] = -1;
}
__global__ void __launch_bounds__(kTopkThreads) topk_radix_kernel(const float* __restrict__ logits,
                                                                  long long logits_stride, int n, int k,
                                                                  int* __restrict__ out, long long out_stride) {
  pdl_launch_dependents();
  pdl_wait();
  topk_radix_row<kTopkThreads>(logits + blockIdx.x * logits_stride, n, k, out + blockIdx.x * out_stride);
}

// Same selection for rows of at most THREADS * ITEMS entries: every thread keeps its ITEMS
// consecutive keys in registers, so the row is read from memory once instead of once per pass.
template <int THREADS, int ITEMS>
__device__ __forceinline__ void topk_radix_reg_body(const float* row, int n, int k, int* dst) {
  constexpr int kTopkThreads = THREADS;
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining;
  __shared__ int s_warp_gt[32], s_warp_eq[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int i0 = tid * ITEMS;

  uint32_t key[ITEMS];
  int cnt = 0;
#pragma unroll
  for (int j = 0; j < ITEMS; ++j) {
    key[j] = i0 + j < n ? f32_order_key(__ldcg(row + i0 + j)) : 0u;  // 0 is below the key of -inf: never eligible
    cnt += key[j] > kNegInfKey;
  }
  if (tid < 256) hist[tid] = 0;
  if (tid == 0) { s_prefix = 0; s_remaining = 0; }
  __syncthreads();
  {
    int wsum = cnt;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, o);
    if (lane == 0 && wsum != 0) atomicAdd(&s_remaining, wsum);
  }
  __syncthreads();
  const int n_eligible = s_remaining;
  __syncthreads();

  uint32_t thr = kNegInfKey + 1;  // select everything eligible
  int need_eq = 0x7fffffff;       // how many entries equal to thr to take
  const bool take_all = n_eligible <= k;
  if (!take_all) {
    if (tid == 0) s_remaining = k;
    uint32_t prefix = 0, mask = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
      // hist is zero here (initially, and re-zeroed by warp 0 after each pass's scan)
#pragma unroll
      for (int j = 0; j < ITEMS; ++j)
        if (key[j] > kNegInfKey && (key[j] & mask) == prefix) atomicAdd(&hist[(key[j] >> shift) & 0xff], 1);
      __syncthreads();
      if (warp == 0) {
        // find the digit where the count of larger-or-equal digits reaches the remaining quota:
        // lane l owns bins 8l .. 8l+7; suffix sums across lanes, then a short scan inside one lane
        const int rem = s_remaining;
        int b[8], ssum = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          b[j] = hist[lane * 8 + j];
          hist[lane * 8 + j] = 0;
          ssum += b[j];
        }
        int suf = ssum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int v = __shfl_down_sync(0xffffffffu, suf, o);
          if (lane + o < 32) suf += v;
        }
        int suf_next = __shfl_down_sync(0xffffffffu, suf, 1);
        if (lane == 31) suf_next = 0;
        if (suf >= rem && suf_next < rem) {
          int r = rem - suf_next, d = 0;
          bool found = false;
#pragma unroll
          for (int j = 7; j >= 0; --j) {
            if (!found) {
              if (b[j] >= r || j == 0) {
                d = j;
                found = true;
              } else {
                r -= b[j];
              }
            }
          }
          s_remaining = r;
          s_prefix = prefix | (static_cast<uint32_t>(lane * 8 + d) << shift);
        }
      }
      __syncthreads();
      prefix = s_prefix;
      mask |= 0xffu << shift;
    }
    thr = prefix;
    need_eq = s_remaining;
  }

  // ordered compaction of the one chunk
  uint32_t gt_mask = 0, eq_mask = 0;
#pragma unroll
  for (int j = 0; j < ITEMS; ++j) {
    if (key[j] > kNegInfKey) {
      if (take_all || key[j] > thr) gt_mask |= 1u << j;
      else if (key[j] == thr) eq_mask |= 1u << j;
    }
  }
  const int my_gt = __popc(gt_mask), my_eq = __popc(eq_mask);
  int sc_gt = my_gt, sc_eq = my_eq;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, sc_gt, o), b = __shfl_up_sync(0xffffffffu, sc_eq, o);
    if (lane >= o) { sc_gt += a; sc_eq += b; }
  }
  if (lane == 31) { s_warp_gt[warp] = sc_gt; s_warp_eq[warp] = sc_eq; }
  __syncthreads();
  int pre_gt = 0, pre_eq = 0, tot_gt = 0, tot_eq = 0;
  for (int w2 = 0; w2 < kTopkThreads / 32; ++w2) {
    const int a = s_warp_gt[w2], b = s_warp_eq[w2];
    if (w2 < warp) { pre_gt += a; pre_eq += b; }
    tot_gt += a; tot_eq += b;
  }
  int eq_before = pre_eq + sc_eq - my_eq;                 // ties before this thread, in index order
  int w = pre_gt + sc_gt - my_gt + min(eq_before, need_eq);  // entries selected before this thread
#pragma unroll
  for (int j = 0; j < ITEMS; ++j) {
    if (gt_mask & (1u << j)) {
      if (w < k) dst[w] = i0 + j;
      ++w;
    } else if (eq_mask & (1u << j)) {
      if (eq_before < need_eq) {
        if (w < k) dst[w] = i0 + j;
        ++w;
      }
      ++eq_before;
    }
  }
  const int n_sel = tot_gt + min(tot_eq, need_eq);
  for (int i = n_sel + tid; i < k; i += kTopkThreads) dst[i] = -1;
}

template <int ITEMS>
__global__ void __launch_bounds__(kTopkThreads) topk_radix_reg_kernel(const float* logits, long long logits_stride, int n,
                                                                      int k, int* out, long long out_stride) {
  pdl_launch_dependents();
  pdl_wait();
  topk_radix_reg_body<kTopkThreads, ITEMS>(logits + blockIdx.x * logits_stride, n, k, out + blockIdx.x * out_stride);
}

// ------------------------------------------------------------------ scoring + selection in one launch
// A cooperative launch: at most one CTA per SM, all resident at once, so they may meet at grid-wide
// barriers (bounded waits; a CTA that gives up sets the status word, still arrives at the remaining
// barriers and leaves).  CTA c of a token scores a contiguous range of keys (256 per pass, the next pass's
// keys already requested while this one runs on the tensor cores), writes the logits, and keeps their
// order-preserving 32-bit images in shared memory.  The k-th largest image is then found by an
// 11 + 11 + 10 bit radix descent over histograms that every CTA adds to in global memory (integer atomics:
// the sums do not depend on arrival order), and the selected positions are written in ascending order at
// offsets that follow from the per-CTA counts.  A row of 131072 keys thus costs four barriers after one
// pass over HBM instead of one CTA reading the row from L2 once per radix digit.
constexpr int kIdxFusedWarps = 16;
constexpr int kIdxFusedThreads = kIdxFusedWarps * 32;
constexpr int kIdxFusedKeys = kIdxFusedWarps * kIdxKeysPerWarp;  // 256 keys per pass
constexpr int kIdxSelMaxCtas = 148;
// per-token work area in global memory (32-bit words), all zero between launches
constexpr int kIdxWorkBarStride = 32;                       // barrier counters 0..3 and the exit counter, a line apart
constexpr int kIdxWorkH1 = 256;                             // [2048] counts by key bits 31..21
constexpr int kIdxWorkH2 = kIdxWorkH1 + 2048;               // [2048] bits 20..10 among the keys of the threshold bin
constexpr int kIdxWorkH3 = kIdxWorkH2 + 2048;               // [1024] bits 9..0
constexpr int kIdxWorkCnt = kIdxWorkH3 + 1024;              // [kIdxSelMaxCtas][2] keys above / equal to the threshold
constexpr int kIdxWorkUsed = kIdxWorkCnt + 2 * kIdxSelMaxCtas;
constexpr int kIdxWorkWords = 6144;                         // per token
static_assert(kIdxWorkUsed <= kIdxWorkWords, "work area");

// ------------------------------------------------------------------ scoring + selection, short rows
// For rows of a few thousand keys: every CTA scores kIdxFusedKeys keys of one query token and counts itself
// done; the CTA that finds itself last for its token then selects that token's top-k from the logits the
// others left in L2, its keys held in registers.  No grid-wide barrier: cheaper than the cooperative
// selection below while one CTA can hold the row (up to 8192 keys); beyond that it reads the row once per
// radix digit from L2 and the cooperative kernel wins (measured: 41 us against 28 us at 16384 keys).
template <int H>
__global__ void __launch_bounds__(kIdxFusedThreads) indexer_topk_kernel(
    const __nv_bfloat16* __restrict__ q,       // [tokens, H, 128]
    const __nv_bfloat16* __restrict__ kcache,  // [T, 128]
    const __nv_bfloat16* __restrict__ w,       // [tokens, H]
    float* logits,                             // [tokens, logits_stride]
    long long logits_stride, int n_keys, const int* __restrict__ pos, int k,
    int* out, long long out_stride,            // [tokens, out_stride] selected indices, ascending, -1 padded
    unsigned* done                             // [tokens] CTAs finished per token; zero between launches
) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [H][pitch]
  __nv_bfloat16* sk = sq + H * kIdxPitch;                          // [kIdxFusedKeys][pitch]
  __shared__ float sw[H];
  __shared__ int s_last;
  const int tok = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int key0 = blockIdx.x * kIdxFusedKeys;

  constexpr int kKIters = kIdxFusedKeys * 16 / kIdxFusedThreads;  // 8
  uint4 kv[kKIters];
#pragma unroll
  for (int it = 0; it < kKIters; ++it) {
    const int i = it * kIdxFusedThreads + threadIdx.x;
    const int r = i >> 4, c = i & 15;
    kv[it] = make_uint4(0, 0, 0, 0);
    if (key0 + r < n_keys) {
      asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(kv[it].x), "=r"(kv[it].y), "=r"(kv[it].z), "=r"(kv[it].w)
                   : "l"(kcache + static_cast<long long>(key0 + r) * 128 + c * 8));
    }
  }
  for (int i = threadIdx.x; i < H * 16; i += kIdxFusedThreads)
    *reinterpret_cast<uint4*>(sq + (i >> 4) * kIdxPitch + (i & 15) * 8) =
        *reinterpret_cast<const uint4*>(q + (static_cast<long long>(tok) * H + (i >> 4)) * 128 + (i & 15) * 8);
#pragma unroll
  for (int it = 0; it < kKIters; ++it) {
    const int i = it * kIdxFusedThreads + threadIdx.x;
    *reinterpret_cast<uint4*>(sk + (i >> 4) * kIdxPitch + (i & 15) * 8) = kv[it];
  }
  for (int i = threadIdx.x; i < H; i += kIdxFusedThreads) sw[i] = bf2f(w[tok * H + i]);
  __syncthreads();

  float acc[H / 8][4];
#pragma unroll
  for (int n = 0; n < H / 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
  const __nv_bfloat16* wk = sk + warp * kIdxKeysPerWarp * kIdxPitch;
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    uint32_t a[4];
    ldmatrix_x4(a, wk + (lane & 15) * kIdxPitch + ks * 16 + (lane >> 4) * 8);
#pragma unroll
    for (int n2 = 0; n2 < H / 16; ++n2) {
      uint32_t b[4];
      ldmatrix_x4(b, sq + (n2 * 16 + (lane & 7) + ((lane >> 4) << 3)) * kIdxPitch + ks * 16 + ((lane >> 3) & 1) * 8);
      const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
      mma_bf16_16816(acc[2 * n2], a, b0);
      mma_bf16_16816(acc[2 * n2 + 1], a, b1);
    }
  }
  const int g = lane >> 2, qd = lane & 3;
  float lo = 0.f, hi = 0.f;
#pragma unroll
  for (int n = 0; n < H / 8; ++n) {
    const float w0 = sw[n * 8 + 2 * qd], w1 = sw[n * 8 + 2 * qd + 1];
    lo += fmaxf(acc[n][0], 0.f) * w0 + fmaxf(acc[n][1], 0.f) * w1;
    hi += fmaxf(acc[n][2], 0.f) * w0 + fmaxf(acc[n][3], 0.f) * w1;
  }
  lo += __shfl_xor_sync(0xffffffffu, lo, 1);
  lo += __shfl_xor_sync(0xffffffffu, lo, 2);
  hi += __shfl_xor_sync(0xffffffffu, hi, 1);
  hi += __shfl_xor_sync(0xffffffffu, hi, 2);
  if (qd == 0) {
    const int last = *pos + tok;
    const int k_lo = key0 + warp * kIdxKeysPerWarp + g, k_hi = k_lo + 8;
    if (k_lo < n_keys) logits[tok * logits_stride + k_lo] = k_lo <= last ? lo : -INFINITY;
    if (k_hi < n_keys) logits[tok * logits_stride + k_hi] = k_hi <= last ? hi : -INFINITY;
  }

  // ---- the last CTA of this token selects ----
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(done + tok, 1u);
    s_last = prev == gridDim.x - 1u ? 1 : 0;
    if (s_last) done[tok] = 0u;  // every CTA of the token has arrived: ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float* row = logits + tok * logits_stride;
  int* dst = out + tok * out_stride;
  if (n_keys <= kIdxFusedThreads * 8)
    topk_radix_reg_body<kIdxFusedThreads, 8>(row, n_keys, k, dst);
  else if (n_keys <= kIdxFusedThreads * 16)
    topk_radix_reg_body<kIdxFusedThreads, 16>(row, n_keys, k, dst);
  else
    topk_radix_row<kIdxFusedThreads>(row, n_keys, k, dst);
}


// ------------------------------------------------------------------ scoring + selection, long rows
// All CTAs of the token arrive; returns false when this CTA gave up (or had given up before).
__device__ __forceinline__ bool idx_grid_barrier(unsigned* ctr, unsigned n_ctas, int* status, bool failed) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    bool ok = !failed;
    __threadfence();
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(ctr) : "memory");
    if (ok) {
      const long long t0 = clock64();
      const long long budget = kWaitBudgetCycles;
      for (;;) {
        unsigned v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
        if (v >= n_ctas) break;
        __nanosleep(32);
        if (clock64() - t0 > budget) {
          ok = false;
          set_status(status, ST_GRID_TIMEOUT);
          break;
        }
      }
    }
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  return s_ok != 0;
}

// Exclusive prefix sum of `v` over the CTA's threads, in thread order; `total` receives the sum.
__device__ __forceinline__ int idx_block_scan(int v, int& total, int* s_warp) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) s_warp[warp] = inc;
  __syncthreads();
  int pre = 0, tot = 0;
#pragma unroll
  for (int w2 = 0; w2 < kIdxFusedWarps; ++w2) {
    const int a = s_warp[w2];
    if (w2 < warp) pre += a;
    tot += a;
  }
  __syncthreads();
  total = tot;
  return pre + inc - v;
}

// The bin where the count of keys in higher-or-equal bins reaches `rem` (1 <= rem <= total), and how many
// keys of that bin are still wanted.  When total < rem nothing is found and only `total` is meaningful.
template <int NB>
__device__ __forceinline__ void idx_find_bin(const int* hist, int rem, int* s_warp, int* s_res, int& bin, int& r,
                                             int& total) {
  constexpr int PER = NB / kIdxFusedThreads;
  int b[PER], s = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    b[j] = hist[threadIdx.x * PER + j];
    s += b[j];
  }
  int tot;
  const int excl = idx_block_scan(s, tot, s_warp);
  const int suf = tot - excl, suf_next = suf - s;  // keys in this thread's bins and above / above only
  if (suf >= rem && suf_next < rem) {
    int rr = rem - suf_next, d = 0;
    bool found = false;
#pragma unroll
    for (int j = PER - 1; j >= 0; --j) {
      if (!found) {
        if (b[j] >= rr || j == 0) {
          d = j;
          found = true;
        } else {
          rr -= b[j];
        }
      }
    }
    s_res[0] = threadIdx.x * PER + d;
    s_res[1] = rr;
  }
  __syncthreads();
  bin = s_res[0];
  r = s_res[1];
  total = tot;
  __syncthreads();
}

// Adds this CTA's histogram to the token's, waits for everybody, and reads the sum back into `hist`.
template <int NB>
__device__ __forceinline__ bool idx_merge_hist(int* hist, unsigned* global_hist, unsigned* bar, unsigned n_ctas,
                                               int* status, bool failed) {
  for (int i = threadIdx.x; i < NB; i += kIdxFusedThreads) {
    const int c = hist[i];
    if (c != 0) atomicAdd(global_hist + i, static_cast<unsigned>(c));
  }
  const bool ok = idx_grid_barrier(bar, n_ctas, status, failed);
  for (int i = threadIdx.x; i < NB; i += kIdxFusedThreads) hist[i] = ok ? static_cast<int>(__ldcg(global_hist + i)) : 0;
  __syncthreads();
  return ok;
}

// grid = (G, tokens) with G * tokens <= SM count; block = 512 threads;
// dynamic smem = (H + 256) * kIdxPitch * 2 + keys_per_cta * 4 bytes.  keys_per_cta is a multiple of 16.
template <int H>
__global__ void __launch_bounds__(kIdxFusedThreads) indexer_select_kernel(
    const __nv_bfloat16* __restrict__ q,       // [tokens, H, 128]
    const __nv_bfloat16* __restrict__ kcache,  // [T, 128]
    const __nv_bfloat16* __restrict__ w,       // [tokens, H]
    float* logits,                             // [tokens, logits_stride]
    long long logits_stride, int n_keys, const int* __restrict__ pos, int k,
    int* out, long long out_stride,            // [tokens, out_stride] selected indices, ascending, -1 padded
    unsigned* work_all,                        // [tokens][kIdxWorkWords], zero between launches
    int keys_per_cta, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [H][pitch]
  __nv_bfloat16* sk = sq + H * kIdxPitch;                          // [kIdxFusedKeys][pitch]
  uint32_t* skeys = reinterpret_cast<uint32_t*>(sk + kIdxFusedKeys * kIdxPitch);  // [keys_per_cta]
  __shared__ int hist[2048];
  __shared__ float sw[H];
  __shared__ int s_warp[kIdxFusedWarps], s_res[2], s_warp_gt[kIdxFusedWarps], s_warp_eq[kIdxFusedWarps];
  __shared__ int s_base[4], s_run[2], s_last;
  const int tok = blockIdx.y, cta = blockIdx.x, n_ctas = gridDim.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  unsigned* work = work_all + static_cast<long long>(tok) * kIdxWorkWords;
  const int key_begin = min(n_keys, cta * keys_per_cta);
  const int n_mine = min(n_keys, key_begin + keys_per_cta) - key_begin;
  const int n_pass = (n_mine + kIdxFusedKeys - 1) / kIdxFusedKeys;
  bool failed = false;

  // ---- scores ----
  constexpr int kKIters = kIdxFusedKeys * 16 / kIdxFusedThreads;  // 8 x 16 bytes per thread and pass
  uint4 kv[kKIters];
  auto request_keys = [&](int pass) {
#pragma unroll
    for (int it = 0; it < kKIters; ++it) {
      const int i = it * kIdxFusedThreads + tid;
      const int r = pass * kIdxFusedKeys + (i >> 4), c = i & 15;
      kv[it] = make_uint4(0, 0, 0, 0);
      if (r < n_mine) {
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(kv[it].x), "=r"(kv[it].y), "=r"(kv[it].z), "=r"(kv[it].w)
                     : "l"(kcache + static_cast<long long>(key_begin + r) * 128 + c * 8));
      }
    }
  };
  if (n_pass > 0) request_keys(0);
  for (int i = tid; i < H * 16; i += kIdxFusedThreads)
    *reinterpret_cast<uint4*>(sq + (i >> 4) * kIdxPitch + (i & 15) * 8) =
        *reinterpret_cast<const uint4*>(q + (static_cast<long long>(tok) * H + (i >> 4)) * 128 + (i & 15) * 8);
  for (int i = tid; i < H; i += kIdxFusedThreads) sw[i] = bf2f(w[tok * H + i]);
  for (int i = tid; i < 2048; i += kIdxFusedThreads) hist[i] = 0;
  const int last = *pos + tok;
  const int g = lane >> 2, qd = lane & 3;
  for (int pass = 0; pass < n_pass; ++pass) {
    __syncthreads();  // the previous pass has read its keys
#pragma unroll
    for (int it = 0; it < kKIters; ++it) {
      const int i = it * kIdxFusedThreads + tid;
      *reinterpret_cast<uint4*>(sk + (i >> 4) * kIdxPitch + (i & 15) * 8) = kv[it];
    }
    if (pass + 1 < n_pass) request_keys(pass + 1);
    __syncthreads();
    if (pass * kIdxFusedKeys + warp * kIdxKeysPerWarp < n_mine) {
      float acc[H / 8][4];
#pragma unroll
      for (int n = 0; n < H / 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
      const __nv_bfloat16* wk = sk + warp * kIdxKeysPerWarp * kIdxPitch;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t a[4];
        ldmatrix_x4(a, wk + (lane & 15) * kIdxPitch + ks * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int n2 = 0; n2 < H / 16; ++n2) {
          uint32_t b[4];
          ldmatrix_x4(b, sq + (n2 * 16 + (lane & 7) + ((lane >> 4) << 3)) * kIdxPitch + ks * 16 + ((lane >> 3) & 1) * 8);
          const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
          mma_bf16_16816(acc[2 * n2], a, b0);
          mma_bf16_16816(acc[2 * n2 + 1], a, b1);
        }
      }
      float lo = 0.f, hi = 0.f;
#pragma unroll
      for (int n = 0; n < H / 8; ++n) {
        const float w0 = sw[n * 8 + 2 * qd], w1 = sw[n * 8 + 2 * qd + 1];
        lo += fmaxf(acc[n][0], 0.f) * w0 + fmaxf(acc[n][1], 0.f) * w1;
        hi += fmaxf(acc[n][2], 0.f) * w0 + fmaxf(acc[n][3], 0.f) * w1;
      }
      lo += __shfl_xor_sync(0xffffffffu, lo, 1);
      lo += __shfl_xor_sync(0xffffffffu, lo, 2);
      hi += __shfl_xor_sync(0xffffffffu, hi, 1);
      hi += __shfl_xor_sync(0xffffffffu, hi, 2);
      if (qd == 0) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int li = pass * kIdxFusedKeys + warp * kIdxKeysPerWarp + g + half * 8;
          if (li < n_mine) {
            const int kg = key_begin + li;
            const float v = kg <= last ? (half == 0 ? lo : hi) : -INFINITY;
            logits[tok * logits_stride + kg] = v;
            const uint32_t key = f32_order_key(v);
            skeys[li] = key;
            if (key > kNegInfKey) atomicAdd(&hist[key >> 21], 1);
          }
        }
      }
    }
  }
  __syncthreads();

  // ---- the k-th largest key: radix descent over the token's merged histograms ----
  failed = !idx_merge_hist<2048>(hist, work + kIdxWorkH1, work + 0 * kIdxWorkBarStride, n_ctas, status, failed);
  int b1, r1, n_eligible;
  idx_find_bin<2048>(hist, k, s_warp, s_res, b1, r1, n_eligible);
  const bool take_all = n_eligible <= k;
  uint32_t thr = kNegInfKey + 1;  // select everything eligible
  int need_eq = 0x7fffffff;       // how many keys equal to thr to take (lowest positions first)
  if (!take_all) {
    for (int i = tid; i < 2048; i += kIdxFusedThreads) hist[i] = 0;
    __syncthreads();
    for (int i = tid; i < n_mine; i += kIdxFusedThreads) {
      const uint32_t key = skeys[i];
      if ((key >> 21) == static_cast<uint32_t>(b1)) atomicAdd(&hist[(key >> 10) & 0x7ffu], 1);
    }
    __syncthreads();
    failed = !idx_merge_hist<2048>(hist, work + kIdxWorkH2, work + 1 * kIdxWorkBarStride, n_ctas, status, failed);
    int b2, r2, tot2;
    idx_find_bin<2048>(hist, r1, s_warp, s_res, b2, r2, tot2);
    const uint32_t prefix22 = (static_cast<uint32_t>(b1) << 11) | static_cast<uint32_t>(b2);
    for (int i = tid; i < 1024; i += kIdxFusedThreads) hist[i] = 0;
    __syncthreads();
    for (int i = tid; i < n_mine; i += kIdxFusedThreads) {
      const uint32_t key = skeys[i];
      if ((key >> 10) == prefix22) atomicAdd(&hist[key & 0x3ffu], 1);
    }
    __syncthreads();
    failed = !idx_merge_hist<1024>(hist, work + kIdxWorkH3, work + 2 * kIdxWorkBarStride, n_ctas, status, failed);
    int b3, r3, tot3;
    idx_find_bin<1024>(hist, r2, s_warp, s_res, b3, r3, tot3);
    thr = (prefix22 << 10) | static_cast<uint32_t>(b3);
    need_eq = r3;
  }

  // ---- how many this CTA selects; where its part of the output starts ----
  {
    int my_gt = 0, my_eq = 0;
    for (int i = tid; i < n_mine; i += kIdxFusedThreads) {
      const uint32_t key = skeys[i];
      if (key > kNegInfKey) {
        if (take_all || key > thr) ++my_gt;
        else if (key == thr) ++my_eq;
      }
    }
    int tot_gt, tot_eq;
    idx_block_scan(my_gt, tot_gt, s_warp);
    idx_block_scan(my_eq, tot_eq, s_warp);
    if (tid == 0) {
      work[kIdxWorkCnt + 2 * cta] = static_cast<unsigned>(tot_gt);
      work[kIdxWorkCnt + 2 * cta + 1] = static_cast<unsigned>(tot_eq);
    }
  }
  failed = !idx_grid_barrier(work + 3 * kIdxWorkBarStride, n_ctas, status, failed);
  {
    const int c_gt = tid < n_ctas && !failed ? static_cast<int>(__ldcg(work + kIdxWorkCnt + 2 * tid)) : 0;
    const int c_eq = tid < n_ctas && !failed ? static_cast<int>(__ldcg(work + kIdxWorkCnt + 2 * tid + 1)) : 0;
    int all_gt, all_eq;
    const int pre_gt = idx_block_scan(c_gt, all_gt, s_warp);
    const int pre_eq = idx_block_scan(c_eq, all_eq, s_warp);
    if (tid == cta) {
      s_base[0] = pre_gt;
      s_base[1] = pre_eq;
      s_base[2] = all_gt;
      s_base[3] = all_eq;
    }
    __syncthreads();
  }
  int* dst = out + tok * out_stride;
  // ordered compaction: thread t of a pass holds eight consecutive keys
  if (tid == 0) {
    s_run[0] = s_base[0] + min(s_base[1], need_eq);  // selected before this CTA
    s_run[1] = s_base[1];                            // keys equal to thr before this CTA
  }
  __syncthreads();
  for (int base = 0; base < n_mine; base += kIdxFusedThreads * 8) {
    const int i0 = base + tid * 8;
    uint32_t gt_mask = 0, eq_mask = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (i0 + j < n_mine) {
        const uint32_t key = skeys[i0 + j];
        if (key > kNegInfKey) {
          if (take_all || key > thr) gt_mask |= 1u << j;
          else if (key == thr) eq_mask |= 1u << j;
        }
      }
    }
    const int my_gt = __popc(gt_mask), my_eq = __popc(eq_mask);
    int sc_gt = my_gt, sc_eq = my_eq;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, sc_gt, o), b = __shfl_up_sync(0xffffffffu, sc_eq, o);
      if (lane >= o) { sc_gt += a; sc_eq += b; }
    }
    if (lane == 31) { s_warp_gt[warp] = sc_gt; s_warp_eq[warp] = sc_eq; }
    __syncthreads();
    int pre_gt = 0, pre_eq = 0, tot_gt = 0, tot_eq = 0;
#pragma unroll
    for (int w2 = 0; w2 < kIdxFusedWarps; ++w2) {
      const int a = s_warp_gt[w2], b = s_warp_eq[w2];
      if (w2 < warp) { pre_gt += a; pre_eq += b; }
      tot_gt += a; tot_eq += b;
    }
    const int base_sel = s_run[0], base_eq = s_run[1];
    int eq_before = base_eq + pre_eq + sc_eq - my_eq;
    const int gt_before = pre_gt + sc_gt - my_gt;
    const int eq_taken_before_pass = min(base_eq, need_eq);
    int wr = base_sel + gt_before + min(eq_before, need_eq) - eq_taken_before_pass;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (gt_mask & (1u << j)) {
        if (wr < k) dst[wr] = key_begin + i0 + j;
        ++wr;
      } else if (eq_mask & (1u << j)) {
        if (eq_before < need_eq) {
          if (wr < k) dst[wr] = key_begin + i0 + j;
          ++wr;
        }
        ++eq_before;
      }
    }
    __syncthreads();
    if (tid == 0) {
      s_run[0] = base_sel + tot_gt + min(base_eq + tot_eq, need_eq) - eq_taken_before_pass;
      s_run[1] = base_eq + tot_eq;
    }
    __syncthreads();
  }
  {
    const int n_sel = min(k, s_base[2] + min(s_base[3], need_eq));
    for (int i = n_sel + cta * kIdxFusedThreads + tid; i < k; i += n_ctas * kIdxFusedThreads) dst[i] = -1;
  }

  // ---- the last CTA out clears the work area for the next launch ----
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const unsigned prev = atomicAdd(work + 4 * kIdxWorkBarStride, 1u);
    s_last = prev == static_cast<unsigned>(n_ctas) - 1u ? 1 : 0;
  }
  __syncthreads();
  if (s_last) {
    __threadfence();
    for (int i = tid; i < kIdxWorkUsed; i += kIdxFusedThreads) work[i] = 0u;
  }
}

}  // namespace tb
