// Sparse MLA decode attention over the latent KV cache (kv_lora 512 + rope 64).
//
// For each query token only the `topk` selected cache rows are touched.  The selected rows
// are split into chunks (flash-decoding); one CTA handles 16 heads x one chunk: it gathers
// its 64-row blocks with one bulk async copy (TMA) per row, computes Q.K^T and P.V with bf16
// tensor-core MMAs in f32, and writes a normalised partial output plus its log-sum-exp.  A
// second small kernel merges the chunks.  Algorithmic HBM traffic: topk x 1152 bytes per token.
#pragma once

#include "common.cuh"
#include "formats.h"

namespace tb {

constexpr int kMlaKeys = 64;
constexpr int kMlaHeads = 16;
constexpr int kMlaDV = 512;
constexpr int kMlaDR = 64;
constexpr int kMlaPitch = 584;   // bf16 elements per smem row: (512 + 64 + 8) -> 1168 bytes
constexpr int kMlaPPitch = 72;   // bf16 elements per P row
constexpr int kMlaThreads = 128;
constexpr int kMlaSmemBytes =
    (kMlaHeads + kMlaKeys) * kMlaPitch * 2 + kMlaHeads * kMlaPPitch * 2 + 2 * 4 * kMlaHeads * 4 + kMlaKeys * 4 + 16;

struct MlaParams {
  const __nv_bfloat16* q_lat;   // [tokens, heads, 512]
  const __nv_bfloat16* q_pe;    // [tokens, heads, 64]
  const __nv_bfloat16* kv;      // [T, 512]
  const __nv_bfloat16* pe;      // [T, 64]
  const int* idx;               // [tokens, topk]
  int topk;
  int heads;
  int n_cache;                  // rows in the cache tensors
  const int* pos;               // position of token 0
  float scale_log2;             // softmax scale * log2(e)
  int blocks_per_split;
  int n_splits;
  float* o_acc;                 // [tokens, heads, n_splits, 512]
  float* lse_acc;               // [tokens, heads, n_splits]
  int* status;
};

__global__ void __launch_bounds__(kMlaThreads) sparse_mla_kernel(const MlaParams p) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(128) uint8_t smem[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem);
  __nv_bfloat16* sKV = sQ + kMlaHeads * kMlaPitch;
  __nv_bfloat16* sP = sKV + kMlaKeys * kMlaPitch;
  float* sMax = reinterpret_cast<float*>(sP + kMlaHeads * kMlaPPitch);  // [4][16]
  float* sSum = sMax + 4 * kMlaHeads;                                   // [4][16]
  int* sValid = reinterpret_cast<int*>(sSum + 4 * kMlaHeads);           // [64]
  uint64_t* bar = reinterpret_cast<uint64_t*>(sValid + kMlaKeys);

  const int split = blockIdx.x, hg = blockIdx.y, tok = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, qd = lane & 3;
  const int pos_s = *p.pos + tok;

  if (tid == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  // Gather of one block of 64 selected rows: one bulk copy per row and part, all completing on `bar`.
  // Returns the number of valid rows (a block without valid rows issues no copy).
  auto issue_gather = [&](int blk) -> int {
    const int key_base = (split * p.blocks_per_split + blk) * kMlaKeys;
    int my_idx = -1;
    bool valid = false;
    if (tid < kMlaKeys) {
      if (key_base + tid < p.topk) my_idx = p.idx[static_cast<long long>(tok) * p.topk + key_base + tid];
      valid = my_idx >= 0 && my_idx < p.n_cache && my_idx <= pos_s;
      sValid[tid] = valid ? 1 : 0;
    }
    const int n_valid = __syncthreads_count(valid ? 1 : 0);
    if (tid == 0 && n_valid > 0) mbar_expect_tx(bar, n_valid * (kMlaDV + kMlaDR) * 2);
    // the rows were last touched through the generic proxy (ldmatrix reads, zero fills): order
    // those accesses before the async-proxy writes of the bulk copies issued below
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (tid < kMlaKeys) {
      __nv_bfloat16* row = sKV + tid * kMlaPitch;
      if (valid) {
        bulk_g2s(row, p.kv + static_cast<long long>(my_idx) * kMlaDV, kMlaDV * 2, bar);
        bulk_g2s(row + kMlaDV, p.pe + static_cast<long long>(my_idx) * kMlaDR, kMlaDR * 2, bar);
      } else {
        for (int c = 0; c < 72; ++c) *reinterpret_cast<uint4*>(row + c * 8) = make_uint4(0, 0, 0, 0);
      }
    }
    return n_valid;
  };
  // the first block's rows are requested before the queries are staged: the two latencies overlap
  int n_valid = p.blocks_per_split > 0 ? issue_gather(0) : 0;
  // stage the 16 query heads: [512 latent | 64 rope]; all of a thread's loads are requested before the
  // first is stored (a load-store loop would pay one memory round trip per iteration)
  constexpr int kQIters = kMlaHeads * 72 / kMlaThreads;  // 9
  uint4 qv[kQIters];
#pragma unroll
  for (int it = 0; it < kQIters; ++it) {
    const int i = it * kMlaThreads + tid;
    const int r = i / 72, c = i % 72;
    const int head = hg * kMlaHeads + r;
    qv[it] = make_uint4(0, 0, 0, 0);
    if (head < p.heads) {
      const long long th = static_cast<long long>(tok) * p.heads + head;
      qv[it] = c < 64 ? *reinterpret_cast<const uint4*>(p.q_lat + th * kMlaDV + c * 8)
                      : *reinterpret_cast<const uint4*>(p.q_pe + th * kMlaDR + (c - 64) * 8);
    }
  }
#pragma unroll
  for (int it = 0; it < kQIters; ++it) {
    const int i = it * kMlaThreads + tid;
    *reinterpret_cast<uint4*>(sQ + (i / 72) * kMlaPitch + (i % 72) * 8) = qv[it];
  }
  __syncthreads();

  uint32_t phase = 0;  // completed phases of `bar` (a block without valid rows issues no copy)
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  float o[16][4];
#pragma unroll
  for (int n = 0; n < 16; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

  for (int blk = 0; blk < p.blocks_per_split; ++blk) {
    // ---- 64 selected rows (block 0 was requested before the loop) ----
    if (blk > 0) n_valid = issue_gather(blk);
    bool gave_up = false;
    if (n_valid > 0) {
      gave_up = !mbar_wait(bar, phase & 1);
      if (gave_up) set_status(p.status, ST_WAIT_FULL_TIMEOUT);
      ++phase;
    }
    // a wait that ran out ends the loop for the whole CTA: no further copies are requested, and the one wait
    // below gives the copies already in flight the same budget again before the kernel returns
    if (__syncthreads_or(gave_up ? 1 : 0)) {
      mbar_wait(bar, (phase - 1) & 1);
      break;
    }

    // ---- S = Q K^T for this warp's 16 keys ----
    float s[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
    const __nv_bfloat16* kbase = sKV + (warp * 16 + (lane & 7) + ((lane >> 4) << 3)) * kMlaPitch + ((lane >> 3) & 1) * 8;
    const __nv_bfloat16* qbase = sQ + (lane & 15) * kMlaPitch + (lane >> 4) * 8;
#pragma unroll 4
    for (int ks = 0; ks < (kMlaDV + kMlaDR) / 16; ++ks) {
      uint32_t a[4], b[4];
      ldmatrix_x4(a, qbase + ks * 16);
      ldmatrix_x4(b, kbase + ks * 16);
      const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
      mma_bf16_16816(s[0], a, b0);
      mma_bf16_16816(s[1], a, b1);
    }
    // scale, mask, block max per head row
    float bmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = warp * 16 + n * 8 + 2 * qd + (j & 1);
        const float v = sValid[key] ? s[n][j] * p.scale_log2 : -INFINITY;
        s[n][j] = v;
        bmax[j >> 1] = fmaxf(bmax[j >> 1], v);
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      bmax[r] = fmaxf(bmax[r], __shfl_xor_sync(0xffffffffu, bmax[r], 1));
      bmax[r] = fmaxf(bmax[r], __shfl_xor_sync(0xffffffffu, bmax[r], 2));
    }
    if (qd == 0) {
      sMax[warp * kMlaHeads + g] = bmax[0];
      sMax[warp * kMlaHeads + g + 8] = bmax[1];
    }
    __syncthreads();
    float alpha[2], m_new[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + 8 * r;
      float m = m_run[r];
#pragma unroll
      for (int w2 = 0; w2 < 4; ++w2) m = fmaxf(m, sMax[w2 * kMlaHeads + row]);
      m_new[r] = m;
      alpha[r] = (m == -INFINITY) ? 1.f : exp2f(m_run[r] - m);
    }
    float bsum[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      float pv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = j >> 1;
        pv[j] = (m_new[r] == -INFINITY) ? 0.f : exp2f(s[n][j] - m_new[r]);
        pv[j] = bf2f(f2bf(pv[j]));  // the sum uses the same rounded probabilities as P.V
        bsum[r] += pv[j];
      }
      const int col = warp * 16 + n * 8 + 2 * qd;
      *reinterpret_cast<uint32_t*>(sP + g * kMlaPPitch + col) = pack_bf16x2(pv[0], pv[1]);
      *reinterpret_cast<uint32_t*>(sP + (g + 8) * kMlaPPitch + col) = pack_bf16x2(pv[2], pv[3]);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      bsum[r] += __shfl_xor_sync(0xffffffffu, bsum[r], 1);
      bsum[r] += __shfl_xor_sync(0xffffffffu, bsum[r], 2);
    }
    if (qd == 0) {
      sSum[warp * kMlaHeads + g] = bsum[0];
      sSum[warp * kMlaHeads + g + 8] = bsum[1];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + 8 * r;
      float sum = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < 4; ++w2) sum += sSum[w2 * kMlaHeads + row];
      l_run[r] = l_run[r] * alpha[r] + sum;
      m_run[r] = m_new[r];
    }
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
      o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
    }
    // ---- O += P V for this warp's 128 latent dims ----
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t a[4];
      ldmatrix_x4(a, sP + (lane & 15) * kMlaPPitch + kk * 16 + (lane >> 4) * 8);
      const __nv_bfloat16* vbase =
          sKV + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kMlaPitch + warp * 128 + (lane >> 4) * 8;
#pragma unroll
      for (int n2 = 0; n2 < 8; ++n2) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vbase + n2 * 16);
        const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
        mma_bf16_16816(o[2 * n2], a, b0);
        mma_bf16_16816(o[2 * n2 + 1], a, b1);
      }
    }
    __syncthreads();  // sKV / sP / sMax are rewritten by the next block
  }

  // ---- normalised partial output and log-sum-exp of this chunk ----
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int head = hg * kMlaHeads + g + 8 * r;
    if (head >= p.heads) continue;
    const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
    const long long base = (static_cast<long long>(tok) * p.heads + head) * p.n_splits + split;
    float* dst = p.o_acc + base * kMlaDV + warp * 128;
#pragma unroll
    for (int n = 0; n < 16; ++n)
      *reinterpret_cast<float2*>(dst + n * 8 + 2 * qd) = make_float2(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
    if (warp == 0 && qd == 0)
      p.lse_acc[base] = l_run[r] > 0.f ? m_run[r] * 0.6931471805599453f + logf(l_run[r]) : -INFINITY;
  }
}

// Merge the chunks: o = sum_i exp(lse_i - lse) * o_i.   grid = (heads, tokens), block = 128; n_splits <= 64.
__global__ void __launch_bounds__(128) sparse_mla_combine_kernel(const float* __restrict__ o_acc,
                                                                 const float* __restrict__ lse_acc, int n_splits,
                                                                 __nv_bfloat16* __restrict__ out,
                                                                 float* __restrict__ lse_out) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float s_w[64];
  __shared__ float s_den, s_mx;
  const int head = blockIdx.x, tok = blockIdx.y, heads = gridDim.x;
  const long long th = static_cast<long long>(tok) * heads + head;
  if (threadIdx.x < 32) {
    // weights of all chunks, computed once by the first warp
    const int lane = threadIdx.x;
    const float l0 = lane < n_splits ? lse_acc[th * n_splits + lane] : -INFINITY;
    const float l1 = lane + 32 < n_splits ? lse_acc[th * n_splits + lane + 32] : -INFINITY;
    const float mx = warp_max(fmaxf(l0, l1));
    const float w0 = mx == -INFINITY ? 0.f : expf(l0 - mx), w1 = mx == -INFINITY ? 0.f : expf(l1 - mx);
    const float den = warp_sum(w0 + w1);
    s_w[lane] = w0;
    s_w[lane + 32] = w1;
    if (lane == 0) {
      s_den = den;
      s_mx = mx;
    }
  }
  // partial outputs in batches of 16 independent loads; the first batch is requested before the
  // barrier, so it overlaps the weights' own load and reductions
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const float* src = o_acc + th * n_splits * kMlaDV + threadIdx.x * 4;
  constexpr int kBatch = 16;
  float4 v[kBatch];
#pragma unroll
  for (int j = 0; j < kBatch; ++j)
    v[j] = j < n_splits ? __ldcs(reinterpret_cast<const float4*>(src + static_cast<long long>(j) * kMlaDV))
                        : make_float4(0.f, 0.f, 0.f, 0.f);
  __syncthreads();
  for (int i0 = 0; i0 < n_splits; i0 += kBatch) {
    float4 nxt[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int i = i0 + kBatch + j;
      nxt[j] = i < n_splits ? __ldcs(reinterpret_cast<const float4*>(src + static_cast<long long>(i) * kMlaDV))
                            : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (i0 + j < n_splits) {
        const float wgt = s_w[i0 + j];
        acc[0] += wgt * v[j].x; acc[1] += wgt * v[j].y; acc[2] += wgt * v[j].z; acc[3] += wgt * v[j].w;
      }
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) v[j] = nxt[j];
  }
  const float den = s_den;
  const float inv = den > 0.f ? 1.f / den : 0.f;
  uint2 o2;
  o2.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
  o2.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
  *reinterpret_cast<uint2*>(out + th * kMlaDV + threadIdx.x * 4) = o2;
  if (threadIdx.x == 0 && lse_out != nullptr) lse_out[th] = den > 0.f ? s_mx + logf(den) : -INFINITY;
}

// Merge of the chunks fused with the value up-projection of the same head: o[h, :] = W_v[h] . o_lat[h] (128 x 512
// e4m3 with block scales, the head's row tile of the packed weight: four 16 KB blocks).  The blocks are requested with
// bulk copies before the wait for the attention launch -- weights depend on nothing -- so they are in shared memory
// when the merged latent vector is; thread r then owns output row r.  Saves the separate product launch, which is
// pure latency at this size (8 MB over the GPU, 1 MB per rank of eight).
// grid = (heads, tokens), block = 128, dynamic smem = kMlaCvSmemBytes; n_splits <= 64; kv_lora 512, v_head_dim 128.
constexpr int kMlaCvSmemBytes = 4 * TB_WBLK_BYTES + kMlaDV * 4 + 16;

__global__ void __launch_bounds__(128) sparse_mla_combine_vproj_kernel(const float* __restrict__ o_acc,
                                                                       const float* __restrict__ lse_acc, int n_splits,
                                                                       __nv_bfloat16* __restrict__ o_lat_out,
                                                                       float* __restrict__ lse_out,
                                                                       const uint8_t* __restrict__ w_v,
                                                                       __nv_bfloat16* __restrict__ o_out, int* status) {
  extern __shared__ __align__(128) uint8_t cv_smem[];
  uint8_t* sW = cv_smem;                                              // [4 k blocks][16448]
  float* s_o = reinterpret_cast<float*>(cv_smem + 4 * TB_WBLK_BYTES);  // [512] merged latent vector (bf16 values)
  uint64_t* bar = reinterpret_cast<uint64_t*>(s_o + kMlaDV);
  __shared__ float s_w[64];
  __shared__ float s_den, s_mx;
  const int head = blockIdx.x, tok = blockIdx.y, heads = gridDim.x;
  const int tid = threadIdx.x;
  if (tid == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
    mbar_expect_tx(bar, 4 * TB_WBLK_BYTES);
    for (int kb = 0; kb < 4; ++kb)
      bulk_g2s(sW + kb * TB_WBLK_BYTES, w_v + (static_cast<long long>(head) * 4 + kb) * TB_WBLK_BYTES, TB_WBLK_BYTES, bar);
  }
  pdl_launch_dependents();
  pdl_wait();
  const long long th = static_cast<long long>(tok) * heads + head;
  if (tid < 32) {
    const int lane = tid;
    const float l0 = lane < n_splits ? lse_acc[th * n_splits + lane] : -INFINITY;
    const float l1 = lane + 32 < n_splits ? lse_acc[th * n_splits + lane + 32] : -INFINITY;
    const float mx = warp_max(fmaxf(l0, l1));
    const float w0 = mx == -INFINITY ? 0.f : expf(l0 - mx), w1 = mx == -INFINITY ? 0.f : expf(l1 - mx);
    const float den = warp_sum(w0 + w1);
    s_w[lane] = w0;
    s_w[lane + 32] = w1;
    if (lane == 0) {
      s_den = den;
      s_mx = mx;
    }
  }
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const float* src = o_acc + th * n_splits * kMlaDV + tid * 4;
  constexpr int kBatch = 16;
  float4 v[kBatch];
#pragma unroll
  for (int j = 0; j < kBatch; ++j)
    v[j] = j < n_splits ? __ldcs(reinterpret_cast<const float4*>(src + static_cast<long long>(j) * kMlaDV))
                        : make_float4(0.f, 0.f, 0.f, 0.f);
  __syncthreads();
  for (int i0 = 0; i0 < n_splits; i0 += kBatch) {
    float4 nxt[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int i = i0 + kBatch + j;
      nxt[j] = i < n_splits ? __ldcs(reinterpret_cast<const float4*>(src + static_cast<long long>(i) * kMlaDV))
                            : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (i0 + j < n_splits) {
        const float wgt = s_w[i0 + j];
        acc[0] += wgt * v[j].x; acc[1] += wgt * v[j].y; acc[2] += wgt * v[j].z; acc[3] += wgt * v[j].w;
      }
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) v[j] = nxt[j];
  }
  const float den = s_den;
  const float inv = den > 0.f ? 1.f / den : 0.f;
  uint2 o2;
  o2.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
  o2.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
  if (o_lat_out != nullptr) *reinterpret_cast<uint2*>(o_lat_out + th * kMlaDV + tid * 4) = o2;
  if (tid == 0 && lse_out != nullptr) lse_out[th] = den > 0.f ? s_mx + logf(den) : -INFINITY;
  // the product sees the same bf16 values the separate launch would read back
  s_o[tid * 4 + 0] = __uint_as_float(o2.x << 16);
  s_o[tid * 4 + 1] = __uint_as_float(o2.x & 0xffff0000u);
  s_o[tid * 4 + 2] = __uint_as_float(o2.y << 16);
  s_o[tid * 4 + 3] = __uint_as_float(o2.y & 0xffff0000u);
  __syncthreads();
  if (!mbar_wait(bar, 0)) {
    set_status(status, ST_WAIT_FULL_TIMEOUT);
    return;
  }
  // output row tid: bytes of W[row, 32 c + 16 kc + b] sit at c * 4096 + (row / 8) * 256 + kc * 128 + (row % 8) * 16 + b
  float y = 0.f;
#pragma unroll
  for (int kb = 0; kb < 4; ++kb) {
    const uint8_t* blk = sW + kb * TB_WBLK_BYTES;
    const uint8_t* rowp = blk + (tid >> 3) * 256 + (tid & 7) * 16;
    float part = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
      for (int kc = 0; kc < 2; ++kc) {
        const uint4 q = *reinterpret_cast<const uint4*>(rowp + c * 4096 + kc * 128);
        const uint32_t wds[4] = {q.x, q.y, q.z, q.w};
        const float* xo = s_o + kb * 128 + c * 32 + kc * 16;
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
          const __half2_raw h01 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(wds[wi] & 0xffffu), __NV_E4M3);
          const __half2_raw h23 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(wds[wi] >> 16), __NV_E4M3);
          const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
          const float2 f23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
          part = fmaf(f01.x, xo[wi * 4 + 0], part);
          part = fmaf(f01.y, xo[wi * 4 + 1], part);
          part = fmaf(f23.x, xo[wi * 4 + 2], part);
          part = fmaf(f23.y, xo[wi * 4 + 3], part);
        }
      }
    }
    y = fmaf(part, *reinterpret_cast<const float*>(blk + TB_WBLK_DATA + (tid >> 3) * 4), y);
  }
  o_out[th * 128 + tid] = f2bf(y);
}

}  // namespace tb
