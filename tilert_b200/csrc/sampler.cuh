// Token sampling from the vocabulary logits: temperature, top-k, top-p (nucleus), seeded; plus the
// top-256 log-probabilities a serving front end exports.  One CTA per token.
//
//   config = (temperature, top_p, top_k, use_top_p) as four floats in device memory (the layout of
//   the reference's SAMPLING_CONFIG scratch tensor, modules/end2end.py:282-289).
//   temperature == 0: greedy (arg-max, ties to the lower token id).
//   Otherwise candidates are the 1024 largest logits (exact, ties to the lower id), sorted by value;
//   top_k in [1, 1024] keeps the first top_k of them (any other value keeps all 1024); with
//   use_top_p the shortest prefix whose probability mass (under the temperature-scaled softmax over
//   the WHOLE vocabulary) reaches top_p is kept; one uniform number picks a token from what is left,
//   in proportion to its probability.  Mass outside the 1024 candidates is never sampled.
//   Log-probabilities are those of the unscaled softmax over the whole vocabulary.
#pragma once

#include "common.cuh"
#include "indexer.cuh"

namespace tb {

constexpr int kSampleCandidates = kTopkThreads;  // 1024: one candidate per thread
constexpr int kSampleTopN = 256;

struct SampleParams {
  const float* logits;  // [tokens, stride]
  long long stride;
  int vocab;
  const float* config;  // (temperature, top_p, top_k, use_top_p)
  unsigned long long seed;
  unsigned long long* step;  // optional device state {step index, CTAs done}: the launch reads the step index
                             // and its last CTA increments it, so a replayed CUDA graph draws new numbers
  unsigned long long step_value;  // used when `step` is null
  int* token;           // [tokens]
  float* token_logprob; // optional [tokens]
  float* topn_logprob;  // optional [tokens, 256]
  int* topn_index;      // optional [tokens, 256]
};

// uniform in [0, 1) from (seed, step, token): splitmix64 finaliser, top 24 bits
__host__ __device__ inline float sample_uniform(unsigned long long seed, unsigned long long step, unsigned long long tok) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (step + 1) + 0xD1B54A32D192ED03ull * (tok + 1);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return static_cast<float>(z >> 40) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ float block_reduce_max(float v, float* red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[threadIdx.x & 31];
  return warp_max(r);
}
__device__ __forceinline__ float block_reduce_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[threadIdx.x & 31];
  return warp_sum(r);
}

__global__ void __launch_bounds__(kTopkThreads) sample_kernel(const SampleParams p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  __shared__ int s_idx[kSampleCandidates];
  __shared__ float s_val[kSampleCandidates];
  __shared__ float s_cum[kSampleCandidates];
  __shared__ float s_warp_tot[32];
  __shared__ int s_pick, s_keep;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tok = blockIdx.x;
  const float* row = p.logits + tok * p.stride;
  const unsigned long long step = p.step != nullptr ? *reinterpret_cast<volatile unsigned long long*>(p.step) : p.step_value;
  const float temperature = p.config[0], top_p = p.config[1];
  const int top_k_cfg = static_cast<int>(p.config[2]);
  const bool use_top_p = p.config[3] != 0.f;

  // ---- softmax normalisers over the whole vocabulary ----
  float m = -INFINITY;
  for (int i = tid; i < p.vocab; i += kTopkThreads) m = fmaxf(m, row[i]);
  m = block_reduce_max(m, red);
  const float inv_t = temperature > 0.f ? 1.0f / temperature : 1.0f;
  float s1 = 0.f, st = 0.f;
  for (int i = tid; i < p.vocab; i += kTopkThreads) {
    const float d = row[i] - m;
    s1 += __expf(d);
    st += __expf(d * inv_t);
  }
  s1 = block_reduce_sum(s1, red);
  st = block_reduce_sum(st, red);
  const float log_s1 = __logf(s1);

  // ---- the 1024 largest logits, then sorted by (value descending, index ascending) ----
  topk_radix_row<kTopkThreads>(row, p.vocab, kSampleCandidates, s_idx);
  __syncthreads();
  s_val[tid] = s_idx[tid] >= 0 ? row[s_idx[tid]] : -INFINITY;
  if (s_idx[tid] < 0) s_idx[tid] = 0x7fffffff;
  __syncthreads();
  for (int size = 2; size <= kSampleCandidates; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const int partner = tid ^ stride;
      if (partner > tid) {
        const bool descending = (tid & size) == 0;
        const float va = s_val[tid], vb = s_val[partner];
        const int ia = s_idx[tid], ib = s_idx[partner];
        const bool a_first = va > vb || (va == vb && ia < ib);  // a belongs before b in the final order
        if (a_first != descending) {
          s_val[tid] = vb; s_val[partner] = va;
          s_idx[tid] = ib; s_idx[partner] = ia;
        }
      }
      __syncthreads();
    }
  }

  // ---- exported log-probabilities ----
  if (p.topn_logprob != nullptr && tid < kSampleTopN) {
    const bool real = s_idx[tid] != 0x7fffffff;
    p.topn_logprob[tok * kSampleTopN + tid] = real ? s_val[tid] - m - log_s1 : -INFINITY;
    p.topn_index[tok * kSampleTopN + tid] = real ? s_idx[tid] : -1;
  }

  // ---- pick ----
  if (tid == 0) {
    s_pick = 0;
    s_keep = 0;
  }
  if (temperature > 0.f) {
    const int k_eff = (top_k_cfg >= 1 && top_k_cfg <= kSampleCandidates) ? top_k_cfg : kSampleCandidates;
    const float w = (tid < k_eff && s_idx[tid] != 0x7fffffff) ? __expf((s_val[tid] - m) * inv_t) : 0.f;
    // inclusive scan of w over the CTA
    float sc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float a = __shfl_up_sync(0xffffffffu, sc, o);
      if (lane >= o) sc += a;
    }
    if (lane == 31) s_warp_tot[warp] = sc;
    __syncthreads();
    float pre = 0.f;
    for (int w2 = 0; w2 < warp; ++w2) pre += s_warp_tot[w2];
    const float cum = pre + sc;
    s_cum[tid] = cum;
    __syncthreads();
    // nucleus: the shortest prefix whose mass reaches top_p of the whole distribution
    const float need = top_p * st;
    if (use_top_p) {
      const float before = tid > 0 ? s_cum[tid - 1] : 0.f;
      if (cum >= need && before < need) s_keep = tid + 1;
    }
    __syncthreads();
    int n_keep = (use_top_p && s_keep > 0) ? s_keep : k_eff;  // never reached: keep every candidate
    if (n_keep > k_eff) n_keep = k_eff;
    const float u = sample_uniform(p.seed, step, static_cast<unsigned long long>(tok));
    const float target = u * s_cum[n_keep - 1];
    {
      const float before = tid > 0 ? s_cum[tid - 1] : 0.f;
      if (tid < n_keep && cum > target && before <= target) s_pick = tid;
    }
    __syncthreads();
  }
  __syncthreads();
  if (tid == 0) {
    const int pick = s_pick;
    p.token[tok] = s_idx[pick];
    if (p.token_logprob != nullptr) p.token_logprob[tok] = s_val[pick] - m - log_s1;
  }
  if (p.step != nullptr && tid == 0) {
    // this CTA has read the step index (above, or it is greedy and does not care): count it done;
    // the last one advances the index for the next launch
    const unsigned long long prev = atomicAdd(p.step + 1, 1ull);
    if (prev == static_cast<unsigned long long>(gridDim.x) - 1ull) {
      p.step[1] = 0ull;
      __threadfence();
      p.step[0] = p.step[0] + 1ull;
    }
  }
}

}  // namespace tb
