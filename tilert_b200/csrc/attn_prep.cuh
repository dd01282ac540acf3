// One launch for the small per-token work between the query-path products and the indexer: the
// indexer head-weight projection (bf16 weights), the latent RMSNorm into the KV cache, the rotary
// embeddings of q_pe / k_pe, and the two indexer rotations.  The five pieces are independent; a
// block's index selects its piece.  Separately they cost five kernel boundaries of a few
// microseconds each on the critical path of a decode step.
#pragma once

#include "elementwise.cuh"
#include "gemv_bf16.cuh"

namespace tb {

struct AttnPrepParams {
  GemvBf16Params wis;  // indexer head weights: out[t, :] = W . RMSNorm(x[t]) (blocks [0, wis_blocks))
  int wis_blocks;
  // latent RMSNorm into the KV cache
  const __nv_bfloat16* kv;
  long long kv_stride;
  const float* kv_gamma;
  float kv_eps;
  int kv_dim;
  __nv_bfloat16* kv_cache;
  int kv_blocks;
  // rotary embedding of q_pe and of the cached k_pe row
  __nv_bfloat16* q_pe;
  int heads;
  int rope;
  __nv_bfloat16* pe_cache;
  int rope_blocks;
  // indexer query rotation
  const __nv_bfloat16* iq;
  __nv_bfloat16* iq_out;
  int idx_heads;
  int iq_blocks;
  // indexer key: LayerNorm -> RoPE -> Hadamard into its cache row
  const __nv_bfloat16* ki;
  __nv_bfloat16* ki_cache;
  const float* ln_w;
  const float* ln_b;
  int ki_blocks;
  const int* pos;
  const float* freqs;
  int n_tokens;
  int cache_rows;  // rows of the three caches (0 = unchecked); a position past them stores nothing and sets the status
  int* status;
};

constexpr int kAttnPrepThreads = kGemvBf16SmallThreads;  // 256: eight warps per block

template <int TOK>
__global__ void __launch_bounds__(kAttnPrepThreads) attn_prep_kernel(const AttnPrepParams p) {
  extern __shared__ __align__(16) float xs[];  // [TOK][k] for the projection blocks
  pdl_launch_dependents();
  int b = blockIdx.x;
  if (b < p.wis_blocks) {
    gemv_bf16_ksplit_body<TOK>(p.wis, b, xs);  // waits for the predecessor itself, after its weight loads
    return;
  }
  b -= p.wis_blocks;
  pdl_wait();
  const int warp = threadIdx.x >> 5;
  constexpr int kWarps = kAttnPrepThreads / 32;
  if (b < p.kv_blocks) {
    rmsnorm_kv_warp(b * kWarps + warp, p.kv, p.kv_stride, p.kv_gamma, p.kv_eps, p.kv_dim, p.pos, p.kv_cache, p.n_tokens, p.cache_rows, p.status);
    return;
  }
  b -= p.kv_blocks;
  if (b < p.rope_blocks) {
    qkv_rope_thread(b * kAttnPrepThreads + threadIdx.x, p.q_pe, p.heads, p.rope, p.pe_cache, p.pos, p.freqs, p.n_tokens, p.cache_rows, p.status);
    return;
  }
  b -= p.rope_blocks;
  if (b < p.iq_blocks) {
    rotate128_warp(b * kWarps + warp, p.iq, p.iq_out, p.idx_heads, p.rope, p.freqs, nullptr, nullptr, nullptr, p.n_tokens);
    return;
  }
  b -= p.iq_blocks;
  if (b < p.ki_blocks)
    rotate128_warp(b * kWarps + warp, p.ki, p.ki_cache, 1, p.rope, p.freqs, p.ln_w, p.ln_b, p.pos, p.n_tokens, p.cache_rows,
                   p.status);
}

}  // namespace tb
