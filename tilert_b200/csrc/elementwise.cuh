// Small per-token kernels between the projections: latent RMSNorm into the KV cache, rotary
// embeddings, and the indexer's (LayerNorm ->) RoPE -> Hadamard transform.  A few KB each;
// launch-latency bound, not bandwidth bound.
#pragma once

#include "common.cuh"

namespace tb {

// Activations may have been written earlier in the SAME launch by other thread blocks (the chained
// streaming launch runs these routines between its products): they are read with L2-only loads, never
// through the non-coherent path a `const __restrict__` pointer would allow.
__device__ __forceinline__ float ld_act(const __nv_bfloat16* p) {
  return bf16_bits_to_f32(__ldcg(reinterpret_cast<const unsigned short*>(p)));
}

// A cache row index past the cache's rows (`cache_rows` > 0) is refused: nothing is stored and the status
// word says so.  The position is device-resident, so only the device can make this check.
__device__ __forceinline__ bool cache_row_ok(int row, int cache_rows, int* status) {
  if (cache_rows <= 0 || (row >= 0 && row < cache_rows)) return true;
  set_status(status, ST_BAD_ARGUMENT);
  return false;
}

// One vector of NV * 256 elements by one warp: every load of the lane up front (8 bf16 per 16-byte load,
// lane-contiguous), one pass.  NV is a template parameter so that only the registers in use exist.
template <int NV>
__device__ __forceinline__ void rmsnorm_vec_warp(const __nv_bfloat16* x, const float* __restrict__ gamma, float eps,
                                                 __nv_bfloat16* dst) {
  const int lane = threadIdx.x & 31;
  constexpr int dim = NV * 256;
  uint4 raw[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) raw[v] = __ldcg(reinterpret_cast<const uint4*>(x + (v * 32 + lane) * 8));
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const uint32_t w4[4] = {raw[v].x, raw[v].y, raw[v].z, raw[v].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = __uint_as_float(w4[j] << 16), b = __uint_as_float(w4[j] & 0xffff0000u);
      ss += a * a + b * b;
    }
  }
  ss = warp_sum(ss);
  const float rinv = rsqrtf(ss / static_cast<float>(dim) + eps);
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int e = (v * 32 + lane) * 8;
    const float4 g0 = *reinterpret_cast<const float4*>(gamma + e), g1 = *reinterpret_cast<const float4*>(gamma + e + 4);
    const uint32_t w4[4] = {raw[v].x, raw[v].y, raw[v].z, raw[v].w};
    const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      o[j] = pack_bf16x2(__uint_as_float(w4[j] << 16) * rinv * gg[2 * j], __uint_as_float(w4[j] & 0xffff0000u) * rinv * gg[2 * j + 1]);
    *reinterpret_cast<uint4*>(dst + e) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// kv [tokens, dim] -> cache[pos + t, dim] = bf16(rmsnorm(kv) * gamma).   One warp per token.
__device__ __forceinline__ void rmsnorm_kv_warp(int tok, const __nv_bfloat16* __restrict__ kv, long long kv_stride,
                                                const float* __restrict__ gamma, float eps, int dim,
                                                const int* __restrict__ pos, __nv_bfloat16* __restrict__ cache,
                                                int n_tokens, int cache_rows = 0, int* status = nullptr) {
  const int lane = threadIdx.x & 31;
  if (tok >= n_tokens) return;
  if (!cache_row_ok(*pos + tok, cache_rows, status)) return;
  const __nv_bfloat16* x = kv + tok * kv_stride;
  __nv_bfloat16* dst = cache + static_cast<long long>(*pos + tok) * dim;
  if ((kv_stride % 8) == 0) {
    if (dim == 512) return rmsnorm_vec_warp<2>(x, gamma, eps, dst);
    if (dim == 256) return rmsnorm_vec_warp<1>(x, gamma, eps, dst);
    if (dim == 1024) return rmsnorm_vec_warp<4>(x, gamma, eps, dst);
  }
  float ss = 0.f;
  for (int i = lane; i < dim; i += 32) {
    const float v = ld_act(x + i);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float rinv = rsqrtf(ss / static_cast<float>(dim) + eps);
  for (int i = lane; i < dim; i += 32) dst[i] = f2bf(ld_act(x + i) * rinv * gamma[i]);
}
__global__ void rmsnorm_kv_kernel(const __nv_bfloat16* __restrict__ kv, long long kv_stride,
                                  const float* __restrict__ gamma, float eps, int dim, const int* __restrict__ pos,
                                  __nv_bfloat16* __restrict__ cache, int n_tokens, int cache_rows, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  rmsnorm_kv_warp(blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), kv, kv_stride, gamma, eps, dim, pos, cache,
                  n_tokens, cache_rows, status);
}

// Interleaved RoPE (pairs (x[2i], x[2i+1])) applied in place to q_pe [tokens, heads, rope] and to the
// cached key rows pe_cache[pos + t, rope].  freqs: [tokens, rope/2, 2] = (cos, sin).
__device__ __forceinline__ void qkv_rope_thread(int idx, __nv_bfloat16* __restrict__ q_pe, int heads, int rope,
                                                __nv_bfloat16* __restrict__ pe_cache, const int* __restrict__ pos,
                                                const float* __restrict__ freqs, int n_tokens, int cache_rows = 0,
                                                int* status = nullptr) {
  const int half = rope / 2;
  const int per_tok = (heads + 1) * half;
  if (idx >= n_tokens * per_tok) return;
  const int tok = idx / per_tok, rem = idx % per_tok;
  const int h = rem / half, i = rem % half;
  const float c = freqs[(tok * half + i) * 2], s = freqs[(tok * half + i) * 2 + 1];
  __nv_bfloat16* v;
  if (h < heads)
    v = q_pe + (static_cast<long long>(tok) * heads + h) * rope + 2 * i;
  else {
    if (!cache_row_ok(*pos + tok, cache_rows, status)) return;
    v = pe_cache + static_cast<long long>(*pos + tok) * rope + 2 * i;
  }
  const float a = bf2f(v[0]), b = bf2f(v[1]);
  v[0] = f2bf(a * c - b * s);
  v[1] = f2bf(a * s + b * c);
}
__global__ void qkv_rope_kernel(__nv_bfloat16* __restrict__ q_pe, int heads, int rope,
                                __nv_bfloat16* __restrict__ pe_cache, const int* __restrict__ pos,
                                const float* __restrict__ freqs, int n_tokens, int cache_rows, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  qkv_rope_thread(blockIdx.x * blockDim.x + threadIdx.x, q_pe, heads, rope, pe_cache, pos, freqs, n_tokens, cache_rows,
                  status);
}

// 128-point Walsh-Hadamard transform of a warp-distributed vector: lane l holds elements
// 4l .. 4l+3.  Natural (Sylvester) ordering.
__device__ __forceinline__ void hadamard128(float (&v)[4]) {
  // strides 1 and 2 inside the lane
  float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
  v[0] = a + c; v[1] = b + d; v[2] = a - c; v[3] = b - d;
  // strides 4 .. 64 across lanes
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const bool upper = (threadIdx.x & o) != 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float other = __shfl_xor_sync(0xffffffffu, v[j], o);
      v[j] = upper ? other - v[j] : v[j] + other;
    }
  }
}

// Indexer rotation: optional LayerNorm (weight, bias, eps 1e-6), non-interleaved RoPE on the first
// `rope` of 128 dims (pairs (x[i], x[i + rope/2])), then Hadamard-128 scaled by 128^-1/2.  Every
// stage rounds to bf16 as the reference's bf16 tensor pipeline does.  One warp per 128-vector.
//   in  [tokens, heads, 128];  out: either [tokens, heads, 128] or cache[pos + t, 128] (heads == 1)
__device__ __forceinline__ void rotate128_warp(int vec, const __nv_bfloat16* __restrict__ in,
                                               __nv_bfloat16* __restrict__ out, int heads, int rope,
                                               const float* __restrict__ freqs, const float* __restrict__ ln_w,
                                               const float* __restrict__ ln_b, const int* __restrict__ pos,
                                               int n_tokens, int cache_rows = 0, int* status = nullptr) {
  const int lane = threadIdx.x & 31;
  if (vec >= n_tokens * heads) return;
  const int tok = vec / heads;
  if (pos != nullptr && !cache_row_ok(*pos + tok, cache_rows, status)) return;
  const __nv_bfloat16* x = in + static_cast<long long>(vec) * 128;
  float v[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = ld_act(x + lane * 4 + j);
  if (ln_w != nullptr) {
    float s = warp_sum(v[0] + v[1] + v[2] + v[3]);
    const float mean = s * (1.0f / 128.0f);
    float d2 = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) d2 += (v[j] - mean) * (v[j] - mean);
    d2 = warp_sum(d2);
    const float rstd = rsqrtf(d2 * (1.0f / 128.0f) + 1e-6f);
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = bf2f(f2bf((v[j] - mean) * rstd * ln_w[lane * 4 + j] + ln_b[lane * 4 + j]));
  }
  // non-interleaved RoPE: element i < rope/2 pairs with element i + rope/2.  With rope = 64 the
  // partner of lane l (< 8) is lane l + 8.
  const int half = rope / 2;
  const int lanes_half = half / 4;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float partner = __shfl_xor_sync(0xffffffffu, v[j], lanes_half);
    const int e = lane * 4 + j;
    if (e < rope) {
      const int i = e < half ? e : e - half;
      const float c = freqs[(tok * half + i) * 2], s = freqs[(tok * half + i) * 2 + 1];
      const float re = e < half ? v[j] : partner, im = e < half ? partner : v[j];
      v[j] = bf2f(f2bf(e < half ? re * c - im * s : re * s + im * c));
    }
  }
  hadamard128(v);
  __nv_bfloat16* dst = out + static_cast<long long>(vec) * 128;
  if (pos != nullptr) dst = out + static_cast<long long>(*pos + tok) * 128;
  const float scale = 0.08838834764831845f;  // 128^-1/2 (a Python scalar in the reference: not rounded to bf16)
#pragma unroll
  for (int j = 0; j < 4; ++j) dst[lane * 4 + j] = f2bf(bf2f(f2bf(v[j])) * scale);
}
__global__ void rotate128_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int heads,
                                 int rope, const float* __restrict__ freqs, const float* __restrict__ ln_w,
                                 const float* __restrict__ ln_b, const int* __restrict__ pos, int n_tokens,
                                 int cache_rows, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  rotate128_warp(blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), in, out, heads, rope, freqs, ln_w, ln_b, pos,
                 n_tokens, cache_rows, status);
}

// MoE routing (sigmoid scores + bias, optional group limiting, top-k, renormalise, scale).
// One warp per token; n_experts <= 256 (8 per lane).
//   scores [tokens, n_experts] f32  ->  probs [tokens, top_k] f32, ids [tokens, top_k] i32,
//   slot_ids [tokens, top_k + 1] i32 = (shared-expert id, ids...), slot_w [tokens, top_k + 1] = (1, probs...)
// Routing of one token by one warp.  On return lane k (< top_k) holds the k-th selected expert in
// `my_id` and its renormalised, scaled weight in `my_w`.
__device__ __forceinline__ void expert_select_warp(const float* __restrict__ scores, const float* __restrict__ bias,
                                                   int n_experts, int n_groups, int n_limited, int top_k,
                                                   float route_scale, int& my_id, float& my_w) {
  const int lane = threadIdx.x & 31;
  const int per_lane = (n_experts + 31) / 32;  // experts e = lane*per_lane + j  (contiguous per lane)
  float orig[8], sel[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int e = lane * per_lane + j;
    if (j < per_lane && e < n_experts) {
      const float s = 1.0f / (1.0f + expf(-__ldcg(scores + e)));
      orig[j] = s;
      sel[j] = bias != nullptr ? s + bias[e] : s;
    } else {
      orig[j] = 0.f;
      sel[j] = -INFINITY;
    }
  }
  if (n_groups > 1) {
    // group score = sum of the two largest biased scores of the group (max if no bias); a group is
    // lanes_per_group consecutive lanes
    const int lanes_per_group = 32 / n_groups;
    float m1 = -INFINITY, m2 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (sel[j] > m1) { m2 = m1; m1 = sel[j]; } else if (sel[j] > m2) { m2 = sel[j]; }
    }
    for (int o = 1; o < lanes_per_group; o <<= 1) {
      const float o1 = __shfl_xor_sync(0xffffffffu, m1, o), o2 = __shfl_xor_sync(0xffffffffu, m2, o);
      const float n1 = fmaxf(m1, o1);
      const float n2 = fmaxf(fminf(m1, o1), fmaxf(m2, o2));
      m1 = n1; m2 = n2;
    }
    const float gscore = bias != nullptr ? m1 + m2 : m1;
    const int my_group = lane / lanes_per_group;
    // rank of my group: number of groups with a larger score, ties to the lower group index
    int rank = 0;
    for (int g = 0; g < n_groups; ++g) {
      const float gs = __shfl_sync(0xffffffffu, gscore, g * lanes_per_group);
      if (gs > gscore || (gs == gscore && g < my_group)) ++rank;
    }
    if (rank >= n_limited) {
#pragma unroll
      for (int j = 0; j < 8; ++j) sel[j] = -INFINITY;
    }
  }
  float wsum = 0.f;
  my_w = 0.f;
  my_id = 0;
  for (int k = 0; k < top_k; ++k) {
    // arg-max over the warp, ties to the lower expert index
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = lane * per_lane + j;
      if (j < per_lane && e < n_experts && (sel[j] > best)) { best = sel[j]; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    float w = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (lane * per_lane + j == best_e) { w = orig[j]; sel[j] = -INFINITY; }
    }
    w = __shfl_sync(0xffffffffu, w, best_e / per_lane);
    wsum += w;
    if (lane == k) { my_w = w; my_id = best_e; }
  }
  my_w = my_w / wsum * route_scale;
}

// Stores one token's routing in the forms the callers read: probs / ids [top_k], and the slot lists
// [top_k + 1] = (shared expert, weight 1) followed by the selected experts.
__device__ __forceinline__ void expert_select_store(int my_id, float my_w, int top_k, int shared_id,
                                                    float* __restrict__ probs, int* __restrict__ ids,
                                                    int* __restrict__ slot_ids, float* __restrict__ slot_w) {
  const int lane = threadIdx.x & 31;
  if (lane < top_k) {
    probs[lane] = my_w;
    ids[lane] = my_id;
    slot_ids[1 + lane] = my_id;
    slot_w[1 + lane] = my_w;
  }
  if (lane == 0) {
    slot_ids[0] = shared_id;
    slot_w[0] = 1.0f;
  }
}

// One warp per token.  Besides the per-token lists, optionally the flat form that lets ONE product launch serve
// every token: flat_ids = [shared, token 0's experts, token 1's experts, ...] and flat_w [n_tokens][1 + n_tokens *
// top_k] = the token's routing weight at its own slots, 1 at the shared slot, 0 elsewhere.
__global__ void expert_select_kernel(const float* __restrict__ scores, const float* __restrict__ bias,
                                     int n_experts, int n_groups, int n_limited, int top_k, float route_scale,
                                     int shared_id, float* __restrict__ probs, int* __restrict__ ids,
                                     int* __restrict__ slot_ids, float* __restrict__ slot_w, int n_tokens,
                                     int* __restrict__ flat_ids, float* __restrict__ flat_w) {
  pdl_launch_dependents();
  pdl_wait();
  const int tok = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (tok >= n_tokens) return;
  int my_id;
  float my_w;
  expert_select_warp(scores + tok * n_experts, bias, n_experts, n_groups, n_limited, top_k, route_scale, my_id, my_w);
  expert_select_store(my_id, my_w, top_k, shared_id, probs + tok * top_k, ids + tok * top_k,
                      slot_ids + tok * (top_k + 1), slot_w + tok * (top_k + 1));
  if (flat_ids != nullptr) {
    const int lane = threadIdx.x & 31, n_flat = 1 + n_tokens * top_k;
    float* row = flat_w + tok * n_flat;
    for (int j = lane; j < n_flat; j += 32) {
      const bool mine = j >= 1 + tok * top_k && j < 1 + (tok + 1) * top_k;
      if (!mine) row[j] = j == 0 ? 1.0f : 0.0f;
    }
    if (lane < top_k) {
      row[1 + tok * top_k + lane] = my_w;
      flat_ids[1 + tok * top_k + lane] = my_id;
    }
    if (tok == 0 && lane == 0) flat_ids[0] = shared_id;
  }
}

}  // namespace tb
