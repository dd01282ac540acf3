// Activation packing: bf16 (or f32) vectors -> X blocks for the weight-streaming GEMM.
//
// Each 128-element block of a token is written as two e4m3 columns, hi = e4m3(x / s) and
// lo = e4m3((x - hi*s) / (s/16)), with s a power of two chosen so the block maximum fits
// e4m3.  hi*s + lo*s/16 equals the bf16 input exactly wherever |x| >= s * 2^-6, so the fp8
// tensor-core product with the weights sees bf16-precision activations.
// An optional RMSNorm (gain gamma) runs first; its bf16 result can also be written out, and
// the reference-format 1x128 quantisation (e4m3 + f32 scale = amax/448) can be emitted too.
#pragma once

#include "common.cuh"
#include "formats.h"

namespace tb {

struct ActPackParams {
  const __nv_bfloat16* x;        // [tokens, k]
  long long x_stride;            // elements between tokens
  int k;                         // multiple of 128
  int n_tokens;                  // 1..4 (split mode) or 1..8 (direct mode, from_q)
  const float* gamma;            // optional RMSNorm gain [k]; nullptr = no normalisation
  float eps;
  const float* seg_scale;        // optional [tokens, n_seg] multiplier folded into the scales
  int kb_per_seg;
  int n_seg;
  uint8_t* xpack;                // [k/128] X blocks
  __nv_bfloat16* out_bf16;       // optional [tokens, k] normalised activations
  long long out_stride;
  uint8_t* out_q;                // optional reference-format e4m3 [tokens, k]
  float* out_qscale;             // optional reference-format scales [tokens, k/128]
};

constexpr int kActPackThreads = 1024;
constexpr int kActPackMaxIter = 5;  // 32 warps * 5 blocks * 128 = k <= 20480

__device__ __forceinline__ float pow2_ceil_scale(float amax) {
  // smallest power of two s with amax / s <= 448 (e4m3 max); 1 for an all-zero block
  if (!(amax > 0.f)) return 1.f;
  int e;
  const float m = frexpf(amax * (1.0f / 448.0f), &e);  // amax/448 = m * 2^e, m in [0.5, 1)
  return ldexpf(1.f, m == 0.5f ? e - 1 : e);
}

// One CTA per token.
__global__ void __launch_bounds__(kActPackThreads) actpack_kernel(const ActPackParams p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  const int tok = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_kb = p.k / TB_KBLOCK;
  const __nv_bfloat16* xr = p.x + tok * p.x_stride;

  float v[kActPackMaxIter][4];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < kActPackMaxIter; ++it) {
    const int kb = warp + it * 32;
    if (kb < n_kb) {
      const uint2 raw = *reinterpret_cast<const uint2*>(xr + kb * TB_KBLOCK + lane * 4);
      v[it][0] = __uint_as_float(raw.x << 16);
      v[it][1] = __uint_as_float(raw.x & 0xffff0000u);
      v[it][2] = __uint_as_float(raw.y << 16);
      v[it][3] = __uint_as_float(raw.y & 0xffff0000u);
      ss += v[it][0] * v[it][0] + v[it][1] * v[it][1] + v[it][2] * v[it][2] + v[it][3] * v[it][3];
    }
  }
  float rinv = 1.f;
  if (p.gamma != nullptr) {
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = (lane < 32) ? red[lane] : 0.f;
    tot = warp_sum(tot);
    rinv = rsqrtf(tot / static_cast<float>(p.k) + p.eps);
  }

#pragma unroll
  for (int it = 0; it < kActPackMaxIter; ++it) {
    const int kb = warp + it * 32;
    if (kb >= n_kb) continue;
    float x4[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float val = v[it][j];
      if (p.gamma != nullptr) {
        val = val * rinv * p.gamma[kb * TB_KBLOCK + lane * 4 + j];
        val = bf2f(f2bf(val));  // the GEMM consumes exactly the bf16 value that is written out
      }
      x4[j] = val;
    }
    if (p.out_bf16 != nullptr) {
      uint2 o;
      o.x = pack_bf16x2(x4[0], x4[1]);
      o.y = pack_bf16x2(x4[2], x4[3]);
      *reinterpret_cast<uint2*>(p.out_bf16 + tok * p.out_stride + kb * TB_KBLOCK + lane * 4) = o;
    }
    float amax = fmaxf(fmaxf(fabsf(x4[0]), fabsf(x4[1])), fmaxf(fabsf(x4[2]), fabsf(x4[3])));
    amax = warp_max(amax);

    if (p.out_q != nullptr) {
      // reference 1x128 activation quantisation: s = max(amax, 1e-4) / 448
      const float s = fmaxf(amax, 1e-4f) * (1.0f / 448.0f);
      uint32_t w = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) w |= static_cast<uint32_t>(f32_to_e4m3(x4[j] / s)) << (8 * j);
      *reinterpret_cast<uint32_t*>(p.out_q + static_cast<long long>(tok) * p.k + kb * TB_KBLOCK + lane * 4) = w;
      if (lane == 0) p.out_qscale[tok * n_kb + kb] = s;
    }

    const float s_hi = pow2_ceil_scale(amax);
    const float s_lo = s_hi * 0.0625f;
    uint32_t whi = 0, wlo = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint8_t h = f32_to_e4m3(x4[j] / s_hi);
      const float r = x4[j] - e4m3_to_f32(h) * s_hi;
      const uint8_t l = f32_to_e4m3(r / s_lo);
      whi |= static_cast<uint32_t>(h) << (8 * j);
      wlo |= static_cast<uint32_t>(l) << (8 * j);
    }
    // element k = 4*lane + j of the block: chunk c = lane/8, half r = (lane%8)/4, quad q = lane%4
    uint8_t* blk = p.xpack + static_cast<long long>(kb) * TB_XBLK_BYTES;
    const int c = lane >> 3, r = (lane >> 2) & 1, q = lane & 3;
    const int col_hi = 2 * tok, col_lo = 2 * tok + 1;
    *reinterpret_cast<uint32_t*>(blk + c * 256 + r * 128 + col_hi * 16 + q * 4) = whi;
    *reinterpret_cast<uint32_t*>(blk + c * 256 + r * 128 + col_lo * 16 + q * 4) = wlo;
    if (lane == 0) {
      float m = 1.f;
      if (p.seg_scale != nullptr) m = p.seg_scale[tok * p.n_seg + kb / p.kb_per_seg];
      float* cs = reinterpret_cast<float*>(blk + TB_XBLK_DATA);
      cs[col_hi] = s_hi * m;
      cs[col_lo] = s_lo * m;
    }
  }
}

// Reference-format quantised activations (e4m3 [tokens, k] + f32 scales [tokens, k/128])
// -> X blocks in direct mode (one column per token).  One warp per k block.
__global__ void xq_repack_kernel(const uint8_t* __restrict__ xq, const float* __restrict__ xs, int n_tokens, int k,
                                 uint8_t* __restrict__ xpack) {
  pdl_launch_dependents();
  pdl_wait();
  const int n_kb = k / TB_KBLOCK;
  const int kb = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (kb >= n_kb) return;
  uint8_t* blk = xpack + static_cast<long long>(kb) * TB_XBLK_BYTES;
  const int c = lane >> 3, r = (lane >> 2) & 1, q = lane & 3;
  for (int tok = 0; tok < 8; ++tok) {
    uint32_t w = 0;
    if (tok < n_tokens)
      w = *reinterpret_cast<const uint32_t*>(xq + static_cast<long long>(tok) * k + kb * TB_KBLOCK + lane * 4);
    *reinterpret_cast<uint32_t*>(blk + c * 256 + r * 128 + tok * 16 + q * 4) = w;
    if (lane == 0) reinterpret_cast<float*>(blk + TB_XBLK_DATA)[tok] = tok < n_tokens ? xs[tok * n_kb + kb] : 0.f;
  }
}

}  // namespace tb
