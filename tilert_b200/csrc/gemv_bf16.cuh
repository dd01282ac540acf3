// bf16-weight GEMV with f32 accumulation for the products that are not FP8 in the checkpoint:
// the MoE router gate, the indexer head-weight projection and the vocabulary head.
// HBM-bound on the weight stream: each warp owns whole rows and keeps several 16-byte
// loads per lane in flight; the (optionally RMS-normalised) activations sit in shared memory.
#pragma once

#include "common.cuh"

namespace tb {

struct GemvBf16Params {
  const void* w;                 // [n, k] bf16 (w_is_f32 = 0) or f32 (w_is_f32 = 1), row-major
  int w_is_f32;
  int n, k;                      // k multiple of 256
  const __nv_bfloat16* x;        // [tokens, k]
  long long x_stride;
  int n_tokens;                  // 1..4
  const float* gamma;            // optional RMSNorm gain
  float eps;
  int round_norm_bf16;           // 1: normalised activations are rounded to bf16 before the product
  __nv_bfloat16* xnorm_out;      // optional [tokens, k] (written by CTA 0)
  long long xnorm_stride;
  // Optional second segment (row-per-warp kernel only): activations [k1, k) come from x2 and are
  // normalised on their own with gamma2 -- the MTP input "concat(enorm(e), hnorm(h))".
  const __nv_bfloat16* x2;       // [tokens, k - k1]; nullptr = one segment
  long long x2_stride;
  int k1;
  const float* gamma2;
  __nv_bfloat16* xnorm2_out;     // optional [tokens, k - k1] (written by CTA 0)
  long long xnorm2_stride;
  void* out;                     // [tokens, n] f32 (out_bf16 = 0) or bf16 (out_bf16 = 1)
  int out_bf16;
  long long out_stride;
};

constexpr int kGemvBf16Threads = 512;

template <int TOK>
__global__ void __launch_bounds__(kGemvBf16Threads) gemv_bf16_kernel(const GemvBf16Params p) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float xs[];  // [TOK][k]
  __shared__ float red[TOK][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;

  // stage (and normalise) the activations; with a second segment each half has its own statistics
  const int k1 = p.x2 != nullptr ? p.k1 : p.k;
  float ss[TOK], ss2[TOK];
#pragma unroll
  for (int t = 0; t < TOK; ++t) ss[t] = ss2[t] = 0.f;
  for (int i = threadIdx.x; i < p.k; i += blockDim.x) {
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
      float v = 0.f;
      if (t < p.n_tokens) v = i < k1 ? bf2f(p.x[t * p.x_stride + i]) : bf2f(p.x2[t * p.x2_stride + i - k1]);
      xs[t * p.k + i] = v;
      if (i < k1) ss[t] += v * v; else ss2[t] += v * v;
    }
  }
  if (p.gamma != nullptr) {
    __shared__ float red2[TOK][32];
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
      const float s = warp_sum(ss[t]), s2 = warp_sum(ss2[t]);
      if (lane == 0) {
        red[t][warp] = s;
        red2[t][warp] = s2;
      }
    }
    __syncthreads();
    float rinv[TOK], rinv2[TOK];
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
      float tot = lane < nwarps ? red[t][lane] : 0.f, tot2 = lane < nwarps ? red2[t][lane] : 0.f;
      tot = warp_sum(tot);
      tot2 = warp_sum(tot2);
      rinv[t] = rsqrtf(tot / static_cast<float>(k1) + p.eps);
      rinv2[t] = rsqrtf(tot2 / static_cast<float>(p.k - k1 > 0 ? p.k - k1 : 1) + p.eps);
    }
    for (int i = threadIdx.x; i < p.k; i += blockDim.x) {
      const float g = i < k1 ? p.gamma[i] : p.gamma2[i - k1];
#pragma unroll
      for (int t = 0; t < TOK; ++t) {
        float v = xs[t * p.k + i] * (i < k1 ? rinv[t] : rinv2[t]) * g;
        if (p.round_norm_bf16) v = bf2f(f2bf(v));
        xs[t * p.k + i] = v;
        if (blockIdx.x == 0 && t < p.n_tokens) {
          if (i < k1) {
            if (p.xnorm_out != nullptr) p.xnorm_out[t * p.xnorm_stride + i] = f2bf(v);
          } else if (p.xnorm2_out != nullptr) {
            p.xnorm2_out[t * p.xnorm2_stride + i - k1] = f2bf(v);
          }
        }
      }
    }
  }
  __syncthreads();

  const int gw = blockIdx.x * nwarps + warp, tw = gridDim.x * nwarps;
  for (int row = gw; row < p.n; row += tw) {
    float acc[TOK];
#pragma unroll
    for (int t = 0; t < TOK; ++t) acc[t] = 0.f;
    if (p.w_is_f32) {
      const float* wr = reinterpret_cast<const float*>(p.w) + static_cast<long long>(row) * p.k;
      for (int k0 = lane * 4; k0 < p.k; k0 += 128) {
        const float4 wv = __ldg(reinterpret_cast<const float4*>(wr + k0));
#pragma unroll
        for (int t = 0; t < TOK; ++t) {
          const float4 xv = *reinterpret_cast<const float4*>(&xs[t * p.k + k0]);
          acc[t] += wv.x * xv.x + wv.y * xv.y + wv.z * xv.z + wv.w * xv.w;
        }
      }
    } else {
      const __nv_bfloat16* wr = reinterpret_cast<const __nv_bfloat16*>(p.w) + static_cast<long long>(row) * p.k;
#pragma unroll 4
      for (int k0 = lane * 8; k0 < p.k; k0 += 256) {
        uint4 wv;
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(wv.x), "=r"(wv.y), "=r"(wv.z), "=r"(wv.w)
                     : "l"(wr + k0));
        const float w0 = __uint_as_float(wv.x << 16), w1 = __uint_as_float(wv.x & 0xffff0000u);
        const float w2 = __uint_as_float(wv.y << 16), w3 = __uint_as_float(wv.y & 0xffff0000u);
        const float w4 = __uint_as_float(wv.z << 16), w5 = __uint_as_float(wv.z & 0xffff0000u);
        const float w6 = __uint_as_float(wv.w << 16), w7 = __uint_as_float(wv.w & 0xffff0000u);
#pragma unroll
        for (int t = 0; t < TOK; ++t) {
          const float4 xa = *reinterpret_cast<const float4*>(&xs[t * p.k + k0]);
          const float4 xb = *reinterpret_cast<const float4*>(&xs[t * p.k + k0 + 4]);
          acc[t] += w0 * xa.x + w1 * xa.y + w2 * xa.z + w3 * xa.w + w4 * xb.x + w5 * xb.y + w6 * xb.z + w7 * xb.w;
        }
      }
    }
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
      const float s = warp_sum(acc[t]);
      if (lane == 0 && t < p.n_tokens) {
        if (p.out_bf16)
          reinterpret_cast<__nv_bfloat16*>(p.out)[t * p.out_stride + row] = f2bf(s);
        else
          reinterpret_cast<float*>(p.out)[t * p.out_stride + row] = s;
      }
    }
  }
}

// Variant for few rows (router gate, indexer head weights): one CTA per pair of rows, the warps
// split K, so the dependent load chain is K / (8 warps * 256) iterations instead of K / 256.
constexpr int kGemvBf16SmallThreads = 256;
constexpr int kGemvBf16SmallRows = 2;

// `block` = index of the row pair; `xs` = [TOK][k] floats of shared memory.  The weights of the
// block's two rows are requested before the wait for the predecessor kernel: they are static, and
// their DRAM latency then overlaps the activation staging and the normalisation.
template <int TOK>
__device__ __forceinline__ void gemv_bf16_ksplit_body(const GemvBf16Params& p, int block, float* xs) {
  __shared__ float red[TOK][8];
  __shared__ float part[kGemvBf16SmallRows][TOK][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kslice = p.k / 8;  // per warp; multiple of 8 elements (k % 256 == 0); at most 1024 (k <= 8192)
  uint4 wpre[kGemvBf16SmallRows][4][2];  // [row][iteration][bf16: .0 only | f32: two halves]
#pragma unroll
  for (int r = 0; r < kGemvBf16SmallRows; ++r) {
    const int row = block * kGemvBf16SmallRows + r;
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int k0 = warp * kslice + lane * 8 + it * 256;
      wpre[r][it][0] = make_uint4(0u, 0u, 0u, 0u);
      wpre[r][it][1] = make_uint4(0u, 0u, 0u, 0u);
      if (row < p.n && k0 < (warp + 1) * kslice) {
        if (p.w_is_f32) {
          const float* wr = reinterpret_cast<const float*>(p.w) + static_cast<long long>(row) * p.k + k0;
          wpre[r][it][0] = __ldg(reinterpret_cast<const uint4*>(wr));
          wpre[r][it][1] = __ldg(reinterpret_cast<const uint4*>(wr + 4));
        } else {
          const __nv_bfloat16* wr = reinterpret_cast<const __nv_bfloat16*>(p.w) + static_cast<long long>(row) * p.k + k0;
          wpre[r][it][0] = __ldg(reinterpret_cast<const uint4*>(wr));
        }
      }
    }
  }
  pdl_wait();
  float ss[TOK];
#pragma unroll
  for (int t = 0; t < TOK; ++t) ss[t] = 0.f;
  // all of this thread's activation loads first (k <= 8192: at most four per token), then the staging:
  // a plain loop would pay one memory round trip per iteration
  uint4 xraw[4][TOK];
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int i = (it * kGemvBf16SmallThreads + threadIdx.x) * 8;
#pragma unroll
    for (int t = 0; t < TOK; ++t)
      xraw[it][t] = (i < p.k && t < p.n_tokens) ? *reinterpret_cast<const uint4*>(p.x + t * p.x_stride + i)
                                                : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int i = (it * kGemvBf16SmallThreads + threadIdx.x) * 8;
    if (i < p.k) {
#pragma unroll
      for (int t = 0; t < TOK; ++t) {
        const uint32_t wv[4] = {xraw[it][t].x, xraw[it][t].y, xraw[it][t].z, xraw[it][t].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a = __uint_as_float(wv[j] << 16), b = __uint_as_float(wv[j] & 0xffff0000u);
          xs[t * p.k + i + 2 * j] = a;
          xs[t * p.k + i + 2 * j + 1] = b;
          ss[t] += a * a + b * b;
        }
      }
    }
  }
  if (p.gamma != nullptr) {
    // gains of this thread's elements (k <= 8192: at most 8 groups of 4), requested before the
    // reduction so their latency hides behind it
    float4 gm[8];
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int i = (it * kGemvBf16SmallThreads + threadIdx.x) * 4;
      gm[it] = i < p.k ? __ldg(reinterpret_cast<const float4*>(p.gamma + i)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
      const float s = warp_sum(ss[t]);
      if (lane == 0) red[t][warp] = s;
    }
    __syncthreads();
    float rinv[TOK];
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
      float tot = lane < 8 ? red[t][lane] : 0.f;
      tot = warp_sum(tot);
      rinv[t] = rsqrtf(tot / static_cast<float>(p.k) + p.eps);
    }
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int i = (it * kGemvBf16SmallThreads + threadIdx.x) * 4;
      if (i < p.k) {
        const float g4[4] = {gm[it].x, gm[it].y, gm[it].z, gm[it].w};
#pragma unroll
        for (int t = 0; t < TOK; ++t) {
          float4 xv = *reinterpret_cast<float4*>(&xs[t * p.k + i]);
          float o[4] = {xv.x * rinv[t] * g4[0], xv.y * rinv[t] * g4[1], xv.z * rinv[t] * g4[2], xv.w * rinv[t] * g4[3]};
          if (p.round_norm_bf16) {
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = bf2f(f2bf(o[j]));
          }
          *reinterpret_cast<float4*>(&xs[t * p.k + i]) = make_float4(o[0], o[1], o[2], o[3]);
          if (p.xnorm_out != nullptr && block == 0 && t < p.n_tokens) {
            uint2 ob;
            ob.x = pack_bf16x2(o[0], o[1]);
            ob.y = pack_bf16x2(o[2], o[3]);
            *reinterpret_cast<uint2*>(p.xnorm_out + t * p.xnorm_stride + i) = ob;
          }
        }
      }
    }
  }
  __syncthreads();

#pragma unroll
  for (int r = 0; r < kGemvBf16SmallRows; ++r) {
    const int row = block * kGemvBf16SmallRows + r;
    float acc[TOK];
#pragma unroll
    for (int t = 0; t < TOK; ++t) acc[t] = 0.f;
    if (row < p.n) {
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int k0 = warp * kslice + lane * 8 + it * 256;
        if (k0 < (warp + 1) * kslice) {
          float wf[8];
          if (p.w_is_f32) {
            const uint4 w0 = wpre[r][it][0], w1 = wpre[r][it][1];
            wf[0] = __uint_as_float(w0.x); wf[1] = __uint_as_float(w0.y); wf[2] = __uint_as_float(w0.z);
            wf[3] = __uint_as_float(w0.w); wf[4] = __uint_as_float(w1.x); wf[5] = __uint_as_float(w1.y);
            wf[6] = __uint_as_float(w1.z); wf[7] = __uint_as_float(w1.w);
          } else {
            const uint4 wv = wpre[r][it][0];
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              wf[2 * j] = __uint_as_float(ww[j] << 16);
              wf[2 * j + 1] = __uint_as_float(ww[j] & 0xffff0000u);
            }
          }
#pragma unroll
          for (int t = 0; t < TOK; ++t) {
            const float4 xa = *reinterpret_cast<const float4*>(&xs[t * p.k + k0]);
            const float4 xb = *reinterpret_cast<const float4*>(&xs[t * p.k + k0 + 4]);
            acc[t] += wf[0] * xa.x + wf[1] * xa.y + wf[2] * xa.z + wf[3] * xa.w + wf[4] * xb.x + wf[5] * xb.y +
                      wf[6] * xb.z + wf[7] * xb.w;
          }
        }
      }
    }
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
      const float s = warp_sum(acc[t]);
      if (lane == 0) part[r][t][warp] = s;
    }
  }
  __syncthreads();
  if (threadIdx.x < kGemvBf16SmallRows * TOK) {
    const int r = threadIdx.x / TOK, t = threadIdx.x % TOK;
    const int row = block * kGemvBf16SmallRows + r;
    if (row < p.n && t < p.n_tokens) {
      float s = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < 8; ++w2) s += part[r][t][w2];
      if (p.out_bf16)
        reinterpret_cast<__nv_bfloat16*>(p.out)[t * p.out_stride + row] = f2bf(s);
      else
        reinterpret_cast<float*>(p.out)[t * p.out_stride + row] = s;
    }
  }
}

template <int TOK>
__global__ void __launch_bounds__(kGemvBf16SmallThreads) gemv_bf16_ksplit_kernel(const GemvBf16Params p) {
  extern __shared__ __align__(16) float xs[];  // [TOK][k]
  pdl_launch_dependents();
  gemv_bf16_ksplit_body<TOK>(p, blockIdx.x, xs);
}

}  // namespace tb
