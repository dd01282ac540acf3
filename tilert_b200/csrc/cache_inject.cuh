// Latent caches handed over by an external prefill in the FP8 wire format (prefill / decode
// disaggregation): per token 512 e4m3 latent values + 4 f32 scales (one per 128 values) = 528 bytes
// in the kv plane, 64 bf16 rope values = 128 bytes in the pe plane, and indexer keys in pages of 64
// tokens: 64 x 128 e4m3 values followed by 64 f32 scales (8448 bytes per page).  The decode side
// keeps bf16 caches, so the rows are dequantised on the way in: latent = e4m3 * scale rounded to
// bf16; indexer key = e4m3 * scale rounded to bf16, then the Hadamard-128 rotation scaled by
// 128^-1/2 (the indexer scores rotated keys against rotated queries).  One warp per token.
#pragma once
#include "elementwise.cuh"

namespace tb {

constexpr int kInjectKvBytes = 528;     // 512 e4m3 + 4 f32
constexpr int kInjectPeBytes = 128;     // 64 bf16
constexpr int kInjectPageTokens = 64;
constexpr int kInjectPageBytes = kInjectPageTokens * 128 + kInjectPageTokens * 4;  // 8448
constexpr int kInjectWarps = 4;

struct CacheInjectParams {
  const uint8_t* kv_raw;   // [seq][528] or nullptr
  const uint8_t* pe_raw;   // [seq][128] or nullptr
  const uint8_t* ki_pages; // [ceil(seq / 64)][8448] or nullptr
  int seq_len;
  int start_pos;           // first cache row written
  __nv_bfloat16* kv_cache; // [T][512]
  __nv_bfloat16* pe_cache; // [T][64]
  __nv_bfloat16* ki_cache; // [T][128]
};

__global__ void __launch_bounds__(kInjectWarps * 32) cache_inject_fp8_kernel(const CacheInjectParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * kInjectWarps + (threadIdx.x >> 5);
  if (t >= p.seq_len) return;
  const long long row = static_cast<long long>(p.start_pos) + t;
  if (p.kv_raw != nullptr) {
    // lane l: values 16l .. 16l+15 of the 512, all in 128-block l / 8
    const uint8_t* src = p.kv_raw + static_cast<long long>(t) * kInjectKvBytes;
    const uint4 q = *reinterpret_cast<const uint4*>(src + lane * 16);
    const float scale = *reinterpret_cast<const float*>(src + 512 + (lane >> 3) * 4);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float a = e4m3_to_f32(static_cast<uint8_t>(w[i] >> (16 * h))) * scale;
        const float b = e4m3_to_f32(static_cast<uint8_t>(w[i] >> (16 * h + 8))) * scale;
        const __nv_bfloat16 ba = f2bf(a), bb = f2bf(b);
        o[i * 2 + h] = static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&ba)) |
                       (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&bb)) << 16);
      }
    }
    uint4* dst = reinterpret_cast<uint4*>(p.kv_cache + row * 512 + lane * 16);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
  if (p.pe_raw != nullptr) {
    const uint32_t v = *reinterpret_cast<const uint32_t*>(p.pe_raw + static_cast<long long>(t) * kInjectPeBytes + lane * 4);
    *reinterpret_cast<uint32_t*>(p.pe_cache + row * 64 + lane * 2) = v;
  }
  if (p.ki_pages != nullptr) {
    const uint8_t* page = p.ki_pages + static_cast<long long>(t / kInjectPageTokens) * kInjectPageBytes;
    const int r = t % kInjectPageTokens;
    const uint32_t q = *reinterpret_cast<const uint32_t*>(page + r * 128 + lane * 4);
    const float scale = *reinterpret_cast<const float*>(page + kInjectPageTokens * 128 + r * 4);
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = bf2f(f2bf(e4m3_to_f32(static_cast<uint8_t>(q >> (8 * j))) * scale));
    hadamard128(v);
    const float hs = 0.08838834764831845f;  // 128^-1/2
    __nv_bfloat16* dst = p.ki_cache + row * 128 + lane * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[j] = f2bf(v[j] * hs);
  }
}

}  // namespace tb
