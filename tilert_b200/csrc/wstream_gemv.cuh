// FP8 weight-streaming skinny GEMM for batch-1 decode (1..8 activation columns).
//
//   out[t, n] = sum_k  W[n, k] * x[t, k]          W: e4m3, 128x128 block scales
//                                                  x: e4m3 columns with per-128 scales
//
// HBM-bound: every weight byte is read exactly once.  One persistent CTA per SM walks a
// contiguous range of (row tile, k block) units (stream-K).  A producer thread stages each
// unit -- one 16448-byte W block and one 1056-byte X block -- into a shared-memory ring with
// bulk async copies (TMA) that complete on mbarriers.  Each ring slot is consumed by TWO warps
// (64 rows each), which feed the e4m3 bytes straight into m16n8k32 tensor-core MMAs and apply
// (weight scale x column scale) in f32 registers once per k block; eight consumer warps work on
// four slots at a time and meet in shared memory when a row tile is complete.  Row tiles that
// straddle two CTAs are finished by the last arriver, which adds the partials in CTA order, so
// the result does not depend on timing.
#pragma once

#include "common.cuh"
#include "formats.h"

namespace tb {

enum Epilogue : int {
  EPI_STORE = 0,     // out = acc (+ residual)
  EPI_SILU_MUL = 1,  // rows g / g+8 of each 16-row group are (gate, up): out = silu(gate) * up
};

struct OutRegion {
  int row_begin;             // first packed row of the region
  int row_end;               // one past the last packed row
  int dtype;                 // 0 = bf16, 1 = f32
  void* ptr;                 // destination of token 0, row row_begin
  long long token_stride;    // elements between tokens
  const int* pos_ptr;        // optional device int: destination starts at token index *pos_ptr
};

// Device-resident state of one rank's all-reduce endpoint.  Everything a call needs (which half
// of the receive buffer to use, what the arrival counter must reach) is derived from `epoch` on
// the device, so a captured CUDA graph can be replayed.
struct AllReduceState {
  unsigned long long epoch;         // completed all-reduce calls on this rank
  unsigned long long arrive;        // incremented once per rank per call, by every rank (peer-written)
  unsigned int local_arrive;        // CTAs of this rank that have pushed their partials (self-resetting)
  unsigned int local_done;          // CTAs of this rank that have finished the call (self-resetting)
};

struct AllReduce {
  int world;                  // 1 = off
  int rank;
  float* recv[8];             // recv[p]: rank p's receive buffer [2 halves][world][4 tokens][n_rows] f32
  AllReduceState* state[8];   // state[p]: rank p's endpoint state (state[rank] is local memory)
};

// Where the activations of a launch come from.
enum XMode : int {
  X_PACKED = 0,  // X blocks prepared beforehand in global memory (bulk-copied with the weights)
  X_BF16 = 1,    // bf16 vectors in global memory; a converter warp normalises (optional RMSNorm),
                 // splits them into two e4m3 terms and writes the X block of each stage itself
};

struct GemvParams {
  const uint8_t* w;
  const uint8_t* x;              // X_PACKED: packed blocks
  int x_mode;
  const __nv_bfloat16* xb;       // X_BF16: [tokens, n_xsegs * n_kb * 128] bf16
  long long xb_stride;           // elements between tokens
  const float* gamma;            // X_BF16: optional RMSNorm gain over the whole vector (n_kb * 128 long)
  float eps;
  const float* seg_scale;        // X_BF16: optional [tokens, n_kb / kb_per_kseg] multipliers (routing weights)
  int n_tiles;
  int n_kb;
  const int* nseg_ids;
  int tiles_per_nseg;
  const int* kseg_ids;
  int kb_per_kseg;
  long long expert_stride;
  int w_kb_per_tile;
  int tiles_per_xseg;
  int n_tokens;
  int only_token;        // >= 0: store only this token's results (per-token expert lists)
  int cols_per_token;
  int epi;
  int n_rows;
  int n_regions;
  OutRegion regions[TB_MAX_REGIONS];
  const __nv_bfloat16* residual;  // optional [tokens, n_rows]
  long long residual_stride;
  float* partial;   // scratch: [2 * grid][8 warps][32 lanes] float4
  int* counters;    // scratch: [n_tiles * 8], zero before the first launch, self-resetting
  int* status;
  unsigned long long* prof;  // optional trace: [grid][16] (see GemvProfSlot)
  AllReduce ar;
};

// Trace slots written per CTA when GemvParams::prof is set (the role of the reference's
// profile_logs tensors, tilert/utils.py:18-45): nanoseconds of %globaltimer.
enum GemvProfSlot : int {
  kGemvProfEntry = 0,         // kernel entry
  kGemvProfReady = 1,         // barriers initialised
  kGemvProfFirstData = 2,     // consumer 0: its first unit's data is in shared memory
  kGemvProfLastUnit = 3,      // consumer 0: its last unit is consumed
  kGemvProfTilesDone = 4,     // consumer 0: all its tile reductions / epilogues are done
  kGemvProfFirstConvert = 5,  // converter 0: first X block written
  kGemvProfIssued = 6,        // producer 0: all its copies issued
  kGemvProfExit = 7,          // consumer 0: end of kernel (after the all-reduce, if any)
  kGemvProfWaitCycles = 8,    // consumer 0: SM cycles spent waiting for data, summed over its units
  kGemvProfMathCycles = 9,    // consumer 0: SM cycles spent consuming, summed over its units
  kGemvProfUnits = 10,        // consumer 0: number of units it consumed
};
__device__ __forceinline__ void gemv_stamp(const GemvParams& p, int slot) {
  if (p.prof != nullptr) p.prof[blockIdx.x * 16 + slot] = globaltimer_ns();
}

#ifndef TB_GEMV_STAGES
#define TB_GEMV_STAGES 12
#endif
constexpr int kGemvStages = TB_GEMV_STAGES;  // multiple of kGemvProducerWarps
constexpr int kGemvConsumerWarps = 8;   // unit i is consumed by warps i % 4 (rows 0-63) and 4 + i % 4 (rows 64-127)
constexpr int kGemvProducerWarps = 4;   // one issuing thread each; unit i is issued by producer i % 4
constexpr int kGemvConverterWarps = 2;  // unit i is converted by converter i % 2 (X_BF16 only)
constexpr int kGemvConsumerThreads = kGemvConsumerWarps * 32;
constexpr int kGemvHelperWarps = kGemvConsumerWarps + kGemvConverterWarps;  // warps that are not producers
constexpr int kGemvThreads = (kGemvConsumerWarps + kGemvProducerWarps + kGemvConverterWarps) * 32;
constexpr int kGemvRedBytes = kGemvConsumerWarps * 4 * 32 * 16;  // per-tile cross-warp reduction buffer
constexpr int kGemvSmemBytes =
    kGemvStages * TB_STAGE_BYTES + kGemvRedBytes + 2 * kGemvStages * 8 + 16 + kGemvHelperWarps * 4 * 4 + 32;

__device__ __forceinline__ long long gemv_range_begin(long long units, int grid, int cta) {
  return units * cta / grid;
}
__device__ __forceinline__ int gemv_owner(long long unit, long long units, int grid) {
  return static_cast<int>(((unit + 1) * grid - 1) / units);
}

__device__ __forceinline__ void gemv_store(const GemvParams& p, int row, int token, float v) {
  if (row >= p.n_rows || token >= p.n_tokens) return;
  if (p.only_token >= 0 && token != p.only_token) return;
  if (p.residual != nullptr) v += bf2f(p.residual[token * p.residual_stride + row]);
#pragma unroll
  for (int i = 0; i < TB_MAX_REGIONS; ++i) {
    if (i < p.n_regions && row >= p.regions[i].row_begin && row < p.regions[i].row_end) {
      const OutRegion& r = p.regions[i];
      long long tok = token;
      if (r.pos_ptr != nullptr) tok += *r.pos_ptr;
      const long long off = tok * r.token_stride + (row - r.row_begin);
      if (r.dtype == 0)
        reinterpret_cast<__nv_bfloat16*>(r.ptr)[off] = f2bf(v);
      else
        reinterpret_cast<float*>(r.ptr)[off] = v;
    }
  }
}

// Final values of one warp's 16 rows x 8 columns (m16n8 accumulator layout).
__device__ __forceinline__ void gemv_epilogue(const GemvParams& p, int tile, int warp, int lane,
                                              const float (&v)[4], int ar_half) {
  const int g = lane >> 2, q = lane & 3;
  const int n16 = tile * 8 + warp;
  float lo[2], hi[2];
  int tok[2], ntok;
  if (p.cols_per_token == 2) {
    lo[0] = v[0] + v[1];
    hi[0] = v[2] + v[3];
    tok[0] = q;
    ntok = 1;
  } else {
    lo[0] = v[0]; lo[1] = v[1];
    hi[0] = v[2]; hi[1] = v[3];
    tok[0] = 2 * q; tok[1] = 2 * q + 1;
    ntok = 2;
  }
  for (int i = 0; i < ntok; ++i) {
    if (p.epi == EPI_SILU_MUL) {
      const float gate = lo[i], up = hi[i];
      const float h = gate / (1.0f + __expf(-gate)) * up;
      gemv_store(p, n16 * 8 + g, tok[i], h);
    } else if (p.ar.world > 1) {
      // push this rank's partial into every rank's receive slot (plain peer stores)
      const int par = ar_half;
      if (tok[i] < p.n_tokens) {
        const long long base = ((static_cast<long long>(par) * p.ar.world + p.ar.rank) * 4 + tok[i]) * p.n_rows;
        const int r0 = n16 * 16 + g, r1 = r0 + 8;
        for (int pr = 0; pr < p.ar.world; ++pr) {
          if (r0 < p.n_rows) p.ar.recv[pr][base + r0] = lo[i];
          if (r1 < p.n_rows) p.ar.recv[pr][base + r1] = hi[i];
        }
      }
    } else {
      gemv_store(p, n16 * 16 + g, tok[i], lo[i]);
      gemv_store(p, n16 * 16 + g + 8, tok[i], hi[i]);
    }
  }
}

__global__ void __launch_bounds__(kGemvThreads, 1) wstream_gemv_kernel(const __grid_constant__ GemvParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  float4* red = reinterpret_cast<float4*>(smem + kGemvStages * TB_STAGE_BYTES);  // [warp][n16 tile][lane]
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kGemvStages * TB_STAGE_BYTES + kGemvRedBytes);
  uint64_t* empty = full + kGemvStages;
  volatile int* cta_error = reinterpret_cast<volatile int*>(empty + kGemvStages);
  float* norm_part = reinterpret_cast<float*>(const_cast<int*>(cta_error) + 4);  // [helper warps][4 tokens]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grid = gridDim.x, cta = blockIdx.x;
  const long long units = static_cast<long long>(p.n_tiles) * p.n_kb;
  // unit indices fit 32 bits (checked on the host); all per-stage index arithmetic is 32-bit --
  // 64-bit divisions in these loops cost more than the stage's data movement
  const int u0 = static_cast<int>(gemv_range_begin(units, grid, cta));
  const int u1 = static_cast<int>(gemv_range_begin(units, grid, cta + 1));

  // The successor may start right away.  Weight prefetch does not depend on the predecessor, so only
  // threads that read activations / routing ids / residuals or write results wait for it (below).
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    gemv_stamp(p, kGemvProfEntry);
    for (int s = 0; s < kGemvStages; ++s) {
      mbar_init(&full[s], p.x_mode == X_BF16 ? 2 : 1);  // producer (+ converter) arrive once per use
      mbar_init(&empty[s], 2);                          // the two consumer warps of the slot
    }
    *cta_error = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) gemv_stamp(p, kGemvProfReady);

  const bool is_consumer = warp < kGemvConsumerWarps;
  const bool is_producer = !is_consumer && warp < kGemvConsumerWarps + kGemvProducerWarps;
  // Producers stream weights, which no kernel of the step writes; they wait for the predecessor only
  // when their addresses depend on it (routing ids) or when they also copy packed activations.
  if (!is_producer || p.x_mode == X_PACKED || p.nseg_ids != nullptr || p.kseg_ids != nullptr) pdl_wait();
  if (p.x_mode == X_BF16 && p.gamma != nullptr && !is_producer) {
    // RMSNorm statistics of the activation vector(s): the non-producer warps split the vector
    // (the producers are already filling the ring), partial sums meet in shared memory.
    const int hw = is_consumer ? warp : warp - kGemvProducerWarps;
    const int n_chunks = p.n_kb * (TB_KBLOCK / 4);  // 8-byte chunks per token
    float ss[4] = {0.f, 0.f, 0.f, 0.f};
    for (int ch = hw * 32 + lane; ch < n_chunks; ch += kGemvHelperWarps * 32) {
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        if (t < p.n_tokens) {
          const uint2 raw = *reinterpret_cast<const uint2*>(p.xb + t * p.xb_stride + ch * 4);
          const float a0 = __uint_as_float(raw.x << 16), a1 = __uint_as_float(raw.x & 0xffff0000u);
          const float a2 = __uint_as_float(raw.y << 16), a3 = __uint_as_float(raw.y & 0xffff0000u);
          ss[t] += a0 * a0 + a1 * a1 + a2 * a2 + a3 * a3;
        }
      }
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float v = warp_sum(ss[t]);
      if (lane == 0) norm_part[hw * 4 + t] = v;
    }
    asm volatile("bar.sync 2, %0;" ::"n"(kGemvHelperWarps * 32) : "memory");
  }

  if (is_producer) {
    // ------------------------------------------------------------ producers
    // Four warps, one issuing thread each; unit i of the CTA's range is issued by producer i % 4
    // into ring slot i % kGemvStages, so no single thread's instruction latency paces the stream.
    if (lane == 0) {
      const int pw = warp - kGemvConsumerWarps;
      const uint64_t pol = policy_evict_first();
      int last_i = -1;
      int t = (u0 + pw) / p.n_kb, kb = (u0 + pw) % p.n_kb;
      for (int u = u0 + pw; u < u1; u += kGemvProducerWarps) {
        const int i = u - u0;
        const int s = i % kGemvStages;
        const uint32_t use = static_cast<uint32_t>(i / kGemvStages);
        if (use > 0 && !mbar_wait(&empty[s], (use - 1) & 1)) {
          set_status(p.status, ST_WAIT_EMPTY_TIMEOUT);
          *cta_error = 1;
          break;
        }
        long long eid = 0;
        int tl = t, kbl = kb;
        if (p.nseg_ids != nullptr) {
          eid = p.nseg_ids[t / p.tiles_per_nseg];
          tl = t % p.tiles_per_nseg;
        }
        if (p.kseg_ids != nullptr) {
          eid = p.kseg_ids[kb / p.kb_per_kseg];
          kbl = kb % p.kb_per_kseg;
        }
        const uint8_t* wsrc =
            p.w + eid * p.expert_stride + (static_cast<long long>(tl) * p.w_kb_per_tile + kbl) * TB_WBLK_BYTES;
        uint8_t* dst = smem + s * TB_STAGE_BYTES;
        if (p.x_mode == X_PACKED) {
          const int xseg = p.tiles_per_xseg > 0 ? t / p.tiles_per_xseg : 0;
          const uint8_t* xsrc = p.x + (static_cast<long long>(xseg) * p.n_kb + kb) * TB_XBLK_BYTES;
          mbar_expect_tx(&full[s], TB_STAGE_BYTES);
          bulk_g2s_stream(dst, wsrc, TB_WBLK_BYTES, &full[s], pol);
          bulk_g2s(dst + TB_WBLK_BYTES, xsrc, TB_XBLK_BYTES, &full[s]);
        } else {
          mbar_expect_tx(&full[s], TB_WBLK_BYTES);
          bulk_g2s_stream(dst, wsrc, TB_WBLK_BYTES, &full[s], pol);
        }
        last_i = i;
        kb += kGemvProducerWarps;
        while (kb >= p.n_kb) {
          kb -= p.n_kb;
          ++t;
        }
      }
      if (pw == 0) gemv_stamp(p, kGemvProfIssued);
      // Do not leave the CTA while this thread's copies may still be landing in its shared memory:
      // wait (bounded) for the last use it issued into each of its ring slots.  On the normal path
      // these have completed already, because the consumers waited on the same phases.
      for (int back = 0; back < kGemvStages && last_i - back >= 0; back += kGemvProducerWarps) {
        const int i = last_i - back;
        mbar_wait(&full[i % kGemvStages], static_cast<uint32_t>(i / kGemvStages) & 1);
      }
    }
  } else if (!is_consumer) {
    // ------------------------------------------------- activation converters (X_BF16 only)
    // Two warps take alternate units.  Each converts the 128 activations of its unit, for every
    // token, into the two-term e4m3 X block of the stage: power-of-two scales, so the scaling is a
    // multiplication and the residual x - hi*s is exact.
    const int cw = warp - (kGemvConsumerWarps + kGemvProducerWarps);  // 0 or 1
    if (p.x_mode == X_BF16 && u0 + cw < u1) {
      const int ntok = p.n_tokens;
      float rinv[4] = {1.f, 1.f, 1.f, 1.f};
      if (p.gamma != nullptr) {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          float tot = 0.f;
#pragma unroll
          for (int w2 = 0; w2 < kGemvHelperWarps; ++w2) tot += norm_part[w2 * 4 + t];
          rinv[t] = rsqrtf(tot / static_cast<float>(p.n_kb * TB_KBLOCK) + p.eps);
        }
      }
      const long long xk = static_cast<long long>(p.n_kb) * TB_KBLOCK;  // activations per x segment
      struct XRaw {
        uint2 v[4];
        float4 g;
      };
      auto fetch = [&](int u) {
        XRaw o;
        const int t = u / p.n_kb, kb = u % p.n_kb;
        const int xseg = p.tiles_per_xseg > 0 ? t / p.tiles_per_xseg : 0;
        const long long off = xseg * xk + static_cast<long long>(kb) * TB_KBLOCK + lane * 4;
#pragma unroll
        for (int tk = 0; tk < 4; ++tk)
          o.v[tk] = tk < ntok ? *reinterpret_cast<const uint2*>(p.xb + tk * p.xb_stride + off) : make_uint2(0, 0);
        o.g = p.gamma != nullptr ? *reinterpret_cast<const float4*>(p.gamma + kb * TB_KBLOCK + lane * 4)
                                 : make_float4(1.f, 1.f, 1.f, 1.f);
        return o;
      };
      // software pipeline over this warp's units (u, u+2, u+4, ...): two requests in flight
      const int ub = u0 + cw;
      XRaw x0 = fetch(ub), x1 = x0, x2 = x0;
      if (ub + 2 < u1) x1 = fetch(ub + 2);
      const int c = lane >> 3, r = (lane >> 2) & 1, q4 = lane & 3;
      for (int u = ub; u < u1; u += 2) {
        const int i = u - u0;
        const int s = i % kGemvStages;
        const uint32_t use = static_cast<uint32_t>(i / kGemvStages);
        if (u + 4 < u1) x2 = fetch(u + 4);
        if (use > 0 && !mbar_wait(&empty[s], (use - 1) & 1)) {
          set_status(p.status, ST_WAIT_EMPTY_TIMEOUT);
          *cta_error = 1;
          break;
        }
        uint8_t* blk = smem + s * TB_STAGE_BYTES + TB_WBLK_BYTES;
        const int kb = u % p.n_kb;
        const float g4[4] = {x0.g.x, x0.g.y, x0.g.z, x0.g.w};
#pragma unroll
        for (int tk = 0; tk < 4; ++tk) {
          if (tk < ntok) {
            const uint2 rw = x0.v[tk];
            float x4[4] = {__uint_as_float(rw.x << 16), __uint_as_float(rw.x & 0xffff0000u),
                           __uint_as_float(rw.y << 16), __uint_as_float(rw.y & 0xffff0000u)};
            if (p.gamma != nullptr) {
#pragma unroll
              for (int j = 0; j < 4; ++j) x4[j] = bf2f(f2bf(x4[j] * rinv[tk] * g4[j]));
            }
            float amax = fmaxf(fmaxf(fabsf(x4[0]), fabsf(x4[1])), fmaxf(fabsf(x4[2]), fabsf(x4[3])));
            amax = warp_max(amax);
            // s_hi = 2^e: the power of two at or just above amax / 448 (at most one step higher when the
            // product below rounds up); exponent clamped so that s_hi / 16 and 1 / s_hi stay normal
            const uint32_t tb = __float_as_uint(amax * (1.0f / 448.0f));
            int e = static_cast<int>(tb >> 23) + ((tb & 0x7fffffu) != 0u ? 1 : 0);
            e = amax > 0.f ? min(max(e, 16), 240) : 127;
            const float s_hi = __uint_as_float(static_cast<uint32_t>(e) << 23);
            const float inv_hi = __uint_as_float(static_cast<uint32_t>(254 - e) << 23);
            const float s_lo = s_hi * 0.0625f, inv_lo = inv_hi * 16.f;
            const __nv_fp8x2_storage_t h01 =
                __nv_cvt_float2_to_fp8x2(make_float2(x4[0] * inv_hi, x4[1] * inv_hi), __NV_SATFINITE, __NV_E4M3);
            const __nv_fp8x2_storage_t h23 =
                __nv_cvt_float2_to_fp8x2(make_float2(x4[2] * inv_hi, x4[3] * inv_hi), __NV_SATFINITE, __NV_E4M3);
            const __half2_raw hr01 = __nv_cvt_fp8x2_to_halfraw2(h01, __NV_E4M3);
            const __half2_raw hr23 = __nv_cvt_fp8x2_to_halfraw2(h23, __NV_E4M3);
            const float2 hf01 = __half22float2(*reinterpret_cast<const __half2*>(&hr01));
            const float2 hf23 = __half22float2(*reinterpret_cast<const __half2*>(&hr23));
            const float r0 = fmaf(-hf01.x, s_hi, x4[0]), r1 = fmaf(-hf01.y, s_hi, x4[1]);
            const float r2 = fmaf(-hf23.x, s_hi, x4[2]), r3 = fmaf(-hf23.y, s_hi, x4[3]);
            const __nv_fp8x2_storage_t l01 =
                __nv_cvt_float2_to_fp8x2(make_float2(r0 * inv_lo, r1 * inv_lo), __NV_SATFINITE, __NV_E4M3);
            const __nv_fp8x2_storage_t l23 =
                __nv_cvt_float2_to_fp8x2(make_float2(r2 * inv_lo, r3 * inv_lo), __NV_SATFINITE, __NV_E4M3);
            const uint32_t whi = static_cast<uint32_t>(h01) | (static_cast<uint32_t>(h23) << 16);
            const uint32_t wlo = static_cast<uint32_t>(l01) | (static_cast<uint32_t>(l23) << 16);
            *reinterpret_cast<uint32_t*>(blk + (c * 32 + (2 * tk) * 4 + q4) * 8 + 4 * r) = whi;
            *reinterpret_cast<uint32_t*>(blk + (c * 32 + (2 * tk + 1) * 4 + q4) * 8 + 4 * r) = wlo;
            if (lane == 0) {
              float mlt = 1.f;
              if (p.seg_scale != nullptr) mlt = p.seg_scale[tk * (p.n_kb / p.kb_per_kseg) + kb / p.kb_per_kseg];
              *reinterpret_cast<float2*>(blk + TB_XBLK_DATA + 8 * tk) = make_float2(s_hi * mlt, s_lo * mlt);
            }
          }
        }
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&full[s]);
          if (u == u0) gemv_stamp(p, kGemvProfFirstConvert);
        }
        x0 = x1;
        x1 = x2;
      }
    }
  } else {
    // ------------------------------------------------------------ consumers
    // Warps w and w + 4 consume units u0 + w, u0 + w + 4, ... (w < 4): rows 0-63 and 64-127 of each
    // 128 x 128 block, four 16-row groups per warp sharing the activation fragments.  When a row tile
    // is complete -- or the CTA's range ends inside it -- the warps add their accumulators through
    // shared memory and warp w finishes 16-row group w.
    const int q = lane & 3;
    const int wq = warp & 3, half = warp >> 2;
    unsigned long long ar_epoch = 0;
    if (p.ar.world > 1) ar_epoch = *reinterpret_cast<volatile unsigned long long*>(&p.ar.state[p.ar.rank]->epoch);
    const int ar_half = static_cast<int>(ar_epoch & 1ull);
    float acc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    bool ok = true;
    long long prof_wait = 0, prof_math = 0, prof_units = 0;

    // Adds the warps' accumulators of row tile t and finishes this warp's 16-row group.
    auto finish_tile = [&](int t) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        red[(warp * 4 + j) * 32 + lane] = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
        acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kGemvConsumerThreads) : "memory");
      // 16-row group `warp` = local group wq of half `half`: partial sums sit with the four warps of that half
      float out[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int w2 = 0; w2 < 4; ++w2) {
        const float4 v = red[((half * 4 + w2) * 4 + wq) * 32 + lane];
        out[0] += v.x; out[1] += v.y; out[2] += v.z; out[3] += v.w;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kGemvConsumerThreads) : "memory");  // red may be rewritten
      const int tile_u0 = t * p.n_kb, tile_u1 = tile_u0 + p.n_kb;
      const int n16 = warp;  // 16-row group inside the tile
      if (u0 <= tile_u0 && u1 >= tile_u1) {
        gemv_epilogue(p, t, n16, lane, out, ar_half);
      } else {
        const int c_first = gemv_owner(tile_u0, units, grid);
        const int c_last = gemv_owner(tile_u1 - 1, units, grid);
        const int my_slot = 2 * cta + ((u0 / p.n_kb) == t ? 0 : 1);
        float4* part = reinterpret_cast<float4*>(p.partial);
        part[(my_slot * 8 + n16) * 32 + lane] = make_float4(out[0], out[1], out[2], out[3]);
        __threadfence();
        __syncwarp();
        int prev = 0;
        if (lane == 0) prev = atomicAdd(&p.counters[t * 8 + n16], 1);
        prev = __shfl_sync(0xffffffffu, prev, 0);
        if (prev == c_last - c_first) {
          __threadfence();
          float sum[4] = {0.f, 0.f, 0.f, 0.f};
          for (int cc = c_first; cc <= c_last; ++cc) {
            const int cu0 = static_cast<int>(gemv_range_begin(units, grid, cc));
            const int slot = 2 * cc + ((cu0 / p.n_kb) == t ? 0 : 1);
            const float4 v = __ldcg(&part[(slot * 8 + n16) * 32 + lane]);
            sum[0] += v.x; sum[1] += v.y; sum[2] += v.z; sum[3] += v.w;
          }
          if (lane == 0) p.counters[t * 8 + n16] = 0;
          gemv_epilogue(p, t, n16, lane, sum, ar_half);
        }
      }
    };

    int cur_t = u0 < u1 ? u0 / p.n_kb : 0;
    const int last_t = u0 < u1 ? (u1 - 1) / p.n_kb : -1;
    for (int u = u0 + wq; u < u1; u += 4) {
      const int t = u / p.n_kb;
      while (cur_t < t) finish_tile(cur_t++);  // every warp passes through every tile boundary, in order
      const int i = u - u0;
      const int s = i % kGemvStages;
      const uint32_t use = static_cast<uint32_t>(i / kGemvStages);
      // A warp that gave up on a wait keeps walking its units without touching the ring, so that it
      // still meets the other warps at every tile boundary (those barriers have no time limit).
      if (!ok || *cta_error) {
        ok = false;
        continue;
      }
      const long long c0 = p.prof != nullptr ? clock64() : 0;
      if (!mbar_wait(&full[s], use & 1)) {
        set_status(p.status, ST_WAIT_FULL_TIMEOUT);
        *cta_error = 1;
        ok = false;
        continue;
      }
      const long long c1 = p.prof != nullptr ? clock64() : 0;
      if (u == u0 && lane == 0) gemv_stamp(p, kGemvProfFirstData);
      const uint8_t* sw = smem + s * TB_STAGE_BYTES;
      const uint8_t* sx = sw + TB_WBLK_BYTES;
      uint2 b[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) b[c] = *reinterpret_cast<const uint2*>(sx + (c * 32 + lane) * 8);
      const float2 cs = *reinterpret_cast<const float2*>(sx + TB_XBLK_DATA + q * 8);
      // four independent accumulation chains (one per 16-row group), each over the four k chunks
      float d[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j) d[j][0] = d[j][1] = d[j][2] = d[j][3] = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 a = *reinterpret_cast<const uint4*>(sw + (((half * 4 + j) * 4 + c) * 32 + lane) * 16);
#ifndef TB_EXP_SKIP_MMA
          mma_e4m3_16832(d[j], a, b[c]);
#else
          d[j][0] += __uint_as_float(a.x ^ b[c].x);
#endif
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 ws = *reinterpret_cast<const float2*>(sw + TB_WBLK_DATA + (half * 4 + j) * 8);
        acc[j][0] = fmaf(d[j][0], ws.x * cs.x, acc[j][0]);
        acc[j][1] = fmaf(d[j][1], ws.x * cs.y, acc[j][1]);
        acc[j][2] = fmaf(d[j][2], ws.y * cs.x, acc[j][2]);
        acc[j][3] = fmaf(d[j][3], ws.y * cs.y, acc[j][3]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
      if (p.prof != nullptr) {
        prof_wait += c1 - c0;
        prof_math += clock64() - c1;
        ++prof_units;
      }
    }
    if (warp == 0 && lane == 0) gemv_stamp(p, kGemvProfLastUnit);
    if (warp == 0 && lane == 0 && p.prof != nullptr) {
      p.prof[blockIdx.x * 16 + kGemvProfWaitCycles] = prof_wait;
      p.prof[blockIdx.x * 16 + kGemvProfMathCycles] = prof_math;
      p.prof[blockIdx.x * 16 + kGemvProfUnits] = prof_units;
    }
    // tiles this warp has not closed yet (including those in which it had no unit)
    while (cur_t <= last_t) finish_tile(cur_t++);
    if (warp == 0 && lane == 0) gemv_stamp(p, kGemvProfTilesDone);
    if (p.ar.world > 1) {
      // ---- one-shot all-reduce over peer memory, fused behind the streaming loop ----
      AllReduceState* self = p.ar.state[p.ar.rank];
      // 1. this CTA's peer stores are done: publish them.  The last CTA of the rank to get here
      //    tells every rank (itself included) that this rank's partial has landed.
      __threadfence_system();
      asm volatile("bar.sync 1, %0;" ::"n"(kGemvConsumerThreads) : "memory");
      if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(&self->local_arrive, 1u);
        if (prev == static_cast<unsigned int>(grid) - 1u) {
          self->local_arrive = 0u;
          __threadfence_system();
          for (int pr = 0; pr < p.ar.world; ++pr)
            asm volatile("red.release.sys.global.add.u64 [%0], 1;" ::"l"(&p.ar.state[pr]->arrive) : "memory");
        }
        // 2. wait (bounded) until every rank has arrived for this call.
        const unsigned long long target = (ar_epoch + 1ull) * static_cast<unsigned long long>(p.ar.world);
        const unsigned long long t0 = globaltimer_ns();
        unsigned long long seen = 0;
        while (ok) {
          asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(&self->arrive) : "memory");
          if (seen >= target) break;
          if (globaltimer_ns() - t0 > kWaitBudgetNs) {
            set_status(p.status, ST_PEER_TIMEOUT);
            *cta_error = 1;
            break;
          }
          __nanosleep(32);
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kGemvConsumerThreads) : "memory");
      // 3. reduce the world's slots for this CTA's share of rows, add the residual, store.
      if (!*cta_error) {
        const float* mine = p.ar.recv[p.ar.rank];
        const int total = p.n_tokens * p.n_rows;
        const int e0 = static_cast<int>(static_cast<long long>(total) * cta / grid);
        const int e1 = static_cast<int>(static_cast<long long>(total) * (cta + 1) / grid);
        for (int e = e0 + static_cast<int>(threadIdx.x); e < e1; e += kGemvConsumerThreads) {
          const int tok = e / p.n_rows, row = e % p.n_rows;
          float v = 0.f;
          for (int r = 0; r < p.ar.world; ++r)
            v += __ldcg(&mine[((static_cast<long long>(ar_half) * p.ar.world + r) * 4 + tok) * p.n_rows + row]);
          gemv_store(p, row, tok, v);
        }
      }
      // 4. the last CTA to finish opens the next call (flips the buffer half).
      asm volatile("bar.sync 1, %0;" ::"n"(kGemvConsumerThreads) : "memory");
      if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(&self->local_done, 1u);
        if (prev == static_cast<unsigned int>(grid) - 1u) {
          self->local_done = 0u;
          __threadfence();
          *reinterpret_cast<volatile unsigned long long*>(&self->epoch) = ar_epoch + 1ull;
        }
      }
    }
    if (warp == 0 && lane == 0) gemv_stamp(p, kGemvProfExit);
  }
}

}  // namespace tb
