// FP8 weight-streaming skinny GEMM for batch-1 decode (1..8 activation columns).
//
//   out[t, n] = sum_k  W[n, k] * x[t, k]          W: e4m3, 128x128 block scales
//                                                  x: e4m3 columns with per-128 scales
//
// HBM-bound: every weight byte is read exactly once.  One persistent CTA per SM walks a
// contiguous range of (row tile, k block) units (stream-K).  A producer thread stages each
// unit -- one 16448-byte W block and one 1056-byte X block -- into a shared-memory ring with
// bulk async copies (TMA) that complete on mbarriers; eight consumer warps each own 16 rows of
// the tile, feed the e4m3 bytes straight into m16n8k32 tensor-core MMAs and apply
// (weight scale x column scale) in f32 registers once per k block.  Row tiles that straddle
// two CTAs are finished by the last arriver, which adds the partials in CTA order, so the
// result does not depend on timing.
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

struct GemvParams {
  const uint8_t* w;
  const uint8_t* x;
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
  AllReduce ar;
};

constexpr int kGemvStages = 12;
constexpr int kGemvConsumerWarps = 8;
constexpr int kGemvThreads = (kGemvConsumerWarps + 1) * 32;
constexpr int kGemvSmemBytes = kGemvStages * TB_STAGE_BYTES + 2 * kGemvStages * 8 + 64;

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
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kGemvStages * TB_STAGE_BYTES);
  uint64_t* empty = full + kGemvStages;
  volatile int* cta_error = reinterpret_cast<volatile int*>(empty + kGemvStages);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grid = gridDim.x, cta = blockIdx.x;
  const long long units = static_cast<long long>(p.n_tiles) * p.n_kb;
  const long long u0 = gemv_range_begin(units, grid, cta);
  const long long u1 = gemv_range_begin(units, grid, cta + 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kGemvStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kGemvConsumerWarps);
    }
    *cta_error = 0;
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == kGemvConsumerWarps) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {
      const uint64_t pol = policy_evict_first();
      long long issued = 0;
      bool ok = true;
      for (long long u = u0; u < u1 && ok; ++u) {
        const long long i = u - u0;
        const int s = static_cast<int>(i % kGemvStages);
        const uint32_t use = static_cast<uint32_t>(i / kGemvStages);
        if (use > 0 && !mbar_wait(&empty[s], (use - 1) & 1)) {
          set_status(p.status, ST_WAIT_EMPTY_TIMEOUT);
          *cta_error = 1;
          ok = false;
          break;
        }
        const int t = static_cast<int>(u / p.n_kb), kb = static_cast<int>(u % p.n_kb);
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
        const int xseg = p.tiles_per_xseg > 0 ? t / p.tiles_per_xseg : 0;
        const uint8_t* xsrc = p.x + (static_cast<long long>(xseg) * p.n_kb + kb) * TB_XBLK_BYTES;
        uint8_t* dst = smem + s * TB_STAGE_BYTES;
        mbar_expect_tx(&full[s], TB_STAGE_BYTES);
        bulk_g2s_stream(dst, wsrc, TB_WBLK_BYTES, &full[s], pol);
        bulk_g2s(dst + TB_WBLK_BYTES, xsrc, TB_XBLK_BYTES, &full[s]);
        ++issued;
      }
      // Do not leave the CTA while copies may still be landing in its shared memory: wait
      // (bounded) for the last issued use of every ring slot.  On the normal path these have
      // all completed already, because the consumers waited on the same phases.
      for (int s = 0; s < kGemvStages; ++s) {
        if (issued > s) {
          const uint32_t last_use = static_cast<uint32_t>((issued - 1 - s) / kGemvStages);
          mbar_wait(&full[s], last_use & 1);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ consumers
    const int q = lane & 3;
    unsigned long long ar_epoch = 0;
    if (p.ar.world > 1) ar_epoch = *reinterpret_cast<volatile unsigned long long*>(&p.ar.state[p.ar.rank]->epoch);
    const int ar_half = static_cast<int>(ar_epoch & 1ull);
    float out[4] = {0.f, 0.f, 0.f, 0.f};
    bool ok = true;
    for (long long u = u0; u < u1; ++u) {
      const long long i = u - u0;
      const int s = static_cast<int>(i % kGemvStages);
      const uint32_t use = static_cast<uint32_t>(i / kGemvStages);
      if (!mbar_wait(&full[s], use & 1)) {
        set_status(p.status, ST_WAIT_FULL_TIMEOUT);
        *cta_error = 1;
        ok = false;
        break;
      }
      const uint8_t* sw = smem + s * TB_STAGE_BYTES;
      const uint8_t* sx = sw + TB_WBLK_BYTES;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 a = *reinterpret_cast<const uint4*>(sw + ((warp * 4 + c) * 32 + lane) * 16);
        const uint2 b = *reinterpret_cast<const uint2*>(sx + (c * 32 + lane) * 8);
        mma_e4m3_16832(acc, a, b);
      }
      const float2 ws = *reinterpret_cast<const float2*>(sw + TB_WBLK_DATA + warp * 8);
      const float2 cs = *reinterpret_cast<const float2*>(sx + TB_XBLK_DATA + q * 8);
      out[0] = fmaf(acc[0], ws.x * cs.x, out[0]);
      out[1] = fmaf(acc[1], ws.x * cs.y, out[1]);
      out[2] = fmaf(acc[2], ws.y * cs.x, out[2]);
      out[3] = fmaf(acc[3], ws.y * cs.y, out[3]);
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);

      const int t = static_cast<int>(u / p.n_kb), kb = static_cast<int>(u % p.n_kb);
      if (kb == p.n_kb - 1 || u == u1 - 1) {
        // this CTA's share of row tile t is complete
        const long long tile_u0 = static_cast<long long>(t) * p.n_kb;
        const long long tile_u1 = tile_u0 + p.n_kb;
        if (u0 <= tile_u0 && u1 >= tile_u1) {
          gemv_epilogue(p, t, warp, lane, out, ar_half);
        } else {
          const int c_first = gemv_owner(tile_u0, units, grid);
          const int c_last = gemv_owner(tile_u1 - 1, units, grid);
          const int my_slot = 2 * cta + ((u0 / p.n_kb) == t ? 0 : 1);
          float4* part = reinterpret_cast<float4*>(p.partial);
          part[(my_slot * 8 + warp) * 32 + lane] = make_float4(out[0], out[1], out[2], out[3]);
          __threadfence();
          __syncwarp();
          int prev = 0;
          if (lane == 0) prev = atomicAdd(&p.counters[t * 8 + warp], 1);
          prev = __shfl_sync(0xffffffffu, prev, 0);
          if (prev == c_last - c_first) {
            __threadfence();
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
            for (int cc = c_first; cc <= c_last; ++cc) {
              const long long cu0 = gemv_range_begin(units, grid, cc);
              const int slot = 2 * cc + ((cu0 / p.n_kb) == t ? 0 : 1);
              const float4 v = __ldcg(&part[(slot * 8 + warp) * 32 + lane]);
              sum[0] += v.x; sum[1] += v.y; sum[2] += v.z; sum[3] += v.w;
            }
            if (lane == 0) p.counters[t * 8 + warp] = 0;
            gemv_epilogue(p, t, warp, lane, sum, ar_half);
          }
        }
        out[0] = out[1] = out[2] = out[3] = 0.f;
      }
    }

    if (p.ar.world > 1) {
      // ---- one-shot all-reduce over peer memory, fused behind the streaming loop ----
      AllReduceState* self = p.ar.state[p.ar.rank];
      // 1. this CTA's peer stores are done: publish them.  The last CTA of the rank to get here
      //    tells every rank (itself included) that this rank's partial has landed.
      __threadfence_system();
      asm volatile("bar.sync 1, 256;" ::: "memory");
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
      asm volatile("bar.sync 1, 256;" ::: "memory");
      // 3. reduce the world's slots for this CTA's share of rows, add the residual, store.
      if (!*cta_error) {
        const float* mine = p.ar.recv[p.ar.rank];
        const int total = p.n_tokens * p.n_rows;
        const int e0 = static_cast<int>(static_cast<long long>(total) * cta / grid);
        const int e1 = static_cast<int>(static_cast<long long>(total) * (cta + 1) / grid);
        for (int e = e0 + static_cast<int>(threadIdx.x); e < e1; e += 256) {
          const int tok = e / p.n_rows, row = e % p.n_rows;
          float v = 0.f;
          for (int r = 0; r < p.ar.world; ++r)
            v += __ldcg(&mine[((static_cast<long long>(ar_half) * p.ar.world + r) * 4 + tok) * p.n_rows + row]);
          gemv_store(p, row, tok, v);
        }
      }
      // 4. the last CTA to finish opens the next call (flips the buffer half).
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(&self->local_done, 1u);
        if (prev == static_cast<unsigned int>(grid) - 1u) {
          self->local_done = 0u;
          __threadfence();
          *reinterpret_cast<volatile unsigned long long*>(&self->epoch) = ar_epoch + 1ull;
        }
      }
    }
  }
}

}  // namespace tb
