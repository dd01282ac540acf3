// FP8 weight-streaming skinny GEMM for batch-1 decode (1..8 activation columns).
//
//   out[t, n] = sum_k  W[n, k] * x[t, k]          W: e4m3, 128x128 block scales
//                                                  x: e4m3 columns with per-128 scales
//
// HBM-bound: every weight byte is read exactly once.  One persistent CTA per SM walks a
// contiguous range of (row tile, k block) units (stream-K).  A producer thread stages each
// unit -- one 16448-byte W block and one 1056-byte X block -- into a shared-memory ring with
// bulk async copies (TMA) that complete on mbarriers.  The tensor-core work of a unit is four
// tcgen05.mma (M = 128 weight rows x N = 16 x K = 32, e4m3 operands read straight from the slot
// through shared-memory descriptors; 8 real activation columns) into the TMEM accumulator that
// belongs to the slot.  Epilogue warps (one thread per weight row) read each accumulator back with
// tcgen05.ld and apply (weight scale x column scale) in f32 registers once per k block.
//
// Every role is a serial loop whose per-unit latency (a barrier wait alone is ~100 cycles) would
// otherwise pace the stream at well under the memory rate, so every role is spread over several
// warps that take units round-robin: 4 producer threads, 2 MMA-issuing threads, 2 groups of 4
// epilogue warps, 2 converter warps.  The two epilogue groups merge their sums through shared
// memory at the end of a row tile.  Row tiles that straddle two CTAs are finished by the last
// arriver, which adds the partials in CTA order, so the result does not depend on timing.
#pragma once

#include "common.cuh"
#include "elementwise.cuh"
#include "formats.h"

namespace tb {

enum Epilogue : int {
  EPI_STORE = 0,     // out = acc (+ residual)
  EPI_SILU_MUL = 1,  // rows g / g+8 of each 16-row group are (gate, up): out = silu(gate) * up
  EPI_ADD_PAIR = 2,  // rows g / g+8 of each 16-row group are the two e4m3 terms of one bf16 weight row: out = sum
};

struct OutRegion {
  int row_begin;             // first packed row of the region
  int row_end;               // one past the last packed row
  int dtype;                 // 0 = bf16, 1 = f32
  void* ptr;                 // destination of token 0, row row_begin
  long long token_stride;    // elements between tokens
  const int* pos_ptr;        // optional device int: destination starts at token index *pos_ptr
  int pos_rows;              // with pos_ptr: rows of the destination (0 = unchecked); a row past them is not stored
  int tok_div;               // > 0: the region is cut into slots of slot_rows rows and slot j keeps only token j / tok_div
  int slot_rows;
};

// All-reduce endpoint of one rank.  A partial sum travels as one 64-bit word {call number, f32 bits}
// written with a single store, so a word that carries the current call number IS the arrival of its
// value: no fence, no counter and no second trip over the link between the data and a flag (a
// naturally aligned 64-bit access is single-copy atomic).  The receive buffer has two halves used
// by alternate calls: a rank can only start call n+2 after every rank has pushed call n+1, which a
// rank does after it has finished reading call n, so a half is never overwritten while it is read.
// The call number is device-resident -- every CTA of a launch adds its share of kArUnit to `calls`
// after it has read it -- so nothing on the host changes between calls and a captured CUDA graph
// can be replayed.
struct AllReduceState {
  unsigned long long calls;  // local only: kArUnit per completed exchange of this rank
};
constexpr unsigned long long kArUnit = 1ull << 20;

struct AllReduce {
  int world;                      // 1 = off
  int rank;
  unsigned long long* recv[8];    // recv[p]: rank p's receive buffer [2 halves][world][4 tokens][n_rows] words
  AllReduceState* state;          // this rank's state (local memory)
};

// Completed exchanges on this endpoint.  When a launch starts (its predecessor has completed) every
// earlier call is whole, and no CTA of this launch can complete the current one before all of them
// have read the counter (each adds its share only afterwards).
__device__ __forceinline__ unsigned long long ar_epoch_of(const AllReduceState* self) {
  return *reinterpret_cast<const volatile unsigned long long*>(&self->calls) / kArUnit;
}
__device__ __forceinline__ uint32_t ar_tag(unsigned long long epoch) {
  return static_cast<uint32_t>(epoch) + 1u;  // never the zero the buffers start with (wraps after 2^32 calls)
}
__device__ __forceinline__ void ar_push(unsigned long long* dst, uint32_t tag, float v) {
  const unsigned long long word = (static_cast<unsigned long long>(tag) << 32) | __float_as_uint(v);
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(word) : "memory");
}
__device__ __forceinline__ unsigned long long ar_peek(const unsigned long long* src) {
  unsigned long long word;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(word) : "l"(src) : "memory");
  return word;
}
// Share of kArUnit that CTA `cta` of `grid` adds to the call counter.
__device__ __forceinline__ unsigned long long ar_share(int cta, int grid) {
  const unsigned long long share = kArUnit / static_cast<unsigned long long>(grid);
  return cta < grid - 1 ? share : kArUnit - share * static_cast<unsigned long long>(grid - 1);
}

// Where the activations of a launch come from.
enum XMode : int {
  X_PACKED = 0,  // X blocks prepared beforehand in global memory (bulk-copied with the weights)
  X_BF16 = 1,    // bf16 vectors in global memory; the kernel normalises them (optional RMSNorm),
                 // splits them into two e4m3 terms and writes the X block of each stage itself
};

// Expert routing done inside the product launch (single-token launches): every producer warp routes
// the token itself from the router scores, so the weight addresses need no separate routing launch;
// CTA 0 also stores the result for the caller and for the down projection that follows.
struct RouteParams {
  const float* scores;  // [n_experts] router logits; nullptr = off (slot ids come from GemvParams::nseg_ids)
  const float* bias;
  int n_experts, n_groups, n_limited, top_k;
  float route_scale;
  int shared_id;        // slot 0: the shared expert's index in the packed expert array
  int slot_base;        // first slot of the list (shared expert, selected experts...) this launch's row segments use
  int for_kseg;         // 1: the slot list indexes the K segments (down projection) instead of the row segments
  float* probs;         // [top_k]
  int* ids;             // [top_k]
  int* slot_ids;        // [top_k + 1]
  float* slot_w;        // [top_k + 1]
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
  uint8_t* xs;                   // X_BF16 scratch: the launch's X blocks [x segments * n_kb], written by all CTAs
  unsigned* xflag;               // X_BF16 scratch: per X block, the launch epoch + 1 once the block is written
  unsigned* xstate;              // X_BF16 scratch: {epoch = completed X_BF16 launches, CTAs done}, self-maintained
  int n_tiles;
  int n_kb;
  const int* nseg_ids;
  RouteParams route;
  int tiles_per_nseg;
  const int* kseg_ids;
  int kb_per_kseg;
  long long expert_stride;
  int w_kb_per_tile;
  int tiles_per_xseg;
  int n_tokens;
  int whole_tiles;       // 1: CTAs take whole row tiles (set by the host when that balances well enough)
  int shared_x;          // X_BF16: 1 when some CTA has more units than ring slots, so the CTAs share the conversion
  int grid_eff;          // chained launches: CTAs that take units of this phase; the rest idle through it
  int cta_base;          // chained launches: first of those CTAs (a short phase sits at the far end of the grid)
  int only_token;        // >= 0: store only this token's results (per-token expert lists)
  int cols_per_token;
  int epi;
  int n_rows;
  int n_regions;
  OutRegion regions[TB_MAX_REGIONS];
  const __nv_bfloat16* residual;  // optional [tokens, n_rows]
  long long residual_stride;
  float* partial;   // scratch: [grid][4 warps][32 lanes][8] 64-bit words {launch number, f32 partial sum}
  unsigned long long* launch_calls;  // scratch: kArUnit per completed launch that used `partial` (self-maintained)
  int* status;
  unsigned long long* prof;  // optional trace: [grid][16] (see GemvProfSlot)
  unsigned stagger_ns;       // pause between one producer's copies of the first pass over the ring (0 = none)
  AllReduce ar;
};

// Trace slots written per CTA when GemvParams::prof is set (the role of the reference's
// profile_logs tensors, tilert/utils.py:18-45): nanoseconds of %globaltimer.
enum GemvProfSlot : int {
  kGemvProfEntry = 0,         // kernel entry
  kGemvProfReady = 1,         // barriers initialised
  kGemvProfFirstData = 2,     // epilogue warp 0: the accumulator of the CTA's first unit is complete
  kGemvProfLastUnit = 3,      // epilogue warp 0: the CTA's last unit is read back
  kGemvProfTilesDone = 4,     // epilogue warp 0: all its tile reductions / epilogues are done
  kGemvProfFirstConvert = 5,  // converter 0: first X block written
  kGemvProfIssued = 6,        // producer 0: all its copies issued
  kGemvProfExit = 7,          // epilogue warp 0: end of kernel (after the all-reduce, if any)
  kGemvProfWaitCycles = 8,    // epilogue warp 0: SM cycles spent waiting for accumulators, summed over its units
  kGemvProfMathCycles = 9,    // epilogue warp 0: SM cycles spent reading back and scaling, summed over its units
  kGemvProfUnits = 10,        // epilogue warp 0: number of units it read back (low 32 bits) and the SM it ran on (high 32)
  kGemvProfMmaWaitFull = 11,  // MMA warp 0: cycles waiting for its slots to fill
  kGemvProfMmaIssue = 12,     // MMA warp 0: cycles issuing MMAs and their commit
  kGemvProfNormDone = 13,     // converter 0: RMSNorm statistics of the activations are ready (%globaltimer)
  kGemvProfProdWait = 14,     // producer 0: cycles waiting for free slots
  kGemvProfConvCycles = 15,   // converter 0: cycles converting (excluding waits)
};
__device__ __forceinline__ void gemv_stamp(const GemvParams& p, int slot) {
  if (p.prof != nullptr) p.prof[blockIdx.x * 16 + slot] = globaltimer_ns();
}

// Per-unit timeline of CTA 0 (SM cycle counter), rows 148.. of the trace (free when the grid has at
// most 148 CTAs): event e of unit i in [kGemvTimelineFirst, +16) goes to
// prof[(148 + e) * 16 + i - kGemvTimelineFirst].  Events: 0 producer saw the slot free, 1 copy issued,
// 3 MMA thread saw the slot full, 4 MMAs committed, 7 epilogue reached the unit, 5 epilogue saw the
// accumulator, 6 epilogue released the slot.
#ifndef TB_TIMELINE_FIRST
#define TB_TIMELINE_FIRST 96
#endif
constexpr int kGemvTimelineFirst = TB_TIMELINE_FIRST;
__device__ __forceinline__ void gemv_timeline(const GemvParams& p, int ev, int i) {
  if (p.prof != nullptr && blockIdx.x == 0 && gridDim.x <= 148 && i >= kGemvTimelineFirst && i < kGemvTimelineFirst + 16)
    p.prof[(148 + ev) * 16 + i - kGemvTimelineFirst] = static_cast<unsigned long long>(clock64());
}

constexpr int kGemvStages = 12;         // ring slots; a multiple of every role's warp count
constexpr int kGemvAccCols = 16;        // TMEM columns per accumulator: N = 16 is the smallest N at M = 128
constexpr int kGemvTmemCols = 256;      // one accumulator per slot; a power of two >= kGemvStages * kGemvAccCols
constexpr int kGemvEpilogueGroups = 2;  // unit i is read back by group i % 2
constexpr int kGemvGroupWarps = 4;      // warps 4g .. 4g+3: TMEM lanes 32(w%4) .. +31 = weight rows of the tile
constexpr int kGemvEpilogueWarps = kGemvEpilogueGroups * kGemvGroupWarps;  // warps 0-7
constexpr int kGemvMmaWarps = 2;        // warps 8-9: one issuing thread each; unit i is issued by MMA warp i % 2
constexpr int kGemvProducerWarps = 4;   // warps 10-13: one issuing thread each; unit i is copied by producer i % 4
constexpr int kGemvConverterWarps = 2;  // warps 14-15: unit i is converted by converter i % 2 (X_BF16 only)
constexpr int kGemvGroupThreads = kGemvGroupWarps * 32;
constexpr int kGemvEpilogueThreads = kGemvEpilogueWarps * 32;
constexpr int kGemvFirstMmaWarp = kGemvEpilogueWarps;
constexpr int kGemvFirstProducerWarp = kGemvFirstMmaWarp + kGemvMmaWarps;
constexpr int kGemvFirstConverterWarp = kGemvFirstProducerWarp + kGemvProducerWarps;
constexpr int kGemvHelperWarps = kGemvEpilogueWarps + kGemvConverterWarps;  // warps that share the norm prologue
constexpr int kGemvThreads = (kGemvFirstConverterWarp + kGemvConverterWarps) * 32;
static_assert(kGemvStages % kGemvProducerWarps == 0 && kGemvStages % kGemvMmaWarps == 0 &&
                  kGemvStages % kGemvEpilogueGroups == 0 && kGemvStages % kGemvConverterWarps == 0,
              "a slot must always be served by the same warp of each role");
static_assert(kGemvStages * kGemvAccCols <= kGemvTmemCols, "one accumulator per slot");
// Ring slot: W block at offset 0, X block at kGemvSlotXOff; both start on a 128-byte line of shared memory
constexpr int kGemvSlotXOff = 16512;
constexpr int kGemvSlotStride = 17664;
constexpr int kGemvBarBytes = 3 * kGemvStages * 8;
constexpr int kGemvMergeBytes = 2 * kGemvGroupThreads * 8 * 4;  // double-buffered sums of epilogue group 1
constexpr int kGemvRouteSlots = 32;  // slot ids per producer warp (top_k + 1 <= 32)
constexpr int kGemvSmemBytes = kGemvStages * kGemvSlotStride + kGemvMergeBytes + kGemvBarBytes + 16 +
                               kGemvHelperWarps * 4 * 4 + kGemvProducerWarps * kGemvRouteSlots * 4 + 32;

// ---- tcgen05 helpers ----
// Shared-memory operand descriptor, K-major, no swizzle: 8-row x 16-byte core matrices; `lbo` =
// bytes between the two core matrices along K, `sbo` = bytes between 8-row groups.
__device__ __forceinline__ uint64_t umma_desc(const void* smem_ptr, uint32_t lbo, uint32_t sbo) {
  return static_cast<uint64_t>((smem_u32(smem_ptr) >> 4) & 0x3fffu) | (static_cast<uint64_t>(lbo >> 4) << 16) |
         (static_cast<uint64_t>(sbo >> 4) << 32) | (1ull << 46);
}
// Instruction descriptor: D = f32, A = B = e4m3, both K-major, N = 16, M = 128.  Only 8 activation
// columns exist: the B descriptor's 8-column group stride is 0, so columns 8-15 repeat columns 0-7
// and are never read back.
constexpr uint32_t kUmmaIdesc = (1u << 4) | (2u << 17) | (8u << 24);
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kUmmaIdesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Issue / completion halves of the same load, so that other work can overlap its latency.  The
// registers must not be read before tmem_ld_wait.
__device__ __forceinline__ void tmem_ld8_issue(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[8]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7])
               :
               : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&d)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) d[i] = __uint_as_float(r[i]);
}

// Bounded wait for a flag in global memory to reach `want` (set with st.release.gpu by another CTA).
__device__ __forceinline__ bool flag_wait(const unsigned* flag, unsigned want, const volatile int* abort) {
  unsigned v;
#pragma unroll 1
  for (int i = 0; i < 16; ++i) {
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v == want) return true;
  }
  const long long t0 = clock64();
  const long long budget = kWaitBudgetCycles;
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      __nanosleep(64);
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if (v == want) return true;
    }
    if (*abort != 0 || clock64() - t0 > budget) return false;
  }
}

// Equal shares: CTA c owns units [begin(c), begin(c+1)), begin(c) = floor(units * c / grid).  Written
// with 32-bit operations only (units < 2^30, grid <= 256): a 64-bit division is a long subroutine,
// and these run at the two moments of a launch when nothing else hides them -- its first and its
// last microsecond.  floor((q g + r) c / g) = q c + floor(r c / g).
__device__ __forceinline__ long long gemv_range_begin(long long units, int grid, int cta) {
  const unsigned u = static_cast<unsigned>(units), g = static_cast<unsigned>(grid), c = static_cast<unsigned>(cta);
  const unsigned q = u / g, r = u - q * g;
  return static_cast<long long>(q * c + (r * c) / g);
}
// The CTA whose range holds `unit`: a float estimate, corrected with the exact range bounds.
__device__ __forceinline__ int gemv_owner(long long unit, long long units, int grid) {
  int c = static_cast<int>((static_cast<float>(unit) + 0.5f) * __fdividef(static_cast<float>(grid), static_cast<float>(units)));
  c = c < 0 ? 0 : (c > grid - 1 ? grid - 1 : c);
  while (c > 0 && gemv_range_begin(units, grid, c) > unit) --c;
  while (c < grid - 1 && gemv_range_begin(units, grid, c + 1) <= unit) ++c;
  return c;
}

__device__ __forceinline__ void gemv_store(const GemvParams& p, int row, int token, float v) {
  if (row >= p.n_rows || token >= p.n_tokens) return;
  if (p.only_token >= 0 && token != p.only_token) return;
  if (p.residual != nullptr) v += bf2f(p.residual[token * p.residual_stride + row]);
#pragma unroll
  for (int i = 0; i < TB_MAX_REGIONS; ++i) {
    if (i < p.n_regions && row >= p.regions[i].row_begin && row < p.regions[i].row_end) {
      const OutRegion& r = p.regions[i];
      if (r.tok_div > 0 && token != ((row - r.row_begin) / r.slot_rows) / r.tok_div) continue;
      long long tok = token;
      if (r.pos_ptr != nullptr) {
        tok += *r.pos_ptr;
        if (r.pos_rows > 0 && (tok < 0 || tok >= r.pos_rows)) {
          set_status(p.status, ST_BAD_ARGUMENT);
          continue;
        }
      }
      const long long off = tok * r.token_stride + (row - r.row_begin);
      if (r.dtype == 0)
        reinterpret_cast<__nv_bfloat16*>(r.ptr)[off] = f2bf(v);
      else
        reinterpret_cast<float*>(r.ptr)[off] = v;
    }
  }
}

// Final values of one weight row (8 accumulator columns) of row tile `tile`; the calling warp holds
// rows 32*warp .. 32*warp+31 of the tile, one per lane.
__device__ __forceinline__ void gemv_epilogue_row(const GemvParams& p, int tile, int warp, int lane,
                                                  const float (&v)[8], unsigned long long ar_epoch) {
  const int row_in_tile = warp * 32 + lane;
  float val[8];
  int ntok;
  if (p.cols_per_token == 2) {
    ntok = 4;
#pragma unroll
    for (int t = 0; t < 4; ++t) val[t] = v[2 * t] + v[2 * t + 1];
  } else {
    ntok = 8;
#pragma unroll
    for (int t = 0; t < 8; ++t) val[t] = v[t];
  }
  if (p.epi == EPI_SILU_MUL || p.epi == EPI_ADD_PAIR) {
    // every 16 packed rows are 8 gate rows followed by their 8 up rows (or 8 leading-term rows followed by
    // their 8 residual-term rows): lane l (bit 3 clear) pairs with l + 8
    const int n16 = (tile * TB_TILE_ROWS + row_in_tile) >> 4;
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      if (t < ntok) {
        const float up = __shfl_xor_sync(0xffffffffu, val[t], 8);
        if ((lane & 8) == 0) {
          const float gate = val[t];
          gemv_store(p, n16 * 8 + (lane & 7), t,
                     p.epi == EPI_SILU_MUL ? __fdividef(gate, 1.0f + __expf(-gate)) * up : gate + up);
        }
      }
    }
    return;
  }
  const int row = tile * TB_TILE_ROWS + row_in_tile;
  if (p.ar.world > 1) {
    // push this rank's partial into every rank's receive slot (plain peer stores)
    if (row < p.n_rows) {
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        if (t < ntok && t < p.n_tokens) {
          const long long idx = ((static_cast<long long>(ar_epoch & 1ull) * p.ar.world + p.ar.rank) * 4 + t) * p.n_rows + row;
          for (int pr = 0; pr < p.ar.world; ++pr) ar_push(&p.ar.recv[pr][idx], ar_tag(ar_epoch), val[t]);
        }
      }
    }
    return;
  }
#pragma unroll
  for (int t = 0; t < 8; ++t)
    if (t < ntok) gemv_store(p, row, t, val[t]);
}

// 1 / rms of each token's activation vector from the per-warp partial sums of squares (1 without a gain).
__device__ __forceinline__ void gemv_rinv(const GemvParams& p, const float* norm_part, float (&rinv)[4]) {
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    rinv[t] = 1.f;
    if (p.gamma != nullptr) {
      float tot = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < kGemvHelperWarps; ++w2) tot += norm_part[w2 * 4 + t];
      rinv[t] = rsqrtf(__fdividef(tot, static_cast<float>(p.n_kb * TB_KBLOCK)) + p.eps);
    }
  }
}

// Converts X block `xb` (x segment xb / n_kb, k block xb % n_kb) of the launch's bf16 activations
// into packed form at `blk` (shared or global memory): per token two e4m3 terms with power-of-two
// scales, so the scaling is a multiplication and the residual x - hi*s is exact.  One warp.
__device__ __forceinline__ void gemv_convert_xblock(const GemvParams& p, int xb, const float (&rinv)[4], uint8_t* blk,
                                                    int lane) {
  const int ntok = p.n_tokens;
  const int kb = xb % p.n_kb;
  const long long off = static_cast<long long>(xb) * TB_KBLOCK + lane * 4;  // x segments are contiguous
  uint2 raw[4];
#pragma unroll
  for (int tk = 0; tk < 4; ++tk)
    raw[tk] = tk < ntok ? *reinterpret_cast<const uint2*>(p.xb + tk * p.xb_stride + off) : make_uint2(0u, 0u);
  const float4 g = p.gamma != nullptr ? *reinterpret_cast<const float4*>(p.gamma + kb * TB_KBLOCK + lane * 4)
                                      : make_float4(1.f, 1.f, 1.f, 1.f);
  const float g4[4] = {g.x, g.y, g.z, g.w};
  const int c = lane >> 3, r = (lane >> 2) & 1, q4 = lane & 3;
#pragma unroll
  for (int tk = 0; tk < 4; ++tk) {
    uint32_t whi = 0u, wlo = 0u;
    float2 sc = make_float2(0.f, 0.f);
    if (tk < ntok) {
      const uint2 rw = raw[tk];
      float x4[4] = {__uint_as_float(rw.x << 16), __uint_as_float(rw.x & 0xffff0000u), __uint_as_float(rw.y << 16),
                     __uint_as_float(rw.y & 0xffff0000u)};
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
      whi = static_cast<uint32_t>(h01) | (static_cast<uint32_t>(h23) << 16);
      wlo = static_cast<uint32_t>(l01) | (static_cast<uint32_t>(l23) << 16);
      float mlt = 1.f;
      if (lane == 0 && p.seg_scale != nullptr) mlt = p.seg_scale[tk * (p.n_kb / p.kb_per_kseg) + kb / p.kb_per_kseg];
      sc = make_float2(s_hi * mlt, s_lo * mlt);
    }
    // columns of absent tokens are written as zeros: the block is read whole by the tensor core
    *reinterpret_cast<uint32_t*>(blk + c * 256 + r * 128 + (2 * tk) * 16 + q4 * 4) = whi;
    *reinterpret_cast<uint32_t*>(blk + c * 256 + r * 128 + (2 * tk + 1) * 16 + q4 * 4) = wlo;
    if (lane == 0) *reinterpret_cast<float2*>(blk + TB_XBLK_DATA + 8 * tk) = sc;
  }
}

__global__ void __launch_bounds__(kGemvThreads, 1) wstream_gemv_kernel(const __grid_constant__ GemvParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  float* merge = reinterpret_cast<float*>(smem + kGemvStages * kGemvSlotStride);  // [2][group threads][8]
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kGemvStages * kGemvSlotStride + kGemvMergeBytes);
  uint64_t* empty = full + kGemvStages;
  uint64_t* acc_full = empty + kGemvStages;
  volatile int* cta_error = reinterpret_cast<volatile int*>(acc_full + kGemvStages);
  volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(const_cast<int*>(cta_error) + 1);
  float* norm_part = reinterpret_cast<float*>(const_cast<int*>(cta_error) + 4);  // [helper warps][4 tokens]
  int* route_ids = reinterpret_cast<int*>(norm_part + kGemvHelperWarps * 4);    // [producer warps][kGemvRouteSlots]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grid = gridDim.x, cta = blockIdx.x;
  const long long units = static_cast<long long>(p.n_tiles) * p.n_kb;
  // unit indices fit 32 bits (checked on the host); all per-stage index arithmetic is 32-bit --
  // 64-bit divisions in these loops cost more than the stage's data movement
  // Ranges: equal shares of units (row tiles may then be split between CTAs and need a fix-up
  // through global memory), or, when the host found that whole row tiles balance well enough,
  // equal shares of tiles (no tile is ever split).
  const int u0 = p.whole_tiles ? static_cast<int>(gemv_range_begin(p.n_tiles, grid, cta)) * p.n_kb
                               : static_cast<int>(gemv_range_begin(units, grid, cta));
  const int u1 = p.whole_tiles ? static_cast<int>(gemv_range_begin(p.n_tiles, grid, cta + 1)) * p.n_kb
                               : static_cast<int>(gemv_range_begin(units, grid, cta + 1));

  // The successor may start right away.  Weight prefetch does not depend on the predecessor, so only
  // threads that read activations / routing ids / residuals or write results wait for it (below).
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    gemv_stamp(p, kGemvProfEntry);
    for (int s = 0; s < kGemvStages; ++s) {
      mbar_init(&full[s], p.x_mode == X_BF16 ? 2 : 1);  // producer (+ converter, or a second producer arrival)
      mbar_init(&empty[s], kGemvGroupWarps);            // the warps of the epilogue group that read the unit back
      mbar_init(&acc_full[s], 1);                       // completion of the unit's MMAs
    }
    *cta_error = 0;
    mbar_fence_init();
  }
  if (warp == kGemvFirstMmaWarp) {
    // tensor memory: one accumulator per ring slot (the whole warp executes the allocation)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(const_cast<uint32_t*>(tmem_base_slot))),
                 "r"(kGemvTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  if (threadIdx.x == 0) gemv_stamp(p, kGemvProfReady);

  const bool is_epilogue = warp < kGemvEpilogueWarps;
  const bool is_mma = warp >= kGemvFirstMmaWarp && warp < kGemvFirstProducerWarp;
  const bool is_producer = warp >= kGemvFirstProducerWarp && warp < kGemvFirstConverterWarp;
  const bool is_converter = warp >= kGemvFirstConverterWarp;
  if (is_converter && p.x_mode == X_BF16 && p.gamma != nullptr) {
    // the norm gain is a weight: pull it into L2 now, so that the conversions that follow the
    // statistics do not start with a DRAM round trip
    const int n_lines = p.n_kb * (TB_KBLOCK * 4 / 128);
    for (int l = (warp - kGemvFirstConverterWarp) * 32 + lane; l < n_lines; l += kGemvConverterWarps * 32)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(p.gamma) + l * 128));
  }
  // Producers stream weights, which no kernel of the step writes; they wait for the predecessor only
  // when their addresses depend on it (routing ids) or when they also copy packed activations.
  if (!is_producer || p.x_mode == X_PACKED || p.nseg_ids != nullptr || p.kseg_ids != nullptr ||
      p.route.scores != nullptr)
    pdl_wait();

  if (p.x_mode == X_BF16 && p.gamma != nullptr && (is_epilogue || is_converter)) {
    // RMSNorm statistics of the activation vector(s): the epilogue and converter warps split the
    // vector (the producers are already filling the ring), partial sums meet in shared memory.
    const int hw = is_epilogue ? warp : warp - kGemvFirstConverterWarp + kGemvEpilogueWarps;
    const int n_chunks = p.n_kb * (TB_KBLOCK / 4);  // 8-byte chunks per token
    float ss[4] = {0.f, 0.f, 0.f, 0.f};
    // batches of independent loads: the whole vector is a few dependent-latency round trips otherwise
    constexpr int kBatch = 8;
    for (int ch0 = hw * 32 + lane; ch0 < n_chunks; ch0 += kBatch * kGemvHelperWarps * 32) {
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        if (t < p.n_tokens) {
          uint2 raw[kBatch];
#pragma unroll
          for (int j = 0; j < kBatch; ++j) {
            const int ch = ch0 + j * kGemvHelperWarps * 32;
            raw[j] = ch < n_chunks ? *reinterpret_cast<const uint2*>(p.xb + t * p.xb_stride + ch * 4) : make_uint2(0u, 0u);
          }
#pragma unroll
          for (int j = 0; j < kBatch; ++j) {
            const float a0 = __uint_as_float(raw[j].x << 16), a1 = __uint_as_float(raw[j].x & 0xffff0000u);
            const float a2 = __uint_as_float(raw[j].y << 16), a3 = __uint_as_float(raw[j].y & 0xffff0000u);
            ss[t] += a0 * a0 + a1 * a1 + a2 * a2 + a3 * a3;
          }
        }
      }
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float v = warp_sum(ss[t]);
      if (lane == 0) norm_part[hw * 4 + t] = v;
    }
    asm volatile("bar.sync 2, %0;" ::"n"(kGemvHelperWarps * 32) : "memory");
    if (warp == kGemvFirstConverterWarp && lane == 0) gemv_stamp(p, kGemvProfNormDone);
  }

  if (is_producer) {
    // ------------------------------------------------------------ producers
    // One issuing thread per warp; unit i of the CTA's range is copied by producer i % 4 into ring
    // slot i % kGemvStages: the W block from the weight tensor and the X block either from the
    // caller's packed activations (X_PACKED) or from the launch's shared X blocks (X_BF16), which
    // the converter warps of all CTAs are writing meanwhile -- a per-block flag says when.
    const int* my_nseg_ids = p.nseg_ids;
    if (p.route.scores != nullptr) {
      // route the token with the whole warp; keep the slot list where this warp's issuing lane reads it
      int my_id;
      float my_w;
      expert_select_warp(p.route.scores, p.route.bias, p.route.n_experts, p.route.n_groups, p.route.n_limited,
                         p.route.top_k, p.route.route_scale, my_id, my_w);
      int* mine = route_ids + (warp - kGemvFirstProducerWarp) * kGemvRouteSlots;
      if (lane < p.route.top_k) mine[1 + lane] = my_id;
      if (lane == 0) mine[0] = p.route.shared_id;
      if (cta == 0 && warp == kGemvFirstProducerWarp)
        expert_select_store(my_id, my_w, p.route.top_k, p.route.shared_id, p.route.probs, p.route.ids,
                            p.route.slot_ids, p.route.slot_w);
      __syncwarp();
      my_nseg_ids = mine;
    }
    if (lane == 0) {
      const int pw = warp - kGemvFirstProducerWarp;
      const uint64_t pol = policy_evict_first();
      const bool shared_x = p.x_mode == X_BF16;
      int last_i = -1;
      long long pw_wait = 0;
      bool failed = false;

      auto w_src = [&](int t, int kb) -> const uint8_t* {
        long long eid = 0;
        int tl = t, kbl = kb;
        if (my_nseg_ids != nullptr) {
          eid = my_nseg_ids[t / p.tiles_per_nseg];
          tl = t % p.tiles_per_nseg;
        }
        if (p.kseg_ids != nullptr) {
          eid = p.kseg_ids[kb / p.kb_per_kseg];
          kbl = kb % p.kb_per_kseg;
        }
        return p.w + eid * p.expert_stride + (static_cast<long long>(tl) * p.w_kb_per_tile + kbl) * TB_WBLK_BYTES;
      };
      auto x_block = [&](int t, int kb) -> int {
        const int xseg = p.tiles_per_xseg > 0 ? t / p.tiles_per_xseg : 0;
        return xseg * p.n_kb + kb;
      };
      // X block of a unit from the shared blocks: wait (bounded) for its flag, then copy.
      auto x_from_shared = [&](int s, int xb, unsigned want) -> bool {
        if (!flag_wait(p.xflag + xb, want, cta_error)) return false;
        // the block was written with ordinary stores by another CTA and is read by the copy engine:
        // order the flag's acquire before the async-proxy read of global memory
        asm volatile("fence.proxy.async.global;" ::: "memory");
        bulk_g2s(smem + s * kGemvSlotStride + kGemvSlotXOff, p.xs + static_cast<long long>(xb) * TB_XBLK_BYTES,
                 TB_XBLK_BYTES, &full[s]);
        return true;
      };

      int u = u0 + pw;
      unsigned want = 0;
      if (shared_x) {
        // The first pass over the ring: weights only, which need nothing from the predecessor (the
        // converter warps write these units' X blocks into the slots).  Only then wait for the
        // predecessor; later units take their X blocks from the launch's shared blocks.
        for (; u < u1 && u - u0 < kGemvStages; u += kGemvProducerWarps) {
          const int s = u - u0;
          // A pause between a producer's copies of the first pass: the launch ramps up instead of putting a full
          // ring per CTA in flight at once while the predecessor's last CTAs are still streaming.
          if (s >= kGemvProducerWarps && p.stagger_ns > 0) __nanosleep(p.stagger_ns);
          mbar_expect_tx(&full[s], TB_WBLK_BYTES);
          bulk_g2s_stream(smem + s * kGemvSlotStride, w_src(u / p.n_kb, u % p.n_kb), TB_WBLK_BYTES, &full[s], pol);
          gemv_timeline(p, 1, s);
          last_i = s;
        }
        pdl_wait();
        want = *reinterpret_cast<const volatile unsigned*>(p.xstate) + 1u;
      }
      int t = u < u1 ? u / p.n_kb : 0, kb = u < u1 ? u % p.n_kb : 0;
      int s = (u - u0) % kGemvStages;
      uint32_t ph_empty = (((u - u0) / kGemvStages) & 1) ^ 1;  // parity of the previous use's release
      for (; u < u1 && !failed; u += kGemvProducerWarps) {
        const int i = u - u0;
        const long long w0 = p.prof != nullptr ? clock64() : 0;
        if (i >= kGemvStages && !mbar_wait(&empty[s], ph_empty, cta_error)) {
          failed = true;
          break;
        }
        if (p.prof != nullptr) pw_wait += clock64() - w0;
        gemv_timeline(p, 0, i);
        uint8_t* dst = smem + s * kGemvSlotStride;
        mbar_expect_tx(&full[s], TB_WBLK_BYTES + TB_XBLK_BYTES);
        bulk_g2s_stream(dst, w_src(t, kb), TB_WBLK_BYTES, &full[s], pol);
        if (shared_x) {
          mbar_arrive(&full[s]);  // stands in for the converter's arrival of the first pass
          if (!x_from_shared(s, x_block(t, kb), want)) {
            failed = true;
            break;
          }
        } else {
          bulk_g2s(dst + kGemvSlotXOff, p.x + static_cast<long long>(x_block(t, kb)) * TB_XBLK_BYTES, TB_XBLK_BYTES,
                   &full[s]);
        }
        gemv_timeline(p, 1, i);
        last_i = i;
        kb += kGemvProducerWarps;
        while (kb >= p.n_kb) {
          kb -= p.n_kb;
          ++t;
        }
        s += kGemvProducerWarps;
        if (s >= kGemvStages) {
          s -= kGemvStages;
          ph_empty ^= 1u;
        }
      }
      if (failed) {
        set_status(p.status, ST_WAIT_EMPTY_TIMEOUT);
        *cta_error = 1;
      }
      if (shared_x) {
        // This producer reads no more X flags.  The last producer of the launch to say so opens the
        // next epoch, which makes every flag of this launch stale.
        const unsigned prev = atomicAdd(p.xstate + 1, 1u);
        if (prev == static_cast<unsigned>(grid * kGemvProducerWarps) - 1u) {
          p.xstate[1] = 0u;
          __threadfence();
          *reinterpret_cast<volatile unsigned*>(p.xstate) = want;
        }
      }
      if (pw == 0) {
        gemv_stamp(p, kGemvProfIssued);
        if (p.prof != nullptr) p.prof[blockIdx.x * 16 + kGemvProfProdWait] = pw_wait;
      }
      // Do not leave the CTA while this thread's copies may still be landing in its shared memory:
      // wait (bounded) for the last use it issued into each of its ring slots.  On the normal path
      // these have completed already, because the MMA-issuing threads waited on the same phases.  (After a
      // failed flag wait a slot may be short of its X block; that wait then runs into the abort flag.)
      for (int back = 0; back < kGemvStages && last_i - back >= 0; back += kGemvProducerWarps) {
        const int i = last_i - back;
        mbar_wait(&full[i % kGemvStages], static_cast<uint32_t>(i / kGemvStages) & 1, cta_error);
      }
    }
  } else if (is_converter) {
    // ------------------------------------------------- activation converters (X_BF16 only)
    // The X blocks of a launch are the same for every CTA, so the CTAs share the conversion (the
    // epilogue warps do this CTA's share before their loop; producers copy the shared blocks into
    // the ring once their flags are up).  That round trip through global memory takes several
    // microseconds, so the units of the first pass over the ring get their X blocks converted here,
    // straight into the slots, by the two converter warps taking alternate units.
    const int cw = warp - kGemvFirstConverterWarp;  // 0 or 1
    if (p.x_mode == X_BF16) {
      float rinv[4];
      gemv_rinv(p, norm_part, rinv);
      for (int u = u0 + cw; u < u1 && u - u0 < kGemvStages; u += kGemvConverterWarps) {
        const int s = u - u0;
        const int t = u / p.n_kb, kb = u % p.n_kb;
        const int xseg = p.tiles_per_xseg > 0 ? t / p.tiles_per_xseg : 0;
        gemv_convert_xblock(p, xseg * p.n_kb + kb, rinv, smem + s * kGemvSlotStride + kGemvSlotXOff, lane);
        // written through the generic proxy, read by the tensor core (async proxy)
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&full[s]);
          if (u == u0) gemv_stamp(p, kGemvProfFirstConvert);
        }
      }
    }
  } else if (is_mma) {
    // ------------------------------------------------------------ tensor-core issue
    // One thread per warp; unit i is issued by MMA warp i % 2.  Per unit: wait for the slot (weights
    // landed, X block written), issue four K = 32 MMAs into the slot's accumulator, and let the
    // hardware signal their completion.  The accumulator is free whenever the slot is full: the
    // epilogue released the slot only after reading the accumulator of the slot's previous unit.
    if (lane == 0) {
      const int mw = warp - kGemvFirstMmaWarp;
      // descriptors differ only in their 14-bit start-address field (16-byte units): one add per operand
      const uint32_t smem16 = smem_u32(smem) >> 4;
      const uint64_t desc_a_hi =
          (static_cast<uint64_t>(128 >> 4) << 16) | (static_cast<uint64_t>(256 >> 4) << 32) | (1ull << 46);
      const uint64_t desc_b_hi = (static_cast<uint64_t>(128 >> 4) << 16) | (1ull << 46);
      int s = mw;
      uint32_t ph_full = 0;
      long long pf_full = 0, pf_issue = 0;
      for (int u = u0 + mw; u < u1; u += kGemvMmaWarps) {
        const long long m0 = p.prof != nullptr ? clock64() : 0;
        if (!mbar_wait(&full[s], ph_full, cta_error)) {
          set_status(p.status, ST_WAIT_FULL_TIMEOUT);
          *cta_error = 1;
          break;
        }
        const long long m1 = p.prof != nullptr ? clock64() : 0;
        gemv_timeline(p, 3, u - u0);
        tc_fence_after();
        const uint32_t wa = smem16 + static_cast<uint32_t>(s) * (kGemvSlotStride >> 4);
        const uint32_t xa = wa + (kGemvSlotXOff >> 4);
        const uint32_t d = tmem_base + static_cast<uint32_t>(s * kGemvAccCols);
#pragma unroll
        for (int c = 0; c < 4; ++c)
          umma_f8(d, desc_a_hi | (wa + c * (4096 >> 4)), desc_b_hi | (xa + c * (256 >> 4)), c > 0 ? 1u : 0u);
        umma_commit(&acc_full[s]);
        gemv_timeline(p, 4, u - u0);
        if (p.prof != nullptr) {
          pf_full += m1 - m0;
          pf_issue += clock64() - m1;
        }
        s += kGemvMmaWarps;
        if (s >= kGemvStages) {
          s -= kGemvStages;
          ph_full ^= 1u;
        }
      }
      if (mw == 0 && p.prof != nullptr) {
        p.prof[blockIdx.x * 16 + kGemvProfMmaWaitFull] = pf_full;
        p.prof[blockIdx.x * 16 + kGemvProfMmaIssue] = pf_issue;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps
    // Two groups of four warps; unit i is read back by group i % 2.  Thread (warp w, lane l) owns
    // weight row 32(w%4) + l of the current row tile: eight f32 sums, one per activation column,
    // over its group's units.  Per unit it waits for the MMAs, reads the accumulator from TMEM and
    // its row's scale and the column scales from the slot, releases the slot, and adds
    // scale * accumulator.  At the end of a row tile group 1 hands its sums to group 0 through
    // shared memory; group 0 finishes the tile.
    const int eg = warp / kGemvGroupWarps, gw = warp % kGemvGroupWarps;
    unsigned long long ar_epoch = 0;
    if (p.ar.world > 1) ar_epoch = ar_epoch_of(p.ar.state);
    // tag of this launch's split-tile partial sums (same scheme as the all-reduce's call number: every
    // CTA adds its share to the counter at its end, after having read it here)
    const uint32_t split_tag =
        ar_tag(*reinterpret_cast<const volatile unsigned long long*>(p.launch_calls) / kArUnit);
    const uint32_t lane_base = static_cast<uint32_t>(gw * 32) << 16;
    if (p.x_mode == X_BF16 && p.shared_x) {
      // (Skipped when no CTA has more units than ring slots: the converter warps cover those.)
      // This CTA's share of the launch's X blocks, while the ring fills: block c, c + grid, ...,
      // spread over the eight epilogue warps; each block's flag is raised behind its stores.
      const unsigned want = *reinterpret_cast<const volatile unsigned*>(p.xstate) + 1u;
      const int n_xsegs = p.tiles_per_xseg > 0 ? p.n_tiles / p.tiles_per_xseg : 1;
      const int n_xblocks = n_xsegs * p.n_kb;
      float rinv[4];
      gemv_rinv(p, norm_part, rinv);
      for (int xb = cta + warp * grid; xb < n_xblocks; xb += kGemvEpilogueWarps * grid) {
        gemv_convert_xblock(p, xb, rinv, p.xs + static_cast<long long>(xb) * TB_XBLK_BYTES, lane);
        // ordinary stores that the copy engines of other CTAs will read: the readers fence between
        // their acquire of the flag and their copy, the writer only has to release
        __syncwarp();
        if (lane == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.xflag + xb), "r"(want) : "memory");
      }
    }
    float out[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) out[c] = 0.f;
    bool ok = true;
    long long prof_wait = 0, prof_math = 0, prof_units = 0;
    int merge_buf = 0;

    // A tile whose k blocks are spread over several CTAs (group 0 only).  The CTA that holds the tile's
    // first unit owns it; every other CTA of the tile leaves its partial sums in its own slot as 64-bit
    // words tagged with the launch number (a tagged word IS the arrival of its value: no fence, no
    // counter), and the owner, which reaches the tile at the very end of its range, picks them up in
    // CTA order -- so the result does not depend on timing -- and finishes the tile.  A CTA is a guest
    // of at most one tile (the one its range starts inside), hence one slot per CTA.
    auto split_tile = [&](int t, const float (&v)[8]) {
      const int tile_u0 = t * p.n_kb, tile_u1 = tile_u0 + p.n_kb;
      unsigned long long* part = reinterpret_cast<unsigned long long*>(p.partial);
      if (u0 > tile_u0) {
        // word j of lane l sits at [j][l]: the 32 lanes of one store (and of the owner's load) cover 256
        // contiguous bytes instead of 32 separate sectors
        unsigned long long* dst = part + static_cast<long long>(cta * 4 + gw) * 256 + lane;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const unsigned long long word = (static_cast<unsigned long long>(split_tag) << 32) | __float_as_uint(v[j]);
          asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(dst + j * 32), "l"(word) : "memory");
        }
        return;
      }
      const int c_last = gemv_owner(tile_u1 - 1, units, grid);
      float sum[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) sum[j] = v[j];
      const long long t0 = clock64();
      const long long budget = kWaitBudgetCycles;
      constexpr int kBatch = 4;  // guests read per round: independent loads, one L2 round trip
      for (int cb = cta + 1; cb <= c_last && ok; cb += kBatch) {
        unsigned long long w[kBatch][8];
        unsigned pending = 0;
#pragma unroll
        for (int g = 0; g < kBatch; ++g)
          if (cb + g <= c_last) pending |= 1u << g;
        while (pending != 0u) {
#pragma unroll
          for (int g = 0; g < kBatch; ++g) {
            if ((pending >> g) & 1u) {
              const unsigned long long* src = part + static_cast<long long>((cb + g) * 4 + gw) * 256 + lane;
#pragma unroll
              for (int j = 0; j < 8; ++j)
                asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w[g][j]) : "l"(src + j * 32) : "memory");
            }
          }
#pragma unroll
          for (int g = 0; g < kBatch; ++g) {
            if ((pending >> g) & 1u) {
              bool all = true;
#pragma unroll
              for (int j = 0; j < 8; ++j) all = all && static_cast<uint32_t>(w[g][j] >> 32) == split_tag;
              if (all) pending &= ~(1u << g);
            }
          }
          // the warp moves on together (tcgen05.ld later needs all its lanes)
          pending = __reduce_or_sync(0xffffffffu, pending);
          if (pending != 0u && (*cta_error != 0 || clock64() - t0 > budget)) {
            set_status(p.status, ST_SPLIT_TIMEOUT);
            *cta_error = 1;
            ok = false;
            break;
          }
        }
        if (!ok) break;
        // Guests are added in rounds of eight: the first four onto the running sum one after the other,
        // the next four summed among themselves first (the chained kernel gathers those two halves with
        // its two epilogue groups at the same time; the grouping is kept the same here so that both
        // kernels give the same bits).
        const bool second_half = ((cb - (cta + 1)) & 4) != 0;
        float half[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) half[j] = 0.f;
#pragma unroll
        for (int g = 0; g < kBatch; ++g) {
          if (cb + g <= c_last) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float v2 = __uint_as_float(static_cast<uint32_t>(w[g][j]));
              if (second_half) half[j] += v2; else sum[j] += v2;
            }
          }
        }
        if (second_half) {
#pragma unroll
          for (int j = 0; j < 8; ++j) sum[j] += half[j];
        }
      }
      if (ok) gemv_epilogue_row(p, t, gw, lane, sum, ar_epoch);
    };

    auto finish_tile = [&](int t) {
      // ---- merge the two groups' sums (every epilogue warp gets here for every tile, on every path) ----
      float* mb = merge + (merge_buf * kGemvGroupThreads + gw * 32 + lane) * 8;
      if (eg == 1) {
        *reinterpret_cast<float4*>(mb) = make_float4(out[0], out[1], out[2], out[3]);
        *reinterpret_cast<float4*>(mb + 4) = make_float4(out[4], out[5], out[6], out[7]);
      }
      asm volatile("bar.sync 3, %0;" ::"n"(kGemvEpilogueThreads) : "memory");
      merge_buf ^= 1;
      if (eg == 0) {
        const float4 m0 = *reinterpret_cast<const float4*>(mb);
        const float4 m1 = *reinterpret_cast<const float4*>(mb + 4);
        out[0] += m0.x; out[1] += m0.y; out[2] += m0.z; out[3] += m0.w;
        out[4] += m1.x; out[5] += m1.y; out[6] += m1.z; out[7] += m1.w;
        const int tile_u0 = t * p.n_kb, tile_u1 = tile_u0 + p.n_kb;
        if (u0 <= tile_u0 && u1 >= tile_u1) {
          gemv_epilogue_row(p, t, gw, lane, out, ar_epoch);
        } else {
          split_tile(t, out);
        }
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) out[c] = 0.f;
    };

    int kb = u0 < u1 ? u0 % p.n_kb : 0, t = u0 < u1 ? u0 / p.n_kb : 0;
    int s = 0;
    uint32_t ph = 0;
    for (int u = u0; u < u1; ++u, ++kb) {
      if (kb == p.n_kb) {
        kb = 0;
        ++t;
      }
      // every decision below is warp-uniform: tcgen05.ld needs the whole warp
      if (((u - u0) & 1) == eg && ok) {
        const long long c0 = p.prof != nullptr ? clock64() : 0;
        if (gw == 0 && lane == 0) gemv_timeline(p, 7, u - u0);
        // acc_full[s] completes after the unit's MMAs, which were issued after full[s] completed:
        // the slot's scales are in shared memory by then.
        if (!__all_sync(0xffffffffu, mbar_wait(&acc_full[s], ph, cta_error))) {
          set_status(p.status, ST_WAIT_FULL_TIMEOUT);
          *cta_error = 1;
          ok = false;
        } else {
          const long long c1 = p.prof != nullptr ? clock64() : 0;
          if (u == u0 && warp == 0 && lane == 0) gemv_stamp(p, kGemvProfFirstData);
          if (gw == 0 && lane == 0) gemv_timeline(p, 5, u - u0);
          tc_fence_after();
          uint32_t dr[8];
          tmem_ld8_issue(tmem_base + lane_base + static_cast<uint32_t>(s * kGemvAccCols), dr);
          const uint8_t* sw = smem + s * kGemvSlotStride;
          const float ws = *reinterpret_cast<const float*>(sw + TB_WBLK_DATA + ((gw * 32 + lane) >> 3) * 4);
          const float4 cs0 = *reinterpret_cast<const float4*>(sw + kGemvSlotXOff + TB_XBLK_DATA);
          const float4 cs1 = *reinterpret_cast<const float4*>(sw + kGemvSlotXOff + TB_XBLK_DATA + 16);
          tmem_ld_wait(dr);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&empty[s]);
          if (gw == 0 && lane == 0) gemv_timeline(p, 6, u - u0);
          out[0] = fmaf(__uint_as_float(dr[0]), ws * cs0.x, out[0]);
          out[1] = fmaf(__uint_as_float(dr[1]), ws * cs0.y, out[1]);
          out[2] = fmaf(__uint_as_float(dr[2]), ws * cs0.z, out[2]);
          out[3] = fmaf(__uint_as_float(dr[3]), ws * cs0.w, out[3]);
          out[4] = fmaf(__uint_as_float(dr[4]), ws * cs1.x, out[4]);
          out[5] = fmaf(__uint_as_float(dr[5]), ws * cs1.y, out[5]);
          out[6] = fmaf(__uint_as_float(dr[6]), ws * cs1.z, out[6]);
          out[7] = fmaf(__uint_as_float(dr[7]), ws * cs1.w, out[7]);
          if (p.prof != nullptr) {
            prof_wait += c1 - c0;
            prof_math += clock64() - c1;
            ++prof_units;
          }
        }
      }
      if (++s == kGemvStages) {
        s = 0;
        ph ^= 1u;
      }
      if (kb == p.n_kb - 1 || u == u1 - 1) {
        if (u == u1 - 1 && warp == 0 && lane == 0) gemv_stamp(p, kGemvProfLastUnit);
        finish_tile(t);
      }
    }
    if (warp == 0 && lane == 0) {
      gemv_stamp(p, kGemvProfTilesDone);
      if (p.prof != nullptr) {
        p.prof[blockIdx.x * 16 + kGemvProfWaitCycles] = prof_wait;
        p.prof[blockIdx.x * 16 + kGemvProfMathCycles] = prof_math;
        p.prof[blockIdx.x * 16 + kGemvProfUnits] = static_cast<unsigned long long>(prof_units) | (static_cast<unsigned long long>(sm_id()) << 32);
      }
    }

    if (threadIdx.x == 0)
      asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(p.launch_calls), "l"(ar_share(cta, grid)) : "memory");

    if (p.ar.world > 1 && eg == 0) {
      // ---- one-shot all-reduce over peer memory, fused behind the streaming loop (group 0) ----
      // This CTA's partials are on their way (every word carries the call number).  Count the CTA
      // towards the call -- a local add, nothing waits on it -- then sum, in rank order, the words of
      // this CTA's share of rows as they arrive, add the residual and store.
      if (threadIdx.x == 0)
        asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(&p.ar.state->calls), "l"(ar_share(cta, grid)) : "memory");
      const unsigned long long* mine = p.ar.recv[p.ar.rank];
      const uint32_t tag = ar_tag(ar_epoch);
      const long long half_base = static_cast<long long>(ar_epoch & 1ull) * p.ar.world;
      const int total = p.n_tokens * p.n_rows;
      const int e0 = static_cast<int>(static_cast<long long>(total) * cta / grid);
      const int e1 = static_cast<int>(static_cast<long long>(total) * (cta + 1) / grid);
      const long long t0 = clock64();
      const long long budget = kWaitBudgetCycles;
      bool alive = ok && !*cta_error;
      for (int e = e0 + static_cast<int>(threadIdx.x); e < e1 && alive; e += kGemvGroupThreads) {
        const int tok = e / p.n_rows, row = e % p.n_rows;
        float v = 0.f;
        unsigned pending = (1u << p.ar.world) - 1u;
        float part[8];
        while (pending != 0u) {
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            if (r < p.ar.world && (pending >> r) & 1u) {
              const unsigned long long word = ar_peek(&mine[((half_base + r) * 4 + tok) * p.n_rows + row]);
              if (static_cast<uint32_t>(word >> 32) == tag) {
                part[r] = __uint_as_float(static_cast<uint32_t>(word));
                pending &= ~(1u << r);
              }
            }
          }
          if (pending != 0u && clock64() - t0 > budget) {
            set_status(p.status, ST_PEER_TIMEOUT);
            alive = false;
            break;
          }
        }
        if (!alive) break;
#pragma unroll
        for (int r = 0; r < 8; ++r)
          if (r < p.ar.world) v += part[r];
        gemv_store(p, row, tok, v);
      }
    }
    if (warp == 0 && lane == 0) gemv_stamp(p, kGemvProfExit);
  }

  // ---- common tail: every warp arrives here on every path; then the tensor memory is returned ----
  tc_fence_before();
  __syncthreads();
  if (warp == kGemvFirstMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kGemvTmemCols)
                 : "memory");
  }
}

}  // namespace tb
