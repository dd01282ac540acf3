// Several dependent FP8 weight-streaming products in ONE persistent launch.
//
// A decode step is a chain of skinny products, each consuming the previous one's output: launched one by
// one, every product pays a pipeline fill (the first weight block lands ~4 us after kernel entry), a tail
// (split-tile fix-up, slowest SM) and a launch boundary -- 8-10 us per product for streams that last
// 2-40 us.  Here the CTAs of one launch (one per SM, all resident) walk through the products ("phases")
// in order and the weight stream never stops: the producer threads run ahead into the next phase's
// weights as ring slots free up, while the activations of the next phase wait on a grid-wide signal.
//
//   * Signals.  Two counters per phase in global memory: "main" (every CTA has stored the phase's results)
//     and "hook" (every CTA has finished the phase's hook, see below).  A CTA raises a signal with a
//     gpu-scope release after a barrier of its storing threads; waiters poll with gpu-scope acquires,
//     bounded, and set the status word when they give up.  Signals complete in index order, because every
//     CTA goes through the phases in order: waiting for the highest needed index is enough.  The last CTA
//     to leave the kernel clears them, so a captured CUDA graph replays without host help.
//   * Hooks.  The small per-token vector work between the products -- latent RMSNorm into the cache, rotary
//     embeddings, indexer rotations -- runs on the two converter warps of every CTA, beside the epilogue
//     warps' main loop of the phase it is attached to and after that phase's dependencies.  (The two bf16
//     row products of a layer, router gate and indexer head weights, are not hooks: packed as two e4m3 terms
//     per row they are phases of the weight stream like every other product.)
//   * Routing.  A phase whose weight addresses depend on the router (routed experts) lets its producer
//     warps wait for the phase that wrote the scores, route the token themselves and only then compute
//     addresses; the shared expert is a phase of its own with static addresses, so the stream covers the
//     routing latency.
//
// Ring slots, TMEM accumulators, the shared X blocks, the split-tile hand-over and the fused all-reduce
// work as in wstream_gemv_kernel; ring positions simply keep counting across phases.  Every wait is
// bounded; thread-block barriers are executed unconditionally (a failed wait skips work, never a barrier).
#pragma once

#include "attn_prep.cuh"
#include "wstream_gemv.cuh"

namespace tb {

constexpr int kChainMaxPhases = 12;
constexpr int kChainMaxHooks = 3;
constexpr int kChainSignals = 2 * kChainMaxPhases;  // main(ph) = 2 ph, hook(ph) = 2 ph + 1; [kChainSignals] = CTAs that left
constexpr int kChainSigStride = 32;                 // one 128-byte line per counter: they are polled, and lines map to L2 slices

enum ChainHookKind : int {
  HOOK_ATTN_PREP = 2,  // latent norm into the cache + rotary embeddings + indexer rotations
};

struct ChainHook {
  int kind;
  AttnPrepParams prep;  // (its head-weight projection is not used here: that product rides the weight stream)
};

struct ChainPhase {
  GemvParams g;
  int wait_sig;     // signal the activation side of this phase (statistics, conversion, hook, residual) waits for; -1 = none
  int w_sig;        // signal the producers wait for before they route / read slot ids; -1 = none
  int hook;         // index into ChainParams::hooks, -1 = none
  int ar_index;     // all-reduce phases before this one in the launch
  int main_target;  // arrivals that complete the main signal: the grid, + 1 when producer 0 of CTA 0 stores routing results
};

struct ChainParams {
  int n_phases;
  unsigned* signals;         // [kChainSignals + 1] counters, kChainSigStride words apart, zero between launches
  unsigned long long* prof;  // optional trace: [phase][grid <= 256][8] %globaltimer stamps (ChainProfSlot)
  int max_inflight;          // weight blocks a CTA keeps in flight at most (a multiple of 4, <= kGemvStages)
  ChainHook hooks[kChainMaxHooks];
  ChainPhase ph[kChainMaxPhases];
};

enum ChainProfSlot : int {
  kChainProfStart = 0,      // dependencies of the phase met (epilogue warp 0)
  kChainProfStats = 1,      // norm statistics ready
  kChainProfHook = 2,       // hook done (0 when the phase has none)
  kChainProfFixupNs = 3,    // nanoseconds this CTA spent collecting split-tile partial sums as a tile's owner
  kChainProfFixupRounds = 4,  // polling rounds that took
  kChainProfTilesDone = 5,  // tile reductions / split-tile fix-ups done
  kChainProfSignal = 6,     // main signal raised (after the all-reduce, if any)
  kChainProfUnits = 7,      // units of this CTA in the phase
};

constexpr int kChainNormBytes = 2 * kGemvHelperWarps * 4 * 4;  // statistics double-buffered by phase parity
constexpr int kChainHookBytes = (sizeof(ChainHook) * kChainMaxHooks + 15) / 16 * 16;  // the hooks' parameters, copied at entry
constexpr int kChainWlandBytes = kGemvStages * 8;  // one more barrier per slot: the slot's weight block has landed
constexpr int kChainSmemBytes = kGemvSmemBytes + kChainNormBytes + 64 + kChainHookBytes + kChainWlandBytes + 16;

// Units [u0, u1) of phase `p` that CTA `cta` takes.  A phase is spread over grid_eff CTAs starting at cta_base:
// all of them for a long product; for a short one only as many as keep a split row tile to a few CTAs (the
// hand-over of a tile's partial sums costs its owner a round trip through L2 per four guests).  `c` receives
// the CTA's index within the phase (-1: not taking part).
__device__ __forceinline__ void chain_range(const GemvParams& p, int cta, int& u0, int& u1, int& c) {
  const int grid = p.grid_eff;
  c = cta - p.cta_base;
  if (c < 0 || c >= grid) {
    c = -1;
    u0 = u1 = 0;
    return;
  }
  if (p.whole_tiles) {
    u0 = static_cast<int>(gemv_range_begin(p.n_tiles, grid, c)) * p.n_kb;
    u1 = static_cast<int>(gemv_range_begin(p.n_tiles, grid, c + 1)) * p.n_kb;
  } else {
    const long long units = static_cast<long long>(p.n_tiles) * p.n_kb;
    u0 = static_cast<int>(gemv_range_begin(units, grid, c));
    u1 = static_cast<int>(gemv_range_begin(units, grid, c + 1));
  }
}
__device__ __forceinline__ void chain_range(const GemvParams& p, int cta, int& u0, int& u1) {
  int c;
  chain_range(p, cta, u0, u1, c);
}

// Bounded wait for a signal counter to reach `target`.  ONE thread per role and CTA polls (the others meet it
// at a thread-block barrier), and it backs off between polls: every poll of every CTA lands on the L2 slice
// that holds the counter, and a slice saturated with polls delays whatever else maps to it by microseconds.
__device__ __forceinline__ bool sig_wait(const unsigned* sig, unsigned target, const volatile int* abort) {
  // Polls are relaxed loads (served by L2); the acquire that orders what follows is one more load of the
  // counter once it has been seen complete.
  unsigned v;
  bool got = false;
#pragma unroll 1
  for (int i = 0; i < 4 && !got; ++i) {
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(sig) : "memory");
    got = v >= target;
  }
  if (!got) {
    const long long t0 = clock64();
    const long long budget = kWaitBudgetCycles;
    while (!got) {
#pragma unroll 1
      for (int i = 0; i < 64 && !got; ++i) {
        __nanosleep(100);
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(sig) : "memory");
        got = v >= target;
      }
      if (!got && (*abort != 0 || clock64() - t0 > budget)) return false;
    }
  }
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(sig) : "memory");
  return v >= target;
}
// Arrivals that complete signal `sig`: the grid for a hook signal, the phase's main_target for a main signal.
__device__ __forceinline__ unsigned sig_target(const ChainParams& cp, int sig) {
  return (sig & 1) ? gridDim.x : static_cast<unsigned>(cp.ph[sig >> 1].main_target);
}
// One arrival on a signal: everything the calling thread has observed (its own stores, and those of the
// threads it met at a barrier) is visible to whoever acquires the counter afterwards.
__device__ __forceinline__ void sig_raise(unsigned* sig) {
  __threadfence();
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(sig), "r"(1u) : "memory");
}

constexpr int kChainEpiBarrier = 4;   // phase-end barrier of the 256 epilogue threads
constexpr int kChainHookBarrier = 5;  // barriers inside the hooks (same 256 threads)
__device__ __forceinline__ void epi_bar(int id) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(kGemvEpilogueThreads) : "memory");
}

// The per-token vector work of attn_prep_kernel -- latent RMSNorm into the cache, rotary embeddings, indexer
// rotations -- spread over the two auxiliary (converter) warps of every CTA: `aw` = this warp's index among
// them, `n_aw` = their number in the launch.  Everything here is a warp- or thread-level routine with a
// handful of registers; it runs beside the epilogue warps' main loop, off the critical path of the products.
__device__ __noinline__ void chain_aux_attn_prep(const AttnPrepParams& a, int aw, int n_aw) {
  const int lane = threadIdx.x & 31;
  const int n_kv = a.n_tokens, n_iq = a.n_tokens * a.idx_heads, n_ki = a.n_tokens;
  const int n_rope = a.n_tokens * (a.heads + 1) * (a.rope / 2);  // thread-level items
  const int rope_warps = (n_rope + 31) / 32;
  const int n_items = n_kv + n_ki + n_iq + rope_warps;
  // from the far end of the grid: the first CTAs carry the most product units when a phase is short
  for (int it = n_aw - 1 - aw; it < n_items; it += n_aw) {
    int b = it;
    if (b < n_kv) {
      rmsnorm_kv_warp(b, a.kv, a.kv_stride, a.kv_gamma, a.kv_eps, a.kv_dim, a.pos, a.kv_cache, a.n_tokens, a.cache_rows, a.status);
      continue;
    }
    b -= n_kv;
    if (b < n_ki) {
      rotate128_warp(b, a.ki, a.ki_cache, 1, a.rope, a.freqs, a.ln_w, a.ln_b, a.pos, a.n_tokens, a.cache_rows, a.status);
      continue;
    }
    b -= n_ki;
    if (b < n_iq) {
      rotate128_warp(b, a.iq, a.iq_out, a.idx_heads, a.rope, a.freqs, nullptr, nullptr, nullptr, a.n_tokens);
      continue;
    }
    b -= n_iq;
    qkv_rope_thread(b * 32 + lane, a.q_pe, a.heads, a.rope, a.pe_cache, a.pos, a.freqs, a.n_tokens, a.cache_rows, a.status);
  }
}

template <bool PROF>
__global__ void __launch_bounds__(kGemvThreads, 1) wstream_chain_kernel(const __grid_constant__ ChainParams cp) {
  extern __shared__ __align__(128) uint8_t smem[];
  float* merge = reinterpret_cast<float*>(smem + kGemvStages * kGemvSlotStride);  // [2][group threads][8]
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kGemvStages * kGemvSlotStride + kGemvMergeBytes);
  uint64_t* empty = full + kGemvStages;
  uint64_t* acc_full = empty + kGemvStages;
  volatile int* cta_error = reinterpret_cast<volatile int*>(acc_full + kGemvStages);
  volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(const_cast<int*>(cta_error) + 1);
  float* norm_all = reinterpret_cast<float*>(const_cast<int*>(cta_error) + 4);  // [2][helper warps][4 tokens]
  int* route_ids = reinterpret_cast<int*>(norm_all + 2 * kGemvHelperWarps * 4);  // [producer warps][kGemvRouteSlots]
  // The hooks are separate functions that take their parameters by reference: a reference into the kernel's
  // parameter space would make every field a dependent load from memory, so they get a shared-memory copy.
  ChainHook* s_hooks = reinterpret_cast<ChainHook*>(
      (reinterpret_cast<uintptr_t>(route_ids + kGemvProducerWarps * kGemvRouteSlots) + 15) & ~static_cast<uintptr_t>(15));
  // wland[s]: the weight block of slot s has landed.  Kept apart from full[s] (which also waits for the X
  // block) so that the producers can bound the weight bytes they have in flight without waiting for
  // activations: see max_inflight.
  uint64_t* wland = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(s_hooks) + kChainHookBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grid = gridDim.x, cta = blockIdx.x;

  pdl_launch_dependents();
  {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(&cp.hooks[0]);
    uint32_t* dst = reinterpret_cast<uint32_t*>(s_hooks);
    for (int i = threadIdx.x; i < static_cast<int>(sizeof(ChainHook) * kChainMaxHooks / 4); i += kGemvThreads) dst[i] = src[i];
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < kGemvStages; ++s) {
      mbar_init(&full[s], 1);                 // the X block: the converting warp's arrival, or the copy's expect-tx arrival
      mbar_init(&wland[s], 1);                // the weight copy's expect-tx arrival
      mbar_init(&empty[s], kGemvGroupWarps);  // the warps of the epilogue group that read the unit back
      mbar_init(&acc_full[s], 1);             // completion of the unit's MMAs
    }
    *cta_error = 0;
    mbar_fence_init();
  }
  if (warp == kGemvFirstMmaWarp) {
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

  const bool is_epilogue = warp < kGemvEpilogueWarps;
  const bool is_mma = warp >= kGemvFirstMmaWarp && warp < kGemvFirstProducerWarp;
  const bool is_producer = warp >= kGemvFirstProducerWarp && warp < kGemvFirstConverterWarp;
  const GemvParams& p0 = cp.ph[0].g;  // scratch shared by all phases: status word, launch counter, X epoch

  if (is_producer) {
    // ------------------------------------------------------------ producers
    // Ring position gi (counted over all phases of this CTA) is copied by producer gi % 4 into slot
    // gi % kGemvStages.  The first kGemvStages units of a phase get their X blocks from this CTA's converter
    // warps; later units copy them from the launch's shared X blocks once their flags are up.
    const int pw = warp - kGemvFirstProducerWarp;
    int* mine = route_ids + pw * kGemvRouteSlots;
    const uint64_t pol = policy_evict_first();
    int ibase = 0, last_gi = -1, j_mine = 0;  // j_mine: copies this producer has issued so far
    const int depth = cp.max_inflight / kGemvProducerWarps;  // of them in flight at most (a ring's worth: no bound)
    bool failed = false, after_pdl = false;
    unsigned want = 0;
    for (int ph = 0; ph < cp.n_phases; ++ph) {
      const ChainPhase& c = cp.ph[ph];
      const GemvParams& p = c.g;
      int u0, u1;
      chain_range(p, cta, u0, u1);
      const int n = u1 - u0;
      const int* my_nseg_ids = p.nseg_ids;
      const int* my_kseg_ids = p.kseg_ids;
      if (p.nseg_ids != nullptr || p.kseg_ids != nullptr || p.route.scores != nullptr) {
        // addresses depend on earlier results: wait for the predecessor kernel, then for the signal
        if (lane == 0) {
          if (!after_pdl) pdl_wait();
          if (pw == 0 && c.w_sig >= 0 && !failed &&
              !sig_wait(cp.signals + c.w_sig * kChainSigStride, sig_target(cp, c.w_sig), cta_error)) {
            set_status(p0.status, ST_CHAIN_TIMEOUT);
            *cta_error = 1;
          }
        }
        after_pdl = true;
        // producer warp 0 polled for all four (its acquire, then this barrier, order the others' reads)
        if (c.w_sig >= 0) asm volatile("bar.sync 6, %0;" ::"n"(kGemvProducerWarps * 32) : "memory");
        failed = failed || *cta_error != 0;
        failed = __shfl_sync(0xffffffffu, failed ? 1 : 0, 0) != 0;
        if (p.route.scores != nullptr) {
          int my_id = 0;
          float my_w = 0.f;
          if (!failed)
            expert_select_warp(p.route.scores, p.route.bias, p.route.n_experts, p.route.n_groups, p.route.n_limited,
                               p.route.top_k, p.route.route_scale, my_id, my_w);
          if (lane < p.route.top_k) mine[1 + lane] = my_id;
          if (lane == 0) mine[0] = p.route.shared_id;
          if (cta == 0 && pw == 0 && p.route.probs != nullptr) {
            if (!failed)
              expert_select_store(my_id, my_w, p.route.top_k, p.route.shared_id, p.route.probs, p.route.ids,
                                  p.route.slot_ids, p.route.slot_w);
            __syncwarp();
            if (lane == 0) sig_raise(cp.signals + 2 * ph * kChainSigStride);  // the extra arrival of main_target
          }
          __syncwarp();
          if (p.route.for_kseg)
            my_kseg_ids = mine;
          else
            my_nseg_ids = mine + p.route.slot_base;
        }
      }
      if (lane == 0 && !failed && n > 0) {
        auto w_src = [&](int t, int kb) -> const uint8_t* {
          long long eid = 0;
          int tl = t, kbl = kb;
          if (my_nseg_ids != nullptr) {
            eid = my_nseg_ids[t / p.tiles_per_nseg];
            tl = t % p.tiles_per_nseg;
          }
          if (my_kseg_ids != nullptr) {
            eid = my_kseg_ids[kb / p.kb_per_kseg];
            kbl = kb % p.kb_per_kseg;
          }
          return p.w + eid * p.expert_stride + (static_cast<long long>(tl) * p.w_kb_per_tile + kbl) * TB_WBLK_BYTES;
        };
        int j = (pw - (ibase & 3) + 4) & 3;  // first unit of the phase that is this producer's
        int t = (u0 + j) / p.n_kb, kb = (u0 + j) % p.n_kb;
        int s = (ibase + j) % kGemvStages;
        uint32_t ph_empty = (((ibase + j) / kGemvStages) & 1) ^ 1;  // parity of the slot's previous release
        for (; j < n; j += kGemvProducerWarps) {
          const int gi = ibase + j;
          if (gi >= kGemvStages && !mbar_wait(&empty[s], ph_empty, cta_error)) {
            failed = true;
            break;
          }
          // Bound the weight bytes in flight: this producer's copy of `depth` turns ago must have landed.  A
          // ring's worth of outstanding copies per SM is several times what saturates the memory, and all of
          // it queues ahead of every small latency-critical access of the phase transitions.
          if (j_mine >= depth) {
            const int gp = gi - depth * kGemvProducerWarps;
            if (gp >= 0 && !mbar_wait(&wland[gp % kGemvStages], static_cast<uint32_t>(gp / kGemvStages) & 1, cta_error)) {
              failed = true;
              break;
            }
          }
          uint8_t* dst = smem + s * kGemvSlotStride;
          mbar_expect_tx(&wland[s], TB_WBLK_BYTES);
          bulk_g2s_stream(dst, w_src(t, kb), TB_WBLK_BYTES, &wland[s], pol);
          if (j >= kGemvStages) {
            // beyond the phase's first pass the X block is copied from the launch's shared blocks
            mbar_expect_tx(&full[s], TB_XBLK_BYTES);
            if (!after_pdl) {
              pdl_wait();
              after_pdl = true;
            }
            if (want == 0u) want = *reinterpret_cast<const volatile unsigned*>(p0.xstate) + 1u;
            const int xseg = p.tiles_per_xseg > 0 ? t / p.tiles_per_xseg : 0;
            const int xb = xseg * p.n_kb + kb;
            if (!flag_wait(p.xflag + xb, want, cta_error)) {
              failed = true;
              break;
            }
            asm volatile("fence.proxy.async.global;" ::: "memory");
            bulk_g2s(dst + kGemvSlotXOff, p.xs + static_cast<long long>(xb) * TB_XBLK_BYTES, TB_XBLK_BYTES, &full[s]);
          }
          ++j_mine;
          last_gi = gi;
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
          set_status(p0.status, ST_WAIT_EMPTY_TIMEOUT);
          *cta_error = 1;
        }
      }
      failed = __shfl_sync(0xffffffffu, failed ? 1 : 0, 0) != 0;
      ibase += n;
    }
    if (lane == 0) {
      // do not leave while this thread's copies may still be landing in shared memory
      for (int back = 0; back < kGemvStages && last_gi - back >= 0; back += kGemvProducerWarps) {
        const int gi = last_gi - back;
        mbar_wait(&wland[gi % kGemvStages], static_cast<uint32_t>(gi / kGemvStages) & 1, cta_error);
        mbar_wait(&full[gi % kGemvStages], static_cast<uint32_t>(gi / kGemvStages) & 1, cta_error);
      }
    }
  } else if (is_mma) {
    // ------------------------------------------------------------ tensor-core issue
    if (lane == 0) {
      const int mw = warp - kGemvFirstMmaWarp;
      int total = 0;
      for (int ph = 0; ph < cp.n_phases; ++ph) {
        int u0, u1;
        chain_range(cp.ph[ph].g, cta, u0, u1);
        total += u1 - u0;
      }
      const uint32_t smem16 = smem_u32(smem) >> 4;
      const uint64_t desc_a_hi =
          (static_cast<uint64_t>(128 >> 4) << 16) | (static_cast<uint64_t>(256 >> 4) << 32) | (1ull << 46);
      const uint64_t desc_b_hi = (static_cast<uint64_t>(128 >> 4) << 16) | (1ull << 46);
      int s = mw;
      uint32_t ph_full = 0;
      for (int gi = mw; gi < total; gi += kGemvMmaWarps) {
        if (!mbar_wait(&wland[s], ph_full, cta_error) || !mbar_wait(&full[s], ph_full, cta_error)) {
          set_status(p0.status, ST_WAIT_FULL_TIMEOUT);
          *cta_error = 1;
          break;
        }
        tc_fence_after();
        const uint32_t wa = smem16 + static_cast<uint32_t>(s) * (kGemvSlotStride >> 4);
        const uint32_t xa = wa + (kGemvSlotXOff >> 4);
        const uint32_t d = tmem_base + static_cast<uint32_t>(s * kGemvAccCols);
#pragma unroll
        for (int c = 0; c < 4; ++c)
          umma_f8(d, desc_a_hi | (wa + c * (4096 >> 4)), desc_b_hi | (xa + c * (256 >> 4)), c > 0 ? 1u : 0u);
        umma_commit(&acc_full[s]);
        s += kGemvMmaWarps;
        if (s >= kGemvStages) {
          s -= kGemvStages;
          ph_full ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------------------------ epilogue warps (0-7) and converter warps (14-15)
    // Static operands that the phases' prologues read with ordinary loads -- the norm gains -- are pulled
    // into L2 now, before the wait for the predecessor.
    if (is_epilogue) {
      for (int ph = 0; ph < cp.n_phases; ++ph) {
        const GemvParams& p = cp.ph[ph].g;
        if (p.gamma == nullptr) continue;
        const int n_lines = p.n_kb * (TB_KBLOCK * 4 / 128);
        for (int l = cta + static_cast<int>(threadIdx.x) * grid; l < n_lines; l += kGemvEpilogueThreads * grid)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(p.gamma) + l * 128));
      }
    }
    pdl_wait();  // everything below reads or writes activations
    const bool conv = !is_epilogue;
    const int cw = warp - kGemvFirstConverterWarp;
    const int hw = is_epilogue ? warp : cw + kGemvEpilogueWarps;
    const int eg = warp / kGemvGroupWarps, gw = warp % kGemvGroupWarps;
    const unsigned want = *reinterpret_cast<const volatile unsigned*>(p0.xstate) + 1u;
    const uint32_t split_tag = ar_tag(*reinterpret_cast<const volatile unsigned long long*>(p0.launch_calls) / kArUnit);
    const uint32_t lane_base = static_cast<uint32_t>(gw * 32) << 16;
    unsigned long long ar_epoch0 = 0;
    for (int ph = 0; ph < cp.n_phases; ++ph)
      if (cp.ph[ph].g.ar.world > 1) {
        ar_epoch0 = ar_epoch_of(cp.ph[ph].g.ar.state);
        break;
      }
    int ibase = 0, merge_buf = 0;
    bool ok = true;

    for (int ph = 0; ph < cp.n_phases; ++ph) {
      const ChainPhase& c = cp.ph[ph];
      const GemvParams& p = c.g;
      int u0, u1, pc;  // pc: this CTA's index within the phase
      chain_range(p, cta, u0, u1, pc);
      const int n = u1 - u0;
      const long long units = static_cast<long long>(p.n_tiles) * p.n_kb;
      // trace slots of this (phase, CTA); the untraced instantiation carries no trace of it in registers
      unsigned long long* const prof = PROF && warp == 0 && lane == 0 ? cp.prof + (ph * 256 + cta) * 8 : nullptr;

      // ---- dependencies of the activation side ----
      if (c.wait_sig >= 0) {
        // epilogue warp 0 polls for the ten helper warps (its acquire, then the barrier, order their reads)
        if (warp == 0 && lane == 0 && ok &&
            !sig_wait(cp.signals + c.wait_sig * kChainSigStride, sig_target(cp, c.wait_sig), cta_error)) {
          set_status(p0.status, ST_CHAIN_TIMEOUT);
          *cta_error = 1;
        }
        asm volatile("bar.sync 2, %0;" ::"n"(kGemvHelperWarps * 32) : "memory");
        ok = ok && *cta_error == 0;
      }
      if (prof != nullptr) prof[kChainProfStart] = globaltimer_ns();

      // ---- RMSNorm statistics: the ten helper warps split the vector(s) ----
      float* norm_part = norm_all + (ph & 1) * kGemvHelperWarps * 4;
      if (p.gamma != nullptr) {
        const int n_chunks = p.n_kb * (TB_KBLOCK / 4);
        float ss[4] = {0.f, 0.f, 0.f, 0.f};
        constexpr int kBatch = 8;
        if (ok) {
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
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float v = warp_sum(ss[t]);
          if (lane == 0) norm_part[hw * 4 + t] = v;
        }
      }
      // Every phase, with or without statistics: the helper warps stay within one phase of each other, which
      // is what lets the statistics be double-buffered by phase parity.
      asm volatile("bar.sync 2, %0;" ::"n"(kGemvHelperWarps * 32) : "memory");
      float rinv[4];
      gemv_rinv(p, norm_part, rinv);
      if (prof != nullptr) prof[kChainProfStats] = globaltimer_ns();

      // ---- the X blocks of the phase's first pass over the ring, straight into the slots: the ten helper
      // warps take them round-robin (the epilogue warps have nothing to read back before these exist; the
      // slots' previous units were released by these same warps before they got here) ----
      for (int j = hw; j < n && j < kGemvStages && ok; j += kGemvHelperWarps) {
        const int gi = ibase + j;
        const int s = gi % kGemvStages;
        // the slot's previous unit must have been read back before its X block is overwritten
        if (gi >= kGemvStages && !mbar_wait(&empty[s], ((gi / kGemvStages) & 1) ^ 1, cta_error)) {
          set_status(p0.status, ST_WAIT_EMPTY_TIMEOUT);
          *cta_error = 1;
          ok = false;
          break;
        }
        const int u = u0 + j;
        const int t = u / p.n_kb, kb = u % p.n_kb;
        const int xseg = p.tiles_per_xseg > 0 ? t / p.tiles_per_xseg : 0;
        gemv_convert_xblock(p, xseg * p.n_kb + kb, rinv, smem + s * kGemvSlotStride + kGemvSlotXOff, lane);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&full[s]);
      }
      if (conv) {
        // ---- auxiliary work attached to this phase, beside the epilogue warps' main loop ----
        if (c.hook >= 0) {
          if (ok) chain_aux_attn_prep(s_hooks[c.hook].prep, cta * kGemvConverterWarps + cw, grid * kGemvConverterWarps);
          asm volatile("bar.sync 7, %0;" ::"n"(kGemvConverterWarps * 32) : "memory");
          if (cw == 0 && lane == 0) sig_raise(cp.signals + (2 * ph + 1) * kChainSigStride);
        }
        ibase += n;
        continue;
      }

      // ---- epilogue warps: this CTA's share of the launch's shared X blocks ----
      if (p.shared_x && ok && pc >= 0) {
        // (only the CTAs that take units of this phase: the others may still be busy with a phase that runs
        // beside it, and every participant's producers wait for these blocks)
        const int n_xsegs = p.tiles_per_xseg > 0 ? p.n_tiles / p.tiles_per_xseg : 1;
        const int n_xblocks = n_xsegs * p.n_kb;
        for (int xb = pc + warp * p.grid_eff; xb < n_xblocks; xb += kGemvEpilogueWarps * p.grid_eff) {
          gemv_convert_xblock(p, xb, rinv, p.xs + static_cast<long long>(xb) * TB_XBLK_BYTES, lane);
          __syncwarp();
          if (lane == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.xflag + xb), "r"(want) : "memory");
        }
      }

      // ---- main loop: read the accumulators back, scale, reduce per row tile ----
      const unsigned long long ar_epoch = ar_epoch0 + static_cast<unsigned long long>(c.ar_index);
      float out[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) out[q] = 0.f;

      // Partial sums of up to four guest CTAs of a split tile, polled until every word carries this launch's
      // tag (bounded), added to `acc` in CTA order.  Guests first .. first + cnt - 1 (phase-local indices).
      auto gather_guests = [&](int first, int cnt, float (&acc)[8], unsigned& rounds) {
        if (cnt <= 0) return;
        const unsigned long long* part = reinterpret_cast<const unsigned long long*>(p.partial);
        const long long t0 = clock64();
        const long long budget = kWaitBudgetCycles;
        constexpr int kBatch = 4;
        unsigned long long w[kBatch][8];
        unsigned pending = (1u << cnt) - 1u;
        while (pending != 0u && ok) {
#pragma unroll
          for (int g = 0; g < kBatch; ++g) {
            if ((pending >> g) & 1u) {
              // word j of lane l sits at [j][l]: the 32 lanes of one load read 256 contiguous bytes
              const unsigned long long* src = part + static_cast<long long>((first + g) * 4 + gw) * 256 + lane;
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
          pending = __reduce_or_sync(0xffffffffu, pending);  // the warp moves on together
          if (PROF) ++rounds;
          if (pending != 0u && (*cta_error != 0 || clock64() - t0 > budget)) {
            set_status(p0.status, ST_SPLIT_TIMEOUT);
            *cta_error = 1;
            ok = false;
          }
        }
        if (!ok) return;
#pragma unroll
        for (int g = 0; g < kBatch; ++g) {
          if (g < cnt) {
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += __uint_as_float(static_cast<uint32_t>(w[g][j]));
          }
        }
      };

      // End of a row tile (every epilogue warp gets here for every tile, on every path; all conditions below
      // are uniform over the CTA, so every barrier is met by all 256 threads).  Group 1 hands its sums to
      // group 0.  A whole tile is finished by group 0.  A tile whose k blocks are spread over several CTAs
      // belongs to the CTA that holds its first unit; every other CTA of the tile (a "guest") leaves its
      // partial sums in its own slot as 64-bit words tagged with the launch number (a tagged word IS the
      // arrival of its value), and the owner -- which reaches the tile at the very end of its range -- picks
      // them up eight guests per round, four by each epilogue group at the same time, in a fixed order:
      // own + (guests 1-4 one after the other) + (guests 5-8 summed among themselves), and so on.
      auto finish_tile = [&](int t) {
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
        }
        const int tile_u0 = t * p.n_kb, tile_u1 = tile_u0 + p.n_kb;
        if (u0 <= tile_u0 && u1 >= tile_u1) {
          if (eg == 0 && ok) gemv_epilogue_row(p, t, gw, lane, out, ar_epoch);
        } else if (u0 > tile_u0) {
          if (eg == 0) {
            unsigned long long* dst = reinterpret_cast<unsigned long long*>(p.partial) +
                                      static_cast<long long>(pc * 4 + gw) * 256 + lane;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const unsigned long long word = (static_cast<unsigned long long>(split_tag) << 32) | __float_as_uint(out[j]);
              asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(dst + j * 32), "l"(word) : "memory");
            }
          }
        } else {
          const int c_last = gemv_owner(tile_u1 - 1, units, p.grid_eff);
          const unsigned long long fix0 = PROF ? globaltimer_ns() : 0ull;
          unsigned fix_rounds = 0;
          for (int first = pc + 1; first <= c_last; first += 2 * 4) {
            const int mine = first + eg * 4;
            const int cnt = c_last - mine + 1 < 4 ? c_last - mine + 1 : 4;
            float* mb2 = merge + (merge_buf * kGemvGroupThreads + gw * 32 + lane) * 8;
            // group 0 adds its guests onto its own sums one after the other; group 1 sums its guests from zero
            float gs[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) gs[j] = eg == 0 ? out[j] : 0.f;
            gather_guests(mine, cnt, gs, fix_rounds);
            if (eg == 0) {
#pragma unroll
              for (int j = 0; j < 8; ++j) out[j] = gs[j];
            } else {
              *reinterpret_cast<float4*>(mb2) = make_float4(gs[0], gs[1], gs[2], gs[3]);
              *reinterpret_cast<float4*>(mb2 + 4) = make_float4(gs[4], gs[5], gs[6], gs[7]);
            }
            asm volatile("bar.sync 3, %0;" ::"n"(kGemvEpilogueThreads) : "memory");
            merge_buf ^= 1;
            if (eg == 0 && c_last >= first + 4) {
              const float4 m0 = *reinterpret_cast<const float4*>(mb2);
              const float4 m1 = *reinterpret_cast<const float4*>(mb2 + 4);
              out[0] += m0.x; out[1] += m0.y; out[2] += m0.z; out[3] += m0.w;
              out[4] += m1.x; out[5] += m1.y; out[6] += m1.z; out[7] += m1.w;
            }
          }
          ok = ok && *cta_error == 0;
          if (PROF && prof != nullptr) {
            prof[kChainProfFixupNs] += globaltimer_ns() - fix0;  // time this CTA spent collecting split-tile partial sums
            prof[kChainProfFixupRounds] += fix_rounds;           // polling rounds of epilogue warp 0
          }
          if (eg == 0 && ok) gemv_epilogue_row(p, t, gw, lane, out, ar_epoch);
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) out[q] = 0.f;
      };

      int kb = n > 0 ? u0 % p.n_kb : 0, t = n > 0 ? u0 / p.n_kb : 0;
      int s = ibase % kGemvStages;
      uint32_t phs = (ibase / kGemvStages) & 1;
      for (int j = 0; j < n; ++j, ++kb) {
        if (kb == p.n_kb) {
          kb = 0;
          ++t;
        }
        if (((ibase + j) & 1) == eg && ok) {
          if (!__all_sync(0xffffffffu, mbar_wait(&acc_full[s], phs, cta_error))) {
            set_status(p0.status, ST_WAIT_FULL_TIMEOUT);
            *cta_error = 1;
            ok = false;
          } else {
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
            out[0] = fmaf(__uint_as_float(dr[0]), ws * cs0.x, out[0]);
            out[1] = fmaf(__uint_as_float(dr[1]), ws * cs0.y, out[1]);
            out[2] = fmaf(__uint_as_float(dr[2]), ws * cs0.z, out[2]);
            out[3] = fmaf(__uint_as_float(dr[3]), ws * cs0.w, out[3]);
            out[4] = fmaf(__uint_as_float(dr[4]), ws * cs1.x, out[4]);
            out[5] = fmaf(__uint_as_float(dr[5]), ws * cs1.y, out[5]);
            out[6] = fmaf(__uint_as_float(dr[6]), ws * cs1.z, out[6]);
            out[7] = fmaf(__uint_as_float(dr[7]), ws * cs1.w, out[7]);
          }
        }
        if (++s == kGemvStages) {
          s = 0;
          phs ^= 1u;
        }
        if (kb == p.n_kb - 1 || j == n - 1) {
          finish_tile(t);
        }
      }
      if (prof != nullptr) {
        prof[kChainProfTilesDone] = globaltimer_ns();
        prof[kChainProfUnits] = static_cast<unsigned long long>(n);
      }

      if (p.ar.world > 1) {
        // ---- one-shot all-reduce over peer memory (group 0), as in wstream_gemv_kernel ----
        if (threadIdx.x == 0)
          asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(&p.ar.state->calls), "l"(ar_share(cta, grid)) : "memory");
        if (eg == 0) {
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
                set_status(p0.status, ST_PEER_TIMEOUT);
                *cta_error = 1;
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
          if (!alive) ok = false;
        }
      }

      // ---- the phase's results of this CTA are stored: raise its main signal ----
      ok = ok && *cta_error == 0;
      epi_bar(kChainEpiBarrier);
      if (threadIdx.x == 0) sig_raise(cp.signals + 2 * ph * kChainSigStride);
      if (prof != nullptr) prof[kChainProfSignal] = globaltimer_ns();
      ibase += n;
    }
    if (threadIdx.x == 0)
      asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(p0.launch_calls), "l"(ar_share(cta, grid)) : "memory");
  }

  // ---- common tail: every warp arrives here on every path; then the tensor memory is returned ----
  tc_fence_before();
  __syncthreads();
  if (warp == kGemvFirstMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kGemvTmemCols)
                 : "memory");
  }
  if (threadIdx.x == 0) {
    // The last CTA to leave clears the signals and opens the next epoch of the shared X blocks: by then
    // every CTA has passed every wait of this launch.
    __threadfence();
    const unsigned prev = atomicAdd(cp.signals + kChainSignals * kChainSigStride, 1u);
    if (prev == static_cast<unsigned>(grid) - 1u) {
      for (int i = 0; i <= kChainSignals; ++i) cp.signals[i * kChainSigStride] = 0u;
      *reinterpret_cast<volatile unsigned*>(p0.xstate) = *reinterpret_cast<const volatile unsigned*>(p0.xstate) + 1u;
      __threadfence();
    }
  }
}

}  // namespace tb
