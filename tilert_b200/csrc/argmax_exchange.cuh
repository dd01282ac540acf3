// Greedy token over a vocabulary that is split across ranks: every rank finds the arg-max of its
// own slice of the f32 logits, pushes the (value, global index) pair into every rank's receive
// slot with plain peer stores, and picks the best pair once all ranks have arrived -- the same
// one-shot exchange (receive-buffer halves, words tagged with the call number, bounded wait) as the all-reduce fused
// into the streaming products (wstream_gemv.cuh), so it takes its place in the same call sequence.
// Ties go to the lowest index, on one rank and between ranks.
#pragma once
#include "wstream_gemv.cuh"

namespace tb {

constexpr int kArgmaxThreads = 1024;

struct ArgmaxParams {
  const float* logits;     // [tokens][stride]: this rank's slice
  long long stride;
  int n_local;             // entries of the slice
  int index_offset;        // global index of entry 0
  int n_tokens;            // 1..4
  int slot_rows;           // row stride of the receive slots (the communicator's max_rows)
  long long* token_out;    // [tokens]
  float* value_out;        // [tokens] or nullptr: the winning logit
  int* status;
  AllReduce ar;
};

__device__ __forceinline__ bool argmax_better(float v, int i, float bv, int bi) {
  return v > bv || (v == bv && i < bi);
}

__global__ void __launch_bounds__(kArgmaxThreads, 1) argmax_exchange_kernel(const __grid_constant__ ArgmaxParams p) {
  __shared__ float s_val[kArgmaxThreads / 32];
  __shared__ int s_idx[kArgmaxThreads / 32];
  __shared__ float s_best_val[4];
  __shared__ int s_best_idx[4];
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int t = 0; t < p.n_tokens; ++t) {
    const float* row = p.logits + t * p.stride;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < p.n_local; i += kArgmaxThreads) {
      const float v = row[i];
      if (argmax_better(v, i, bv, bi)) {
        bv = v;
        bi = i;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (argmax_better(ov, oi, bv, bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      s_val[warp] = bv;
      s_idx[warp] = bi;
    }
    __syncthreads();
    if (warp == 0) {
      bv = s_val[lane];
      bi = s_idx[lane];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (argmax_better(ov, oi, bv, bi)) {
          bv = ov;
          bi = oi;
        }
      }
      if (lane == 0) {
        s_best_val[t] = bv;
        s_best_idx[t] = bi == 0x7fffffff ? 0x7fffffff : bi + p.index_offset;
      }
    }
    __syncthreads();
  }
  if (p.ar.world <= 1) {
    if (threadIdx.x < p.n_tokens) {
      p.token_out[threadIdx.x] = s_best_idx[threadIdx.x];
      if (p.value_out != nullptr) p.value_out[threadIdx.x] = s_best_val[threadIdx.x];
    }
    return;
  }
  // ---- exchange: slot of rank r, token t = words 0 (value) and 1 (index bits) of [half][r][t][slot_rows],
  //      each tagged with the call number like the all-reduce's partial sums ----
  if (threadIdx.x == 0) {
    const unsigned long long epoch = ar_epoch_of(p.ar.state);
    const uint32_t tag = ar_tag(epoch);
    const long long half = static_cast<long long>(epoch & 1ull);
    for (int t = 0; t < p.n_tokens; ++t) {
      const long long idx = ((half * p.ar.world + p.ar.rank) * 4 + t) * p.slot_rows;
      for (int pr = 0; pr < p.ar.world; ++pr) {
        ar_push(&p.ar.recv[pr][idx], tag, s_best_val[t]);
        ar_push(&p.ar.recv[pr][idx + 1], tag, __int_as_float(s_best_idx[t]));
      }
    }
    asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(&p.ar.state->calls), "l"(kArUnit) : "memory");
    const unsigned long long* mine = p.ar.recv[p.ar.rank];
    const long long t0 = clock64();
    const long long budget = kWaitBudgetCycles;
    for (int t = 0; t < p.n_tokens; ++t) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int r = 0; r < p.ar.world; ++r) {
        const long long idx = ((half * p.ar.world + r) * 4 + t) * p.slot_rows;
        unsigned long long wv, wi;
        for (;;) {
          wv = ar_peek(&mine[idx]);
          wi = ar_peek(&mine[idx + 1]);
          if (static_cast<uint32_t>(wv >> 32) == tag && static_cast<uint32_t>(wi >> 32) == tag) break;
          if (clock64() - t0 > budget) {
            set_status(p.status, ST_PEER_TIMEOUT);
            return;
          }
        }
        const float v = __uint_as_float(static_cast<uint32_t>(wv));
        const int i = static_cast<int>(static_cast<uint32_t>(wi));
        if (argmax_better(v, i, bv, bi)) {
          bv = v;
          bi = i;
        }
      }
      p.token_out[t] = bi;
      if (p.value_out != nullptr) p.value_out[t] = bv;
    }
  }
}

}  // namespace tb
