// out = all_reduce(partial) + residual over the communicator's peer buffers, as a launch of its own: the role of the
// reference's padded_allreduce_add_op (tilert/models/deepseek_v3_2/ops/padded_allreduce_add.py:17-41).  Same exchange
// as the all-reduce fused into the streaming products (wstream_gemv.cuh): every rank writes each of its values as one
// 64-bit word {call number, f32 bits} into every rank's receive slot, then sums, in rank order, the words of its own
// slots as they arrive (bounded wait, status word on time-out).  It counts as one call of the communicator's sequence.
#pragma once

#include "wstream_gemv.cuh"

namespace tb {

struct ArAddParams {
  const __nv_bfloat16* partial;   // [n_tokens, n_rows] this rank's addend
  const __nv_bfloat16* residual;  // [n_tokens, n_rows] added once after the reduction, or null
  __nv_bfloat16* out;             // [n_tokens, n_rows]
  int n_tokens, n_rows;
  AllReduce ar;
  int* status;
};

constexpr int kArAddThreads = 256;

__global__ void __launch_bounds__(kArAddThreads) allreduce_add_kernel(const __grid_constant__ ArAddParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int total = p.n_tokens * p.n_rows;
  const int cta = blockIdx.x, grid = gridDim.x;
  const int e0 = static_cast<int>(static_cast<long long>(total) * cta / grid);
  const int e1 = static_cast<int>(static_cast<long long>(total) * (cta + 1) / grid);
  if (p.ar.world <= 1) {
    for (int e = e0 + static_cast<int>(threadIdx.x); e < e1; e += kArAddThreads) {
      float v = bf2f(p.partial[e]);
      if (p.residual != nullptr) v += bf2f(p.residual[e]);
      p.out[e] = f2bf(v);
    }
    return;
  }
  const unsigned long long epoch = ar_epoch_of(p.ar.state);
  const uint32_t tag = ar_tag(epoch);
  const long long half_base = static_cast<long long>(epoch & 1ull) * p.ar.world;
  for (int e = e0 + static_cast<int>(threadIdx.x); e < e1; e += kArAddThreads) {
    const int tok = e / p.n_rows, row = e % p.n_rows;
    const float v = bf2f(p.partial[e]);
    const long long idx = ((half_base + p.ar.rank) * 4 + tok) * p.n_rows + row;
    for (int pr = 0; pr < p.ar.world; ++pr) ar_push(&p.ar.recv[pr][idx], tag, v);
  }
  // every thread of this CTA has read the call number: count the CTA towards the call (a local add, nothing waits
  // on it; the number only changes when the last CTA has added its share)
  __syncthreads();
  if (threadIdx.x == 0)
    asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(&p.ar.state->calls), "l"(ar_share(cta, grid)) : "memory");
  const unsigned long long* mine = p.ar.recv[p.ar.rank];
  const long long t0 = clock64();
  const long long budget = kWaitBudgetCycles;
  for (int e = e0 + static_cast<int>(threadIdx.x); e < e1; e += kArAddThreads) {
    const int tok = e / p.n_rows, row = e % p.n_rows;
    unsigned pending = (1u << p.ar.world) - 1u;
    float part[8];
    while (pending != 0u) {
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r < p.ar.world && ((pending >> r) & 1u)) {
          const unsigned long long word = ar_peek(&mine[((half_base + r) * 4 + tok) * p.n_rows + row]);
          if (static_cast<uint32_t>(word >> 32) == tag) {
            part[r] = __uint_as_float(static_cast<uint32_t>(word));
            pending &= ~(1u << r);
          }
        }
      }
      if (pending != 0u && clock64() - t0 > budget) {
        set_status(p.status, ST_PEER_TIMEOUT);
        return;
      }
    }
    float v = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (r < p.ar.world) v += part[r];
    if (p.residual != nullptr) v += bf2f(p.residual[e]);
    p.out[e] = f2bf(v);
  }
}

}  // namespace tb
