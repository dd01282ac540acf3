// Shared device helpers for the sm_100a decode kernels: mbarrier / bulk-copy (TMA) PTX
// wrappers with bounded waits, warp MMA wrappers, bf16 helpers and the per-device status
// word that a kernel sets instead of trapping when a wait runs out.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb {

// ---- status codes written to the device status word (first error wins) ----
enum Status : int {
  ST_OK = 0,
  ST_WAIT_FULL_TIMEOUT = 1,   // consumer gave up waiting for a bulk copy to land
  ST_WAIT_EMPTY_TIMEOUT = 2,  // producer gave up waiting for a free ring slot
  ST_PEER_TIMEOUT = 3,        // all-reduce gave up waiting for a peer's arrival
  ST_BAD_ARGUMENT = 4,
  ST_SPLIT_TIMEOUT = 5,       // a row tile's owner gave up waiting for another CTA's partial sums
  ST_CHAIN_TIMEOUT = 6,       // a phase of a chained launch gave up waiting for an earlier phase's signal
  ST_GRID_TIMEOUT = 7,        // a CTA of a cooperative launch gave up waiting for the others at a grid-wide barrier
};

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ unsigned sm_id() {
  unsigned v;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(v));
  return v;
}

__device__ __forceinline__ void set_status(int* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- programmatic dependent launch ----
// Kernels are launched with programmatic stream serialisation: a kernel may start while its
// predecessor in the stream is still running.  `pdl_wait` blocks until the predecessor has completed
// and its memory is visible (nothing produced by earlier kernels may be read, and nothing they might
// still read or write may be written, before it); `pdl_launch_dependents` lets the successor start.
// Both are no-ops in a launch without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- mbarrier ----
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: returns false (and the caller bails out) when the budget runs out.  The budget is
// counted on the SM's cycle counter, read only after a batch of failed polls: reading %globaltimer
// costs about as much as a whole pipeline stage, and a waiting consumer is the normal state of a
// bandwidth-bound kernel.
constexpr long long kDefaultWaitBudgetCycles = 1000000000ll;  // about half a second at ~2 GHz
// The budget lives in device memory so that a host call can shorten it (tilert_b200_set_wait_budget);
// it is read only on the slow path of a wait, after a few hundred failed polls.
__device__ long long g_wait_budget_cycles = kDefaultWaitBudgetCycles;
__device__ __forceinline__ long long wait_budget_cycles() {
  return *reinterpret_cast<const volatile long long*>(&g_wait_budget_cycles);
}
#define kWaitBudgetCycles (::tb::wait_budget_cycles())
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
#pragma unroll 1
  for (int i = 0; i < 32; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > kWaitBudgetCycles) return false;
  }
}

// Same, but also gives up (returns false) soon after another warp of the CTA has raised `abort`, so
// that one role's failure does not make every other role sit out its own full budget.  The flag is
// read only on the slow path.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const volatile int* abort) {
#pragma unroll 1
  for (int i = 0; i < 32; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort != 0 || clock64() - t0 > kWaitBudgetCycles) return false;
  }
}

// ---- bulk async copy (TMA, untiled): global -> this CTA's shared memory ----
// Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// Same with an L2 evict-first hint for data that is streamed exactly once.
__device__ __forceinline__ void bulk_g2s_stream(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                                uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::
          "r"(smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// ---- warp MMA ----
// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem_row)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem_row)));
}

// ---- small numeric helpers ----
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) { return __uint_as_float(uint32_t(b) << 16); }
__device__ __forceinline__ float bf2f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ __nv_bfloat16 f2bf(float v) { return __float2bfloat16_rn(v); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint8_t f32_to_e4m3(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float e4m3_to_f32(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(v, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace tb
