// C ABI of the decode path: argument checks, parameter blocks and kernel launches.
// Declarations and the reference operator each entry point replaces: include/tilert_b200.h.
#include "../../include/tilert_b200.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "actpack.cuh"
#include "elementwise.cuh"
#include "gemv_bf16.cuh"
#include "attn_prep.cuh"
#include "indexer.cuh"
#include "sparse_mla.cuh"
#include "allreduce_add.cuh"
#include "sampler.cuh"
#include "wstream_gemv.cuh"
#include "wstream_chain.cuh"
#include "argmax_exchange.cuh"
#include "cache_inject.cuh"

using namespace tb;

namespace {

thread_local std::string g_last_error;
long long g_launches = 0;

int fail(int code, const char* fmt, const char* detail = "") {
  char buf[512];
  snprintf(buf, sizeof(buf), fmt, detail);
  g_last_error = buf;
  return code;
}
#define TB_CUDA(expr)                                                        \
  do {                                                                       \
    cudaError_t e__ = (expr);                                                \
    if (e__ != cudaSuccess) return fail(TB_ECUDA, #expr ": %s", cudaGetErrorString(e__)); \
  } while (0)
#define TB_REQUIRE(cond) \
  do {                   \
    if (!(cond)) return fail(TB_EINVAL, "requirement failed: %s", #cond); \
  } while (0)

// Every kernel is launched with programmatic stream serialisation (see pdl_wait in common.cuh);
// TILERT_B200_PDL=0 in the environment switches it off.
bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("TILERT_B200_PDL");
    return e == nullptr || e[0] != '0';
  }();
  return on;
}
template <typename... KArgs, typename... Args>
cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

constexpr int kMaxGrid = 256;                       // CTAs a GEMV launch may use (>= SM count)
constexpr size_t kPartialBytes = 2ull * kMaxGrid * 8 * 32 * 16;  // = kMaxGrid slots x 4 warps x 32 lanes x 8 words x 8 bytes
constexpr int kMaxTiles = 1 << 13;                  // row tiles of one streaming product
constexpr size_t kXpackScratchBytes = 2ull << 20;   // activation blocks of the widest K (2048 blocks)
constexpr int kMaxXBlocks = 1984;                   // X blocks one launch may convert (fits kXpackScratchBytes)
constexpr size_t kXFlagBytes = (kMaxXBlocks + 64) * sizeof(unsigned);  // flags, then {epoch, done}
constexpr size_t kSmallScratchBytes = 64ull << 10;  // slot ids / weights for routing
constexpr size_t kMoeFlatBytes = 2ull << 20;  // expert hidden states of up to 4 tokens x 33 slots x 4096 values, bf16
constexpr size_t kIdxWorkBytes = 8ull * kIdxWorkWords * 4;  // the indexer's selection work area, eight query tokens
constexpr size_t kChainSignalBytes = (kChainSignals + 1) * kChainSigStride * sizeof(unsigned);

}  // namespace

// Byte range written by a recorded phase (or its hook) and the signal that says it is complete.
struct ChainRange {
  const char* lo;
  const char* hi;
  int sig;
};
// Streaming products recorded between tilert_b200_chain_begin and tilert_b200_chain_end: they run as the
// phases of one wstream_chain_kernel launch.
struct ChainRecorder {
  bool active = false;
  ChainParams params;
  int n_hooks = 0;
  int pending_hook = -1;  // recorded hook that waits for the next product to attach to
  int x_blocks = 0;       // shared X blocks handed out so far
  int n_ar = 0;
  std::vector<ChainRange> outs;
};

struct TbContext {
  int device = 0;
  int num_sms = 0;
  float* partial = nullptr;
  float* chain_partial = nullptr;      // split-tile slots of chained launches: one region per phase
  unsigned* chain_signals = nullptr;   // signal counters of chained launches (self-clearing)
  unsigned* idx_work = nullptr;        // histograms and barrier counters of the indexer's selection (self-clearing)
  int grid_limit = 0;                  // > 0: streaming launches use at most this many CTAs (tilert_b200_set_grid_limit)
  // Several tokens through the experts in ONE launch each (gate/up, down): the gate/up launch leaves every token's
  // column for every (token, expert) slot here, [tokens][1 + tokens * top_k][inter] bf16, and remembers whose
  // hidden_out it belongs to; the down launch that gets that hidden_out reads this instead.
  void* moe_flat = nullptr;
  const void* moe_flat_owner = nullptr;
  int moe_flat_tokens = 0, moe_flat_inter = 0, moe_flat_topk = 0;
  unsigned long long* chain_prof = nullptr;  // caller-owned trace of chained launches, see tilert_b200_set_chain_profile
  ChainRecorder rec;
  unsigned long long* launch_calls = nullptr;  // device-resident launch number of the streaming kernel
  int* status = nullptr;
  uint8_t* xpack = nullptr;
  uint8_t* xshared = nullptr;  // X blocks converted inside a streaming launch, shared by its CTAs
  unsigned* xflags = nullptr;  // their ready flags, then the launch-epoch state
  uint8_t* small = nullptr;
  unsigned long long* prof = nullptr;  // caller-owned trace buffer, see tilert_b200_set_profile
  int prof_records = 1;                // records in the buffer; streaming launch k writes record k % prof_records
  long long prof_next = 0;
};

struct TbComm {
  TbContext* ctx = nullptr;
  int world = 1, rank = 0, max_rows = 0;
  void* buffers[8] = {};
};

namespace {

size_t comm_state_offset(int world, int max_rows) {
  // [2 halves][world][4 tokens][max_rows] 64-bit words {call number, f32}, then the endpoint state
  size_t b = 2ull * world * 4 * max_rows * sizeof(unsigned long long);
  return (b + 255) / 256 * 256;
}

// Whole tiles per CTA when that balances well enough -- short rows (few k blocks per tile) with many
// tiles when the busiest CTA then has at most 20 % more than the average, any row length at 4 % --
// otherwise equal shares of units with split-tile fix-up.
void set_partition(GemvParams& p, int grid) {
  const int max_tiles = (p.n_tiles + grid - 1) / grid;
  const long long busiest = static_cast<long long>(max_tiles) * grid, all = p.n_tiles;
  const bool short_rows = p.n_kb <= 16 && p.n_tiles >= grid / 2 && busiest * 5 <= all * 6;
  // Long rows too when whole tiles balance within 4 %: the fix-up of split tiles costs more than that.
  const bool balanced = p.n_tiles >= grid / 2 && busiest * 25 <= all * 26;
  p.whole_tiles = (short_rows || balanced) ? 1 : 0;
}

// Most units any CTA takes under the launch's partition; decides whether the CTAs share the activation
// conversion (a CTA converts only the X blocks of its first pass over the ring by itself).
int max_cta_units(const GemvParams& p, int grid) {
  if (p.whole_tiles) return (p.n_tiles + grid - 1) / grid * p.n_kb;
  const long long units = static_cast<long long>(p.n_tiles) * p.n_kb;
  return static_cast<int>((units + grid - 1) / grid);
}

const char* cptr(const void* p) { return reinterpret_cast<const char*>(p); }

// Highest signal among the recorded outputs that overlap [ptr, ptr + bytes); -1 when nothing recorded writes there.
int chain_dep(const ChainRecorder& r, const void* ptr, long long bytes) {
  if (ptr == nullptr || bytes <= 0) return -1;
  int best = -1;
  for (const ChainRange& o : r.outs)
    if (cptr(ptr) < o.hi && cptr(ptr) + bytes > o.lo && o.sig > best) best = o.sig;
  return best;
}
void chain_out(ChainRecorder& r, const void* ptr, long long bytes, int sig) {
  if (ptr != nullptr && bytes > 0) r.outs.push_back({cptr(ptr), cptr(ptr) + bytes, sig});
}
int imax(int a, int b) { return a > b ? a : b; }

int chain_grid(const TbContext* ctx) { return ctx->num_sms < kMaxGrid ? ctx->num_sms : kMaxGrid; }

// Appends a streaming product to the chain being recorded.  Dependencies come from the recorded outputs
// that the product's inputs overlap: activations, residual and routing weights decide when the activation
// side may start, slot ids and router scores when the producers may compute weight addresses.
int record_phase(TbContext* ctx, GemvParams& p) {
  ChainRecorder& r = ctx->rec;
  if (r.params.n_phases >= kChainMaxPhases) return fail(TB_ESTATE, "chain: too many products in one chain%s");
  if (p.x_mode != X_BF16) return fail(TB_EINVAL, "chain: only products on bf16 activations can be chained%s");
  const int ph = r.params.n_phases;
  const long long units = static_cast<long long>(p.n_tiles) * p.n_kb;
  const int grid = chain_grid(ctx);
  p.grid_eff = units < grid ? static_cast<int>(units) : grid;
  // A short product is not spread thinner than eight CTAs per row tile: every further CTA inside a tile is
  // one more partial sum its owner must collect through L2 (a round trip per four), and a product this
  // small gains nothing from more CTAs.  It then sits at the far end of the grid, away from the CTAs that
  // earlier short phases loaded.
  if (static_cast<long long>(p.n_tiles) * 8 < p.grid_eff) p.grid_eff = p.n_tiles * 8;
  p.cta_base = p.grid_eff < grid ? grid - p.grid_eff : 0;
  if (ph > 0) {
    const GemvParams& prev = r.params.ph[ph - 1].g;
    // short phases alternate between the two ends of the grid, so that they do not pile up on the same CTAs
    if (p.grid_eff < grid && prev.grid_eff < grid && prev.cta_base > 0) p.cta_base = 0;
  }
  set_partition(p, p.grid_eff);
  p.shared_x = max_cta_units(p, p.grid_eff) > kGemvStages ? 1 : 0;
  p.partial = ctx->chain_partial + static_cast<size_t>(ph) * (kPartialBytes / sizeof(float));
  p.launch_calls = ctx->launch_calls;
  p.status = ctx->status;
  p.prof = nullptr;
  const int n_xsegs = p.tiles_per_xseg > 0 ? p.n_tiles / p.tiles_per_xseg : 1;
  TB_REQUIRE(p.tiles_per_xseg <= 0 || p.n_tiles % p.tiles_per_xseg == 0);
  const int n_xblocks = n_xsegs * p.n_kb;
  if (r.x_blocks + n_xblocks > kMaxXBlocks) return fail(TB_ESTATE, "chain: the chained products need too many X blocks%s");
  p.xs = ctx->xshared + static_cast<size_t>(r.x_blocks) * TB_XBLK_BYTES;
  p.xflag = ctx->xflags + r.x_blocks;
  p.xstate = ctx->xflags + kMaxXBlocks;
  r.x_blocks += n_xblocks;

  ChainPhase& c = r.params.ph[ph];
  c.hook = r.pending_hook;
  r.pending_hook = -1;
  c.ar_index = r.n_ar;
  if (p.ar.world > 1) ++r.n_ar;
  c.main_target = grid;

  // a down projection that reads the slot list an earlier recorded product routes: route it here too, so
  // that its weight addresses do not wait for that product to finish
  if (p.kseg_ids != nullptr) {
    for (int q = 0; q < ph; ++q) {
      const RouteParams& rq = r.params.ph[q].g.route;
      if (rq.scores != nullptr && rq.slot_ids == p.kseg_ids) {
        p.route = rq;
        p.route.for_kseg = 1;
        p.route.slot_base = 0;
        p.route.probs = nullptr;
        p.kseg_ids = nullptr;
        break;
      }
    }
  }
  // activation-side dependencies
  int dep = chain_dep(r, p.xb, (static_cast<long long>(p.n_tokens - 1) * p.xb_stride + static_cast<long long>(n_xblocks) * TB_KBLOCK) * 2);
  dep = imax(dep, chain_dep(r, p.residual, (static_cast<long long>(p.n_tokens - 1) * p.residual_stride + p.n_rows) * 2));
  if (p.seg_scale != nullptr)
    dep = imax(dep, chain_dep(r, p.seg_scale, static_cast<long long>(p.n_tokens) * (p.n_kb / p.kb_per_kseg) * 4));
  if (c.hook >= 0) dep = imax(dep, 2 * ph - 2);  // the vector work reads cache rows and vectors of every earlier product
  c.wait_sig = dep;
  if (ph > 0) {
    // A full-width phase that does not wait for the short phase recorded just before it (router gate ->
    // shared expert: both read the same vector) takes only the CTAs that phase left idle: the two then run
    // side by side instead of one after the other on the short phase's CTAs.
    const GemvParams& prev = r.params.ph[ph - 1].g;
    const bool independent = dep < 2 * (ph - 1) && p.nseg_ids == nullptr && p.kseg_ids == nullptr && p.route.scores == nullptr;
    if (independent && p.grid_eff == grid && prev.grid_eff * 3 <= grid && units >= 4ll * grid) {
      p.grid_eff = grid - prev.grid_eff;
      p.cta_base = prev.cta_base > 0 ? 0 : prev.grid_eff;
      set_partition(p, p.grid_eff);
      p.shared_x = max_cta_units(p, p.grid_eff) > kGemvStages ? 1 : 0;
    }
  }
  // weight-address dependencies
  int wdep = -1;
  if (p.nseg_ids != nullptr) wdep = imax(wdep, chain_dep(r, p.nseg_ids, 4ll * (p.n_tiles / p.tiles_per_nseg)));
  if (p.kseg_ids != nullptr) wdep = imax(wdep, chain_dep(r, p.kseg_ids, 4ll * (p.n_kb / p.kb_per_kseg)));
  if (p.route.scores != nullptr) {
    wdep = imax(wdep, chain_dep(r, p.route.scores, 4ll * p.route.n_experts));
    if (p.route.probs != nullptr) c.main_target = grid + 1;  // producer 0 of CTA 0 stores the routing results
  }
  c.w_sig = wdep;

  // outputs
  for (int i = 0; i < p.n_regions; ++i) {
    const OutRegion& reg = p.regions[i];
    if (reg.pos_ptr != nullptr) continue;  // cache rows: only hooks read them, and those wait for every earlier product
    const long long esz = reg.dtype == 0 ? 2 : 4;
    chain_out(r, reg.ptr, (static_cast<long long>(p.n_tokens - 1) * reg.token_stride + (reg.row_end - reg.row_begin)) * esz, 2 * ph);
  }
  if (p.route.scores != nullptr && p.route.probs != nullptr) {
    chain_out(r, p.route.probs, 4ll * p.route.top_k, 2 * ph);
    chain_out(r, p.route.ids, 4ll * p.route.top_k, 2 * ph);
    chain_out(r, p.route.slot_ids, 4ll * (p.route.top_k + 1), 2 * ph);
    chain_out(r, p.route.slot_w, 4ll * (p.route.top_k + 1), 2 * ph);
  }
  if (c.hook >= 0) {
    const AttnPrepParams& a = r.params.hooks[c.hook].prep;
    chain_out(r, a.q_pe, 2ll * a.n_tokens * a.heads * a.rope, 2 * ph + 1);
    chain_out(r, a.iq_out, 2ll * a.n_tokens * a.idx_heads * 128, 2 * ph + 1);
  }
  c.g = p;
  ++r.params.n_phases;
  return TB_OK;
}

int launch_gemv(TbContext* ctx, GemvParams& p, cudaStream_t st) {
  static bool attr_set[64] = {};
  if (!attr_set[ctx->device & 63]) {
    TB_CUDA(cudaFuncSetAttribute(wstream_gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvSmemBytes));
    TB_CUDA(cudaFuncSetAttribute(wstream_chain_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kChainSmemBytes));
    TB_CUDA(cudaFuncSetAttribute(wstream_chain_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kChainSmemBytes));
    attr_set[ctx->device & 63] = true;
  }
  TB_REQUIRE(p.n_tiles > 0 && p.n_kb > 0);
  TB_REQUIRE(p.n_tiles <= kMaxTiles);
  const long long units = static_cast<long long>(p.n_tiles) * p.n_kb;
  TB_REQUIRE(units < (1ll << 30));
  if (ctx->rec.active) return record_phase(ctx, p);
  int grid = ctx->num_sms < kMaxGrid ? ctx->num_sms : kMaxGrid;
  if (ctx->grid_limit > 0 && ctx->grid_limit < grid) grid = ctx->grid_limit;  // SMs left to a concurrent stream
  if (units < grid) grid = static_cast<int>(units);
  if (static_cast<long long>(p.n_tiles) * 8 < grid) grid = p.n_tiles * 8;  // at most eight CTAs inside a row tile
  set_partition(p, grid);
  p.grid_eff = grid;
  p.shared_x = max_cta_units(p, grid) > kGemvStages ? 1 : 0;
  p.partial = ctx->partial;
  p.launch_calls = ctx->launch_calls;
  p.status = ctx->status;
  if (p.x_mode == X_BF16) {
    const int n_xsegs = p.tiles_per_xseg > 0 ? p.n_tiles / p.tiles_per_xseg : 1;
    TB_REQUIRE(p.tiles_per_xseg <= 0 || p.n_tiles % p.tiles_per_xseg == 0);
    TB_REQUIRE(static_cast<long long>(n_xsegs) * p.n_kb <= kMaxXBlocks);
    p.xs = ctx->xshared;
    p.xflag = ctx->xflags;
    p.xstate = ctx->xflags + kMaxXBlocks;
  }
  p.prof = ctx->prof;
  if (ctx->prof != nullptr) p.prof += (ctx->prof_next++ % ctx->prof_records) * (256 * 16);
  // Pause between one producer's three copies of the first pass over the ring (long launches only).  Without it a
  // CTA that starts early under programmatic dependent launch puts twelve copies in flight at once and takes
  // bandwidth from the predecessor's slowest CTAs, which everybody then waits for: measured on the layer step,
  // 0.2072 ms without, 0.2023 ms with 1.2-2 us, slower again from 3 us.  TILERT_B200_STAGGER_NS overrides.
  static const unsigned stagger_ns = [] {
    const char* e = getenv("TILERT_B200_STAGGER_NS");
    return e != nullptr ? static_cast<unsigned>(atoi(e)) : 1500u;
  }();
  p.stagger_ns = stagger_ns;
  TB_CUDA(launch(wstream_gemv_kernel, dim3(grid), dim3(kGemvThreads), kGemvSmemBytes, st, p));
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  return TB_OK;
}

// Operators that cannot become part of a chained launch refuse to run while one is being recorded.
#define TB_NOT_CHAINABLE(ctx)                                                                          \
  do {                                                                                                 \
    if ((ctx) != nullptr && (ctx)->rec.active)                                                         \
      return fail(TB_ESTATE, "%s cannot be recorded into a chain (end the chain first)", __func__);    \
  } while (0)

void gemv_defaults(GemvParams& p) {
  memset(&p, 0, sizeof(p));
  p.only_token = -1;
  p.cols_per_token = 2;
  p.epi = EPI_STORE;
  p.ar.world = 1;
}

void set_region(GemvParams& p, int row_begin, int rows, void* ptr, long long token_stride, int dtype = 0,
                const int* pos = nullptr, int pos_rows = 0) {
  if (rows <= 0 || ptr == nullptr) return;
  OutRegion& r = p.regions[p.n_regions++];
  r.row_begin = row_begin;
  r.row_end = row_begin + rows;
  r.dtype = dtype;
  r.ptr = ptr;
  r.token_stride = token_stride;
  r.pos_ptr = pos;
  r.pos_rows = pos_rows;
}

int set_comm(GemvParams& p, TbComm* comm, int n_rows) {
  if (comm == nullptr || comm->world <= 1) return TB_OK;
  TB_REQUIRE(n_rows == comm->max_rows);  // slot stride of the receive buffers
  p.ar.world = comm->world;
  p.ar.rank = comm->rank;
  const size_t off = comm_state_offset(comm->world, comm->max_rows);
  for (int r = 0; r < comm->world; ++r) p.ar.recv[r] = reinterpret_cast<unsigned long long*>(comm->buffers[r]);
  p.ar.state = reinterpret_cast<AllReduceState*>(reinterpret_cast<uint8_t*>(comm->buffers[comm->rank]) + off);
  return TB_OK;
}

void set_x_bf16(GemvParams& p, const void* x, long long stride, const float* gamma = nullptr, float eps = 0.f,
                const float* seg_scale = nullptr) {
  p.x_mode = X_BF16;
  p.xb = reinterpret_cast<const __nv_bfloat16*>(x);
  p.xb_stride = stride;
  p.gamma = gamma;
  p.eps = eps;
  p.seg_scale = seg_scale;
}

int launch_actpack(const ActPackParams& p, cudaStream_t st) {
  TB_REQUIRE(p.k % TB_KBLOCK == 0 && p.k / TB_KBLOCK <= 32 * kActPackMaxIter);
  TB_REQUIRE(p.n_tokens >= 1 && p.n_tokens <= 4);
  TB_CUDA(launch(actpack_kernel, dim3(p.n_tokens), dim3(kActPackThreads), 0, st, p));
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  return TB_OK;
}

// Plain (no norm) packing of a flat [tokens, k] bf16 array that may exceed the single-CTA limit of
// the normalising kernel: split into chunks of at most 32*kActPackMaxIter blocks.
int pack_flat(const void* x, int tokens, int k, const float* seg_scale, int n_seg, uint8_t* xpack,
              cudaStream_t st) {
  const int max_k = 32 * kActPackMaxIter * TB_KBLOCK;
  TB_REQUIRE(seg_scale == nullptr || k <= max_k);
  for (int k0 = 0; k0 < k; k0 += max_k) {
    ActPackParams p{};
    p.x = reinterpret_cast<const __nv_bfloat16*>(x) + k0;
    p.x_stride = k;
    p.k = (k - k0) < max_k ? (k - k0) : max_k;
    p.n_tokens = tokens;
    p.seg_scale = seg_scale;
    p.n_seg = n_seg;
    p.kb_per_seg = n_seg > 0 ? (k / TB_KBLOCK) / n_seg : 1;
    p.xpack = xpack + static_cast<size_t>(k0 / TB_KBLOCK) * TB_XBLK_BYTES;
    int rc = launch_actpack(p, st);
    if (rc != TB_OK) return rc;
  }
  return TB_OK;
}

}  // namespace

// ------------------------------------------------------------------------------- runtime
extern "C" const char* tilert_b200_last_error(void) { return g_last_error.c_str(); }
extern "C" int tilert_b200_dsa_temp_vars_size(void) { return 56; }
extern "C" size_t tilert_b200_context_bytes(void) {
  return kPartialBytes * (1 + kChainMaxPhases) + 1024 + 2 * kXpackScratchBytes + kXFlagBytes + kSmallScratchBytes + kIdxWorkBytes + kMoeFlatBytes;
}
extern "C" size_t tilert_b200_xpack_bytes(int dim) { return static_cast<size_t>(dim / TB_KBLOCK) * TB_XBLK_BYTES; }

extern "C" int tilert_b200_init(int device, TbContext** ctx_out) {
  TB_REQUIRE(ctx_out != nullptr);
  TB_CUDA(cudaSetDevice(device));
  TbContext* c = new TbContext();
  c->device = device;
  cudaDeviceProp prop;
  TB_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major < 10) {
    delete c;
    return fail(TB_ESTATE, "this library is built for sm_100a only; device is %s", prop.name);
  }
  c->num_sms = prop.multiProcessorCount;
  TB_CUDA(cudaMalloc(&c->partial, kPartialBytes));
  TB_CUDA(cudaMalloc(&c->chain_partial, kPartialBytes * kChainMaxPhases));
  TB_CUDA(cudaMemset(c->chain_partial, 0, kPartialBytes * kChainMaxPhases));
  TB_CUDA(cudaMalloc(&c->chain_signals, kChainSignalBytes));
  TB_CUDA(cudaMemset(c->chain_signals, 0, kChainSignalBytes));
  TB_CUDA(cudaMalloc(&c->moe_flat, kMoeFlatBytes));
  TB_CUDA(cudaMemset(c->moe_flat, 0, kMoeFlatBytes));
  TB_CUDA(cudaMalloc(&c->idx_work, kIdxWorkBytes));
  TB_CUDA(cudaMemset(c->idx_work, 0, kIdxWorkBytes));
  TB_CUDA(cudaMalloc(&c->status, 256));
  TB_CUDA(cudaMalloc(&c->launch_calls, 256));
  TB_CUDA(cudaMemset(c->launch_calls, 0, 256));
  TB_CUDA(cudaMalloc(&c->xpack, kXpackScratchBytes));
  TB_CUDA(cudaMalloc(&c->xshared, kXpackScratchBytes));
  TB_CUDA(cudaMalloc(&c->xflags, kXFlagBytes));
  TB_CUDA(cudaMemset(c->xshared, 0, kXpackScratchBytes));
  TB_CUDA(cudaMemset(c->xflags, 0, kXFlagBytes));
  TB_CUDA(cudaMalloc(&c->small, kSmallScratchBytes));
  TB_CUDA(cudaMemset(c->partial, 0, kPartialBytes));
  TB_CUDA(cudaMemset(c->status, 0, 256));
  TB_CUDA(cudaMemset(c->xpack, 0, kXpackScratchBytes));
  TB_CUDA(cudaMemset(c->small, 0, kSmallScratchBytes));
  TB_CUDA(cudaDeviceSynchronize());
  *ctx_out = c;
  return TB_OK;
}

extern "C" int tilert_b200_default_context(int device, TbContext** ctx_out) {
  // one context per device and process, shared by every binding that asks for it (ctypes, the dispatcher
  // registration library): their launches then use one set of scratch, in stream order
  static std::mutex mu;
  static TbContext* ctxs[64] = {};
  TB_REQUIRE(ctx_out != nullptr && device >= 0 && device < 64);
  std::lock_guard<std::mutex> lock(mu);
  if (ctxs[device] == nullptr) {
    const int rc = tilert_b200_init(device, &ctxs[device]);
    if (rc != TB_OK) return rc;
  }
  *ctx_out = ctxs[device];
  return TB_OK;
}

extern "C" int tilert_b200_destroy(TbContext* ctx) {
  if (ctx == nullptr) return TB_OK;
  cudaSetDevice(ctx->device);
  cudaFree(ctx->partial);
  cudaFree(ctx->chain_partial);
  cudaFree(ctx->chain_signals);
  cudaFree(ctx->idx_work);
  cudaFree(ctx->moe_flat);
  cudaFree(ctx->launch_calls);
  cudaFree(ctx->status);
  cudaFree(ctx->xpack);
  cudaFree(ctx->xshared);
  cudaFree(ctx->xflags);
  cudaFree(ctx->small);
  delete ctx;
  return TB_OK;
}

extern "C" int tilert_b200_status(TbContext* ctx, int* status_out) {
  TB_REQUIRE(ctx != nullptr && status_out != nullptr);
  TB_CUDA(cudaSetDevice(ctx->device));
  TB_CUDA(cudaDeviceSynchronize());
  TB_CUDA(cudaMemcpy(status_out, ctx->status, sizeof(int), cudaMemcpyDeviceToHost));
  if (*status_out != 0) {
    // a launch that gave up may have left signal counters of a chained launch half-way: start clean
    TB_CUDA(cudaMemset(ctx->status, 0, sizeof(int)));
    TB_CUDA(cudaMemset(ctx->chain_signals, 0, kChainSignalBytes));
    TB_CUDA(cudaMemset(ctx->idx_work, 0, kIdxWorkBytes));
  }
  return TB_OK;
}

extern "C" int tilert_b200_set_grid_limit(TbContext* ctx, int max_ctas) {
  TB_REQUIRE(ctx != nullptr && max_ctas >= 0);
  ctx->grid_limit = max_ctas;
  return TB_OK;
}

extern "C" int tilert_b200_set_wait_budget(TbContext* ctx, long long cycles) {
  TB_REQUIRE(ctx != nullptr);
  TB_CUDA(cudaSetDevice(ctx->device));
  const long long v = cycles > 0 ? cycles : kDefaultWaitBudgetCycles;
  TB_CUDA(cudaMemcpyToSymbol(g_wait_budget_cycles, &v, sizeof(v)));
  return TB_OK;
}

// ------------------------------------------------------------------------------ chained launches
extern "C" int tilert_b200_chain_begin(TbContext* ctx) {
  TB_REQUIRE(ctx != nullptr);
  if (ctx->rec.active) return fail(TB_ESTATE, "chain: a chain is already being recorded%s");
  ChainRecorder& r = ctx->rec;
  memset(&r.params, 0, sizeof(r.params));
  r.n_hooks = 0;
  r.pending_hook = -1;
  r.x_blocks = 0;
  r.n_ar = 0;
  r.outs.clear();
  r.active = true;
  return TB_OK;
}

extern "C" int tilert_b200_chain_abort(TbContext* ctx) {
  TB_REQUIRE(ctx != nullptr);
  ctx->rec.active = false;
  return TB_OK;
}

extern "C" int tilert_b200_chain_end(TbContext* ctx, void* stream) {
  TB_REQUIRE(ctx != nullptr);
  ChainRecorder& r = ctx->rec;
  if (!r.active) return fail(TB_ESTATE, "chain: no chain is being recorded%s");
  r.active = false;
  if (r.pending_hook >= 0) return fail(TB_ESTATE, "chain: the last recorded operator needs a following product to attach to%s");
  if (r.params.n_phases == 0) return TB_OK;
  r.params.signals = ctx->chain_signals;
  r.params.prof = ctx->chain_prof;
  static const int inflight = [] {
    // TILERT_B200_INFLIGHT: 4, 8 or 12 weight blocks in flight per CTA (tuning knob)
    const char* e = getenv("TILERT_B200_INFLIGHT");
    const int v = e != nullptr ? atoi(e) : 8;
    return v >= 12 ? 12 : (v >= 8 ? 8 : 4);
  }();
  r.params.max_inflight = inflight;
  static_assert(sizeof(ChainParams) <= 24 * 1024, "kernel parameter space");
  if (r.params.prof != nullptr)
    TB_CUDA(launch(wstream_chain_kernel<true>, dim3(chain_grid(ctx)), dim3(kGemvThreads), kChainSmemBytes,
                   static_cast<cudaStream_t>(stream), r.params));
  else
    TB_CUDA(launch(wstream_chain_kernel<false>, dim3(chain_grid(ctx)), dim3(kGemvThreads), kChainSmemBytes,
                   static_cast<cudaStream_t>(stream), r.params));
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  return TB_OK;
}

extern "C" int tilert_b200_set_chain_profile(TbContext* ctx, unsigned long long* trace) {
  TB_REQUIRE(ctx != nullptr);
  ctx->chain_prof = trace;
  return TB_OK;
}

extern "C" int tilert_b200_num_sms(TbContext* ctx) { return ctx != nullptr ? ctx->num_sms : 0; }
extern "C" long long tilert_b200_launch_count(void) { return g_launches; }
extern "C" int tilert_b200_set_profile(TbContext* ctx, unsigned long long* trace) {
  TB_REQUIRE(ctx != nullptr);
  ctx->prof = trace;
  ctx->prof_records = 1;
  ctx->prof_next = 0;
  return TB_OK;
}
extern "C" int tilert_b200_set_profile_ring(TbContext* ctx, unsigned long long* trace, int n_records) {
  TB_REQUIRE(ctx != nullptr && n_records >= 1);
  ctx->prof = trace;
  ctx->prof_records = n_records;
  ctx->prof_next = 0;
  return TB_OK;
}
extern "C" int tilert_b200_dev_alloc(size_t bytes, void** dev_ptr_out) {
  TB_REQUIRE(dev_ptr_out != nullptr && bytes > 0);
  TB_CUDA(cudaMalloc(dev_ptr_out, bytes));
  TB_CUDA(cudaMemset(*dev_ptr_out, 0, bytes));
  TB_CUDA(cudaDeviceSynchronize());
  return TB_OK;
}
extern "C" int tilert_b200_dev_free(void* dev_ptr) {
  TB_CUDA(cudaFree(dev_ptr));
  return TB_OK;
}

// ------------------------------------------------------------------------------ p2p plumbing
extern "C" size_t tilert_b200_comm_buffer_bytes(int world, int max_rows) {
  return comm_state_offset(world, max_rows) + 256;
}
extern "C" int tilert_b200_ipc_export(void* dev_ptr, uint8_t handle_out[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  TB_CUDA(cudaIpcGetMemHandle(&h, dev_ptr));
  memcpy(handle_out, &h, 64);
  return TB_OK;
}
extern "C" int tilert_b200_ipc_import(const uint8_t handle[64], void** dev_ptr_out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  TB_CUDA(cudaIpcOpenMemHandle(dev_ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
  return TB_OK;
}
extern "C" int tilert_b200_ipc_close(void* dev_ptr) {
  TB_CUDA(cudaIpcCloseMemHandle(dev_ptr));
  return TB_OK;
}
extern "C" int tilert_b200_comm_create(TbContext* ctx, int world, int rank, void* const* buffers, int max_rows,
                                       TbComm** comm_out) {
  TB_REQUIRE(ctx != nullptr && comm_out != nullptr && buffers != nullptr);
  TB_REQUIRE(world >= 1 && world <= 8 && rank >= 0 && rank < world && max_rows > 0);
  TbComm* c = new TbComm();
  c->ctx = ctx;
  c->world = world;
  c->rank = rank;
  c->max_rows = max_rows;
  for (int r = 0; r < world; ++r) {
    if (buffers[r] == nullptr) {
      delete c;
      return fail(TB_EINVAL, "comm buffer pointer is null%s");
    }
    c->buffers[r] = buffers[r];
  }
  *comm_out = c;
  return TB_OK;
}
extern "C" int tilert_b200_comm_destroy(TbComm* comm) {
  delete comm;
  return TB_OK;
}

// --------------------------------------------------------------------- activation preparation
extern "C" int tilert_rmsnorm_quant_op(TbContext* ctx, const void* x, const float* gamma, float eps, int tokens,
                                       int dim, void* out, uint8_t* q_out, float* q_scale_out,
                                       const float* seg_scale, int n_seg, uint8_t* xpack, void* stream) {
  TB_NOT_CHAINABLE(ctx);
  TB_REQUIRE(ctx != nullptr && x != nullptr);
  TB_REQUIRE((q_out == nullptr) == (q_scale_out == nullptr));
  if (xpack == nullptr) xpack = ctx->xpack;  // caller only wants the bf16 / reference-format outputs
  if (gamma == nullptr && out == nullptr && q_out == nullptr)
    return pack_flat(x, tokens, dim, seg_scale, n_seg, xpack, static_cast<cudaStream_t>(stream));
  ActPackParams p{};
  p.x = reinterpret_cast<const __nv_bfloat16*>(x);
  p.x_stride = dim;
  p.k = dim;
  p.n_tokens = tokens;
  p.gamma = gamma;
  p.eps = eps;
  p.seg_scale = seg_scale;
  p.n_seg = n_seg;
  p.kb_per_seg = n_seg > 0 ? (dim / TB_KBLOCK) / n_seg : 1;
  p.xpack = xpack;
  p.out_bf16 = reinterpret_cast<__nv_bfloat16*>(out);
  p.out_stride = dim;
  p.out_q = q_out;
  p.out_qscale = q_scale_out;
  return launch_actpack(p, static_cast<cudaStream_t>(stream));
}

extern "C" int tilert_xq_repack_op(TbContext* ctx, const uint8_t* x_q, const float* x_scale, int tokens, int dim,
                                   uint8_t* xpack, void* stream) {
  TB_NOT_CHAINABLE(ctx);
  TB_REQUIRE(ctx != nullptr && x_q != nullptr && x_scale != nullptr && xpack != nullptr);
  TB_REQUIRE(dim % TB_KBLOCK == 0 && tokens >= 1 && tokens <= 8);
  const int n_kb = dim / TB_KBLOCK;
  xq_repack_kernel<<<(n_kb + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(x_q, x_scale, tokens, dim, xpack);
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  return TB_OK;
}

// ------------------------------------------------------------------- FP8 streaming products
extern "C" int tilert_projx_wqkva_op(TbContext* ctx, const uint8_t* xpack, int cols_per_token,
                                     const uint8_t* w_packed, int tokens, int dim, int q_lora, int kv_lora, int rope,
                                     int ki_dim, const int* cur_pos, void* q_out, void* kv_out, void* pe_cache,
                                     int cache_rows, void* ki_out, void* stream) {
  TB_REQUIRE(ctx != nullptr && xpack != nullptr && w_packed != nullptr);
  TB_REQUIRE(dim % TB_KBLOCK == 0 && (cols_per_token == 1 || cols_per_token == 2));
  TB_REQUIRE(tokens >= 1 && tokens * cols_per_token <= 8);
  TB_REQUIRE(rope == 0 || cur_pos != nullptr);
  const int rows = q_lora + kv_lora + rope + ki_dim;
  GemvParams p;
  gemv_defaults(p);
  p.w = w_packed;
  p.x = xpack;
  p.n_tiles = (rows + TB_TILE_ROWS - 1) / TB_TILE_ROWS;
  p.n_kb = dim / TB_KBLOCK;
  p.w_kb_per_tile = p.n_kb;
  p.n_tokens = tokens;
  p.cols_per_token = cols_per_token;
  p.n_rows = rows;
  set_region(p, 0, q_lora, q_out, q_lora);
  set_region(p, q_lora, kv_lora, kv_out, kv_lora);
  set_region(p, q_lora + kv_lora, rope, pe_cache, rope, 0, cur_pos, cache_rows);
  set_region(p, q_lora + kv_lora + rope, ki_dim, ki_out, ki_dim);
  return launch_gemv(ctx, p, static_cast<cudaStream_t>(stream));
}

extern "C" int tilert_rmsnorm_projx_wqkva_op(TbContext* ctx, const void* x, const float* gamma, float eps,
                                             const uint8_t* w_packed, int tokens, int dim, int q_lora, int kv_lora,
                                             int rope, int ki_dim, const int* cur_pos, void* q_out, void* kv_out,
                                             void* pe_cache, int cache_rows, void* ki_out, void* stream) {
  TB_REQUIRE(ctx != nullptr && x != nullptr && gamma != nullptr && w_packed != nullptr);
  TB_REQUIRE(dim % TB_KBLOCK == 0 && tokens >= 1 && tokens <= 4);
  TB_REQUIRE(rope == 0 || cur_pos != nullptr);
  const int rows = q_lora + kv_lora + rope + ki_dim;
  GemvParams p;
  gemv_defaults(p);
  p.w = w_packed;
  set_x_bf16(p, x, dim, gamma, eps);
  p.n_tiles = (rows + TB_TILE_ROWS - 1) / TB_TILE_ROWS;
  p.n_kb = dim / TB_KBLOCK;
  p.w_kb_per_tile = p.n_kb;
  p.n_tokens = tokens;
  p.n_rows = rows;
  set_region(p, 0, q_lora, q_out, q_lora);
  set_region(p, q_lora, kv_lora, kv_out, kv_lora);
  set_region(p, q_lora + kv_lora, rope, pe_cache, rope, 0, cur_pos, cache_rows);
  set_region(p, q_lora + kv_lora + rope, ki_dim, ki_out, ki_dim);
  return launch_gemv(ctx, p, static_cast<cudaStream_t>(stream));
}

extern "C" int tilert_rmsnorm_proj_q_op(TbContext* ctx, const void* q, const float* gamma, float eps,
                                        const uint8_t* w_packed, int tokens, int q_lora, int heads, int nope,
                                        int rope, int iq_heads, int iq_dim, void* q_nope, void* q_pe, void* iq,
                                        void* stream) {
  TB_REQUIRE(ctx != nullptr && q != nullptr && gamma != nullptr && w_packed != nullptr);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  TB_REQUIRE(tokens >= 1 && tokens <= 4 && q_lora % TB_KBLOCK == 0);
  const int r_nope = heads * nope, r_pe = heads * rope, r_iq = iq_heads * iq_dim;
  GemvParams p;
  gemv_defaults(p);
  p.w = w_packed;
  set_x_bf16(p, q, q_lora, gamma, eps);
  p.n_rows = r_nope + r_pe + r_iq;
  p.n_tiles = (p.n_rows + TB_TILE_ROWS - 1) / TB_TILE_ROWS;
  p.n_kb = q_lora / TB_KBLOCK;
  p.w_kb_per_tile = p.n_kb;
  p.n_tokens = tokens;
  set_region(p, 0, r_nope, q_nope, r_nope);
  set_region(p, r_nope, r_pe, q_pe, r_pe);
  set_region(p, r_nope + r_pe, r_iq, iq, r_iq);
  return launch_gemv(ctx, p, st);
}

extern "C" int tilert_projq_wqb_op(TbContext* ctx, const void* q_nope, const uint8_t* w_packed, int tokens,
                                   int heads, int nope, int kv_lora, void* out, void* stream) {
  TB_REQUIRE(ctx != nullptr && q_nope != nullptr && w_packed != nullptr && out != nullptr);
  TB_REQUIRE(nope % TB_KBLOCK == 0 && kv_lora % TB_TILE_ROWS == 0);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  TB_REQUIRE(tokens >= 1 && tokens <= 4);
  GemvParams p;
  gemv_defaults(p);
  p.w = w_packed;
  set_x_bf16(p, q_nope, static_cast<long long>(heads) * nope);
  p.n_rows = heads * kv_lora;
  p.n_tiles = p.n_rows / TB_TILE_ROWS;
  p.n_kb = nope / TB_KBLOCK;
  p.w_kb_per_tile = p.n_kb;
  p.tiles_per_xseg = kv_lora / TB_TILE_ROWS;
  p.n_tokens = tokens;
  set_region(p, 0, p.n_rows, out, p.n_rows);
  return launch_gemv(ctx, p, st);
}

extern "C" int tilert_projo_wkvb_op(TbContext* ctx, const void* o_lat, const uint8_t* w_packed, int tokens,
                                    int heads, int kv_lora, int v_dim, void* out, void* stream) {
  TB_REQUIRE(ctx != nullptr && o_lat != nullptr && w_packed != nullptr && out != nullptr);
  TB_REQUIRE(kv_lora % TB_KBLOCK == 0 && v_dim % TB_TILE_ROWS == 0);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  TB_REQUIRE(tokens >= 1 && tokens <= 4);
  GemvParams p;
  gemv_defaults(p);
  p.w = w_packed;
  set_x_bf16(p, o_lat, static_cast<long long>(heads) * kv_lora);
  p.n_rows = heads * v_dim;
  p.n_tiles = p.n_rows / TB_TILE_ROWS;
  p.n_kb = kv_lora / TB_KBLOCK;
  p.w_kb_per_tile = p.n_kb;
  p.tiles_per_xseg = v_dim / TB_TILE_ROWS;
  p.n_tokens = tokens;
  set_region(p, 0, p.n_rows, out, p.n_rows);
  return launch_gemv(ctx, p, st);
}

extern "C" int tilert_unproj_o_allreduce_op(TbContext* ctx, const void* vec, const uint8_t* w_packed,
                                            const void* x_residual, int tokens, int k, int n, void* out,
                                            TbComm* comm, void* stream) {
  TB_REQUIRE(ctx != nullptr && vec != nullptr && w_packed != nullptr && out != nullptr);
  TB_REQUIRE(k % TB_KBLOCK == 0);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  TB_REQUIRE(tokens >= 1 && tokens <= 4);
  int rc = TB_OK;
  GemvParams p;
  gemv_defaults(p);
  p.w = w_packed;
  set_x_bf16(p, vec, k);
  p.n_rows = n;
  p.n_tiles = (n + TB_TILE_ROWS - 1) / TB_TILE_ROWS;
  p.n_kb = k / TB_KBLOCK;
  p.w_kb_per_tile = p.n_kb;
  p.n_tokens = tokens;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(x_residual);
  p.residual_stride = n;
  set_region(p, 0, n, out, n);
  rc = set_comm(p, comm, n);
  if (rc != TB_OK) return rc;
  return launch_gemv(ctx, p, st);
}

extern "C" int tilert_expert_select_up_gate_silu_op(TbContext* ctx, const void* hidden, const float* gamma, float eps,
                                                    const float* scores, const float* bias, const uint8_t* w_packed,
                                                    long long expert_stride, int tokens, int dim, int inter,
                                                    int n_experts, int n_groups, int n_limited_groups, int top_k,
                                                    float route_scale, void* hidden_out, float* probs_out,
                                                    int* idx_out, int* slot_ids, float* slot_w, void* stream) {
  TB_REQUIRE(ctx != nullptr && hidden != nullptr && scores != nullptr && w_packed != nullptr);
  TB_REQUIRE(hidden_out != nullptr && probs_out != nullptr && idx_out != nullptr && tokens >= 1 && tokens <= 4);
  TB_REQUIRE(n_experts <= 256 && top_k <= 31 && (n_groups == 1 || (32 % n_groups == 0 && n_experts % 32 == 0)));
  TB_REQUIRE((2 * inter) % TB_TILE_ROWS == 0 && dim % TB_KBLOCK == 0);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (slot_ids == nullptr) slot_ids = reinterpret_cast<int*>(ctx->small);
  if (slot_w == nullptr) slot_w = reinterpret_cast<float*>(ctx->small + 4096);
  const int n_slots = top_k + 1;
  ctx->moe_flat_owner = nullptr;
  auto base = [&](GemvParams& p) {
    gemv_defaults(p);
    p.w = w_packed;
    set_x_bf16(p, hidden, dim, gamma, eps);
    p.tiles_per_nseg = 2 * inter / TB_TILE_ROWS;
    p.n_kb = dim / TB_KBLOCK;
    p.w_kb_per_tile = p.n_kb;
    p.expert_stride = expert_stride;
    p.n_tokens = tokens;
    p.epi = EPI_SILU_MUL;
  };
  auto route = [&](GemvParams& p, int t) {
    p.route.scores = scores + static_cast<long long>(t) * n_experts;
    p.route.bias = bias;
    p.route.n_experts = n_experts;
    p.route.n_groups = n_groups;
    p.route.n_limited = n_limited_groups;
    p.route.top_k = top_k;
    p.route.route_scale = route_scale;
    p.route.shared_id = n_experts;
    p.route.probs = probs_out + t * top_k;
    p.route.ids = idx_out + t * top_k;
    p.route.slot_ids = slot_ids + t * n_slots;
    p.route.slot_w = slot_w + t * n_slots;
  };
  if (ctx->rec.active) {
    // Chained: the shared expert (static addresses, every token at once) is a phase of its own, so that
    // the stream covers the routing; then one phase per token for its routed experts, each routed by the
    // producer warps themselves.
    GemvParams ps;
    base(ps);
    ps.w = w_packed + static_cast<long long>(n_experts) * expert_stride;
    ps.tiles_per_nseg = 0;
    ps.n_tiles = 2 * inter / TB_TILE_ROWS;
    ps.n_rows = inter;
    set_region(ps, 0, inter, hidden_out, static_cast<long long>(n_slots) * inter);
    int rc = launch_gemv(ctx, ps, st);
    if (rc != TB_OK) return rc;
    for (int t = 0; t < tokens; ++t) {
      GemvParams p;
      base(p);
      route(p, t);
      p.route.slot_base = 1;
      p.n_tiles = top_k * p.tiles_per_nseg;
      p.only_token = tokens > 1 ? t : -1;
      p.n_rows = top_k * inter;
      set_region(p, 0, p.n_rows, reinterpret_cast<__nv_bfloat16*>(hidden_out) + inter, static_cast<long long>(n_slots) * inter);
      rc = launch_gemv(ctx, p, st);
      if (rc != TB_OK) return rc;
    }
    return TB_OK;
  }
  // One token: the product launch routes the token itself.
  if (tokens == 1) {
    GemvParams p;
    base(p);
    p.n_tiles = n_slots * p.tiles_per_nseg;
    route(p, 0);
    p.n_rows = n_slots * inter;
    set_region(p, 0, p.n_rows, hidden_out, p.n_rows);
    return launch_gemv(ctx, p, st);
  }
  // Several tokens: a routing launch, then ONE product launch over the flat slot list [shared, token 0's experts,
  // token 1's experts, ...].  Every slot's rows are computed for every token anyway (the tokens are columns of the
  // same activation block), so all of them are stored in the context's flat buffer, where the down product finds
  // its input; hidden_out [tokens][top_k + 1][inter] gets the shared rows of every token and, of the routed slots,
  // the owning token's rows only.
  const int n_flat = 1 + tokens * top_k;
  TB_REQUIRE(static_cast<size_t>(tokens) * n_flat * inter * 2 <= kMoeFlatBytes);
  int* flat_ids = reinterpret_cast<int*>(ctx->small + 16384);      // [n_flat]
  float* flat_w = reinterpret_cast<float*>(ctx->small + 16896);    // [tokens][n_flat]
  TB_CUDA(launch(expert_select_kernel, dim3((tokens + 3) / 4), dim3(128), 0, st, scores, bias, n_experts, n_groups,
                 n_limited_groups, top_k, route_scale, n_experts, probs_out, idx_out, slot_ids, slot_w, tokens, flat_ids,
                 flat_w));
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  GemvParams p;
  base(p);
  p.n_tiles = n_flat * p.tiles_per_nseg;
  p.nseg_ids = flat_ids;
  p.n_rows = n_flat * inter;
  __nv_bfloat16* ho = reinterpret_cast<__nv_bfloat16*>(hidden_out);
  set_region(p, 0, p.n_rows, ctx->moe_flat, static_cast<long long>(n_flat) * inter);
  set_region(p, 0, inter, ho, static_cast<long long>(n_slots) * inter);
  // routed slot 1 + t * top_k + j of the flat list is slot 1 + j of token t: row r goes to r + t * inter
  set_region(p, inter, tokens * top_k * inter, ho + inter, inter);
  p.regions[2].tok_div = top_k;
  p.regions[2].slot_rows = inter;
  int rc = launch_gemv(ctx, p, st);
  if (rc != TB_OK) return rc;
  ctx->moe_flat_owner = hidden_out;
  ctx->moe_flat_tokens = tokens;
  ctx->moe_flat_inter = inter;
  ctx->moe_flat_topk = top_k;
  return TB_OK;
}

extern "C" int tilert_expert_down_allreduce_op(TbContext* ctx, const void* vec, const uint8_t* w_packed,
                                               long long expert_stride, const int* slot_ids, const float* slot_w,
                                               const void* x_residual, int tokens, int inter, int dim, int n_slots,
                                               void* out, TbComm* comm, void* stream) {
  TB_REQUIRE(ctx != nullptr && vec != nullptr && w_packed != nullptr && out != nullptr);
  TB_REQUIRE(inter % TB_KBLOCK == 0);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (slot_ids == nullptr) slot_ids = reinterpret_cast<const int*>(ctx->small);
  if (slot_w == nullptr) slot_w = reinterpret_cast<const float*>(ctx->small + 4096);
  TB_REQUIRE(tokens >= 1 && tokens <= 4);
  int rc = TB_OK;
  if (tokens > 1 && !ctx->rec.active && ctx->moe_flat_owner == vec && ctx->moe_flat_tokens == tokens &&
      ctx->moe_flat_inter == inter && ctx->moe_flat_topk == n_slots - 1) {
    // Several tokens in one launch: the K dimension is the flat slot list of the gate/up launch that produced
    // `vec` (its flat buffer holds every token's column for every slot); a token's weight is its routing weight
    // at its own slots, 1 at the shared slot and 0 at the other tokens' slots.
    const int n_flat = 1 + tokens * (n_slots - 1);
    GemvParams p;
    gemv_defaults(p);
    p.w = w_packed;
    set_x_bf16(p, ctx->moe_flat, static_cast<long long>(n_flat) * inter, nullptr, 0.f,
               reinterpret_cast<const float*>(ctx->small + 16896));
    p.n_rows = dim;
    p.n_tiles = (dim + TB_TILE_ROWS - 1) / TB_TILE_ROWS;
    p.kb_per_kseg = inter / TB_KBLOCK;
    p.n_kb = n_flat * p.kb_per_kseg;
    p.w_kb_per_tile = p.kb_per_kseg;
    p.kseg_ids = reinterpret_cast<const int*>(ctx->small + 16384);
    p.expert_stride = expert_stride;
    p.n_tokens = tokens;
    p.residual = reinterpret_cast<const __nv_bfloat16*>(x_residual);
    p.residual_stride = dim;
    set_region(p, 0, dim, out, dim);
    rc = set_comm(p, comm, dim);
    if (rc != TB_OK) return rc;
    return launch_gemv(ctx, p, st);
  }
  for (int t = 0; t < tokens; ++t) {
    GemvParams p;
    gemv_defaults(p);
    p.w = w_packed;
    set_x_bf16(p, vec, static_cast<long long>(n_slots) * inter, nullptr, 0.f, slot_w);
    p.n_rows = dim;
    p.n_tiles = (dim + TB_TILE_ROWS - 1) / TB_TILE_ROWS;
    p.kb_per_kseg = inter / TB_KBLOCK;
    p.n_kb = n_slots * p.kb_per_kseg;
    p.w_kb_per_tile = p.kb_per_kseg;
    p.kseg_ids = slot_ids + t * n_slots;
    p.expert_stride = expert_stride;
    p.n_tokens = tokens;
    p.only_token = tokens > 1 ? t : -1;
    p.residual = reinterpret_cast<const __nv_bfloat16*>(x_residual);
    p.residual_stride = dim;
    set_region(p, 0, dim, out, dim);
    rc = set_comm(p, comm, dim);
    if (rc != TB_OK) return rc;
    rc = launch_gemv(ctx, p, st);
    if (rc != TB_OK) return rc;
  }
  return TB_OK;
}

extern "C" int tilert_rmsnorm_up_gate_silu_op(TbContext* ctx, const void* x, const float* gamma, float eps,
                                              const uint8_t* w_packed, int tokens, int dim, int inter, void* out,
                                              void* stream) {
  TB_REQUIRE(ctx != nullptr && x != nullptr && gamma != nullptr && w_packed != nullptr && out != nullptr);
  TB_REQUIRE((2 * inter) % TB_TILE_ROWS == 0);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  TB_REQUIRE(tokens >= 1 && tokens <= 4 && dim % TB_KBLOCK == 0);
  GemvParams p;
  gemv_defaults(p);
  p.w = w_packed;
  set_x_bf16(p, x, dim, gamma, eps);
  p.n_tiles = 2 * inter / TB_TILE_ROWS;
  p.n_kb = dim / TB_KBLOCK;
  p.w_kb_per_tile = p.n_kb;
  p.n_tokens = tokens;
  p.epi = EPI_SILU_MUL;
  p.n_rows = inter;
  set_region(p, 0, inter, out, inter);
  return launch_gemv(ctx, p, st);
}

extern "C" int tilert_rmsnorm_proj_rows2_op(TbContext* ctx, const void* x, const float* gamma, float eps,
                                            const uint8_t* w_packed, int tokens, int dim, int n, void* out,
                                            int out_is_f32, void* stream) {
  TB_REQUIRE(ctx != nullptr && x != nullptr && w_packed != nullptr && out != nullptr);
  TB_REQUIRE(tokens >= 1 && tokens <= 4 && dim % TB_KBLOCK == 0 && n >= 1);
  GemvParams p;
  gemv_defaults(p);
  p.w = w_packed;
  set_x_bf16(p, x, dim, gamma, eps);
  const int packed_rows = (n + 7) / 8 * 16;  // 8 leading-term rows + 8 residual-term rows per 8 source rows
  p.n_tiles = (packed_rows + TB_TILE_ROWS - 1) / TB_TILE_ROWS;
  p.n_kb = dim / TB_KBLOCK;
  p.w_kb_per_tile = p.n_kb;
  p.n_tokens = tokens;
  p.epi = EPI_ADD_PAIR;
  p.n_rows = n;
  set_region(p, 0, n, out, n, out_is_f32 ? 1 : 0);
  return launch_gemv(ctx, p, static_cast<cudaStream_t>(stream));
}

extern "C" int tilert_down_allreduce_op(TbContext* ctx, const void* vec, const uint8_t* w_packed,
                                        const void* x_residual, int tokens, int inter, int dim, void* out,
                                        TbComm* comm, void* stream) {
  return tilert_unproj_o_allreduce_op(ctx, vec, w_packed, x_residual, tokens, inter, dim, out, comm, stream);
}

// ------------------------------------------------------------------------------ bf16 products
namespace {
// The per-token vector work recorded into a chain: it runs on the converter warps beside the next recorded
// product, once that product's (and its own) inputs are complete.
int record_hook(TbContext* ctx, const AttnPrepParams& prep) {
  ChainRecorder& r = ctx->rec;
  if (r.pending_hook >= 0) return fail(TB_ESTATE, "chain: two attn_prep operators in a row (a product must follow each)%s");
  if (r.n_hooks >= kChainMaxHooks) return fail(TB_ESTATE, "chain: too many attn_prep operators in one chain%s");
  if (prep.wis.w != nullptr)
    return fail(TB_EINVAL, "chain: pass w_is = NULL to a recorded attn_prep (the head weights are a product of "
                           "their own, tilert_rmsnorm_proj_rows2_op)%s");
  ChainHook& h = r.params.hooks[r.n_hooks];
  h.kind = HOOK_ATTN_PREP;
  h.prep = prep;
  r.pending_hook = r.n_hooks++;
  return TB_OK;
}

int launch_gemv_bf16(TbContext* ctx, GemvBf16Params& p, cudaStream_t st) {
  TB_REQUIRE(p.n_tokens >= 1 && p.n_tokens <= 4);
  TB_REQUIRE(p.k % 256 == 0);
  if (ctx->rec.active)
    return fail(TB_ESTATE, "a bf16 row product cannot be recorded into a chain (pack the weight with "
                           "pack_bf16_two_term and use tilert_rmsnorm_proj_rows2_op)%s");
  const int tok_t = p.n_tokens == 1 ? 1 : (p.n_tokens == 2 ? 2 : 4);
  const size_t smem = static_cast<size_t>(tok_t) * p.k * sizeof(float);
  const int warps = kGemvBf16Threads / 32;
  int grid = (p.n + warps - 1) / warps;
  const int cap = ctx->num_sms * 2;
  if (grid > cap) grid = cap;
  static bool attr_set = false;
  if (!attr_set) {
    TB_CUDA(cudaFuncSetAttribute(gemv_bf16_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    TB_CUDA(cudaFuncSetAttribute(gemv_bf16_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    TB_CUDA(cudaFuncSetAttribute(gemv_bf16_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_set = true;
  }
  TB_REQUIRE(smem <= 200 * 1024);
  if (p.n <= 2048 && p.k <= 8192 && p.x2 == nullptr) {
    static bool attr2_set = false;
    if (!attr2_set) {
      TB_CUDA(cudaFuncSetAttribute(gemv_bf16_ksplit_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
      TB_CUDA(cudaFuncSetAttribute(gemv_bf16_ksplit_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
      TB_CUDA(cudaFuncSetAttribute(gemv_bf16_ksplit_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      attr2_set = true;
    }
    const int g2 = (p.n + kGemvBf16SmallRows - 1) / kGemvBf16SmallRows;
    if (tok_t == 1)
      TB_CUDA(launch(gemv_bf16_ksplit_kernel<1>, dim3(g2), dim3(kGemvBf16SmallThreads), smem, st, p));
    else if (tok_t == 2)
      TB_CUDA(launch(gemv_bf16_ksplit_kernel<2>, dim3(g2), dim3(kGemvBf16SmallThreads), smem, st, p));
    else
      TB_CUDA(launch(gemv_bf16_ksplit_kernel<4>, dim3(g2), dim3(kGemvBf16SmallThreads), smem, st, p));
  } else if (tok_t == 1)
    TB_CUDA(launch(gemv_bf16_kernel<1>, dim3(grid), dim3(kGemvBf16Threads), smem, st, p));
  else if (tok_t == 2)
    TB_CUDA(launch(gemv_bf16_kernel<2>, dim3(grid), dim3(kGemvBf16Threads), smem, st, p));
  else
    TB_CUDA(launch(gemv_bf16_kernel<4>, dim3(grid), dim3(kGemvBf16Threads), smem, st, p));
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  return TB_OK;
}
}  // namespace

extern "C" int tilert_proj_w_op(TbContext* ctx, const void* x, const float* gamma, float eps, const void* w,
                                int tokens, int n, int k, void* out, void* stream) {
  TB_REQUIRE(ctx != nullptr && x != nullptr && w != nullptr && out != nullptr);
  GemvBf16Params p{};
  p.gamma = gamma;
  p.eps = eps;
  p.w = w;
  p.n = n;
  p.k = k;
  p.x = reinterpret_cast<const __nv_bfloat16*>(x);
  p.x_stride = k;
  p.n_tokens = tokens;
  p.out = out;
  p.out_bf16 = 1;
  p.out_stride = n;
  return launch_gemv_bf16(ctx, p, static_cast<cudaStream_t>(stream));
}

extern "C" int tilert_rmsnorm_expert_proj_op(TbContext* ctx, const void* x, const float* gamma, float eps,
                                             const void* w_gate, int gate_is_f32, int tokens, int dim,
                                             int n_experts, float* scores_out, void* hidden_out, void* stream) {
  TB_REQUIRE(ctx != nullptr && x != nullptr && w_gate != nullptr && scores_out != nullptr);  // gamma == NULL: x is already normalised
  GemvBf16Params p{};
  p.w = w_gate;
  p.w_is_f32 = gate_is_f32;
  p.n = n_experts;
  p.k = dim;
  p.x = reinterpret_cast<const __nv_bfloat16*>(x);
  p.x_stride = dim;
  p.n_tokens = tokens;
  p.gamma = gamma;
  p.eps = eps;
  p.round_norm_bf16 = 1;
  p.xnorm_out = reinterpret_cast<__nv_bfloat16*>(hidden_out);
  p.xnorm_stride = dim;
  p.out = scores_out;
  p.out_stride = n_experts;
  return launch_gemv_bf16(ctx, p, static_cast<cudaStream_t>(stream));
}

extern "C" int tilert_rmsnorm_head_proj_op(TbContext* ctx, const void* x, const float* gamma, float eps,
                                           const void* w, int tokens, int dim, int vocab, void* x_norm_out,
                                           float* logits_out, void* stream) {
  TB_REQUIRE(ctx != nullptr && x != nullptr && gamma != nullptr && w != nullptr && logits_out != nullptr);
  GemvBf16Params p{};
  p.w = w;
  p.n = vocab;
  p.k = dim;
  p.x = reinterpret_cast<const __nv_bfloat16*>(x);
  p.x_stride = dim;
  p.n_tokens = tokens;
  p.gamma = gamma;
  p.eps = eps;
  p.round_norm_bf16 = 0;
  p.xnorm_out = reinterpret_cast<__nv_bfloat16*>(x_norm_out);
  p.xnorm_stride = dim;
  p.out = logits_out;
  p.out_stride = vocab;
  return launch_gemv_bf16(ctx, p, static_cast<cudaStream_t>(stream));
}

// Multi-token-prediction input: (optionally enorm / hnorm, then) concat and eh_proj [dim, 2*dim] bf16.
// At most two tokens fit the kernel's shared memory at 2*dim = 14336; more tokens take two launches.
namespace {
// Rows [row_begin, row_begin + n_rows) of the product (n_rows <= 0: all of them); `out` is the full [tokens, dim] tensor.
int launch_eh_proj(TbContext* ctx, const void* e, const void* h, const float* gamma_e, const float* gamma_h, float eps,
                   const void* w, int tokens, int dim, void* e_norm_out, void* h_norm_out, void* out,
                   cudaStream_t st, int row_begin = 0, int n_rows = 0) {
  TB_REQUIRE(tokens >= 1 && tokens <= 4 && dim % 128 == 0);
  if (n_rows <= 0) {
    row_begin = 0;
    n_rows = dim;
  }
  TB_REQUIRE(row_begin >= 0 && row_begin + n_rows <= dim);
  for (int t0 = 0; t0 < tokens; t0 += 2) {
    const int nt = tokens - t0 < 2 ? tokens - t0 : 2;
    GemvBf16Params p{};
    p.w = reinterpret_cast<const __nv_bfloat16*>(w) + static_cast<long long>(row_begin) * 2 * dim;
    p.n = n_rows;
    p.k = 2 * dim;
    p.k1 = dim;
    p.x = reinterpret_cast<const __nv_bfloat16*>(e) + static_cast<long long>(t0) * dim;
    p.x_stride = dim;
    p.x2 = reinterpret_cast<const __nv_bfloat16*>(h) + static_cast<long long>(t0) * dim;
    p.x2_stride = dim;
    p.n_tokens = nt;
    p.gamma = gamma_e;
    p.gamma2 = gamma_h;
    p.eps = eps;
    p.round_norm_bf16 = 1;
    if (e_norm_out != nullptr) p.xnorm_out = reinterpret_cast<__nv_bfloat16*>(e_norm_out) + static_cast<long long>(t0) * dim;
    p.xnorm_stride = dim;
    if (h_norm_out != nullptr) p.xnorm2_out = reinterpret_cast<__nv_bfloat16*>(h_norm_out) + static_cast<long long>(t0) * dim;
    p.xnorm2_stride = dim;
    p.out = reinterpret_cast<__nv_bfloat16*>(out) + static_cast<long long>(t0) * dim + row_begin;
    p.out_bf16 = 1;
    p.out_stride = dim;
    const int rc = launch_gemv_bf16(ctx, p, st);
    if (rc != TB_OK) return rc;
  }
  return TB_OK;
}
}  // namespace

extern "C" int tilert_eh_proj_allreduce_op(TbContext* ctx, const void* e_norm, const void* h_norm, const void* w,
                                           int tokens, int dim, void* out, void* stream) {
  TB_REQUIRE(ctx != nullptr && e_norm != nullptr && h_norm != nullptr && w != nullptr && out != nullptr);
  return launch_eh_proj(ctx, e_norm, h_norm, nullptr, nullptr, 0.f, w, tokens, dim, nullptr, nullptr, out,
                        static_cast<cudaStream_t>(stream));
}

extern "C" int tilert_mtp_preprocess_op(TbContext* ctx, const void* e, const void* h, const float* gamma_e,
                                        const float* gamma_h, float eps, const void* w, int tokens, int dim,
                                        void* e_norm_out, void* h_norm_out, void* out, void* stream) {
  TB_REQUIRE(ctx != nullptr && e != nullptr && h != nullptr && gamma_e != nullptr && gamma_h != nullptr);
  TB_REQUIRE(w != nullptr && out != nullptr);
  return launch_eh_proj(ctx, e, h, gamma_e, gamma_h, eps, w, tokens, dim, e_norm_out, h_norm_out, out,
                        static_cast<cudaStream_t>(stream));
}

extern "C" int tilert_padded_allreduce_add_op(TbContext* ctx, const void* partial, const void* x_residual, int tokens,
                                              int n, void* out, TbComm* comm, void* stream) {
  TB_NOT_CHAINABLE(ctx);
  TB_REQUIRE(ctx != nullptr && partial != nullptr && out != nullptr && tokens >= 1 && tokens <= 4 && n >= 1);
  ArAddParams p{};
  p.partial = reinterpret_cast<const __nv_bfloat16*>(partial);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(x_residual);
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.n_tokens = tokens;
  p.n_rows = n;
  p.ar.world = 1;
  p.status = ctx->status;
  if (comm != nullptr && comm->world > 1) {
    TB_REQUIRE(n == comm->max_rows);  // slot stride of the receive buffers
    p.ar.world = comm->world;
    p.ar.rank = comm->rank;
    const size_t off = comm_state_offset(comm->world, comm->max_rows);
    for (int r = 0; r < comm->world; ++r) p.ar.recv[r] = reinterpret_cast<unsigned long long*>(comm->buffers[r]);
    p.ar.state = reinterpret_cast<AllReduceState*>(reinterpret_cast<uint8_t*>(comm->buffers[comm->rank]) + off);
  }
  const int grid = std::max(1, std::min(16, (tokens * n + 4 * kArAddThreads - 1) / (4 * kArAddThreads)));
  TB_CUDA(launch(allreduce_add_kernel, dim3(grid), dim3(kArAddThreads), 0, static_cast<cudaStream_t>(stream), p));
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  return TB_OK;
}

extern "C" int tilert_mtp_preprocess_rows_op(TbContext* ctx, const void* e, const void* h, const float* gamma_e,
                                             const float* gamma_h, float eps, const void* w, int tokens, int dim,
                                             int row_begin, int n_rows, void* e_norm_out, void* h_norm_out, void* out,
                                             void* stream) {
  TB_REQUIRE(ctx != nullptr && e != nullptr && h != nullptr && gamma_e != nullptr && gamma_h != nullptr);
  TB_REQUIRE(w != nullptr && out != nullptr && n_rows >= 1);
  return launch_eh_proj(ctx, e, h, gamma_e, gamma_h, eps, w, tokens, dim, e_norm_out, h_norm_out, out,
                        static_cast<cudaStream_t>(stream), row_begin, n_rows);
}

// -------------------------------------------------------------------- per-token vector operators
extern "C" int tilert_rmsnorm_kv_op(TbContext* ctx, const void* kv, const float* gamma, float eps, int tokens,
                                    int dim, const int* cur_pos, void* kv_cache, int cache_rows, void* stream) {
  TB_NOT_CHAINABLE(ctx);
  TB_REQUIRE(ctx != nullptr && kv != nullptr && gamma != nullptr && cur_pos != nullptr && kv_cache != nullptr);
  rmsnorm_kv_kernel<<<(tokens + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(kv), dim, gamma, eps, dim, cur_pos,
      reinterpret_cast<__nv_bfloat16*>(kv_cache), tokens, cache_rows, ctx->status);
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  return TB_OK;
}

extern "C" int tilert_qkv_rope_op(TbContext* ctx, void* q_pe, int heads, int rope, void* pe_cache,
                                  const int* cur_pos, const float* freqs, int tokens, int cache_rows, void* stream) {
  TB_NOT_CHAINABLE(ctx);
  TB_REQUIRE(ctx != nullptr && q_pe != nullptr && pe_cache != nullptr && cur_pos != nullptr && freqs != nullptr);
  const int total = tokens * (heads + 1) * (rope / 2);
  qkv_rope_kernel<<<(total + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(q_pe), heads, rope, reinterpret_cast<__nv_bfloat16*>(pe_cache), cur_pos,
      freqs, tokens, cache_rows, ctx->status);
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  return TB_OK;
}

extern "C" int tilert_rotate_op(TbContext* ctx, const void* in, void* out, int heads, int rope, const float* freqs,
                                int tokens, void* stream) {
  TB_NOT_CHAINABLE(ctx);
  TB_REQUIRE(ctx != nullptr && in != nullptr && out != nullptr && freqs != nullptr);
  TB_REQUIRE(rope == 64);
  const int vecs = tokens * heads;
  rotate128_kernel<<<(vecs + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(in), reinterpret_cast<__nv_bfloat16*>(out), heads, rope, freqs, nullptr,
      nullptr, nullptr, tokens, 0, nullptr);
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  return TB_OK;
}

extern "C" int tilert_layernorm_rope_rotate_op(TbContext* ctx, const void* in, const int* cur_pos, void* k_cache,
                                               const float* weight, const float* bias, const float* freqs, int rope,
                                               int tokens, int cache_rows, void* stream) {
  TB_NOT_CHAINABLE(ctx);
  TB_REQUIRE(ctx != nullptr && in != nullptr && cur_pos != nullptr && k_cache != nullptr);
  TB_REQUIRE(weight != nullptr && bias != nullptr && freqs != nullptr && rope == 64);
  rotate128_kernel<<<(tokens + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(in), reinterpret_cast<__nv_bfloat16*>(k_cache), 1, rope, freqs, weight,
      bias, cur_pos, tokens, cache_rows, ctx->status);
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  return TB_OK;
}

extern "C" int tilert_attn_prep_op(TbContext* ctx, const void* x, const float* in_gamma, float eps, const void* w_is,
                                   int idx_heads, int dim, void* idx_w_out, const void* kv, const float* kv_gamma,
                                   int kv_dim, void* kv_cache, void* q_pe, int heads, int rope, void* pe_cache,
                                   const void* iq, void* iq_out, const void* ki, void* ki_cache, const float* ln_w,
                                   const float* ln_b, const float* freqs, const int* cur_pos, int tokens,
                                   int cache_rows, void* stream) {
  TB_REQUIRE(ctx != nullptr && kv != nullptr && (w_is == nullptr || (x != nullptr && idx_w_out != nullptr)));
  TB_REQUIRE(kv_gamma != nullptr && kv_cache != nullptr && q_pe != nullptr && pe_cache != nullptr && iq != nullptr);
  TB_REQUIRE(iq_out != nullptr && ki != nullptr && ki_cache != nullptr && ln_w != nullptr && ln_b != nullptr);
  TB_REQUIRE(freqs != nullptr && cur_pos != nullptr && tokens >= 1 && tokens <= 4 && rope == 64);
  TB_REQUIRE(dim % 256 == 0 && dim <= 8192);
  AttnPrepParams p{};
  p.wis.gamma = in_gamma;
  p.wis.eps = eps;
  p.wis.w = w_is;
  p.wis.n = idx_heads;
  p.wis.k = dim;
  p.wis.x = reinterpret_cast<const __nv_bfloat16*>(x);
  p.wis.x_stride = dim;
  p.wis.n_tokens = tokens;
  p.wis.out = idx_w_out;
  p.wis.out_bf16 = 1;
  p.wis.out_stride = idx_heads;
  constexpr int kWarps = kAttnPrepThreads / 32;
  p.wis_blocks = w_is != nullptr ? (idx_heads + kGemvBf16SmallRows - 1) / kGemvBf16SmallRows : 0;
  p.kv = reinterpret_cast<const __nv_bfloat16*>(kv);
  p.kv_stride = kv_dim;
  p.kv_gamma = kv_gamma;
  p.kv_eps = eps;
  p.kv_dim = kv_dim;
  p.kv_cache = reinterpret_cast<__nv_bfloat16*>(kv_cache);
  p.kv_blocks = (tokens + kWarps - 1) / kWarps;
  p.q_pe = reinterpret_cast<__nv_bfloat16*>(q_pe);
  p.heads = heads;
  p.rope = rope;
  p.pe_cache = reinterpret_cast<__nv_bfloat16*>(pe_cache);
  p.rope_blocks = (tokens * (heads + 1) * (rope / 2) + kAttnPrepThreads - 1) / kAttnPrepThreads;
  p.iq = reinterpret_cast<const __nv_bfloat16*>(iq);
  p.iq_out = reinterpret_cast<__nv_bfloat16*>(iq_out);
  p.idx_heads = idx_heads;
  p.iq_blocks = (tokens * idx_heads + kWarps - 1) / kWarps;
  p.ki = reinterpret_cast<const __nv_bfloat16*>(ki);
  p.ki_cache = reinterpret_cast<__nv_bfloat16*>(ki_cache);
  p.ln_w = ln_w;
  p.ln_b = ln_b;
  p.ki_blocks = (tokens + kWarps - 1) / kWarps;
  p.pos = cur_pos;
  p.freqs = freqs;
  p.n_tokens = tokens;
  p.cache_rows = cache_rows;
  p.status = ctx->status;
  static bool attr_set[64] = {};
  if (!attr_set[ctx->device & 63]) {
    TB_CUDA(cudaFuncSetAttribute(attn_prep_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    TB_CUDA(cudaFuncSetAttribute(attn_prep_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    TB_CUDA(cudaFuncSetAttribute(attn_prep_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_set[ctx->device & 63] = true;
  }
  if (ctx->rec.active) return record_hook(ctx, p);
  const int grid = p.wis_blocks + p.kv_blocks + p.rope_blocks + p.iq_blocks + p.ki_blocks;
  const int tok = tokens == 1 ? 1 : (tokens == 2 ? 2 : 4);
  const size_t smem = static_cast<size_t>(tok) * dim * sizeof(float);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (tok == 1)
    TB_CUDA(launch(attn_prep_kernel<1>, dim3(grid), dim3(kAttnPrepThreads), smem, st, p));
  else if (tok == 2)
    TB_CUDA(launch(attn_prep_kernel<2>, dim3(grid), dim3(kAttnPrepThreads), smem, st, p));
  else
    TB_CUDA(launch(attn_prep_kernel<4>, dim3(grid), dim3(kAttnPrepThreads), smem, st, p));
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  return TB_OK;
}

// ------------------------------------------------------------------ indexer and sparse attention
extern "C" int tilert_sparse_index_op(TbContext* ctx, const void* q, const void* k_cache, const void* weights,
                                      float* logits, long long logits_stride, int heads, int tokens, int n_keys,
                                      const int* cur_pos, void* stream) {
  TB_NOT_CHAINABLE(ctx);
  TB_REQUIRE(ctx != nullptr && q != nullptr && k_cache != nullptr && weights != nullptr && logits != nullptr);
  TB_REQUIRE(cur_pos != nullptr && n_keys > 0 && (heads == 16 || heads == 32 || heads == 64));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid((n_keys + 63) / 64, tokens);
  const size_t smem = static_cast<size_t>(heads + 64) * kIdxPitch * 2;
  const __nv_bfloat16* qq = reinterpret_cast<const __nv_bfloat16*>(q);
  const __nv_bfloat16* kk = reinterpret_cast<const __nv_bfloat16*>(k_cache);
  const __nv_bfloat16* ww = reinterpret_cast<const __nv_bfloat16*>(weights);
  if (heads == 64)
    TB_CUDA(launch(indexer_logits_kernel<64>, dim3(grid), dim3(kIdxWarps * 32), smem, st, qq, kk, ww, logits, logits_stride, n_keys, cur_pos, 0));
  else if (heads == 32)
    TB_CUDA(launch(indexer_logits_kernel<32>, dim3(grid), dim3(kIdxWarps * 32), smem, st, qq, kk, ww, logits, logits_stride, n_keys, cur_pos, 0));
  else
    TB_CUDA(launch(indexer_logits_kernel<16>, dim3(grid), dim3(kIdxWarps * 32), smem, st, qq, kk, ww, logits, logits_stride, n_keys, cur_pos, 0));
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  return TB_OK;
}

extern "C" int tilert_topk_accurate_op(TbContext* ctx, const float* logits, long long logits_stride, int rows, int n,
                                       int k, int* indices, void* stream) {
  TB_NOT_CHAINABLE(ctx);
  TB_REQUIRE(ctx != nullptr && logits != nullptr && indices != nullptr && rows >= 1 && n >= 0 && k >= 1);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long out_stride = k;
  if (n <= kTopkThreads * 4)
    TB_CUDA(launch(topk_radix_reg_kernel<4>, dim3(rows), dim3(kTopkThreads), 0, st, logits, logits_stride, n, k, indices,
                   out_stride));
  else if (n <= kTopkThreads * 8)
    TB_CUDA(launch(topk_radix_reg_kernel<8>, dim3(rows), dim3(kTopkThreads), 0, st, logits, logits_stride, n, k, indices,
                   out_stride));
  else
    TB_CUDA(launch(topk_radix_kernel, dim3(rows), dim3(kTopkThreads), 0, st, logits, logits_stride, n, k, indices,
                   out_stride));
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  return TB_OK;
}

extern "C" int tilert_sparse_index_topk_op(TbContext* ctx, const void* q, const void* k_cache, const void* weights,
                                           float* logits, long long logits_stride, int heads, int tokens, int n_keys,
                                           const int* cur_pos, int k, int* indices, void* stream) {
  TB_NOT_CHAINABLE(ctx);
  TB_REQUIRE(ctx != nullptr && q != nullptr && k_cache != nullptr && weights != nullptr && logits != nullptr);
  TB_REQUIRE(cur_pos != nullptr && indices != nullptr && n_keys > 0 && k >= 1 && tokens >= 1 && tokens <= 8);
  TB_REQUIRE(heads == 16 || heads == 32 || heads == 64);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* qq = reinterpret_cast<const __nv_bfloat16*>(q);
  const __nv_bfloat16* kk = reinterpret_cast<const __nv_bfloat16*>(k_cache);
  const __nv_bfloat16* ww = reinterpret_cast<const __nv_bfloat16*>(weights);
  const long long out_stride = k;
  static bool attr_set[64] = {};
  constexpr size_t kIdxSelSmemMax = 200 * 1024;
  if (!attr_set[ctx->device & 63]) {
    TB_CUDA(cudaFuncSetAttribute(indexer_topk_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    TB_CUDA(cudaFuncSetAttribute(indexer_topk_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    TB_CUDA(cudaFuncSetAttribute(indexer_topk_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    TB_CUDA(cudaFuncSetAttribute(indexer_select_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, kIdxSelSmemMax));
    TB_CUDA(cudaFuncSetAttribute(indexer_select_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, kIdxSelSmemMax));
    TB_CUDA(cudaFuncSetAttribute(indexer_select_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kIdxSelSmemMax));
    attr_set[ctx->device & 63] = true;
  }
  if (n_keys <= kIdxFusedThreads * 16) {
    // short rows: the last thread block of a token selects, the row in its registers
    const dim3 grid((n_keys + kIdxFusedKeys - 1) / kIdxFusedKeys, tokens);
    const size_t smem = static_cast<size_t>(heads + kIdxFusedKeys) * kIdxPitch * 2;
    unsigned* done = reinterpret_cast<unsigned*>(ctx->small + 8192);  // [8], zero between launches
    if (heads == 64)
      TB_CUDA(launch(indexer_topk_kernel<64>, grid, dim3(kIdxFusedThreads), smem, st, qq, kk, ww, logits, logits_stride, n_keys, cur_pos, k, indices, out_stride, done));
    else if (heads == 32)
      TB_CUDA(launch(indexer_topk_kernel<32>, grid, dim3(kIdxFusedThreads), smem, st, qq, kk, ww, logits, logits_stride, n_keys, cur_pos, k, indices, out_stride, done));
    else
      TB_CUDA(launch(indexer_topk_kernel<16>, grid, dim3(kIdxFusedThreads), smem, st, qq, kk, ww, logits, logits_stride, n_keys, cur_pos, k, indices, out_stride, done));
    ++g_launches;
    TB_CUDA(cudaGetLastError());
    return TB_OK;
  }
  // scoring and selection in one cooperative launch: at most one thread block per SM over all tokens, every block
  // a contiguous range of keys (a multiple of 16)
  int sel_sms = std::min(kIdxSelMaxCtas, ctx->num_sms);
  if (ctx->grid_limit > 0) sel_sms = std::min(sel_sms, ctx->grid_limit);  // SMs left to a concurrent streaming launch
  const int max_g = std::max(1, sel_sms / tokens);
  const int n_ctas = std::min((n_keys + kIdxFusedKeys - 1) / kIdxFusedKeys, max_g);
  const int keys_per_cta = (((n_keys + n_ctas - 1) / n_ctas) + 15) & ~15;
  const dim3 grid(n_ctas, tokens);
  const size_t smem = static_cast<size_t>(heads + kIdxFusedKeys) * kIdxPitch * 2 + static_cast<size_t>(keys_per_cta) * 4;
  if (smem > kIdxSelSmemMax) return fail(TB_EINVAL, "sparse_index_topk: too many keys per thread block for its shared memory%s");
  if (heads == 64)
    TB_CUDA(launch(indexer_select_kernel<64>, grid, dim3(kIdxFusedThreads), smem, st, qq, kk, ww, logits, logits_stride, n_keys, cur_pos, k, indices, out_stride, ctx->idx_work, keys_per_cta, ctx->status));
  else if (heads == 32)
    TB_CUDA(launch(indexer_select_kernel<32>, grid, dim3(kIdxFusedThreads), smem, st, qq, kk, ww, logits, logits_stride, n_keys, cur_pos, k, indices, out_stride, ctx->idx_work, keys_per_cta, ctx->status));
  else
    TB_CUDA(launch(indexer_select_kernel<16>, grid, dim3(kIdxFusedThreads), smem, st, qq, kk, ww, logits, logits_stride, n_keys, cur_pos, k, indices, out_stride, ctx->idx_work, keys_per_cta, ctx->status));
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  return TB_OK;
}

namespace {
// The attention launch, then the merge of its chunks: alone, or fused with the value up-projection (w_v != NULL).
int launch_sparse_mla(TbContext* ctx, const void* q, const void* q_pe, const void* kv, const void* k_pe,
                      const int* indices, int topk, const int* cur_pos, int heads, int tokens, int n_cache,
                      float softmax_scale, int split_size, void* out, float* out_acc, float* lse, float* lse_acc,
                      const uint8_t* w_v, void* o_out, cudaStream_t st) {
  TB_NOT_CHAINABLE(ctx);
  TB_REQUIRE(ctx != nullptr && q != nullptr && q_pe != nullptr && kv != nullptr && k_pe != nullptr);
  TB_REQUIRE(indices != nullptr && cur_pos != nullptr && out_acc != nullptr && lse_acc != nullptr);
  TB_REQUIRE(split_size > 0 && split_size % kMlaKeys == 0 && topk > 0);
  TB_REQUIRE(w_v != nullptr ? o_out != nullptr : out != nullptr);
  static bool attr_set = false;
  if (!attr_set) {
    TB_CUDA(cudaFuncSetAttribute(sparse_mla_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmemBytes));
    TB_CUDA(cudaFuncSetAttribute(sparse_mla_combine_vproj_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kMlaCvSmemBytes));
    attr_set = true;
  }
  MlaParams p{};
  p.q_lat = reinterpret_cast<const __nv_bfloat16*>(q);
  p.q_pe = reinterpret_cast<const __nv_bfloat16*>(q_pe);
  p.kv = reinterpret_cast<const __nv_bfloat16*>(kv);
  p.pe = reinterpret_cast<const __nv_bfloat16*>(k_pe);
  p.idx = indices;
  p.topk = topk;
  p.heads = heads;
  p.n_cache = n_cache;
  p.pos = cur_pos;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.blocks_per_split = split_size / kMlaKeys;
  p.n_splits = (topk + split_size - 1) / split_size;
  TB_REQUIRE(p.n_splits <= 64);
  p.o_acc = out_acc;
  p.lse_acc = lse_acc;
  p.status = ctx->status;
  const dim3 grid(p.n_splits, (heads + kMlaHeads - 1) / kMlaHeads, tokens);
  TB_CUDA(launch(sparse_mla_kernel, dim3(grid), dim3(kMlaThreads), kMlaSmemBytes, st, p));
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  if (w_v != nullptr)
    TB_CUDA(launch(sparse_mla_combine_vproj_kernel, dim3(dim3(heads, tokens)), dim3(128), kMlaCvSmemBytes, st, out_acc,
                   lse_acc, p.n_splits, reinterpret_cast<__nv_bfloat16*>(out), lse, w_v,
                   reinterpret_cast<__nv_bfloat16*>(o_out), ctx->status));
  else
    TB_CUDA(launch(sparse_mla_combine_kernel, dim3(dim3(heads, tokens)), dim3(128), 0, st, out_acc, lse_acc, p.n_splits,
                   reinterpret_cast<__nv_bfloat16*>(out), lse));
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  return TB_OK;
}
}  // namespace

extern "C" int tilert_flash_sparse_mla_op(TbContext* ctx, const void* q, const void* q_pe, const void* kv,
                                          const void* k_pe, const int* indices, int topk, const int* cur_pos,
                                          int heads, int tokens, int n_cache, float softmax_scale, int split_size,
                                          void* out, float* out_acc, float* lse, float* lse_acc, void* stream) {
  return launch_sparse_mla(ctx, q, q_pe, kv, k_pe, indices, topk, cur_pos, heads, tokens, n_cache, softmax_scale,
                           split_size, out, out_acc, lse, lse_acc, nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int tilert_flash_sparse_mla_vproj_op(TbContext* ctx, const void* q, const void* q_pe, const void* kv,
                                                const void* k_pe, const int* indices, int topk, const int* cur_pos,
                                                int heads, int tokens, int n_cache, float softmax_scale,
                                                int split_size, void* out, float* out_acc, float* lse, float* lse_acc,
                                                const uint8_t* w_v_packed, int kv_lora, int v_dim, void* o_out,
                                                void* stream) {
  TB_REQUIRE(w_v_packed != nullptr && o_out != nullptr && kv_lora == kMlaDV && v_dim == TB_TILE_ROWS);
  return launch_sparse_mla(ctx, q, q_pe, kv, k_pe, indices, topk, cur_pos, heads, tokens, n_cache, softmax_scale,
                           split_size, out, out_acc, lse, lse_acc, w_v_packed, o_out, static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------------------ sampling
extern "C" int tilert_sample_op(TbContext* ctx, const float* logits, long long logits_stride, int tokens, int vocab,
                                const float* config_dev, unsigned long long seed, unsigned long long* step_dev,
                                unsigned long long step_value, int* token_out, float* token_logprob_out,
                                float* topn_logprob_out, int* topn_index_out, void* stream) {
  TB_NOT_CHAINABLE(ctx);
  TB_REQUIRE(ctx != nullptr && logits != nullptr && config_dev != nullptr && token_out != nullptr);
  TB_REQUIRE(tokens >= 1 && vocab >= 1 && logits_stride >= vocab);
  TB_REQUIRE((topn_logprob_out == nullptr) == (topn_index_out == nullptr));
  SampleParams p{};
  p.logits = logits;
  p.stride = logits_stride;
  p.vocab = vocab;
  p.config = config_dev;
  p.seed = seed;
  p.step = step_dev;
  p.step_value = step_value;
  p.token = token_out;
  p.token_logprob = token_logprob_out;
  p.topn_logprob = topn_logprob_out;
  p.topn_index = topn_index_out;
  TB_CUDA(launch(sample_kernel, dim3(tokens), dim3(kTopkThreads), 0, static_cast<cudaStream_t>(stream), p));
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  return TB_OK;
}

// ------------------------------------------------------------------ cache injection (FP8 wire format)
extern "C" int tilert_inject_cache_fp8_op(TbContext* ctx, const uint8_t* kv_raw, const uint8_t* pe_raw,
                                          const uint8_t* ki_pages, int seq_len, int start_pos, int cache_rows,
                                          void* kv_cache, void* pe_cache, void* ki_cache, void* stream) {
  TB_NOT_CHAINABLE(ctx);
  TB_REQUIRE(ctx != nullptr && seq_len >= 0 && start_pos >= 0 && start_pos + seq_len <= cache_rows);
  TB_REQUIRE((kv_raw == nullptr) == (kv_cache == nullptr) && (pe_raw == nullptr) == (pe_cache == nullptr) &&
             (ki_pages == nullptr) == (ki_cache == nullptr));
  TB_REQUIRE(reinterpret_cast<uintptr_t>(kv_raw) % 16 == 0 && reinterpret_cast<uintptr_t>(pe_raw) % 4 == 0 &&
             reinterpret_cast<uintptr_t>(ki_pages) % 4 == 0 && reinterpret_cast<uintptr_t>(kv_cache) % 16 == 0);
  if (seq_len == 0) return TB_OK;
  CacheInjectParams p{};
  p.kv_raw = kv_raw;
  p.pe_raw = pe_raw;
  p.ki_pages = ki_pages;
  p.seq_len = seq_len;
  p.start_pos = start_pos;
  p.kv_cache = reinterpret_cast<__nv_bfloat16*>(kv_cache);
  p.pe_cache = reinterpret_cast<__nv_bfloat16*>(pe_cache);
  p.ki_cache = reinterpret_cast<__nv_bfloat16*>(ki_cache);
  const int grid = (seq_len + kInjectWarps - 1) / kInjectWarps;
  TB_CUDA(launch(cache_inject_fp8_kernel, dim3(grid), dim3(kInjectWarps * 32), 0, static_cast<cudaStream_t>(stream), p));
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  return TB_OK;
}

// ------------------------------------------------------------------ greedy token across ranks
extern "C" int tilert_argmax_exchange_op(TbContext* ctx, const float* logits, long long logits_stride, int tokens,
                                         int n_local, int index_offset, TbComm* comm, long long* token_out,
                                         float* value_out, void* stream) {
  TB_NOT_CHAINABLE(ctx);
  TB_REQUIRE(ctx != nullptr && logits != nullptr && token_out != nullptr);
  TB_REQUIRE(tokens >= 1 && tokens <= 4 && n_local >= 1 && logits_stride >= n_local && index_offset >= 0);
  ArgmaxParams p{};
  p.logits = logits;
  p.stride = logits_stride;
  p.n_local = n_local;
  p.index_offset = index_offset;
  p.n_tokens = tokens;
  p.token_out = token_out;
  p.value_out = value_out;
  p.status = ctx->status;
  p.ar.world = 1;
  if (comm != nullptr && comm->world > 1) {
    TB_REQUIRE(comm->max_rows >= 2);
    p.slot_rows = comm->max_rows;
    p.ar.world = comm->world;
    p.ar.rank = comm->rank;
    const size_t off = comm_state_offset(comm->world, comm->max_rows);
    for (int r = 0; r < comm->world; ++r) p.ar.recv[r] = reinterpret_cast<unsigned long long*>(comm->buffers[r]);
    p.ar.state = reinterpret_cast<AllReduceState*>(reinterpret_cast<uint8_t*>(comm->buffers[comm->rank]) + off);
  }
  TB_CUDA(launch(argmax_exchange_kernel, dim3(1), dim3(kArgmaxThreads), 0, static_cast<cudaStream_t>(stream), p));
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  return TB_OK;
}

// ------------------------------------------------------------ allocation-free entry point
// Scratch for tilert_b200_matvec_fp8_static: partial sums of row tiles shared by several CTAs
// (kMaxGrid slots of 8 KB, every word tagged with the launch number), a status word, the ready flags
// of a launch's shared X blocks with their epoch, the X blocks themselves, and the launch number
// (last 256 bytes; never cleared, the kernel maintains it).  It lives in the library image, so every
// GPU that loads the library holds these ~2.4 MB until exit.
namespace {
constexpr int kStaticMaxTiles = 1024;                                   // rows <= 131072
constexpr int kStaticMaxKBlocks = 256;                                  // k <= 32768
constexpr size_t kStaticXBytes = static_cast<size_t>(kStaticMaxKBlocks) * TB_XBLK_BYTES;   // shared X blocks
constexpr size_t kStaticXFlagBytes = (kStaticMaxKBlocks + 64) * sizeof(unsigned);           // flags + epoch state
constexpr size_t kStaticLaunchCallsOffset = kPartialBytes + 256 + kStaticXFlagBytes + kStaticXBytes;
constexpr size_t kStaticScratchBytes = kStaticLaunchCallsOffset + 256;  // + the launch number (never cleared)
}  // namespace
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
struct StaticScratchView {
  unsigned char* base = nullptr;  // DEVICE address of g_static_scratch on this device
  int num_sms = 0;
};
StaticScratchView g_static_view[64];
std::mutex g_static_mutex;  // guards the one-time set-up per device
}  // namespace

extern "C" int tilert_b200_matvec_fp8_static(const void* x, const uint8_t* w_packed, const void* residual,
                                             int tokens, int k, int n, void* out, int* status_out_dev,
                                             void* stream) {
  TB_REQUIRE(x != nullptr && w_packed != nullptr && out != nullptr);
  TB_REQUIRE(tokens >= 1 && tokens <= 4 && k > 0 && k % TB_KBLOCK == 0 && n > 0);
  const int n_tiles = (n + TB_TILE_ROWS - 1) / TB_TILE_ROWS;
  if (n_tiles > kStaticMaxTiles)
    return fail(TB_EINVAL, "tilert_b200_matvec_fp8_static: n exceeds the static scratch (at most 131072 rows)%s");
  if (k / TB_KBLOCK > kStaticMaxKBlocks)
    return fail(TB_EINVAL, "tilert_b200_matvec_fp8_static: k exceeds the static scratch (at most 32768)%s");
  TB_REQUIRE(static_cast<long long>(n_tiles) * (k / TB_KBLOCK) < (1ll << 30));
  int device = 0;
  TB_CUDA(cudaGetDevice(&device));
  TB_REQUIRE(device >= 0 && device < 64);
  StaticScratchView& view = g_static_view[device];
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (view.base == nullptr) {
    // One-time set-up for this device (it must be the current device, which it is).  In host code
    // the array's name is only a handle: the address a kernel can use comes from the runtime.
    void* dev_addr = nullptr;
    TB_CUDA(cudaGetSymbolAddress(&dev_addr, g_static_scratch));
    int sms = 0;
    TB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    TB_CUDA(cudaFuncSetAttribute(wstream_gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvSmemBytes));
    view.num_sms = sms;
    view.base = static_cast<unsigned char*>(dev_addr);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* partial = reinterpret_cast<float*>(view.base);
  int* status = reinterpret_cast<int*>(view.base + kPartialBytes);
  // The array keeps whatever the previous call left: the status word must start at zero (the partial
  // sums need no clearing: stale words carry an older launch number).
  // The same goes for the X-block flags and their epoch state, which follow the status word.
  unsigned* xflags = reinterpret_cast<unsigned*>(view.base + kPartialBytes + 256);
  uint8_t* xshared = view.base + kPartialBytes + 256 + kStaticXFlagBytes;
  TB_CUDA(cudaMemsetAsync(status, 0, 256 + kStaticXFlagBytes, st));
  GemvParams p;
  gemv_defaults(p);
  p.w = w_packed;
  set_x_bf16(p, x, k);
  p.n_rows = n;
  p.n_tiles = n_tiles;
  p.n_kb = k / TB_KBLOCK;
  p.w_kb_per_tile = p.n_kb;
  p.n_tokens = tokens;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.residual_stride = n;
  set_region(p, 0, n, out, n);
  p.partial = partial;
  p.launch_calls = reinterpret_cast<unsigned long long*>(view.base + kStaticLaunchCallsOffset);
  p.status = status;
  p.xs = xshared;
  p.xflag = xflags;
  p.xstate = xflags + kStaticMaxKBlocks;
  const long long units = static_cast<long long>(p.n_tiles) * p.n_kb;
  int grid = view.num_sms < kMaxGrid ? view.num_sms : kMaxGrid;
  if (units < grid) grid = static_cast<int>(units);
  set_partition(p, grid);
  p.grid_eff = grid;
  p.shared_x = max_cta_units(p, grid) > kGemvStages ? 1 : 0;
  TB_CUDA(launch(wstream_gemv_kernel, dim3(grid), dim3(kGemvThreads), kGemvSmemBytes, st, p));
  ++g_launches;
  TB_CUDA(cudaGetLastError());
  if (status_out_dev != nullptr)
    TB_CUDA(cudaMemcpyAsync(status_out_dev, status, sizeof(int), cudaMemcpyDeviceToDevice, st));
  return TB_OK;
}
