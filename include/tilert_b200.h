/*
 * tilert_b200 -- C ABI of the B200-native batch-1 FP8 decode path.
 *
 * The reference library (libtilert_dsv32.so, loaded by tilert/__init__.py:43-77) registers its
 * kernels as PyTorch operators `torch.ops.tilert.<name>`; the Python wrappers under
 * tilert/models/deepseek_v3_2/ops/ are the only callers.  Every function below replaces one of
 * those operators (the wrapper's file:line is cited) with plain pointers and sizes, so it can be
 * bound from ctypes, a PyTorch extension or any other FFI.
 *
 * Conventions
 *   - every pointer is a CUDA device pointer on the context's device unless marked "host";
 *   - bf16 tensors are passed as `const void*` / `void*`, e4m3 bytes as `uint8_t*`;
 *   - outputs are caller-allocated (the reference operators also write into caller tensors);
 *   - `stream` is a `cudaStream_t`; calls are asynchronous on it;
 *   - the return value is 0 on success, a negative TB_E* code otherwise; `tilert_b200_last_error`
 *     gives the message.  A kernel that gives up on a bounded wait records a positive code in the
 *     context's device status word, read with `tilert_b200_status`;
 *   - a context owns scratch memory used by the calls made with it: calls made with one context must be
 *     ordered on one stream.  Whatever the context, streaming launches (every FP8 product, chained launches, the
 *     indexer's selection, `tilert_b200_matvec_fp8_static`) must not overlap on a device: each needs all of its
 *     thread blocks resident at once (they wait on one another, bounded), so two of them running side by side from
 *     different streams can each be left half resident, wait out their budget and return a status code.
 *
 * Weight operands named `*_packed` are in the library's block format (128x128 e4m3 tiles in
 * the tensor core's shared-memory operand order followed by their scales, see tilert_b200/csrc/formats.h); they are
 * produced from HF-format tensors (e4m3 weight + f32 `weight_scale_inv` per 128x128 block) by
 * `tilert_b200.pack`.  Activation operands named `xpack` are in the matching activation block
 * format, produced by the rmsnorm/pack operators below.
 */
#ifndef TILERT_B200_H_
#define TILERT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TB_OK 0
#define TB_ECUDA (-1)     /* a CUDA runtime call failed */
#define TB_EINVAL (-2)    /* bad argument (shape not supported, null pointer, ...) */
#define TB_ESTATE (-3)    /* library state error (no context, comm not set up) */

typedef struct TbContext TbContext;
typedef struct TbComm TbComm;

/* ---- runtime -------------------------------------------------------------------------- */

/* tilert_init_op / tilert_force_init_op (tilert/tilert_init.py:11-18): create the per-device
 * context (scratch for split tiles, status word). */
int tilert_b200_init(int device, TbContext** ctx_out);
int tilert_b200_destroy(TbContext* ctx);
/* The process-wide context of `device`, created on first use and never destroyed: what the ctypes binding and
 * the dispatcher registration library (libtilert_dsv32.so) both use, so that they share one set of scratch. */
int tilert_b200_default_context(int device, TbContext** ctx_out);
/* Reads and clears the device status word (synchronises the device).  0 = no kernel gave up. */
int tilert_b200_status(TbContext* ctx, int* status_out);
const char* tilert_b200_last_error(void);
int tilert_b200_num_sms(TbContext* ctx);
/* dsa_temp_vars_size (tilert/models/deepseek_v3_2/temp_var_indices.py:109-118): number of named
 * scratch tensors the driver shares with Python. */
int tilert_b200_dsa_temp_vars_size(void);
/* Bytes of scratch a context allocates (for memory planning). */
size_t tilert_b200_context_bytes(void);
/* Number of kernels this library has launched in this process (monotonic; includes launches that
 * were recorded into a CUDA graph during stream capture). */
long long tilert_b200_launch_count(void);
/* Tracing, the role of the reference's `profile_logs` argument (tilert/utils.py:18-45): while
 * `trace` (device memory, u64 [256][16]) is set, every weight-streaming launch records per CTA eight
 * %globaltimer stamps (entry, ready, first data, last unit, tiles done, first conversion, copies
 * issued, exit) and counters of its first epilogue, MMA, producer and converter warps (cycles waiting /
 * working, units); rows 148-155 hold a per-unit timeline of CTA 0 (units 96-111, SM cycles).  NULL
 * switches tracing off. */
int tilert_b200_set_profile(TbContext* ctx, unsigned long long* trace);
/* Same with room for several launches: `trace` is u64 [n_records][256][16] and the k-th streaming
 * launch after this call writes record k % n_records (one decode step = one record per product). */
int tilert_b200_set_profile_ring(TbContext* ctx, unsigned long long* trace, int n_records);
/* Caps the thread blocks of the streaming launches and of the cooperative indexer selection made with this context
 * from now on (0 = one per SM).  A launch with fewer blocks than SMs leaves the others to kernels of another stream:
 * either kernels whose blocks do NOT wait on one another (the layer runs the per-token vector work and the indexer's
 * short-row scoring + selection beside the absorbed-q product this way), or ONE other capped launch, when the two
 * caps add up to at most the SM count, so that both are always fully resident (the layer runs the cooperative
 * long-row selection on 84 SMs beside the absorbed-q product on 64).  Host-side state: it applies to the launches
 * issued while it is set, also when they are captured in a graph. */
int tilert_b200_set_grid_limit(TbContext* ctx, int max_ctas);

/* Upper bound, in SM clock cycles, of every bounded wait in the library's kernels on the context's device
 * (default 1e9, about half a second; cycles <= 0 restores it).  A wait that runs out makes its kernel
 * return early with a status code (tilert_b200_status); tests use a short bound to exercise that path. */
int tilert_b200_set_wait_budget(TbContext* ctx, long long cycles);

/* ---- chained launches ------------------------------------------------------------------- */
/* The reference runs a whole decode step as ONE native call (dsa_show_hands,
 * tilert/models/deepseek_v3_2/modules/end2end.py:99-104,551-558).  Between chain_begin and chain_end the
 * FP8 product operators below are recorded instead of launched, and chain_end launches them as the
 * phases of one persistent kernel whose weight stream runs through the phase boundaries (activations of
 * a phase wait on a grid-wide signal of the phases that produce them).  tilert_rmsnorm_expert_proj_op,
 * tilert_proj_w_op and tilert_attn_prep_op may be recorded too: they run on spare warps at the start of
 * the product recorded after them.  Any other operator returns TB_ESTATE while a chain is being recorded.
 * Limits: 12 products and 3 such operators per chain.  Every CTA of the launch must be resident at once
 * (as for the single products), so chained launches of different streams must not overlap on a device. */
int tilert_b200_chain_begin(TbContext* ctx);
int tilert_b200_chain_end(TbContext* ctx, void* stream);
int tilert_b200_chain_abort(TbContext* ctx);
/* Trace of chained launches: while `trace` (device memory, u64 [12][256][8], zeroed by the caller) is set,
 * epilogue warp 0 of every CTA records per phase the %globaltimer at: dependencies met, norm statistics
 * ready, hook done, first accumulator complete, last unit read back, tiles reduced, main signal raised;
 * slot 7 = the CTA's units in the phase.  NULL switches it off. */
int tilert_b200_set_chain_profile(TbContext* ctx, unsigned long long* trace);

/* ---- peer-to-peer plumbing for the fused all-reduce ------------------------------------ */
/* The reference exchanges raw buffer addresses between its per-GPU threads
 * (tilert/models/deepseek_v3_2/modules/end2end.py:491-501).  With one process per GPU the same
 * exchange goes through CUDA IPC handles (64 opaque bytes each, sent over any host channel). */
size_t tilert_b200_comm_buffer_bytes(int world, int max_rows);
/* Zero-filled device allocation made directly with cudaMalloc (IPC handles need the base address
 * of an allocation, which a sub-allocating framework allocator does not give). */
int tilert_b200_dev_alloc(size_t bytes, void** dev_ptr_out);
int tilert_b200_dev_free(void* dev_ptr);
int tilert_b200_ipc_export(void* dev_ptr, uint8_t handle_out[64]);
int tilert_b200_ipc_import(const uint8_t handle[64], void** dev_ptr_out);
int tilert_b200_ipc_close(void* dev_ptr);
/* `buffers[r]` is rank r's communication buffer (own allocation for r == rank, imported mapping
 * otherwise), each `tilert_b200_comm_buffer_bytes(world, max_rows)` bytes and zero-filled before
 * any rank's first call.  Every rank must issue the same sequence of all-reduce / exchange operators on
 * the communicator (same count, same order): a call that no peer matches waits for its bounded time,
 * sets the status word to 3 and leaves the ranks' call numbers apart for good. */
int tilert_b200_comm_create(TbContext* ctx, int world, int rank, void* const* buffers, int max_rows,
                            TbComm** comm_out);
int tilert_b200_comm_destroy(TbComm* comm);

/* ---- activation preparation ------------------------------------------------------------ */

/* rmsnorm_quant_op / rmsnorm_op (tilert/models/deepseek_v3_2/ops/rmsnorm_quant.py:19-64).
 * x [tokens, dim] bf16 -> out bf16 (optional), q_out e4m3 + q_scale_out f32 [tokens, dim/128]
 * (optional, reference 1x128 quantisation), and xpack (the operand of the FP8 products).
 * gamma == NULL skips the normalisation (plain packing).  seg_scale (optional, [tokens, n_seg])
 * multiplies the scales of each run of dim/n_seg activations (routing weights). */
int tilert_rmsnorm_quant_op(TbContext* ctx, const void* x, const float* gamma, float eps, int tokens, int dim,
                            void* out, uint8_t* q_out, float* q_scale_out, const float* seg_scale, int n_seg,
                            uint8_t* xpack, void* stream);
/* Re-lays reference-format quantised activations (e4m3 [tokens, dim] + f32 [tokens, dim/128]) as
 * xpack with one column per token (cols_per_token = 1). */
int tilert_xq_repack_op(TbContext* ctx, const uint8_t* x_q, const float* x_scale, int tokens, int dim,
                        uint8_t* xpack, void* stream);
size_t tilert_b200_xpack_bytes(int dim);

/* ---- FP8 weight-streaming products ----------------------------------------------------- */

/* projx_wqkva_op (ops/projx_wqkva.py:22-48) and projx_wqaki_op (ops/projx_wqaki.py:11-44) in one
 * launch: rows of w_packed are [q_a (q_lora) | kv_a (kv_lora) | k_pe (rope) | indexer wk (ki_dim)];
 * any of the four parts may have size 0.  k_pe is written to pe_cache[*cur_pos + t]. */
int tilert_projx_wqkva_op(TbContext* ctx, const uint8_t* xpack, int cols_per_token, const uint8_t* w_packed,
                          int tokens, int dim, int q_lora, int kv_lora, int rope, int ki_dim, const int* cur_pos,
                          void* q_out, void* kv_out, void* pe_cache, int cache_rows, void* ki_out, void* stream);

/* RMSNormProjxWqkva.tilert_forward (ops/rmsnorm_projx_wqkva.py:473-509) as ONE launch: the RMSNorm
 * (rmsnorm_quant_op) runs inside the product kernel, which reads the bf16 hidden state directly. */
int tilert_rmsnorm_projx_wqkva_op(TbContext* ctx, const void* x, const float* gamma, float eps,
                                  const uint8_t* w_packed, int tokens, int dim, int q_lora, int kv_lora, int rope,
                                  int ki_dim, const int* cur_pos, void* q_out, void* kv_out, void* pe_cache,
                                  int cache_rows, void* ki_out, void* stream);

/* rmsnorm_proj_qb_op (ops/rmsnorm_projq_wqb.py:21-43) and rmsnorm_proj_qi_op
 * (ops/rmsnorm_projq_wqi.py:21-40) in one launch: RMSNorm(q) then rows
 * [q_nope (heads*nope) | q_pe (heads*rope) | iq (iq_heads*iq_dim)]. */
int tilert_rmsnorm_proj_q_op(TbContext* ctx, const void* q, const float* gamma, float eps, const uint8_t* w_packed,
                             int tokens, int q_lora, int heads, int nope, int rope, int iq_heads, int iq_dim,
                             void* q_nope, void* q_pe, void* iq, void* stream);

/* projq_wqb_op (ops/projq_wqb.py:24-54): q_lat[t,h,:] = q_nope[t,h,:] . W_kvb_nope[h]  (per-head). */
int tilert_projq_wqb_op(TbContext* ctx, const void* q_nope, const uint8_t* w_packed, int tokens, int heads,
                        int nope, int kv_lora, void* out, void* stream);
/* projo_wkvb_op (ops/projo_wkvb.py:24-54): o[t,h,:] = o_lat[t,h,:] . W_kvb_v[h]^T  (per-head). */
int tilert_projo_wkvb_op(TbContext* ctx, const void* o_lat, const uint8_t* w_packed, int tokens, int heads,
                         int kv_lora, int v_dim, void* out, void* stream);

/* unproj_o_allreduce_op (ops/unproj_o_allreduce.py:23-58): out = all_reduce(W_o_shard . vec) + x_residual.
 * comm == NULL: single GPU, no reduction.  The reduction runs inside the product kernel. */
int tilert_unproj_o_allreduce_op(TbContext* ctx, const void* vec, const uint8_t* w_packed, const void* x_residual,
                                 int tokens, int k, int n, void* out, TbComm* comm, void* stream);

/* padded_allreduce_add_op (ops/padded_allreduce_add.py:17-41): out = all_reduce(partial) + x_residual, bf16
 * [tokens, n], as a launch of its own over the communicator's peer buffers (n must be the communicator's row
 * count); one call of the communicator's sequence.  comm == NULL: out = partial + x_residual. */
int tilert_padded_allreduce_add_op(TbContext* ctx, const void* partial, const void* x_residual, int tokens, int n,
                                   void* out, TbComm* comm, void* stream);

/* expert_select_up_gate_silu_op (ops/expert_sel_up_gate_silu.py:23-48): routing (sigmoid + bias,
 * group-limited top-k, renormalise, scale) then SiLU(W1 x) * (W3 x) for the shared expert and the
 * selected routed experts.  hidden [tokens, dim] bf16 is the normalised post-attention state
 * (hidden_out of rmsnorm_expert_proj_op) when gamma == NULL; with gamma (f32 [dim]) it is the raw state
 * and the RMSNorm (eps) runs inside the launch, so the product need not wait for the router's copy.  w_packed: [n_experts + 1] experts, `expert_stride` bytes apart, the
 * shared expert last; rows of each expert interleave gate and up in groups of 8.
 * hidden_out [tokens, top_k + 1, inter] bf16 (slot 0 = shared expert).
 * slot_ids / slot_w [tokens, top_k + 1]: expert id and weight per slot (inputs of the down op).
 * Under tensor parallelism every rank holds an `inter`-row slice of every expert.
 * One token: one launch that also routes.  Several tokens (<= 4): a routing launch, then ONE product launch over the
 * flat slot list [shared, token 0's experts, token 1's experts, ...] -- the shared expert is streamed once and every
 * (token, expert) pair once; besides hidden_out the launch leaves every token's column of every slot in a buffer
 * of the context, which the down operator uses when it is given this hidden_out next. */
int tilert_expert_select_up_gate_silu_op(TbContext* ctx, const void* hidden, const float* gamma, float eps,
                                         const float* scores, const float* bias, const uint8_t* w_packed, long long expert_stride,
                                         int tokens, int dim, int inter, int n_experts, int n_groups,
                                         int n_limited_groups, int top_k, float route_scale, void* hidden_out,
                                         float* probs_out, int* idx_out, int* slot_ids, float* slot_w,
                                         void* stream);

/* expert_down_allreduce_op (ops/expert_down_allreduce.py:23-63):
 * out = all_reduce(sum_slots w_slot * W2[slot_ids] . vec[slot]) + x_residual.  Several tokens: ONE launch when
 * `vec` is the hidden_out of the preceding expert_select_up_gate_silu_op call on this context (K = the flat slot
 * list, a token's weight 0 at the other tokens' slots), else one launch per token. */
int tilert_expert_down_allreduce_op(TbContext* ctx, const void* vec, const uint8_t* w_packed,
                                    long long expert_stride, const int* slot_ids, const float* slot_w,
                                    const void* x_residual, int tokens, int inter, int dim, int n_slots, void* out,
                                    TbComm* comm, void* stream);

/* rmsnorm_up_gate_silu_op (ops/rmsnorm_up_gate_silu.py:26-44): dense FFN first half. */
int tilert_rmsnorm_up_gate_silu_op(TbContext* ctx, const void* x, const float* gamma, float eps,
                                   const uint8_t* w_packed, int tokens, int dim, int inter, void* out, void* stream);
/* down_allreduce_op (ops/down_allreduce.py:24-59): dense FFN second half + all-reduce + residual. */
int tilert_down_allreduce_op(TbContext* ctx, const void* vec, const uint8_t* w_packed, const void* x_residual,
                             int tokens, int inter, int dim, void* out, TbComm* comm, void* stream);

/* rmsnorm_expert_proj_op / proj_w_op (ops/rmsnorm_expert_proj.py:151-169, ops/projx_wis.py:21-40) on the FP8
 * weight stream: a bf16 weight [n, dim] packed by tilert_b200.pack.pack_bf16_two_term as two e4m3 rows per
 * source row (leading and residual term, exact for bf16) goes through the same streaming kernel as the FP8
 * products, whose epilogue adds the two rows.  out[t, :] = W . RMSNorm(x[t]) (gamma NULL: x as is),
 * f32 (out_is_f32) or bf16.  In a chained launch this makes the router a product like the others -- the
 * routed experts' weight addresses wait for its signal -- instead of bf16 loads on spare warps. */
int tilert_rmsnorm_proj_rows2_op(TbContext* ctx, const void* x, const float* gamma, float eps, const uint8_t* w_packed,
                                 int tokens, int dim, int n, void* out, int out_is_f32, void* stream);

/* ---- bf16 products --------------------------------------------------------------------- */

/* proj_w_op (ops/projx_wis.py:21-40): out[t, :] = W[n, k] . x[t, :]   (bf16 in, bf16 out).
 * gamma != NULL: x is the raw hidden state and RMSNorm(x) * gamma (kept in f32) is applied first. */
int tilert_proj_w_op(TbContext* ctx, const void* x, const float* gamma, float eps, const void* w, int tokens, int n,
                     int k, void* out, void* stream);
/* rmsnorm_expert_proj_op (ops/rmsnorm_expert_proj.py:151-169): hidden_out = bf16(RMSNorm(x)),
 * scores_out[t, :] = W_gate . hidden_out[t, :] in f32.  w_gate is bf16 (gate_is_f32 = 0) or f32.
 * gamma == NULL: x is already normalised (hidden_out may then be NULL). */
int tilert_rmsnorm_expert_proj_op(TbContext* ctx, const void* x, const float* gamma, float eps, const void* w_gate,
                                  int gate_is_f32, int tokens, int dim, int n_experts, float* scores_out,
                                  void* hidden_out, void* stream);
/* rmsnorm_head_proj_op (ops/rmsnorm_head_proj.py:19-39): f32 logits of a vocabulary shard. */
int tilert_rmsnorm_head_proj_op(TbContext* ctx, const void* x, const float* gamma, float eps, const void* w,
                                int tokens, int dim, int vocab, void* x_norm_out, float* logits_out, void* stream);

/* eh_proj_allreduce_op (ops/eh_proj_allreduce.py:23-60; golden :252-277): out[t, :] = W_eh[dim, 2*dim] .
 * concat(e_norm[t], h_norm[t])   (bf16 in, bf16 weights, bf16 out).  Every rank computes the whole
 * product: the reference's K-sharding + all-reduce of this 205 MB bf16 weight is not reproduced. */
int tilert_eh_proj_allreduce_op(TbContext* ctx, const void* e_norm, const void* h_norm, const void* w, int tokens,
                                int dim, void* out, void* stream);
/* mtp_preprocess_layer (modules/mtp_preprocess.py:20-28; golden :197-229) for already embedded tokens:
 * e_norm = RMSNorm(e) * gamma_e, h_norm = RMSNorm(h) * gamma_h (both rounded to bf16 and optionally
 * written out), then eh_proj as above, in one launch per two tokens. */
int tilert_mtp_preprocess_op(TbContext* ctx, const void* e, const void* h, const float* gamma_e,
                             const float* gamma_h, float eps, const void* w, int tokens, int dim, void* e_norm_out,
                             void* h_norm_out, void* out, void* stream);
/* The same for output rows [row_begin, row_begin + n_rows) only (`w` is still the whole [dim, 2 dim] weight, `out` the
 * whole [tokens, dim] tensor, of which only those columns are written).  With the ranks of a tensor-parallel group
 * each taking dim / world rows into a buffer that is zero elsewhere, padded_allreduce_add_op assembles the vector on
 * every rank: each rank streams 1 / world of eh_proj (the reference splits K and all-reduces,
 * ops/eh_proj_allreduce.py:159-183; rows keep every output's sum on one rank, so the result is bit-identical to the
 * unsharded product). */
int tilert_mtp_preprocess_rows_op(TbContext* ctx, const void* e, const void* h, const float* gamma_e,
                                  const float* gamma_h, float eps, const void* w, int tokens, int dim, int row_begin,
                                  int n_rows, void* e_norm_out, void* h_norm_out, void* out, void* stream);

/* ---- per-token vector operators -------------------------------------------------------- */

/* rmsnorm_kv_op (ops/rmsnorm_kv.py:20-43): kv_cache[*cur_pos + t] = bf16(RMSNorm(kv[t]) * gamma). */
int tilert_rmsnorm_kv_op(TbContext* ctx, const void* kv, const float* gamma, float eps, int tokens, int dim,
                         const int* cur_pos, void* kv_cache, int cache_rows, void* stream);
/* qkv_rope_op (ops/qkv_rope.py:21-50): interleaved RoPE in place on q_pe [tokens, heads, rope] and on
 * pe_cache[*cur_pos + t].  freqs [tokens, rope/2, 2] f32 = (cos, sin). */
int tilert_qkv_rope_op(TbContext* ctx, void* q_pe, int heads, int rope, void* pe_cache, const int* cur_pos,
                       const float* freqs, int tokens, int cache_rows, void* stream);
/* rotate_op (ops/rotate.py:61-105): non-interleaved RoPE on the first `rope` dims + Hadamard-128. */
int tilert_rotate_op(TbContext* ctx, const void* in, void* out, int heads, int rope, const float* freqs,
                     int tokens, void* stream);
/* layernorm_rope_rotate_op (ops/layernorm_rope_rotate.py:23-83): LayerNorm -> RoPE -> Hadamard into
 * k_cache[*cur_pos + t]. */
int tilert_layernorm_rope_rotate_op(TbContext* ctx, const void* in, const int* cur_pos, void* k_cache,
                                    const float* weight, const float* bias, const float* freqs, int rope,
                                    int tokens, int cache_rows, void* stream);
/* proj_w_op + rmsnorm_kv_op + qkv_rope_op + rotate_op + layernorm_rope_rotate_op in one launch (the five
 * operators above, ops/projx_wis.py:21-40, ops/rmsnorm_kv.py:20-43, ops/qkv_rope.py:21-50,
 * ops/rotate.py:61-105, ops/layernorm_rope_rotate.py:23-83): they are independent of one another, and
 * separately each costs a kernel boundary on the critical path of a decode step.  Arguments and
 * results are those of the five operators: x [tokens, dim] raw hidden state with its input-norm gain,
 * w_is [idx_heads, dim] bf16 -> idx_w_out [tokens, idx_heads] bf16; kv [tokens, kv_dim] -> kv_cache row;
 * q_pe [tokens, heads, rope] and the pe_cache row rotated in place; iq [tokens, idx_heads, 128] ->
 * iq_out; ki [tokens, 128] -> ki_cache row.  Results are bit-identical to the separate operators.
 * w_is may be NULL (the head weights then come from elsewhere, e.g. tilert_rmsnorm_proj_rows2_op). */
int tilert_attn_prep_op(TbContext* ctx, const void* x, const float* in_gamma, float eps, const void* w_is,
                        int idx_heads, int dim, void* idx_w_out, const void* kv, const float* kv_gamma, int kv_dim,
                        void* kv_cache, void* q_pe, int heads, int rope, void* pe_cache, const void* iq, void* iq_out,
                        const void* ki, void* ki_cache, const float* ln_w, const float* ln_b, const float* freqs,
                        const int* cur_pos, int tokens, int cache_rows, void* stream);

/* `cache_rows` (operators above that write the cache row of position *cur_pos + t): the number of rows the
 * cache tensors hold, 0 = unchecked.  The position lives in device memory, so only the kernel can check it:
 * a row at or past cache_rows is not written and the status word becomes 4 (bad argument). */

/* ---- DSA indexer and sparse attention ---------------------------------------------------- */

/* sparse_index_op (ops/sparse_index.py:11-69): logits[t, j] = sum_h w[t,h] relu(q[t,h] . k_cache[j])
 * for j < n_keys, -inf where j > *cur_pos + t.  heads in {16, 32, 64}, head dim 128. */
int tilert_sparse_index_op(TbContext* ctx, const void* q, const void* k_cache, const void* weights, float* logits,
                           long long logits_stride, int heads, int tokens, int n_keys, const int* cur_pos,
                           void* stream);
/* topk_accurate_op (ops/topk.py:60-109): exact top-k of each of `rows` logit rows (entries >= n or
 * equal to -inf never selected); indices ascending, unused slots -1. */
int tilert_topk_accurate_op(TbContext* ctx, const float* logits, long long logits_stride, int rows, int n, int k,
                            int* indices, void* stream);
/* sparse_index_topk_dsv32_op (ops/sparse_index.py:72-128): the two above with the same results, as ONE
 * cooperative launch: at most one thread block per SM (tokens <= 8 share them), each scoring a contiguous range
 * of keys; the k-th largest score is found over histograms that all blocks add to, meeting at four grid-wide
 * barriers (bounded waits: status word 7 when a block gives up), and every block writes its part of the
 * ascending index list.  Uses a work area of the context that the launch clears itself. */
int tilert_sparse_index_topk_op(TbContext* ctx, const void* q, const void* k_cache, const void* weights,
                                float* logits, long long logits_stride, int heads, int tokens, int n_keys,
                                const int* cur_pos, int k, int* indices, void* stream);
/* flash_sparse_mla_op (ops/flash_sparse_mla.py:18-93): softmax((q.kv + q_pe.pe) * scale) . kv over the
 * selected rows.  out_acc [tokens, heads, n_splits, 512] f32 and lse_acc [tokens, heads, n_splits] f32
 * with n_splits = ceil(topk / split_size); split_size a multiple of 64. */
int tilert_flash_sparse_mla_op(TbContext* ctx, const void* q, const void* q_pe, const void* kv, const void* k_pe,
                               const int* indices, int topk, const int* cur_pos, int heads, int tokens, int n_cache,
                               float softmax_scale, int split_size, void* out, float* out_acc, float* lse,
                               float* lse_acc, void* stream);
/* flash_sparse_mla_op followed by projo_wkvb_op (ops/projo_wkvb.py) in two launches instead of three: the merge of
 * the attention chunks also multiplies each head's latent output with that head's W_kv_b value rows (w_v_packed:
 * [heads] row tiles of 128 x 512, as projo_wkvb_op takes them; kv_lora 512, v_dim 128) and writes o_out
 * [tokens, heads, 128] bf16.  `out` (the latent output) may be NULL. */
int tilert_flash_sparse_mla_vproj_op(TbContext* ctx, const void* q, const void* q_pe, const void* kv, const void* k_pe,
                                     const int* indices, int topk, const int* cur_pos, int heads, int tokens,
                                     int n_cache, float softmax_scale, int split_size, void* out, float* out_acc,
                                     float* lse, float* lse_acc, const uint8_t* w_v_packed, int kv_lora, int v_dim,
                                     void* o_out, void* stream);

/* ---- sampling --------------------------------------------------------------------------- */

/* The sampling step the reference runs inside its driver (configuration and outputs visible in
 * modules/end2end.py:253-311, 665-703: SAMPLING_CONFIG = (temperature, top_p, top_k, use_top_p),
 * TOP_N_LOG_PROBS / TOP_N_INDICES [.., 256], TOP_P_SCORES = log-probability of the sampled token;
 * the algorithm itself is inside its binary and is restated here in the standard form).
 *   logits [tokens, logits_stride] f32 (first `vocab` entries of a row are used);
 *   config_dev: 4 floats in device memory; temperature 0 = greedy arg-max (ties to the lower id);
 *   candidates are the 1024 largest logits; top_k in [1, 1024] keeps the first top_k, any other value
 *   all 1024; with use_top_p the shortest prefix reaching top_p of the temperature-scaled softmax mass
 *   of the whole vocabulary is kept; one uniform number from (seed, step, token index) picks a token.
 *   step_dev: optional device state of two u64 {step, scratch}, zero before first use: the launch reads
 *   the step and its last block increments it (so a replayed CUDA graph draws new numbers); NULL uses
 *   step_value.  token_logprob_out / topn_* may be NULL; log-probabilities are those of the unscaled
 *   softmax over the whole vocabulary, top-n sorted by descending probability. */
int tilert_sample_op(TbContext* ctx, const float* logits, long long logits_stride, int tokens, int vocab,
                     const float* config_dev, unsigned long long seed, unsigned long long* step_dev,
                     unsigned long long step_value, int* token_out, float* token_logprob_out, float* topn_logprob_out,
                     int* topn_index_out, void* stream);

/* ---- latent caches from an external prefill, FP8 wire format -------------------------------- */

/* The decode side of prefill / decode disaggregation: tilert/pd_vllm/profiles/mla_nsa.py:16-41 (layout),
 * :186-232 (_dequant_kv, _dequant_ki) followed by DSAv32Generator.inject_cache
 * (tilert/models/deepseek_v3_2/generator.py:419-484), as one launch per layer.
 *
 *   kv_raw   [seq_len, 528] bytes: 512 e4m3 latent values + 4 f32 scales (one per 128 values);
 *   pe_raw   [seq_len, 128] bytes: 64 bf16 rope values;
 *   ki_pages [ceil(seq_len / 64), 8448] bytes: 64 x 128 e4m3 indexer-key values, then 64 f32 scales;
 *   rows start_pos .. start_pos + seq_len - 1 of kv_cache [cache_rows, 512], pe_cache [cache_rows, 64] and
 *   ki_cache [cache_rows, 128] (bf16) are written: latent = e4m3 * scale rounded to bf16; indexer key =
 *   e4m3 * scale rounded to bf16, then Hadamard-128 scaled by 128^-1/2.  A plane and its cache may both be
 *   NULL to skip it.  kv_raw and kv_cache must be 16-byte aligned, the other planes 4-byte aligned. */
int tilert_inject_cache_fp8_op(TbContext* ctx, const uint8_t* kv_raw, const uint8_t* pe_raw, const uint8_t* ki_pages,
                               int seq_len, int start_pos, int cache_rows, void* kv_cache, void* pe_cache,
                               void* ki_cache, void* stream);

/* ---- greedy token over a vocabulary split across ranks ----------------------------------- */

/* The arg-max that follows rmsnorm_head_proj_op when every rank holds vocab / world rows of the head
 * (the reference keeps LOGITS_OUT as f32[1, 4, vocab / 8] per device and leaves PREDICTED_TOKENS,
 * tilert/models/deepseek_v3_2/modules/end2end.py:617-651, temp_var_indices.py:15-76; the exchange
 * itself is inside its native library).  Every rank takes the arg-max of its slice, stores the
 * (value, global index) pair into every rank's receive slot over peer memory and, once all ranks
 * have arrived (bounded wait, status word on time-out), picks the largest value, lowest index on ties.
 * It is one call in the communicator's sequence, like a fused all-reduce: every rank must issue it
 * at the same point of its stream.
 *
 *   logits [tokens, logits_stride] f32, of which n_local entries per row are this rank's slice,
 *   entry 0 being global index index_offset; tokens 1..4; comm NULL or of world 1: local arg-max only;
 *   token_out [tokens] int64; value_out [tokens] f32 or NULL. */
int tilert_argmax_exchange_op(TbContext* ctx, const float* logits, long long logits_stride, int tokens, int n_local,
                              int index_offset, TbComm* comm, long long* token_out, float* value_out, void* stream);

/* ---- allocation-free product ------------------------------------------------------------ */

/* No counterpart in the reference.  out[t, :] = W . x[t, :] (+ residual[t, :]) with the same FP8
 * weight-streaming kernel as unproj_o_allreduce_op on one GPU, for callers that must not allocate
 * device memory: code running under a host runtime that owns the whole memory pool and forbids
 * cudaMalloc from plug-ins, or a serving loop with a frozen memory budget in which an allocation
 * would synchronise the device.  It takes no TbContext (creating one allocates) and calls no
 * cudaMalloc, cudaFree or allocating library routine.  Its scratch -- the partial sums of row tiles
 * whose k blocks are spread over several thread blocks (64-bit words tagged with the launch number, so
 * they need neither counters nor clearing), a status word, and the converted activation blocks with
 * their ready flags -- is a fixed ~2.4 MB array inside the library image, held by every GPU that
 * loads the library until the process exits.
 *
 *   x [tokens, k] bf16, w_packed for [n, k], residual [tokens, n] bf16 or NULL, out [tokens, n] bf16;
 *   tokens 1..4, k a multiple of 128 and at most 32768, n at most 131072 rows (a larger k or n
 *   returns TB_EINVAL);
 *   status_out_dev: optional device int that receives the kernel's status word (0 = completed).  It is
 *   the only way to learn that a bounded wait of this call ran out (the word inside the array is
 *   cleared by the next call): callers that need error detection must pass it.
 *
 * The first call on each device looks up the array's device address and sets a function
 * attribute (under a lock, so first calls from several host threads are safe); make that call outside
 * any stream capture.  All calls on a device share the one array: the status word, the ready flags and
 * their epoch are cleared at the start of every call, and two calls whose kernels overlap on the GPU
 * (different streams) race on it -- serialise them. */
int tilert_b200_matvec_fp8_static(const void* x, const uint8_t* w_packed, const void* residual, int tokens, int k,
                                  int n, void* out, int* status_out_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TILERT_B200_H_ */
