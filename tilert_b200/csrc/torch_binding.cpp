// Registers the decode operators with the PyTorch dispatcher under the names and argument orders the
// reference's Python wrappers call (`torch.ops.tilert.<op>`, tilert/models/deepseek_v3_2/ops/*.py; the
// reference's own library does this from C++ too and is loaded with `torch.ops.load_library`,
// tilert/__init__.py:68-77).  Every operator forwards to the C ABI of libtilert_b200.so (include/tilert_b200.h),
// writes into caller-allocated outputs and returns nothing.  Weight operands are this library's packed
// tensors (tilert_b200.pack); trailing `model_arch` / `kernel_type` strings, `profile_logs` tensors, `flag`
// epochs and the empty int64 placeholder tensors of the reference signatures are accepted and ignored.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <optional>
#include <string>

#include "../../include/tilert_b200.h"

namespace {

using at::Tensor;
using OptTensor = std::optional<Tensor>;

void check(int rc) { TORCH_CHECK(rc == 0, "tilert_b200 call failed (", rc, "): ", tilert_b200_last_error()); }

TbContext* ctx_of(const Tensor& t) {
  TORCH_CHECK(t.is_cuda(), "tilert ops need CUDA tensors (there is no CPU path)");
  TbContext* c = nullptr;
  check(tilert_b200_default_context(t.get_device(), &c));
  return c;
}
void* stream_of(const Tensor& t) { return c10::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

const Tensor& need(const Tensor& t, at::ScalarType dt, const char* name) {
  TORCH_CHECK(t.scalar_type() == dt, name, " must be a ", c10::toString(dt), " tensor, got ", c10::toString(t.scalar_type()));
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
  return t;
}
void* ptr(const Tensor& t) { return t.data_ptr(); }
void* ptr(const OptTensor& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }
int rows_of(const Tensor& cache) { return static_cast<int>(cache.size(-2)); }

constexpr auto BF16 = at::kBFloat16;
constexpr auto F32 = at::kFloat;
constexpr auto I32 = at::kInt;
constexpr float kEps = 1e-6f;

using Str = std::string;

void tilert_init_op() {}

int64_t dsa_temp_vars_size() { return tilert_b200_dsa_temp_vars_size(); }

Tensor alloc_misc_ws(int64_t num_max_insts, int64_t device_id) {
  // the reference's instruction workspace (tilert/utils.py:62) has no role here: kernels take their parameters at launch
  return at::zeros({std::max<int64_t>(num_max_insts, 1), 16}, at::TensorOptions().dtype(at::kLong).device(at::kCUDA, device_id));
}

void rmsnorm_op(const Tensor& x, const Tensor& gamma, Tensor out, Str, Str, OptTensor) {
  need(x, BF16, "x"); need(gamma, F32, "gamma"); need(out, BF16, "out");
  check(tilert_rmsnorm_quant_op(ctx_of(x), ptr(x), gamma.data_ptr<float>(), kEps, x.size(-2), x.size(-1), ptr(out), nullptr,
                                nullptr, nullptr, 0, nullptr, stream_of(x)));
}

void rmsnorm_quant_op(const Tensor& x, const Tensor& gamma, Tensor out, Tensor q_out, Tensor q_scale_out, Str, Str, OptTensor,
                      OptTensor) {
  need(x, BF16, "x"); need(gamma, F32, "gamma"); need(out, BF16, "out"); need(q_scale_out, F32, "q_scale_out");
  check(tilert_rmsnorm_quant_op(ctx_of(x), ptr(x), gamma.data_ptr<float>(), kEps, x.size(-2), x.size(-1), ptr(out),
                                static_cast<uint8_t*>(ptr(q_out)), q_scale_out.data_ptr<float>(), nullptr, 0, nullptr, stream_of(x)));
}

void projx_wqkva_op(const Tensor& x_q, const Tensor& x_scale, const Tensor& w, const Tensor& cur_pos, Tensor q_out, Tensor kv_out,
                    Tensor pe_cache, Str, Str, OptTensor, OptTensor) {
  need(x_scale, F32, "x_scale"); need(cur_pos, I32, "cur_pos"); need(q_out, BF16, "q_out"); need(kv_out, BF16, "kv_out");
  need(pe_cache, BF16, "pe_cache");
  const int tokens = x_q.size(-2), dim = x_q.size(-1);
  Tensor xpack = at::zeros({static_cast<int64_t>(tilert_b200_xpack_bytes(dim))}, x_scale.options().dtype(at::kByte));
  TbContext* c = ctx_of(q_out);
  check(tilert_xq_repack_op(c, static_cast<const uint8_t*>(ptr(x_q)), x_scale.data_ptr<float>(), tokens, dim,
                            xpack.data_ptr<uint8_t>(), stream_of(q_out)));
  check(tilert_projx_wqkva_op(c, xpack.data_ptr<uint8_t>(), 1, w.data_ptr<uint8_t>(), tokens, dim, q_out.size(-1), kv_out.size(-1),
                              pe_cache.size(-1), 0, cur_pos.data_ptr<int>(), ptr(q_out), ptr(kv_out), ptr(pe_cache),
                              rows_of(pe_cache), nullptr, stream_of(q_out)));
}

void proj_w_op(const Tensor& x, const Tensor& w, Tensor out, Str, Str, OptTensor) {
  need(x, BF16, "x"); need(w, BF16, "w"); need(out, BF16, "out");
  check(tilert_proj_w_op(ctx_of(x), ptr(x), nullptr, kEps, ptr(w), x.size(-2), w.size(0), w.size(1), ptr(out), stream_of(x)));
}

void rmsnorm_proj_qb_op(const Tensor& q, const Tensor& w, OptTensor, const Tensor& gamma, Tensor q_nope, Tensor q_pe, Str, Str,
                        OptTensor, OptTensor) {
  need(q, BF16, "q"); need(gamma, F32, "gamma"); need(q_nope, BF16, "q_nope"); need(q_pe, BF16, "q_pe");
  check(tilert_rmsnorm_proj_q_op(ctx_of(q), ptr(q), gamma.data_ptr<float>(), kEps, w.data_ptr<uint8_t>(), q.size(-2), q.size(-1),
                                 q_nope.size(-2), q_nope.size(-1), q_pe.size(-1), 0, 0, ptr(q_nope), ptr(q_pe), nullptr, stream_of(q)));
}

void rmsnorm_kv_op(const Tensor& kv, const Tensor& gamma, const Tensor& cur_pos, Tensor kv_cache, Str, Str, OptTensor) {
  need(kv, BF16, "kv"); need(gamma, F32, "gamma"); need(cur_pos, I32, "cur_pos"); need(kv_cache, BF16, "kv_cache");
  check(tilert_rmsnorm_kv_op(ctx_of(kv), ptr(kv), gamma.data_ptr<float>(), kEps, kv.size(-2), kv.size(-1), cur_pos.data_ptr<int>(),
                             ptr(kv_cache), rows_of(kv_cache), stream_of(kv)));
}

void qkv_rope_op(Tensor q_pe, Tensor pe_cache, const Tensor& rope_freqs, const Tensor& cur_pos, Str, Str, OptTensor) {
  need(q_pe, BF16, "q_pe"); need(pe_cache, BF16, "pe_cache"); need(rope_freqs, F32, "rope_freqs"); need(cur_pos, I32, "cur_pos");
  check(tilert_qkv_rope_op(ctx_of(q_pe), ptr(q_pe), q_pe.size(-2), q_pe.size(-1), ptr(pe_cache), cur_pos.data_ptr<int>(),
                           rope_freqs.data_ptr<float>(), q_pe.size(-3), rows_of(pe_cache), stream_of(q_pe)));
}

void rotate_op(const Tensor& x_in, Tensor out, const Tensor& freqs, Str, Str, OptTensor) {
  need(x_in, BF16, "x_in"); need(out, BF16, "out"); need(freqs, F32, "freqs");
  TORCH_CHECK(x_in.size(-1) == 128, "dim must be 128");
  check(tilert_rotate_op(ctx_of(x_in), ptr(x_in), ptr(out), x_in.size(-2), 64, freqs.data_ptr<float>(), x_in.size(-3), stream_of(x_in)));
}

void layernorm_rope_rotate_op(const Tensor& x_in, const Tensor& cur_pos, Tensor k_cache, const Tensor& weight, const Tensor& bias,
                              const Tensor& freqs, Str, Str, OptTensor) {
  need(x_in, BF16, "x_in"); need(cur_pos, I32, "cur_pos"); need(k_cache, BF16, "k_cache"); need(weight, F32, "weight");
  need(bias, F32, "bias"); need(freqs, F32, "freqs");
  TORCH_CHECK(x_in.size(-1) == 128, "dim must be 128");
  check(tilert_layernorm_rope_rotate_op(ctx_of(x_in), ptr(x_in), cur_pos.data_ptr<int>(), ptr(k_cache), weight.data_ptr<float>(),
                                        bias.data_ptr<float>(), freqs.data_ptr<float>(), 64, x_in.size(-2), rows_of(k_cache),
                                        stream_of(x_in)));
}

Tensor pos_tensor(int64_t cur_pos, const Tensor& like) {
  // the reference passes the position of these two operators as a host integer (ops/sparse_index.py:67,126)
  return at::full({1}, cur_pos, like.options().dtype(I32));
}

void sparse_index_op(const Tensor& q, const Tensor& k_cache, const Tensor& weights, Tensor logits, int64_t cur_pos, Str, Str,
                     OptTensor) {
  need(q, BF16, "q"); need(k_cache, BF16, "k_cache"); need(weights, BF16, "weights"); need(logits, F32, "logits");
  const Tensor pos = pos_tensor(cur_pos, q);
  check(tilert_sparse_index_op(ctx_of(q), ptr(q), ptr(k_cache), ptr(weights), logits.data_ptr<float>(), logits.size(-1), q.size(-2),
                               q.size(-3), k_cache.size(-2), pos.data_ptr<int>(), stream_of(q)));
}

void sparse_index_topk_dsv32_op(const Tensor& q, const Tensor& k_cache, const Tensor& weights, Tensor logits, int64_t cur_pos,
                                Tensor indices, OptTensor, OptTensor) {
  need(q, BF16, "q"); need(k_cache, BF16, "k_cache"); need(weights, BF16, "weights"); need(logits, F32, "logits");
  need(indices, I32, "indices");
  const Tensor pos = pos_tensor(cur_pos, q);
  check(tilert_sparse_index_topk_op(ctx_of(q), ptr(q), ptr(k_cache), ptr(weights), logits.data_ptr<float>(), logits.size(-1),
                                    q.size(-2), q.size(-3), k_cache.size(-2), pos.data_ptr<int>(), indices.size(-1),
                                    indices.data_ptr<int>(), stream_of(q)));
}

void topk_accurate_op(const Tensor& logits, Tensor indices, int64_t seq_len, OptTensor, Str, Str, OptTensor, int64_t) {
  need(logits, F32, "logits"); need(indices, I32, "indices");
  check(tilert_topk_accurate_op(ctx_of(logits), logits.data_ptr<float>(), logits.size(-1), logits.numel() / logits.size(-1), seq_len,
                                indices.size(-1), indices.data_ptr<int>(), stream_of(logits)));
}

void topk_approximate_op(const Tensor& logits, Tensor indices, int64_t seq_len, Str, Str, OptTensor) {
  // one selection kernel serves both names: the exact top-k is a valid answer to the approximate one
  topk_accurate_op(logits, indices, seq_len, std::nullopt, "", "", std::nullopt, 1);
}

void projq_wqb_op(const Tensor& q_nope, const Tensor& w, OptTensor, Tensor out, Str, Str, OptTensor) {
  need(q_nope, BF16, "q_nope"); need(out, BF16, "out");
  check(tilert_projq_wqb_op(ctx_of(out), ptr(q_nope), w.data_ptr<uint8_t>(), q_nope.size(-3), q_nope.size(-2), q_nope.size(-1),
                            out.size(-1), ptr(out), stream_of(out)));
}

void flash_sparse_mla_op(const Tensor& q, const Tensor& q_pe, const Tensor& kv, const Tensor& k_pe, const Tensor& indices,
                         const Tensor& cur_pos, Tensor out, Tensor out_acc, OptTensor lse, Tensor lse_acc, int64_t split_size, Str,
                         Str, OptTensor, OptTensor, double softmax_scale) {
  TORCH_CHECK(softmax_scale > 0, "flash_sparse_mla_op: softmax_scale must be given (the reference derives it from its model "
                                 "arguments inside the native library)");
  need(q, BF16, "q"); need(q_pe, BF16, "q_pe"); need(kv, BF16, "kv"); need(k_pe, BF16, "k_pe"); need(indices, I32, "indices");
  need(cur_pos, I32, "cur_pos"); need(out, BF16, "out"); need(out_acc, F32, "out_acc"); need(lse_acc, F32, "lse_acc");
  check(tilert_flash_sparse_mla_op(ctx_of(q), ptr(q), ptr(q_pe), ptr(kv), ptr(k_pe), indices.data_ptr<int>(), indices.size(-1),
                                   cur_pos.data_ptr<int>(), q.size(-2), q.size(-3), kv.size(-2), static_cast<float>(softmax_scale),
                                   split_size, ptr(out), out_acc.data_ptr<float>(), static_cast<float*>(ptr(lse)),
                                   lse_acc.data_ptr<float>(), stream_of(q)));
}

void projo_wkvb_op(const Tensor& o, const Tensor& w, OptTensor, Tensor out, Str, Str, OptTensor, OptTensor) {
  need(o, BF16, "o"); need(out, BF16, "out");
  check(tilert_projo_wkvb_op(ctx_of(out), ptr(o), w.data_ptr<uint8_t>(), o.size(-3), o.size(-2), o.size(-1), out.size(-1), ptr(out),
                             stream_of(out)));
}

void unproj_o_allreduce_op(const Tensor& vec, const Tensor& w, OptTensor, const Tensor& x_residual, int64_t, Tensor out, OptTensor,
                           Str, Str) {
  need(vec, BF16, "vec"); need(out, BF16, "out"); need(x_residual, BF16, "x_residual");
  const int tokens = out.size(-2);
  check(tilert_unproj_o_allreduce_op(ctx_of(out), ptr(vec), w.data_ptr<uint8_t>(), ptr(x_residual), tokens, vec.numel() / tokens,
                                     out.size(-1), ptr(out), nullptr, stream_of(out)));
}

void padded_allreduce_add_op(const Tensor& partial_buf, const Tensor& x_in, int64_t, Tensor vec_out, OptTensor, Str, Str) {
  need(partial_buf, BF16, "partial_buf"); need(x_in, BF16, "x_in"); need(vec_out, BF16, "vec_out");
  check(tilert_padded_allreduce_add_op(ctx_of(vec_out), ptr(partial_buf), ptr(x_in), vec_out.size(-2), vec_out.size(-1),
                                       ptr(vec_out), nullptr, stream_of(vec_out)));
}

void down_allreduce_op(const Tensor& vec, const Tensor& w, OptTensor, const Tensor& x_residual, int64_t, Tensor out, Str, Str,
                       OptTensor) {
  unproj_o_allreduce_op(vec, w, std::nullopt, x_residual, 0, out, std::nullopt, "", "");
}

void rmsnorm_expert_proj_op(const Tensor& x, const Tensor& gamma, const Tensor& w_gate, Tensor scores_out, Tensor hidden_out, Str,
                            Str, OptTensor) {
  need(x, BF16, "x"); need(gamma, F32, "gamma"); need(scores_out, F32, "scores_out"); need(hidden_out, BF16, "hidden_out");
  TORCH_CHECK(w_gate.scalar_type() == BF16 || w_gate.scalar_type() == F32, "w_gate must be bfloat16 or float32");
  check(tilert_rmsnorm_expert_proj_op(ctx_of(x), ptr(x), gamma.data_ptr<float>(), kEps, ptr(w_gate), w_gate.scalar_type() == F32,
                                      x.size(-2), x.size(-1), w_gate.size(0), scores_out.data_ptr<float>(), ptr(hidden_out),
                                      stream_of(x)));
}

void expert_select_up_gate_silu_op(const Tensor& hidden, const Tensor& scores, OptTensor bias, const Tensor& w, Tensor hidden_out,
                                   Tensor probs_out, Tensor idx_out, OptTensor, Str, Str, int64_t n_groups, int64_t n_limited_groups,
                                   double route_scale, OptTensor slot_ids, OptTensor slot_w) {
  need(hidden, BF16, "hidden"); need(scores, F32, "scores"); need(hidden_out, BF16, "hidden_out"); need(probs_out, F32, "probs_out");
  need(idx_out, I32, "idx_out");
  check(tilert_expert_select_up_gate_silu_op(
      ctx_of(hidden), ptr(hidden), nullptr, kEps, scores.data_ptr<float>(), static_cast<const float*>(ptr(bias)), w.data_ptr<uint8_t>(),
      w.stride(0) * w.element_size(), scores.size(-2), hidden.size(-1), hidden_out.size(-1), scores.size(-1), n_groups,
      n_limited_groups, probs_out.size(-1), static_cast<float>(route_scale), ptr(hidden_out), probs_out.data_ptr<float>(),
      idx_out.data_ptr<int>(), static_cast<int*>(ptr(slot_ids)), static_cast<float*>(ptr(slot_w)), stream_of(hidden)));
}

void expert_down_allreduce_op(const Tensor& vec, const Tensor& w, OptTensor, const Tensor& indices, const Tensor& scores,
                              const Tensor& x_residual, int64_t, Tensor out, OptTensor, Str, Str, OptTensor slot_ids, OptTensor slot_w) {
  need(vec, BF16, "vec"); need(out, BF16, "out"); need(x_residual, BF16, "x_residual");
  const int tokens = vec.size(-3), n_slots = vec.size(-2), inter = vec.size(-1);
  Tensor ids, wts;
  if (slot_ids.has_value() && slot_w.has_value()) {
    ids = *slot_ids;
    wts = *slot_w;
  } else {
    // the reference hands over routed indices and weights only; slot 0 is the shared expert (the last packed slot), weight 1
    const int n_routed = indices.size(-1);
    ids = at::cat({at::full({tokens, 1}, w.size(0) - 1, indices.options().dtype(I32)), indices.view({tokens, n_routed}).to(I32)}, 1)
              .contiguous();
    wts = at::cat({at::ones({tokens, 1}, scores.options().dtype(F32)), scores.view({tokens, n_routed}).to(F32)}, 1).contiguous();
  }
  check(tilert_expert_down_allreduce_op(ctx_of(out), ptr(vec), w.data_ptr<uint8_t>(), w.stride(0) * w.element_size(),
                                        ids.data_ptr<int>(), wts.data_ptr<float>(), ptr(x_residual), tokens, inter, out.size(-1),
                                        n_slots, ptr(out), nullptr, stream_of(out)));
}

void rmsnorm_up_gate_silu_op(const Tensor& x, const Tensor& gamma, const Tensor& w, Tensor out, Str, Str, OptTensor) {
  need(x, BF16, "x"); need(gamma, F32, "gamma"); need(out, BF16, "out");
  const int tokens = x.size(-2);
  check(tilert_rmsnorm_up_gate_silu_op(ctx_of(x), ptr(x), gamma.data_ptr<float>(), kEps, w.data_ptr<uint8_t>(), tokens, x.size(-1),
                                       out.numel() / tokens, ptr(out), stream_of(x)));
}

void rmsnorm_head_proj_op(const Tensor& x, const Tensor& gamma, const Tensor& w, OptTensor x_norm_out, Tensor logits_out, Str, Str,
                          OptTensor) {
  need(x, BF16, "x"); need(gamma, F32, "gamma"); need(w, BF16, "w"); need(logits_out, F32, "logits_out");
  check(tilert_rmsnorm_head_proj_op(ctx_of(x), ptr(x), gamma.data_ptr<float>(), kEps, ptr(w), x.size(-2), x.size(-1), w.size(0),
                                    ptr(x_norm_out), logits_out.data_ptr<float>(), stream_of(x)));
}

void eh_proj_allreduce_op(const Tensor& e_norm, const Tensor& h_norm, const Tensor& w, int64_t, Tensor out, OptTensor, Str, Str,
                          OptTensor) {
  need(e_norm, BF16, "e_norm"); need(h_norm, BF16, "h_norm"); need(w, BF16, "w"); need(out, BF16, "out");
  check(tilert_eh_proj_allreduce_op(ctx_of(w), ptr(e_norm), ptr(h_norm), ptr(w), e_norm.size(-2), e_norm.size(-1), ptr(out),
                                    stream_of(w)));
}

}  // namespace

#define TB_S "str model_arch, str kernel_type, Tensor? profile_logs=None"

TORCH_LIBRARY(tilert, m) {
  m.def("tilert_init_op() -> ()", &tilert_init_op);
  m.def("tilert_force_init_op() -> ()", &tilert_init_op);
  m.def("dsa_temp_vars_size() -> int", &dsa_temp_vars_size);
  m.def("alloc_misc_ws(int num_max_insts, int device_id) -> Tensor", &alloc_misc_ws);
  m.def("rmsnorm_op(Tensor x, Tensor gamma, Tensor(a!) out, " TB_S ") -> ()", &rmsnorm_op);
  m.def("rmsnorm_quant_op(Tensor x, Tensor gamma, Tensor(a!) out, Tensor(b!) q_out, Tensor(c!) q_scale_out, " TB_S
        ", Tensor? placeholder=None) -> ()", &rmsnorm_quant_op);
  m.def("projx_wqkva_op(Tensor x_q, Tensor x_scale, Tensor w, Tensor cur_pos, Tensor(a!) q_out, Tensor(b!) kv_out, "
        "Tensor(c!) pe_cache, " TB_S ", Tensor? placeholder=None) -> ()", &projx_wqkva_op);
  m.def("proj_w_op(Tensor x, Tensor w, Tensor(a!) out, " TB_S ") -> ()", &proj_w_op);
  m.def("rmsnorm_proj_qb_op(Tensor q, Tensor w, Tensor? w_scales, Tensor gamma, Tensor(a!) q_nope, Tensor(b!) q_pe, "
        "str model_arch, str algorithm, Tensor? profile_logs=None, Tensor? placeholder=None) -> ()", &rmsnorm_proj_qb_op);
  m.def("rmsnorm_kv_op(Tensor kv, Tensor gamma, Tensor cur_pos, Tensor(a!) kv_cache, " TB_S ") -> ()", &rmsnorm_kv_op);
  m.def("qkv_rope_op(Tensor(a!) q_pe, Tensor(b!) pe_cache, Tensor rope_freqs, Tensor cur_pos, " TB_S ") -> ()", &qkv_rope_op);
  m.def("rotate_op(Tensor x_in, Tensor(a!) out, Tensor freqs, " TB_S ") -> ()", &rotate_op);
  m.def("layernorm_rope_rotate_op(Tensor x_in, Tensor cur_pos, Tensor(a!) k_cache, Tensor weight, Tensor bias, Tensor freqs, " TB_S
        ") -> ()", &layernorm_rope_rotate_op);
  m.def("sparse_index_op(Tensor q, Tensor k_cache, Tensor weights, Tensor(a!) logits, int cur_pos, " TB_S ") -> ()", &sparse_index_op);
  m.def("sparse_index_topk_dsv32_op(Tensor q, Tensor k_cache, Tensor weights, Tensor(a!) logits, int cur_pos, Tensor(b!) indices, "
        "Tensor? workspace=None, Tensor? profile_logs=None) -> ()", &sparse_index_topk_dsv32_op);
  m.def("topk_accurate_op(Tensor logits, Tensor(a!) indices, int seq_len, Tensor? indices_ws, " TB_S ", int ratio=1) -> ()",
        &topk_accurate_op);
  m.def("topk_approximate_op(Tensor logits, Tensor(a!) indices, int seq_len, " TB_S ") -> ()", &topk_approximate_op);
  m.def("projq_wqb_op(Tensor q_nope, Tensor w, Tensor? w_scales, Tensor(a!) out, " TB_S ") -> ()", &projq_wqb_op);
  m.def("flash_sparse_mla_op(Tensor q, Tensor q_pe, Tensor kv, Tensor k_pe, Tensor indices, Tensor cur_pos, Tensor(a!) out, "
        "Tensor(b!) out_acc, Tensor(c!)? lse, Tensor(d!) lse_acc, int split_size, " TB_S
        ", Tensor? placeholder=None, float softmax_scale=-1.0) -> ()", &flash_sparse_mla_op);
  m.def("projo_wkvb_op(Tensor o, Tensor w, Tensor? w_scales, Tensor(a!) out, " TB_S ", Tensor? placeholder=None) -> ()", &projo_wkvb_op);
  m.def("unproj_o_allreduce_op(Tensor vec, Tensor w, Tensor? w_scale, Tensor x_residual, int flag, Tensor(a!) out, "
        "Tensor? profile_logs, str model_arch, str kernel_type) -> ()", &unproj_o_allreduce_op);
  m.def("padded_allreduce_add_op(Tensor partial_buf, Tensor x_in, int flag, Tensor(a!) vec_out, Tensor? profile_logs, "
        "str model_arch, str compute_kernel_type=\"bf16\") -> ()", &padded_allreduce_add_op);
  m.def("down_allreduce_op(Tensor vec, Tensor w, Tensor? w_scale, Tensor x_residual, int flag, Tensor(a!) out, " TB_S ") -> ()",
        &down_allreduce_op);
  m.def("rmsnorm_expert_proj_op(Tensor x, Tensor gamma, Tensor w_gate, Tensor(a!) scores_out, Tensor(b!) hidden_out, " TB_S ") -> ()",
        &rmsnorm_expert_proj_op);
  m.def("expert_select_up_gate_silu_op(Tensor hidden, Tensor scores, Tensor? bias, Tensor w, Tensor(a!) hidden_out, "
        "Tensor(b!) probs_out, Tensor(c!) idx_out, Tensor? profile_logs, str model_arch, str algorithm, int n_groups=8, "
        "int n_limited_groups=4, float route_scale=2.5, Tensor(d!)? slot_ids=None, Tensor(e!)? slot_w=None) -> ()",
        &expert_select_up_gate_silu_op);
  m.def("expert_down_allreduce_op(Tensor vec, Tensor w, Tensor? w_scale, Tensor indices, Tensor scores, Tensor x_residual, int flag, "
        "Tensor(a!) out, Tensor? profile_logs, str model_arch, str kernel_type, Tensor? slot_ids=None, Tensor? slot_w=None) -> ()",
        &expert_down_allreduce_op);
  m.def("rmsnorm_up_gate_silu_op(Tensor x, Tensor gamma, Tensor w, Tensor(a!) out, " TB_S ") -> ()", &rmsnorm_up_gate_silu_op);
  m.def("rmsnorm_head_proj_op(Tensor x, Tensor gamma, Tensor w, Tensor(a!)? x_norm_out, Tensor(b!) logits_out, " TB_S ") -> ()",
        &rmsnorm_head_proj_op);
  m.def("eh_proj_allreduce_op(Tensor e_norm, Tensor h_norm, Tensor w, int flag, Tensor(a!) out, Tensor? profile_logs, "
        "str model_arch, str kernel_type, Tensor? placeholder=None) -> ()", &eh_proj_allreduce_op);
}
