"""``torch.ops.tilert.*``: the dispatcher names and argument orders the reference's Python wrappers call
(tilert/models/deepseek_v3_2/ops/*.py; the list is the set of ``torch.ops.tilert.<name>(...)`` call
sites there), bound to this library's operators.

The reference loads its native library with ``torch.ops.load_library`` (tilert/__init__.py:68-77) and
its wrappers then call ``torch.ops.tilert.<op>``.  ``register()`` defines the same operator names with
the same positional argument order, so that a reference-style wrapper runs unchanged on this backend.
Weight operands are this library's packed tensors (``tilert_b200.pack``): the reference's own packed
layouts are private to its binary.  Trailing ``model_arch`` / ``kernel_type`` strings, ``profile_logs``
tensors, ``flag`` epochs and the empty ``int64`` placeholder tensors are accepted and ignored.

Every operator writes into caller-allocated outputs and returns nothing, like the reference's.
"""

from __future__ import annotations

import torch

from .models.deepseek_v3_2 import ops as _ops

_LIB: torch.library.Library | None = None

# name -> (schema, implementation).  ``Tensor(a!)`` marks the caller-allocated outputs.
_S = "str model_arch, str kernel_type, Tensor? profile_logs"


def _rmsnorm_kv_op(kv, gamma, cur_pos, kv_cache, model_arch, kernel_type, profile_logs=None):
    _ops.rmsnorm_kv(kv, gamma, cur_pos, kv_cache)


def _qkv_rope_op(q_pe, pe_cache, rope_freqs, cur_pos, model_arch, kernel_type, profile_logs=None):
    _ops.qkv_rope(q_pe, pe_cache, rope_freqs, cur_pos)


def _rotate_op(x_in, out, freqs, model_arch, kernel_type, profile_logs=None):
    _ops.rotate(x_in, out, freqs)


def _layernorm_rope_rotate_op(x_in, cur_pos, k_cache, weight, bias, freqs, model_arch, kernel_type, profile_logs=None):
    _ops.layernorm_rope_rotate(x_in, cur_pos, k_cache, weight, bias, freqs)


def _proj_w_op(x, w, out, model_arch, kernel_type, profile_logs=None):
    _ops.projx_wis(x, w, out)


def _rmsnorm_quant_op(x, gamma, out, q_out, q_scale_out, model_arch, kernel_type, profile_logs=None, placeholder=None):
    _ops.rmsnorm_quant(x, gamma, out, q_out, q_scale_out)


def _projq_wqb_op(q_nope, w, w_scales, out, model_arch, kernel_type, profile_logs=None):
    _ops.projq_wqb(q_nope, w, w_scales, out)


def _projo_wkvb_op(o, w, w_scales, out, model_arch, kernel_type, profile_logs=None, placeholder=None):
    _ops.projo_wkvb(o, w, w_scales, out)


def _unproj_o_allreduce_op(vec, w, w_scale, x_residual, flag, out, profile_logs, model_arch, kernel_type):
    _ops.unproj_o_allreduce(vec, w, w_scale, x_residual, flag, out)


def _rmsnorm_expert_proj_op(x, gamma, w_gate, scores_out, hidden_out, model_arch, kernel_type, profile_logs=None):
    _ops.rmsnorm_expert_proj(x, gamma, w_gate, scores_out, hidden_out)


def _rmsnorm_up_gate_silu_op(x, gamma, w, out, model_arch, kernel_type, profile_logs=None):
    _ops.rmsnorm_up_gate_silu(x, gamma, w, out)


def _down_allreduce_op(vec, w, w_scale, x_residual, flag, out, model_arch, kernel_type, profile_logs=None):
    _ops.down_allreduce(vec, w, w_scale, x_residual, flag, out)


def _rmsnorm_head_proj_op(x, gamma, w, x_norm_out, logits_out, model_arch, kernel_type, profile_logs=None):
    _ops.rmsnorm_head_proj(x, gamma, w, x_norm_out, logits_out)


def _eh_proj_allreduce_op(e_norm, h_norm, w, flag, out, profile_logs, model_arch, kernel_type, placeholder=None):
    _ops.eh_proj_allreduce(e_norm, h_norm, w, flag, out)


def _sparse_index_op(q, k_cache, weights, logits, cur_pos, model_arch, kernel_type, profile_logs=None):
    # the reference passes cur_pos as a host int here (ops/sparse_index.py:67)
    pos = torch.tensor([cur_pos], dtype=torch.int32, device=q.device)
    _ops.sparse_index(q, k_cache, weights, logits, pos, n_keys=k_cache.shape[-2])


def _topk_accurate_op(logits, indices, seq_len, indices_ws, model_arch, kernel_type, profile_logs=None, ratio=1):
    _ops.topk_accurate(logits, seq_len, indices.shape[-1], indices=indices)


def _flash_sparse_mla_op(q, q_pe, kv, k_pe, indices, cur_pos, out, out_acc, lse, lse_acc, split_size, model_arch,
                         kernel_type, profile_logs=None, placeholder=None, softmax_scale=-1.0):
    if softmax_scale <= 0:
        raise RuntimeError("flash_sparse_mla_op: softmax_scale must be given (the reference derives it from its "
                           "model arguments inside the native library)")
    _ops.flash_sparse_mla(q, q_pe, kv, k_pe, indices, cur_pos, out, softmax_scale=softmax_scale, split_size=split_size,
                          out_acc=out_acc, lse=lse, lse_acc=lse_acc)


def _rmsnorm_op(x, gamma, out, model_arch, kernel_type, profile_logs=None):
    _ops.rmsnorm(x, gamma, out)


def _projx_wqkva_op(x_q, x_scale, w, cur_pos, q_out, kv_out, pe_cache, model_arch, kernel_type, profile_logs=None,
                    placeholder=None):
    _ops.projx_wqkva(x_q, x_scale, w, cur_pos, q_out, kv_out, pe_cache)


def _rmsnorm_proj_qb_op(q, w, w_scales, gamma, q_nope, q_pe, model_arch, algorithm, profile_logs=None, placeholder=None):
    # ``w`` packed by pack.pack_q_b_rows; the indexer rows it may carry are not written here
    _ops.rmsnorm_proj_q(q, gamma, w, q_nope, q_pe)


def _sparse_index_topk_dsv32_op(q, k_cache, weights, logits, cur_pos, indices, workspace=None, profile_logs=None):
    pos = torch.tensor([cur_pos], dtype=torch.int32, device=q.device)
    _ops.sparse_index_topk(q, k_cache, weights, logits, indices, pos, n_keys=k_cache.shape[-2])


def _topk_approximate_op(logits, indices, seq_len, model_arch, kernel_type, profile_logs=None):
    # one selection kernel serves both names: the exact top-k is a valid answer to the approximate one
    _ops.topk_accurate(logits, seq_len, indices.shape[-1], indices=indices)


def _expert_select_up_gate_silu_op(hidden, scores, bias, w, hidden_out, probs_out, idx_out, profile_logs, model_arch,
                                   algorithm, n_groups=8, n_limited_groups=4, route_scale=2.5, slot_ids=None,
                                   slot_w=None):
    _ops.expert_select_up_gate_silu(hidden, scores, bias, w, hidden_out, probs_out, idx_out, dim=hidden.shape[-1],
                                    n_groups=n_groups, n_limited_groups=n_limited_groups, route_scale=route_scale,
                                    slot_ids=slot_ids, slot_w=slot_w)


def _expert_down_allreduce_op(vec, w, w_scale, indices, scores, x_residual, flag, out, profile_logs, model_arch,
                              kernel_type, slot_ids=None, slot_w=None):
    if slot_ids is None or slot_w is None:
        # the reference hands over routed indices and weights only; slot 0 is the shared expert (the last
        # packed slot) with weight 1
        tokens, n_routed = indices.shape[-2], indices.shape[-1]
        shared = torch.full((tokens, 1), w.shape[0] - 1, dtype=torch.int32, device=indices.device)
        slot_ids = torch.cat([shared, indices.view(tokens, n_routed).to(torch.int32)], dim=1).contiguous()
        slot_w = torch.cat([torch.ones(tokens, 1, device=scores.device), scores.view(tokens, n_routed).float()],
                           dim=1).contiguous()
    _ops.expert_down_allreduce(vec, w, w_scale, indices, scores, x_residual, flag, out, slot_ids=slot_ids, slot_w=slot_w)


def _alloc_misc_ws(num_max_insts, device_id):
    # the reference's instruction workspace (utils.py:62) has no role here: kernels take their parameters
    # at launch; a small zeroed tensor keeps callers that hold on to it working
    return torch.zeros(max(int(num_max_insts), 1), 16, dtype=torch.int64, device=torch.device("cuda", device_id))


_OPS = {
    "rmsnorm_kv_op": (f"(Tensor kv, Tensor gamma, Tensor cur_pos, Tensor(a!) kv_cache, {_S}=None) -> ()", _rmsnorm_kv_op),
    "qkv_rope_op": (f"(Tensor(a!) q_pe, Tensor(b!) pe_cache, Tensor rope_freqs, Tensor cur_pos, {_S}=None) -> ()",
                    _qkv_rope_op),
    "rotate_op": (f"(Tensor x_in, Tensor(a!) out, Tensor freqs, {_S}=None) -> ()", _rotate_op),
    "layernorm_rope_rotate_op": (f"(Tensor x_in, Tensor cur_pos, Tensor(a!) k_cache, Tensor weight, Tensor bias, "
                                 f"Tensor freqs, {_S}=None) -> ()", _layernorm_rope_rotate_op),
    "proj_w_op": (f"(Tensor x, Tensor w, Tensor(a!) out, {_S}=None) -> ()", _proj_w_op),
    "rmsnorm_quant_op": (f"(Tensor x, Tensor gamma, Tensor(a!) out, Tensor(b!) q_out, Tensor(c!) q_scale_out, {_S}=None, "
                         "Tensor? placeholder=None) -> ()", _rmsnorm_quant_op),
    "projq_wqb_op": (f"(Tensor q_nope, Tensor w, Tensor? w_scales, Tensor(a!) out, {_S}=None) -> ()", _projq_wqb_op),
    "projo_wkvb_op": (f"(Tensor o, Tensor w, Tensor? w_scales, Tensor(a!) out, {_S}=None, Tensor? placeholder=None) -> ()",
                      _projo_wkvb_op),
    "unproj_o_allreduce_op": ("(Tensor vec, Tensor w, Tensor? w_scale, Tensor x_residual, int flag, Tensor(a!) out, "
                              "Tensor? profile_logs, str model_arch, str kernel_type) -> ()", _unproj_o_allreduce_op),
    "rmsnorm_expert_proj_op": (f"(Tensor x, Tensor gamma, Tensor w_gate, Tensor(a!) scores_out, Tensor(b!) hidden_out, "
                               f"{_S}=None) -> ()", _rmsnorm_expert_proj_op),
    "rmsnorm_up_gate_silu_op": (f"(Tensor x, Tensor gamma, Tensor w, Tensor(a!) out, {_S}=None) -> ()",
                                _rmsnorm_up_gate_silu_op),
    "down_allreduce_op": (f"(Tensor vec, Tensor w, Tensor? w_scale, Tensor x_residual, int flag, Tensor(a!) out, {_S}=None)"
                          " -> ()", _down_allreduce_op),
    "rmsnorm_head_proj_op": (f"(Tensor x, Tensor gamma, Tensor w, Tensor(a!)? x_norm_out, Tensor(b!) logits_out, {_S}=None)"
                             " -> ()", _rmsnorm_head_proj_op),
    "eh_proj_allreduce_op": ("(Tensor e_norm, Tensor h_norm, Tensor w, int flag, Tensor(a!) out, Tensor? profile_logs, "
                             "str model_arch, str kernel_type, Tensor? placeholder=None) -> ()", _eh_proj_allreduce_op),
    "sparse_index_op": (f"(Tensor q, Tensor k_cache, Tensor weights, Tensor(a!) logits, int cur_pos, {_S}=None) -> ()",
                        _sparse_index_op),
    "topk_accurate_op": (f"(Tensor logits, Tensor(a!) indices, int seq_len, Tensor? indices_ws, {_S}=None, int ratio=1)"
                         " -> ()", _topk_accurate_op),
    "rmsnorm_op": (f"(Tensor x, Tensor gamma, Tensor(a!) out, {_S}=None) -> ()", _rmsnorm_op),
    "projx_wqkva_op": (f"(Tensor x_q, Tensor x_scale, Tensor w, Tensor cur_pos, Tensor(a!) q_out, Tensor(b!) kv_out, "
                       f"Tensor(c!) pe_cache, {_S}=None, Tensor? placeholder=None) -> ()", _projx_wqkva_op),
    "rmsnorm_proj_qb_op": ("(Tensor q, Tensor w, Tensor? w_scales, Tensor gamma, Tensor(a!) q_nope, Tensor(b!) q_pe, "
                           "str model_arch, str algorithm, Tensor? profile_logs=None, Tensor? placeholder=None) -> ()",
                           _rmsnorm_proj_qb_op),
    "sparse_index_topk_dsv32_op": ("(Tensor q, Tensor k_cache, Tensor weights, Tensor(a!) logits, int cur_pos, "
                                   "Tensor(b!) indices, Tensor? workspace=None, Tensor? profile_logs=None) -> ()",
                                   _sparse_index_topk_dsv32_op),
    "topk_approximate_op": (f"(Tensor logits, Tensor(a!) indices, int seq_len, {_S}=None) -> ()", _topk_approximate_op),
    "expert_select_up_gate_silu_op": ("(Tensor hidden, Tensor scores, Tensor? bias, Tensor w, Tensor(a!) hidden_out, "
                                      "Tensor(b!) probs_out, Tensor(c!) idx_out, Tensor? profile_logs, str model_arch, "
                                      "str algorithm, int n_groups=8, int n_limited_groups=4, float route_scale=2.5, "
                                      "Tensor(d!)? slot_ids=None, Tensor(e!)? slot_w=None) -> ()",
                                      _expert_select_up_gate_silu_op),
    "expert_down_allreduce_op": ("(Tensor vec, Tensor w, Tensor? w_scale, Tensor indices, Tensor scores, "
                                 "Tensor x_residual, int flag, Tensor(a!) out, Tensor? profile_logs, str model_arch, "
                                 "str kernel_type, Tensor? slot_ids=None, Tensor? slot_w=None) -> ()",
                                 _expert_down_allreduce_op),
    "flash_sparse_mla_op": ("(Tensor q, Tensor q_pe, Tensor kv, Tensor k_pe, Tensor indices, Tensor cur_pos, "
                            "Tensor(a!) out, Tensor(b!) out_acc, Tensor(c!)? lse, Tensor(d!) lse_acc, int split_size, "
                            f"{_S}=None, Tensor? placeholder=None, float softmax_scale=-1.0) -> ()", _flash_sparse_mla_op),
}


def op_names() -> list[str]:
    """Names registered under ``torch.ops.tilert`` by :func:`register`."""
    return ["tilert_init_op", "tilert_force_init_op", "dsa_temp_vars_size", "alloc_misc_ws", *_OPS]


def register() -> None:
    """Define the ``tilert`` operator namespace (once per process; a second call is a no-op).

    Raises ``RuntimeError`` if another library has already defined the namespace (the reference's own
    ``libtilert*.so`` loaded in the same process): the two backends cannot be mixed."""
    global _LIB
    if _LIB is not None:
        return
    import tilert_b200 as tb
    from .models.deepseek_v3_2.temp_var_indices import TEMP_VARS_SIZE

    lib = torch.library.Library("tilert", "DEF")
    lib.define("tilert_init_op() -> ()")
    lib.impl("tilert_init_op", lambda: tb.tilert_init(torch.cuda.current_device()) and None, "CompositeExplicitAutograd")
    lib.define("tilert_force_init_op() -> ()")
    lib.impl("tilert_force_init_op", lambda: tb.tilert_init(torch.cuda.current_device()) and None,
             "CompositeExplicitAutograd")
    lib.define("alloc_misc_ws(int num_max_insts, int device_id) -> Tensor")
    lib.impl("alloc_misc_ws", _alloc_misc_ws, "CompositeExplicitAutograd")
    lib.define("dsa_temp_vars_size() -> int")
    lib.impl("dsa_temp_vars_size", lambda: TEMP_VARS_SIZE, "CompositeExplicitAutograd")
    for name, (schema, fn) in _OPS.items():
        lib.define(name + schema)
        lib.impl(name, fn, "CompositeExplicitAutograd")
    _LIB = lib
