"""Operator wrappers of the decode path, named after the reference's
(tilert/models/deepseek_v3_2/ops/*.py).  Each wrapper checks dtypes/devices like the reference
wrapper does (ValueError on a bad argument), then calls the C ABI with raw pointers on the
current CUDA stream.  All outputs are caller-allocated tensors, as in the reference.

Operands called ``*_packed`` come from ``tilert_b200.pack``; ``xpack`` buffers are uint8 tensors of
``xpack_bytes(dim)`` bytes produced by ``rmsnorm_quant`` / ``act_pack``.
"""

from __future__ import annotations

import ctypes

import torch

import tilert_b200 as _tb

BF16 = torch.bfloat16
F32 = torch.float32
I32 = torch.int32
U8 = torch.uint8


def _p(t: torch.Tensor | None):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ctx(t: torch.Tensor):
    return ctypes.c_void_p(_tb.tilert_init(t.device.index))


def _rows(cache: torch.Tensor | None) -> int:
    """Rows of a cache tensor [..., T, d]: the kernels refuse to write a position at or past it."""
    return 0 if cache is None else int(cache.shape[-2])


def _need(t: torch.Tensor | None, dtype, name: str, optional: bool = False) -> None:
    if t is None:
        if optional:
            return
        raise ValueError(f"{name} must be given")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be a {dtype} tensor, got {t.dtype}.")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path).")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous.")


def set_grid_limit(device, max_ctas: int) -> None:
    """Cap the thread blocks of the streaming launches issued from now on (0 = one per SM); see
    ``tilert_b200_set_grid_limit``."""
    import ctypes

    dev = torch.device(device)
    _tb.check(_tb.lib().tilert_b200_set_grid_limit(ctypes.c_void_p(_tb.tilert_init(dev.index or 0)), max_ctas))


def num_sms(device) -> int:
    """SMs of the device (the grid of a streaming launch)."""
    dev = torch.device(device)
    return int(_tb.lib().tilert_b200_num_sms(ctypes.c_void_p(_tb.tilert_init(dev.index or 0))))


class chain:
    """Record the FP8 products issued inside the ``with`` block and launch them as ONE persistent
    kernel at its end (``tilert_b200_chain_begin`` / ``_end``): the role of the reference's single native
    call per decode step (modules/end2end.py:99-104).  ``rmsnorm_expert_proj``, ``projx_wis`` and
    ``attn_prep`` may be recorded as well (they run at the start of the product that follows them);
    any other operator raises inside the block.  ``enabled=False`` makes the block a no-op wrapper, so
    that callers can switch between chained and separate launches."""

    def __init__(self, device, enabled: bool = True):
        self.ctx = ctypes.c_void_p(_tb.tilert_init(torch.device(device).index)) if enabled else None

    def __enter__(self):
        if self.ctx is not None:
            _tb.check(_tb.lib().tilert_b200_chain_begin(self.ctx))
        return self

    def __exit__(self, exc_type, exc, tb):
        if self.ctx is None:
            return False
        if exc_type is not None:
            _tb.lib().tilert_b200_chain_abort(self.ctx)
            return False
        _tb.check(_tb.lib().tilert_b200_chain_end(self.ctx, _stream()))
        return False


def xpack_bytes(dim: int) -> int:
    return (dim // 128) * 1056


def new_xpack(dim: int, device) -> torch.Tensor:
    return torch.zeros(xpack_bytes(dim), dtype=U8, device=device)


# ------------------------------------------------------------------ activation preparation
def rmsnorm_quant(x, gamma, out, q_out, q_scale_out, profile_logs=None, *, model_arch="deepseek_v3_2",
                  eps=1e-6, xpack=None):
    """ops/rmsnorm_quant.py:19-64.  ``out`` / ``q_out`` / ``q_scale_out`` may be None."""
    _need(x, BF16, "x")
    _need(gamma, F32, "gamma", optional=True)
    _need(out, BF16, "out", optional=True)
    _need(q_out, torch.float8_e4m3fn, "q_out", optional=True)
    _need(q_scale_out, F32, "q_scale_out", optional=True)
    tokens, dim = x.shape[-2], x.shape[-1]
    _tb.check(_tb.lib().tilert_rmsnorm_quant_op(_ctx(x), _p(x), _p(gamma), eps, tokens, dim, _p(out), _p(q_out),
                                                _p(q_scale_out), None, 0, _p(xpack), _stream()))


def rmsnorm(x, gamma, out, profile_logs=None, *, model_arch="deepseek_v3_2", eps=1e-6):
    """ops/rmsnorm_quant.py:19-52 (the unquantised variant)."""
    rmsnorm_quant(x, gamma, out, None, None, profile_logs, model_arch=model_arch, eps=eps)


def act_pack(x, xpack, seg_scale=None):
    """Pack bf16 activations [tokens, dim] for the FP8 products (no reference counterpart: the
    reference kernels read bf16 activations directly)."""
    _need(x, BF16, "x")
    _need(xpack, U8, "xpack")
    _need(seg_scale, F32, "seg_scale", optional=True)
    tokens, dim = x.shape[-2], x.shape[-1]
    n_seg = 0 if seg_scale is None else seg_scale.shape[-1]
    _tb.check(_tb.lib().tilert_rmsnorm_quant_op(_ctx(x), _p(x), None, 0.0, tokens, dim, None, None, None,
                                                _p(seg_scale), n_seg, _p(xpack), _stream()))


def xq_repack(x_q, x_scale, xpack):
    _need(x_q, torch.float8_e4m3fn, "x_q")
    _need(x_scale, F32, "x_scale")
    tokens, dim = x_q.shape[-2], x_q.shape[-1]
    _tb.check(_tb.lib().tilert_xq_repack_op(_ctx(x_q), _p(x_q), _p(x_scale), tokens, dim, _p(xpack), _stream()))


# ---------------------------------------------------------------- FP8 streaming products
def projx_wqkva_packed(xpack, cols_per_token, w_packed, tokens, dim, q_lora, kv_lora, rope, ki_dim, cur_pos,
                       q_out, kv_out, pe_cache, ki_out):
    """Fused q_a / kv_a / k_pe / indexer-k product on packed activations."""
    _need(cur_pos, I32, "cur_pos", optional=rope == 0)
    _tb.check(_tb.lib().tilert_projx_wqkva_op(_ctx(w_packed), _p(xpack), cols_per_token, _p(w_packed), tokens, dim,
                                              q_lora, kv_lora, rope, ki_dim, _p(cur_pos), _p(q_out), _p(kv_out),
                                              _p(pe_cache), _rows(pe_cache), _p(ki_out), _stream()))


def rmsnorm_projx_wqkva(x, gamma, w_packed, cur_pos, q_out, kv_out, pe_cache, ki_out=None, *, eps=1e-6):
    """RMSNormProjxWqkva.tilert_forward (ops/rmsnorm_projx_wqkva.py:473-509) in one launch: RMSNorm,
    q_a / kv_a / k_pe (into ``pe_cache[cur_pos]``) and, when the packed weight carries them, the indexer
    key rows."""
    _need(x, BF16, "x")
    _need(gamma, F32, "gamma")
    _need(cur_pos, I32, "cur_pos")
    _need(q_out, BF16, "q_out")
    _need(kv_out, BF16, "kv_out")
    _need(pe_cache, BF16, "pe_cache")
    _need(ki_out, BF16, "ki_out", optional=True)
    tokens, dim = x.shape[-2], x.shape[-1]
    ki_dim = 0 if ki_out is None else ki_out.shape[-1]
    _tb.check(_tb.lib().tilert_rmsnorm_projx_wqkva_op(_ctx(x), _p(x), _p(gamma), eps, _p(w_packed), tokens, dim,
                                                      q_out.shape[-1], kv_out.shape[-1], pe_cache.shape[-1], ki_dim,
                                                      _p(cur_pos), _p(q_out), _p(kv_out), _p(pe_cache), _rows(pe_cache),
                                                      _p(ki_out), _stream()))


def projx_wqkva(x_in, x_scale, w_packed, cur_pos, q_out, kv_out, pe_cache, profile_logs=None, *,
                model_arch="deepseek_v3_2", ki_out=None):
    """ops/projx_wqkva.py:22-48: quantised activations (e4m3 + 1x128 f32 scales) in, q / kv out, k_pe
    written to ``pe_cache[cur_pos]``.  ``ki_out`` additionally emits the indexer key rows when the
    packed weight carries them (the reference's projx_wqaki, ops/projx_wqaki.py:11-44)."""
    _need(x_in, torch.float8_e4m3fn, "x_in")
    _need(x_scale, F32, "x_scale")
    _need(q_out, BF16, "q_out")
    _need(kv_out, BF16, "kv_out")
    _need(pe_cache, BF16, "pe_cache")
    tokens, dim = x_in.shape[-2], x_in.shape[-1]
    xp = new_xpack(dim, x_in.device)
    xq_repack(x_in, x_scale, xp)
    ki_dim = 0 if ki_out is None else ki_out.shape[-1]
    projx_wqkva_packed(xp, 1, w_packed, tokens, dim, q_out.shape[-1], kv_out.shape[-1], pe_cache.shape[-1], ki_dim,
                       cur_pos, q_out, kv_out, pe_cache, ki_out)


def rmsnorm_proj_q(q, gamma, w_packed, q_nope, q_pe, iq=None, *, eps=1e-6):
    """ops/rmsnorm_projq_wqb.py:21-43 (+ ops/rmsnorm_projq_wqi.py:21-40 when ``iq`` is given)."""
    _need(q, BF16, "q")
    _need(gamma, F32, "gamma")
    _need(q_nope, BF16, "q_nope", optional=True)
    _need(q_pe, BF16, "q_pe", optional=True)
    _need(iq, BF16, "iq", optional=True)
    tokens, q_lora = q.shape[-2], q.shape[-1]
    heads = 0 if q_nope is None else q_nope.shape[-2]
    nope = 0 if q_nope is None else q_nope.shape[-1]
    rope = 0 if q_pe is None else q_pe.shape[-1]
    iq_heads = 0 if iq is None else iq.shape[-2]
    iq_dim = 0 if iq is None else iq.shape[-1]
    _tb.check(_tb.lib().tilert_rmsnorm_proj_q_op(_ctx(q), _p(q), _p(gamma), eps, _p(w_packed), tokens, q_lora, heads,
                                                 nope, rope, iq_heads, iq_dim, _p(q_nope), _p(q_pe), _p(iq),
                                                 _stream()))


def projq_wqb(q_nope, w_packed, w_scales, out, profile_logs=None, compute_kernel_type="fp8mma", *,
              model_arch="deepseek_v3_2"):
    """ops/projq_wqb.py:24-54 (``w_scales`` is unused: scales travel inside ``w_packed``)."""
    _need(q_nope, BF16, "q_nope")
    _need(out, BF16, "out")
    tokens, heads, nope = q_nope.shape[-3], q_nope.shape[-2], q_nope.shape[-1]
    _tb.check(_tb.lib().tilert_projq_wqb_op(_ctx(out), _p(q_nope), _p(w_packed), tokens, heads, nope, out.shape[-1],
                                            _p(out), _stream()))


def projo_wkvb(o_lat, w_packed, w_scales, out, profile_logs=None, compute_kernel_type="fp8mma", *,
               model_arch="deepseek_v3_2"):
    """ops/projo_wkvb.py:24-54."""
    _need(o_lat, BF16, "o_lat")
    _need(out, BF16, "out")
    tokens, heads, c = o_lat.shape[-3], o_lat.shape[-2], o_lat.shape[-1]
    _tb.check(_tb.lib().tilert_projo_wkvb_op(_ctx(out), _p(o_lat), _p(w_packed), tokens, heads, c, out.shape[-1],
                                             _p(out), _stream()))


def unproj_o_allreduce(vec_in, w_packed, w_scale, x_in, flag, hidden_out, profile_logs=None, *,
                       model_arch="deepseek_v3_2", comm=None):
    """ops/unproj_o_allreduce.py:23-58.  ``flag`` (the reference's caller-supplied epoch) is ignored:
    the epoch lives in device memory."""
    _need(vec_in, BF16, "vec_in")
    _need(hidden_out, BF16, "hidden_out")
    _need(x_in, BF16, "x_in", optional=True)
    tokens = hidden_out.shape[-2]
    k = vec_in.numel() // tokens
    _tb.check(_tb.lib().tilert_unproj_o_allreduce_op(_ctx(hidden_out), _p(vec_in), _p(w_packed), _p(x_in), tokens, k,
                                                     hidden_out.shape[-1], _p(hidden_out),
                                                     None if comm is None else ctypes.c_void_p(comm), _stream()))


def padded_allreduce_add(partial_buf, x_in, flag, vec_out, profile_logs=None, *, model_arch="deepseek_v3_2",
                         compute_kernel_type="bf16", comm=None):
    """ops/padded_allreduce_add.py:17-41: ``vec_out = all_reduce(partial_buf) + x_in`` (bf16 [1, L, dim]).  ``flag`` is
    ignored: the call number lives in device memory."""
    _need(partial_buf, BF16, "partial_buf")
    _need(vec_out, BF16, "vec_out")
    _need(x_in, BF16, "x_in", optional=True)
    tokens = vec_out.shape[-2]
    _tb.check(_tb.lib().tilert_padded_allreduce_add_op(_ctx(vec_out), _p(partial_buf), _p(x_in), tokens,
                                                       vec_out.shape[-1], _p(vec_out),
                                                       None if comm is None else ctypes.c_void_p(comm), _stream()))


def rmsnorm_expert_proj(x, gamma, w_gate, scores_out, hidden_out, profile_logs=None, *,
                        model_arch="deepseek_v3_2", eps=1e-6):
    """ops/rmsnorm_expert_proj.py:151-169."""
    _need(x, BF16, "x")
    _need(gamma, F32, "gamma", optional=True)  # None: x is already normalised
    _need(scores_out, F32, "scores_out")
    _need(hidden_out, BF16, "hidden_out", optional=True)
    if w_gate.dtype not in (BF16, F32):
        raise ValueError("w_gate must be bfloat16 or float32")
    tokens, dim = x.shape[-2], x.shape[-1]
    _tb.check(_tb.lib().tilert_rmsnorm_expert_proj_op(_ctx(x), _p(x), _p(gamma), eps, _p(w_gate),
                                                      int(w_gate.dtype == F32), tokens, dim, w_gate.shape[0],
                                                      _p(scores_out), _p(hidden_out), _stream()))


def rmsnorm_proj_rows2(x, gamma, w_packed2, out, *, eps=1e-6):
    """``out = W . RMSNorm(x)`` for a bf16 weight packed as two e4m3 terms per row (``pack.pack_bf16_two_term``)
    on the FP8 weight stream: the router gate (ops/rmsnorm_expert_proj.py:151-169, f32 ``out``) and the indexer
    head weights (ops/projx_wis.py:21-40, bf16 ``out``).  ``gamma`` None: ``x`` is used as it is."""
    _need(x, BF16, "x")
    _need(gamma, F32, "gamma", optional=True)
    _need(w_packed2, U8, "w_packed2")
    if out.dtype not in (BF16, F32):
        raise ValueError("out must be bfloat16 or float32")
    tokens, dim = x.shape[-2], x.shape[-1]
    _tb.check(_tb.lib().tilert_rmsnorm_proj_rows2_op(_ctx(x), _p(x), _p(gamma), eps, _p(w_packed2), tokens, dim,
                                                     out.shape[-1], _p(out), int(out.dtype == F32), _stream()))


def expert_select_up_gate_silu(hidden_in, scores, bias, w_packed, hidden_out, probs_out, idx_out,
                               profile_logs=None, *, model_arch="deepseek_v3_2", dim, n_groups, n_limited_groups,
                               route_scale, slot_ids=None, slot_w=None, gamma=None, eps=1e-6):
    """ops/expert_sel_up_gate_silu.py:23-48.  ``hidden_in`` is the bf16 post-attention norm output (or, with
    ``gamma``, the raw state: the RMSNorm then runs inside the launch);
    ``w_packed`` is [n_experts + 1, tiles, kblocks, 16448] with the shared expert last."""
    _need(hidden_in, BF16, "hidden_in")
    _need(gamma, F32, "gamma", optional=True)
    _need(scores, F32, "scores")
    _need(bias, F32, "bias", optional=True)
    _need(hidden_out, BF16, "hidden_out")
    _need(probs_out, F32, "probs_out")
    _need(idx_out, I32, "idx_out")
    tokens = scores.shape[-2]
    n_experts = scores.shape[-1]
    top_k = probs_out.shape[-1]
    inter = hidden_out.shape[-1]
    stride = w_packed.stride(0) * w_packed.element_size()
    _tb.check(_tb.lib().tilert_expert_select_up_gate_silu_op(
        _ctx(scores), _p(hidden_in), _p(gamma), eps, _p(scores), _p(bias), _p(w_packed), stride, tokens, dim, inter, n_experts,
        n_groups, n_limited_groups, top_k, route_scale, _p(hidden_out), _p(probs_out), _p(idx_out), _p(slot_ids),
        _p(slot_w), _stream()))


def expert_down_allreduce(vec_in, w_packed, w_scale, indices, scores, x_in, flag, hidden_out, profile_logs=None, *,
                          model_arch="deepseek_v3_2", slot_ids, slot_w, comm=None):
    """ops/expert_down_allreduce.py:23-63.  ``slot_ids`` / ``slot_w`` are the per-slot expert ids and
    weights written by ``expert_select_up_gate_silu`` (slot 0 = shared expert, weight 1)."""
    _need(vec_in, BF16, "vec_in")
    _need(hidden_out, BF16, "hidden_out")
    tokens, n_slots, inter = vec_in.shape[-3], vec_in.shape[-2], vec_in.shape[-1]
    stride = w_packed.stride(0) * w_packed.element_size()
    _tb.check(_tb.lib().tilert_expert_down_allreduce_op(
        _ctx(hidden_out), _p(vec_in), _p(w_packed), stride, _p(slot_ids), _p(slot_w), _p(x_in), tokens, inter,
        hidden_out.shape[-1], n_slots, _p(hidden_out), None if comm is None else ctypes.c_void_p(comm), _stream()))


def rmsnorm_up_gate_silu(x, gamma, w_packed, out, profile_logs=None, *, model_arch="deepseek_v3_2", eps=1e-6):
    """ops/rmsnorm_up_gate_silu.py:26-44."""
    _need(x, BF16, "x")
    _need(gamma, F32, "gamma")
    _need(out, BF16, "out")
    tokens, dim = x.shape[-2], x.shape[-1]
    _tb.check(_tb.lib().tilert_rmsnorm_up_gate_silu_op(_ctx(x), _p(x), _p(gamma), eps, _p(w_packed), tokens, dim,
                                                       out.numel() // tokens, _p(out), _stream()))


def down_allreduce(vec_in, w_packed, w_scale, x_in, flag, hidden_out, profile_logs=None, *,
                   model_arch="deepseek_v3_2", comm=None):
    """ops/down_allreduce.py:24-59."""
    _need(vec_in, BF16, "vec_in")
    _need(hidden_out, BF16, "hidden_out")
    tokens = hidden_out.shape[-2]
    _tb.check(_tb.lib().tilert_down_allreduce_op(_ctx(hidden_out), _p(vec_in), _p(w_packed), _p(x_in), tokens,
                                                 vec_in.numel() // tokens, hidden_out.shape[-1], _p(hidden_out),
                                                 None if comm is None else ctypes.c_void_p(comm), _stream()))


# ------------------------------------------------------------------------ bf16 products
def projx_wis(x, w, out, profile_logs=None, *, model_arch="deepseek_v3_2", gamma=None, eps=1e-6):
    """ops/projx_wis.py:21-40: indexer head weights, bf16 weight [heads, dim].  With ``gamma`` the input
    is the raw hidden state and the RMSNorm runs inside the kernel."""
    _need(x, BF16, "x")
    _need(w, BF16, "w")
    _need(out, BF16, "out")
    _need(gamma, F32, "gamma", optional=True)
    _tb.check(_tb.lib().tilert_proj_w_op(_ctx(x), _p(x), _p(gamma), eps, _p(w), x.shape[-2], w.shape[0], w.shape[1],
                                         _p(out), _stream()))


def rmsnorm_head_proj(x, gamma, w, x_norm_out, logits_out, profile_logs=None, *, model_arch="deepseek_v3_2",
                      eps=1e-6):
    """ops/rmsnorm_head_proj.py:19-39."""
    _need(x, BF16, "x")
    _need(gamma, F32, "gamma")
    _need(w, BF16, "w")
    _need(logits_out, F32, "logits_out")
    _need(x_norm_out, BF16, "x_norm_out", optional=True)
    _tb.check(_tb.lib().tilert_rmsnorm_head_proj_op(_ctx(x), _p(x), _p(gamma), eps, _p(w), x.shape[-2], x.shape[-1],
                                                    w.shape[0], _p(x_norm_out), _p(logits_out), _stream()))


def inject_cache_fp8(kv_raw, pe_raw, ki_pages, seq_len, start_pos, kv_cache, pe_cache, ki_cache):
    """Latent caches of one layer from an external prefill in the FP8 wire format (pd_vllm/profiles/mla_nsa.py:
    16-41, 186-232, then generator.py:419-484): ``kv_raw`` uint8 [seq, 528], ``pe_raw`` uint8 [seq, 128],
    ``ki_pages`` uint8 [ceil(seq / 64), 8448] are dequantised into rows ``start_pos ..`` of the bf16 caches
    (the indexer keys also get their Hadamard rotation).  A plane may be None together with its cache."""
    for t, name in ((kv_raw, "kv_raw"), (pe_raw, "pe_raw"), (ki_pages, "ki_pages")):
        _need(t, torch.uint8, name, optional=True)
    for t, name in ((kv_cache, "kv_cache"), (pe_cache, "pe_cache"), (ki_cache, "ki_cache")):
        _need(t, BF16, name, optional=True)
    if seq_len == 0:
        return
    ref = next(t for t in (kv_cache, pe_cache, ki_cache) if t is not None)
    if kv_raw is not None and (kv_raw.numel() < seq_len * 528 or kv_cache is None):
        raise ValueError("kv_raw must hold seq_len rows of 528 bytes and come with kv_cache")
    if pe_raw is not None and (pe_raw.numel() < seq_len * 128 or pe_cache is None):
        raise ValueError("pe_raw must hold seq_len rows of 128 bytes and come with pe_cache")
    if ki_pages is not None and (ki_pages.numel() < (seq_len + 63) // 64 * 8448 or ki_cache is None):
        raise ValueError("ki_pages must hold ceil(seq_len / 64) pages of 8448 bytes and come with ki_cache")
    _tb.check(_tb.lib().tilert_inject_cache_fp8_op(_ctx(ref), _p(kv_raw), _p(pe_raw), _p(ki_pages), seq_len, start_pos,
                                                   ref.shape[-2], _p(kv_cache), _p(pe_cache), _p(ki_cache), _stream()))


def argmax_exchange(logits, index_offset, token_out, value_out=None, *, comm=None):
    """Greedy token over a vocabulary split across ranks (the arg-max behind the reference's
    ``PREDICTED_TOKENS``, modules/end2end.py:617-651): ``logits`` [..., S, vocab / world] f32 is this rank's
    slice starting at global index ``index_offset``; ``token_out`` int64 [S] receives the same token on
    every rank.  Without ``comm`` it is a local arg-max."""
    _need(logits, F32, "logits")
    _need(token_out, torch.int64, "token_out")
    _need(value_out, F32, "value_out", optional=True)
    tokens = logits.shape[-2]
    _tb.check(_tb.lib().tilert_argmax_exchange_op(_ctx(logits), _p(logits), logits.stride(-2), tokens, logits.shape[-1],
                                                  index_offset, None if comm is None else ctypes.c_void_p(comm),
                                                  _p(token_out), _p(value_out), _stream()))


# ------------------------------------------------------------- per-token vector operators
def eh_proj_allreduce(vec_in_enorm, vec_in_hnorm, w, flag, hidden_out, profile_logs=None, *,
                      model_arch="deepseek_v3_2"):
    """ops/eh_proj_allreduce.py:23-60.  ``w`` is eh_proj.weight [dim, 2*dim] bf16; ``flag`` is unused."""
    _need(vec_in_enorm, BF16, "vec_in_enorm")
    _need(vec_in_hnorm, BF16, "vec_in_hnorm")
    _need(w, BF16, "w")
    _need(hidden_out, BF16, "hidden_out")
    tokens, dim = vec_in_enorm.shape[-2], vec_in_enorm.shape[-1]
    _tb.check(_tb.lib().tilert_eh_proj_allreduce_op(_ctx(w), _p(vec_in_enorm), _p(vec_in_hnorm), _p(w), tokens, dim,
                                                    _p(hidden_out), _stream()))


def mtp_preprocess(e, h, gamma_e, gamma_h, w, hidden_out, profile_logs=None, *, model_arch="deepseek_v3_2", eps=1e-6,
                   e_norm_out=None, h_norm_out=None):
    """modules/mtp_preprocess.py:20-28 for already embedded tokens: enorm, hnorm, concat, eh_proj."""
    _need(e, BF16, "e")
    _need(h, BF16, "h")
    _need(gamma_e, F32, "gamma_e")
    _need(gamma_h, F32, "gamma_h")
    _need(w, BF16, "w")
    _need(hidden_out, BF16, "hidden_out")
    _need(e_norm_out, BF16, "e_norm_out", optional=True)
    _need(h_norm_out, BF16, "h_norm_out", optional=True)
    tokens, dim = e.shape[-2], e.shape[-1]
    _tb.check(_tb.lib().tilert_mtp_preprocess_op(_ctx(w), _p(e), _p(h), _p(gamma_e), _p(gamma_h), eps, _p(w), tokens,
                                                 dim, _p(e_norm_out), _p(h_norm_out), _p(hidden_out), _stream()))


def mtp_preprocess_rows(e, h, gamma_e, gamma_h, w, hidden_out, row_begin, n_rows, *, eps=1e-6):
    """``mtp_preprocess`` for output rows [row_begin, row_begin + n_rows) only: one rank's share when eh_proj is split
    by rows over a tensor-parallel group (``hidden_out`` is the whole [1, S, dim] tensor; only those columns change)."""
    _need(e, BF16, "e")
    _need(h, BF16, "h")
    _need(gamma_e, F32, "gamma_e")
    _need(gamma_h, F32, "gamma_h")
    _need(w, BF16, "w")
    _need(hidden_out, BF16, "hidden_out")
    tokens, dim = e.shape[-2], e.shape[-1]
    _tb.check(_tb.lib().tilert_mtp_preprocess_rows_op(_ctx(w), _p(e), _p(h), _p(gamma_e), _p(gamma_h), eps, _p(w), tokens,
                                                      dim, row_begin, n_rows, None, None, _p(hidden_out), _stream()))


def rmsnorm_kv(kv, gamma, cur_pos, kv_cache, profile_logs=None, *, model_arch="deepseek_v3_2", eps=1e-6):
    """ops/rmsnorm_kv.py:20-43."""
    _need(kv, BF16, "kv")
    _need(gamma, F32, "gamma")
    _need(cur_pos, I32, "cur_pos")
    _need(kv_cache, BF16, "kv_cache")
    _tb.check(_tb.lib().tilert_rmsnorm_kv_op(_ctx(kv), _p(kv), _p(gamma), eps, kv.shape[-2], kv.shape[-1],
                                             _p(cur_pos), _p(kv_cache), _rows(kv_cache), _stream()))


def qkv_rope(q_pe, pe_cache, rope_freqs, cur_pos, profile_logs=None, *, model_arch="deepseek_v3_2"):
    """ops/qkv_rope.py:21-50.  ``rope_freqs`` f32 [tokens, rope/2, 2] = (cos, sin)."""
    _need(q_pe, BF16, "q_pe")
    _need(pe_cache, BF16, "pe_cache")
    _need(rope_freqs, F32, "rope_freqs")
    _need(cur_pos, I32, "cur_pos")
    tokens, heads, rope = q_pe.shape[-3], q_pe.shape[-2], q_pe.shape[-1]
    _tb.check(_tb.lib().tilert_qkv_rope_op(_ctx(q_pe), _p(q_pe), heads, rope, _p(pe_cache), _p(cur_pos),
                                           _p(rope_freqs), tokens, _rows(pe_cache), _stream()))


def rotate(x_in, out, freqs, profile_logs=None, *, model_arch="deepseek_v3_2", rope=64):
    """ops/rotate.py:61-105."""
    _need(x_in, BF16, "x_in")
    _need(out, BF16, "out")
    _need(freqs, F32, "freqs")
    if x_in.shape[-1] != 128:
        raise ValueError("dim must be 128")
    tokens, heads = x_in.shape[-3], x_in.shape[-2]
    _tb.check(_tb.lib().tilert_rotate_op(_ctx(x_in), _p(x_in), _p(out), heads, rope, _p(freqs), tokens, _stream()))


def layernorm_rope_rotate(x_in, cur_pos, k_cache, weight, bias, freqs, profile_logs=None, *,
                          model_arch="deepseek_v3_2", rope=64):
    """ops/layernorm_rope_rotate.py:23-83."""
    _need(x_in, BF16, "x_in")
    _need(cur_pos, I32, "cur_pos")
    _need(k_cache, BF16, "k_cache")
    _need(weight, F32, "weight")
    _need(bias, F32, "bias")
    _need(freqs, F32, "freqs")
    if x_in.shape[-1] != 128:
        raise ValueError("dim must be 128")
    _tb.check(_tb.lib().tilert_layernorm_rope_rotate_op(_ctx(x_in), _p(x_in), _p(cur_pos), _p(k_cache), _p(weight),
                                                        _p(bias), _p(freqs), rope, x_in.shape[-2], _rows(k_cache), _stream()))


def attn_prep(x, in_gamma, w_is, idx_w_out, kv, kv_gamma, kv_cache, q_pe, pe_cache, iq, iq_out, ki, ki_cache,
              ln_weight, ln_bias, freqs, cur_pos, *, eps=1e-6, rope=64):
    """projx_wis + rmsnorm_kv + qkv_rope + rotate + layernorm_rope_rotate in one launch
    (ops/projx_wis.py:21-40, ops/rmsnorm_kv.py:20-43, ops/qkv_rope.py:21-50, ops/rotate.py:61-105,
    ops/layernorm_rope_rotate.py:23-83); same arguments and bit-identical results."""
    for t, nm in ((kv, "kv"), (kv_cache, "kv_cache"), (q_pe, "q_pe"), (pe_cache, "pe_cache"), (iq, "iq"),
                  (iq_out, "iq_out"), (ki, "ki"), (ki_cache, "ki_cache")):
        _need(t, BF16, nm)
    for t, nm in ((x, "x"), (w_is, "w_is"), (idx_w_out, "idx_w_out")):  # w_is None: no head-weight projection here
        _need(t, BF16, nm, optional=w_is is None)
    for t, nm in ((in_gamma, "in_gamma"), (kv_gamma, "kv_gamma"), (ln_weight, "ln_weight"), (ln_bias, "ln_bias"),
                  (freqs, "freqs")):
        _need(t, F32, nm)
    _need(cur_pos, I32, "cur_pos")
    if iq.shape[-1] != 128 or ki.shape[-1] != 128:
        raise ValueError("dim must be 128")
    tokens, heads = q_pe.shape[-3], q_pe.shape[-2]
    _tb.check(_tb.lib().tilert_attn_prep_op(
        _ctx(kv), _p(x), _p(in_gamma), eps, _p(w_is), iq.shape[-2], 0 if w_is is None else w_is.shape[1], _p(idx_w_out),
        _p(kv), _p(kv_gamma),
        kv.shape[-1], _p(kv_cache), _p(q_pe), heads, rope, _p(pe_cache), _p(iq), _p(iq_out), _p(ki), _p(ki_cache),
        _p(ln_weight), _p(ln_bias), _p(freqs), _p(cur_pos), tokens,
        min(_rows(kv_cache), _rows(pe_cache), _rows(ki_cache)), _stream()))


# ------------------------------------------------------------ indexer and sparse attention
def sparse_index(q, kv, weights, logits, cur_pos, profile_logs=None, compute_kernel_type="bf16", *,
                 model_arch="deepseek_v3_2", n_keys=None):
    """ops/sparse_index.py:11-69.  ``cur_pos`` is an int32 device tensor (position of token 0)."""
    _need(q, BF16, "q")
    _need(kv, BF16, "kv")
    _need(weights, BF16, "weights")
    _need(logits, F32, "logits")
    _need(cur_pos, I32, "cur_pos")
    heads, dim = q.shape[-2], q.shape[-1]
    if heads not in (16, 32, 64):
        raise ValueError(f"Unsupported head size: {heads}.")
    if dim != 128:
        raise ValueError("dim must be 128")
    tokens = q.shape[-3]
    n_keys = kv.shape[-2] if n_keys is None else n_keys
    _tb.check(_tb.lib().tilert_sparse_index_op(_ctx(q), _p(q), _p(kv), _p(weights), _p(logits), logits.shape[-1],
                                               heads, tokens, n_keys, _p(cur_pos), _stream()))


def topk_accurate(logits, n, topk, indices=None, profile_logs=None, *, model_arch="deepseek_v3_2"):
    """ops/topk.py:60-109: exact top-k of the first ``n`` logits of each row."""
    if logits.dtype != F32:
        raise ValueError("logits must be a float32 tensor.")
    _need(logits, F32, "logits")
    rows = logits.numel() // logits.shape[-1]
    if indices is None:
        indices = torch.empty(rows, topk, dtype=I32, device=logits.device)
    _tb.check(_tb.lib().tilert_topk_accurate_op(_ctx(logits), _p(logits), logits.shape[-1], rows, n, topk,
                                                _p(indices), _stream()))
    return indices


def sparse_index_topk(q, kv, weights, logits, indices, cur_pos, profile_logs=None, *, n_keys=None):
    """ops/sparse_index.py:72-128."""
    _need(indices, I32, "indices")
    _need(q, BF16, "q")
    _need(cur_pos, I32, "cur_pos")
    heads = q.shape[-2]
    tokens = q.shape[-3]
    n_keys = kv.shape[-2] if n_keys is None else n_keys
    _tb.check(_tb.lib().tilert_sparse_index_topk_op(_ctx(q), _p(q), _p(kv), _p(weights), _p(logits),
                                                    logits.shape[-1], heads, tokens, n_keys, _p(cur_pos),
                                                    indices.shape[-1], _p(indices), _stream()))


def flash_sparse_mla(q, q_pe, kv, k_pe, indices, cur_pos, output, profile_logs=None, *, softmax_scale,
                     model_arch="deepseek_v3_2", split_size=64, out_acc=None, lse=None, lse_acc=None, w_v=None, o_out=None):
    """ops/flash_sparse_mla.py:18-93.  With ``w_v`` (the packed value rows of kv_b) and ``o_out`` [.., heads, 128] the
    merge of the attention chunks also does the value up-projection (ops/projo_wkvb.py): one launch less."""
    _need(q, BF16, "q")
    _need(q_pe, BF16, "q_pe")
    _need(kv, BF16, "kv")
    _need(k_pe, BF16, "k_pe")
    _need(indices, I32, "indices")
    _need(cur_pos, I32, "cur_pos")
    _need(output, BF16, "output")
    tokens, heads = q.shape[-3], q.shape[-2]
    topk = indices.shape[-1]
    n_splits = (topk + split_size - 1) // split_size
    if out_acc is None:
        out_acc = torch.empty(tokens, heads, n_splits, 512, dtype=F32, device=q.device)
    if lse_acc is None:
        lse_acc = torch.empty(tokens, heads, n_splits, dtype=F32, device=q.device)
    if w_v is not None:
        _need(o_out, BF16, "o_out")
        _tb.check(_tb.lib().tilert_flash_sparse_mla_vproj_op(_ctx(q), _p(q), _p(q_pe), _p(kv), _p(k_pe), _p(indices), topk,
                                                             _p(cur_pos), heads, tokens, kv.shape[-2], softmax_scale,
                                                             split_size, _p(output), _p(out_acc), _p(lse), _p(lse_acc),
                                                             _p(w_v), q.shape[-1], o_out.shape[-1], _p(o_out), _stream()))
        return
    _tb.check(_tb.lib().tilert_flash_sparse_mla_op(_ctx(q), _p(q), _p(q_pe), _p(kv), _p(k_pe), _p(indices), topk,
                                                   _p(cur_pos), heads, tokens, kv.shape[-2], softmax_scale,
                                                   split_size, _p(output), _p(out_acc), _p(lse), _p(lse_acc),
                                                   _stream()))


# ------------------------------------------------------------------------------ sampling
def sample(logits, config, token_out, *, seed=0, step=None, step_value=0, token_logprob=None, topn_logprobs=None,
           topn_indices=None, vocab=None):
    """The driver's sampling step (modules/end2end.py:253-311, 665-703): ``config`` is the f32
    ``SAMPLING_CONFIG`` tensor (temperature, top_p, top_k, use_top_p); ``step`` an optional int64[2] device
    tensor that makes replayed CUDA graphs draw new numbers; outputs as ``TOP_P_SCORES`` /
    ``TOP_N_LOG_PROBS`` / ``TOP_N_INDICES``."""
    _need(logits, F32, "logits")
    _need(config, F32, "config")
    _need(token_out, I32, "token_out")
    _need(token_logprob, F32, "token_logprob", optional=True)
    _need(topn_logprobs, F32, "topn_logprobs", optional=True)
    _need(topn_indices, I32, "topn_indices", optional=True)
    if step is not None and (step.dtype != torch.int64 or step.numel() < 2 or not step.is_cuda):
        raise ValueError("step must be an int64 CUDA tensor of two elements")
    rows = logits.numel() // logits.shape[-1]
    n = logits.shape[-1] if vocab is None else vocab
    seed &= (1 << 63) - 1
    _tb.check(_tb.lib().tilert_sample_op(_ctx(logits), _p(logits), logits.shape[-1], rows, n, _p(config), seed, _p(step),
                                         step_value, _p(token_out), _p(token_logprob), _p(topn_logprobs),
                                         _p(topn_indices), _stream()))

