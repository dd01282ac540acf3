"""One decoder layer of the batch-1 decode path: packed weights, scratch tensors, latent caches and
the operator sequence.

The reference keeps these as registries (tilert/models/deepseek_v3_2/modules/mla_v2.py,
modules/moe.py, modules/mlp.py, modules/dsa.py:105-229) and runs the sequence inside its native
library; here the sequence is explicit Python over the operator wrappers, and a whole step can be
captured in a CUDA graph.  Sharding is symmetric: every rank holds ``n_heads / world`` attention
heads and a ``1 / world`` slice of every expert's intermediate dimension; the row-parallel
products (o_proj, down_proj) reduce inside their kernels.
"""

from __future__ import annotations

import math
import os

import torch

from tilert_b200 import pack
from . import ops
from .model_args import ModelArgs

BF16 = torch.bfloat16
F32 = torch.float32
I32 = torch.int32


def precompute_freqs(args: ModelArgs) -> torch.Tensor:
    """(cos, sin) table [max_seq_len, rope/2, 2] f32 with the YaRN correction of
    tilert/models/utils.py:17-118."""
    dim, base = args.qk_rope_head_dim, args.rope_theta
    freqs = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    if args.rope_factor is not None and args.max_seq_len > args.original_seq_len:
        def corr(n_rot):
            return dim * math.log(args.original_seq_len / (n_rot * 2 * math.pi)) / (2 * math.log(base))
        low = float(max(math.floor(corr(args.beta_fast)), 0))
        high = float(min(math.ceil(corr(args.beta_slow)), dim - 1))
        if low == high:
            high += 0.001
        ramp = torch.clamp((torch.arange(dim // 2, dtype=torch.float32) - low) / (high - low), 0, 1)
        smooth = 1 - ramp
        freqs = freqs / args.rope_factor * (1 - smooth) + freqs * smooth
    ang = torch.outer(torch.arange(args.max_seq_len), freqs)
    return torch.view_as_real(torch.polar(torch.ones_like(ang), ang)).contiguous()


# The two-stream step.  Up to FORK_MAX_KEYS keys the indexer's scoring + selection is the short-row kernel, whose
# thread blocks never wait on one another: it and the vector launch take whatever SMs the product beside them
# (capped at FORK_PRODUCT_CTAS of the 148 SMs) leaves free.  Beyond that the selection is a cooperative launch whose
# blocks meet at grid-wide barriers: it and the product then get fixed shares of the SMs that add up to the SM count
# (FORK_LONG_PRODUCT_SHARE of them for the product, the rest for the selection), so both are always fully resident
# whatever the order they start in.
FORK_MAX_KEYS = 8192
FORK_PRODUCT_CTAS = int(os.environ.get("TILERT_B200_FORK_CTAS", "112"))  # 96-128 measure the same within 0.5 %
FORK_LONG_PRODUCT_SHARE = 64 / 148  # of the SM count; the selection gets the rest


_SIDE_STREAMS: dict = {}


def _side_stream(dev: torch.device) -> "torch.cuda.Stream":
    """One second stream per device, shared by all layers."""
    if dev not in _SIDE_STREAMS:
        _SIDE_STREAMS[dev] = torch.cuda.Stream(device=dev)
    return _SIDE_STREAMS[dev]


def softmax_scale(args: ModelArgs) -> float:
    """tilert/models/deepseek_v3_2/ops/flash_sparse_mla.py:125-130."""
    scale = (args.qk_nope_head_dim + args.qk_rope_head_dim) ** -0.5
    mscale = 1.0 if args.rope_factor is None else 0.1 * math.log(args.rope_factor) + 1.0
    return scale * mscale * mscale


class LayerWeights:
    """Packed per-rank weights of one layer, built from an HF-keyed FP8 state dict."""

    def __init__(self, args: ModelArgs, sd: dict[str, torch.Tensor], li: int, device, world: int = 1, rank: int = 0,
                 expert_ids: list[int] | None = None):
        a = args
        dev = torch.device(device)
        p = f"model.layers.{li}"
        at = f"{p}.self_attn"

        def g(key):
            return sd[key].to(dev)

        def f32(key):
            return sd[key].to(dev, F32).contiguous()

        hl = a.n_heads // world
        h0 = rank * hl
        hd = a.qk_nope_head_dim + a.qk_rope_head_dim
        self.in_norm = f32(f"{p}.input_layernorm.weight")
        self.post_norm = f32(f"{p}.post_attention_layernorm.weight")
        self.q_norm = f32(f"{at}.q_a_layernorm.weight")
        self.kv_norm = f32(f"{at}.kv_a_layernorm.weight")
        self.k_norm_w = f32(f"{at}.indexer.k_norm.weight")
        self.k_norm_b = f32(f"{at}.indexer.k_norm.bias")
        self.wis = g(f"{at}.indexer.weights_proj.weight").to(BF16).contiguous()
        # the same weight as two e4m3 terms per row (exact for bf16): rides the FP8 weight stream in chained launches
        self.wis2 = pack.pack_bf16_two_term(self.wis)
        # q_a | kv_a | k_pe | indexer wk: replicated on every rank
        self.w_qkva = pack.pack_concat([
            (g(f"{at}.q_a_proj.weight"), g(f"{at}.q_a_proj.weight_scale_inv")),
            (g(f"{at}.kv_a_proj_with_mqa.weight"), g(f"{at}.kv_a_proj_with_mqa.weight_scale_inv")),
            (g(f"{at}.indexer.wk.weight"), g(f"{at}.indexer.wk.weight_scale_inv")),
        ])
        # q_b: this rank's heads, plus the (replicated) indexer query projection
        wq_b, sq_b = g(f"{at}.q_b_proj.weight"), g(f"{at}.q_b_proj.weight_scale_inv")
        rs_full = pack.row_scales(sq_b, wq_b.shape[0])
        rows = slice(h0 * hd, (h0 + hl) * hd)
        self.w_qb = pack.pack_q_b_rows(wq_b.view(torch.uint8)[rows], rs_full[rows], hl, a.qk_nope_head_dim,
                                       a.qk_rope_head_dim, g(f"{at}.indexer.wq_b.weight"),
                                       g(f"{at}.indexer.wq_b.weight_scale_inv"))
        wkv_b, skv_b = g(f"{at}.kv_b_proj.weight"), g(f"{at}.kv_b_proj.weight_scale_inv")
        per_head = a.qk_nope_head_dim + a.v_head_dim
        kv_rows = slice(h0 * per_head, (h0 + hl) * per_head)
        kv_srows = slice(h0 * per_head // 128, (h0 + hl) * per_head // 128)
        self.w_absorb = pack.pack_kv_b_absorb(wkv_b[kv_rows], skv_b[kv_srows], hl, a.qk_nope_head_dim, a.v_head_dim)
        self.w_v = pack.pack_kv_b_v(wkv_b[kv_rows], skv_b[kv_srows], hl, a.qk_nope_head_dim, a.v_head_dim)
        w_o, s_o = g(f"{at}.o_proj.weight"), g(f"{at}.o_proj.weight_scale_inv")
        oc = slice(h0 * a.v_head_dim, (h0 + hl) * a.v_head_dim)
        ocs = slice(h0 * a.v_head_dim // 128, (h0 + hl) * a.v_head_dim // 128)
        self.w_o = pack.pack_matrix(w_o[:, oc].contiguous(), s_o[:, ocs].contiguous())

        m = f"{p}.mlp"
        self.dense = li < a.n_dense_layers
        if self.dense:
            il = a.inter_dim // world
            r = slice(rank * il, (rank + 1) * il)
            rs_ = slice(rank * il // 128, (rank + 1) * il // 128)
            self.w_gu = pack.pack_gate_up(g(f"{m}.gate_proj.weight")[r], g(f"{m}.gate_proj.weight_scale_inv")[rs_],
                                          g(f"{m}.up_proj.weight")[r], g(f"{m}.up_proj.weight_scale_inv")[rs_])
            self.w_down = pack.pack_matrix(g(f"{m}.down_proj.weight")[:, r].contiguous(),
                                           g(f"{m}.down_proj.weight_scale_inv")[:, rs_].contiguous())
            self.inter_local = il
        else:
            il = a.moe_inter_dim // world
            r = slice(rank * il, (rank + 1) * il)
            rs_ = slice(rank * il // 128, (rank + 1) * il // 128)
            self.router = g(f"{m}.gate.weight").contiguous()
            # bf16 in HF checkpoints: packed like wis2 for the weight stream; an f32 gate keeps its row product
            self.router2 = pack.pack_bf16_two_term(self.router) if self.router.dtype == BF16 else None
            self.router_bias = f32(f"{m}.gate.e_score_correction_bias")
            n_e = a.n_routed_experts
            gu_tiles, n_kb = 2 * il // 128, a.dim // 128
            # [n_experts + 1] slots, the shared expert last; experts absent from the state dict stay zero
            self.w_gu = torch.zeros(n_e + 1, gu_tiles, n_kb, pack.WBLK_BYTES, dtype=torch.uint8, device=dev)
            self.w_down = torch.zeros(n_e + 1, a.dim // 128, il // 128, pack.WBLK_BYTES, dtype=torch.uint8, device=dev)
            present = range(n_e) if expert_ids is None else expert_ids
            for slot, name in [(n_e, "shared_experts")] + [(e, f"experts.{e}") for e in present]:
                k = f"{m}.{name}"
                self.w_gu[slot] = pack.pack_gate_up(g(f"{k}.gate_proj.weight")[r], g(f"{k}.gate_proj.weight_scale_inv")[rs_],
                                                    g(f"{k}.up_proj.weight")[r], g(f"{k}.up_proj.weight_scale_inv")[rs_])
                self.w_down[slot] = pack.pack_matrix(g(f"{k}.down_proj.weight")[:, r].contiguous(),
                                                     g(f"{k}.down_proj.weight_scale_inv")[:, rs_].contiguous())
            self.inter_local = il

    def weight_bytes(self, args: ModelArgs) -> int:
        """Bytes of weights one decode step of this layer streams from HBM on this rank."""
        n = sum(t.numel() for t in (self.w_qkva, self.w_qb, self.w_absorb, self.w_v, self.w_o))
        n += self.wis.numel() * 2
        if self.dense:
            n += self.w_gu.numel() + self.w_down.numel()
        else:
            per = self.w_gu[0].numel() + self.w_down[0].numel()
            n += per * (args.n_activated_experts + args.n_shared_experts) + self.router.numel() * self.router.element_size()
        return n


class LayerScratch:
    """The per-step scratch tensors of a decoder layer (one rank).  Layers run one after the other, so a model
    can give all its layers ONE of these -- the reference does the same with its ``temp_vars`` list
    (modules/dsa.py:105-229), and ``from_temp_vars`` builds a scratch set on top of such a list, indexed by
    ``DsaTempVarIdx``.  The layer output alternates between two buffers, because a layer still reads its input
    (the previous layer's output) while it writes its own."""

    def __init__(self, args: ModelArgs, device, cache_len: int, max_tokens: int = 1, world: int = 1):
        a, dev, s = args, torch.device(device), max_tokens
        hl = a.n_heads // world
        z = lambda *shape, dtype=BF16: torch.zeros(*shape, dtype=dtype, device=dev)  # noqa: E731
        self.q_a = z(1, s, a.q_lora_rank)
        self.kv = z(1, s, a.kv_lora_rank)
        self.ki = z(1, s, a.index_head_dim)
        self.idx_w = z(1, s, a.index_n_heads)
        self.q_nope = z(1, s, hl, a.qk_nope_head_dim)
        self.q_pe = z(1, s, hl, a.qk_rope_head_dim)
        self.iq = z(1, s, a.index_n_heads, a.index_head_dim)
        self.iq_rt = z(1, s, a.index_n_heads, a.index_head_dim)
        self.idx_logits = z(1, s, cache_len, dtype=F32)
        self.sel = torch.full((1, s, a.index_topk), -1, dtype=I32, device=dev)
        self.q_lat = z(1, s, hl, a.kv_lora_rank)
        self.o_lat = z(1, s, hl, a.kv_lora_rank)
        n_splits = (a.index_topk + 63) // 64
        self.o_acc = z(1, s, hl, n_splits, a.kv_lora_rank, dtype=F32)
        self.lse = z(1, s, hl, dtype=F32)
        self.lse_acc = z(1, s, hl, n_splits, dtype=F32)
        self.o = z(1, s, hl, a.v_head_dim)
        self.h = z(1, s, a.dim)
        self.h_norm = z(1, s, a.dim)
        self.outs = [z(1, s, a.dim), z(1, s, a.dim)]
        n_slots = a.n_activated_experts + 1
        self.scores = z(1, s, a.n_routed_experts, dtype=F32)
        self.probs = z(1, s, a.n_activated_experts, dtype=F32)
        self.eidx = z(1, s, a.n_activated_experts, dtype=I32)
        self.slot_ids = z(s, n_slots, dtype=I32)
        self.slot_w = z(s, n_slots, dtype=F32)
        dense_local = a.inter_dim // world if a.n_dense_layers > 0 else 0
        self.ffn_flat = z(s * max(n_slots * (a.moe_inter_dim // world), dense_local))

    @classmethod
    def from_temp_vars(cls, args: ModelArgs, tv: list[torch.Tensor], cache_len: int, max_tokens: int = 1,
                       world: int = 1) -> "LayerScratch":
        """A scratch set whose tensors ARE the driver's ``temp_vars`` (tilert/models/deepseek_v3_2/
        temp_var_indices.py:15-76), so that code reading ``temp_vars[Idx.X]`` after a step sees the step's values."""
        from .temp_var_indices import Idx

        a, s = args, max_tokens
        hl = a.n_heads // world
        n_splits = (a.index_topk + 63) // 64
        n_slots = a.n_activated_experts + 1
        self = cls.__new__(cls)

        def take(idx, *shape):
            t = tv[idx]
            n = 1
            for d in shape:
                n *= d
            if t.numel() < n:
                raise ValueError(f"temp_vars[{Idx(idx).name}] holds {t.numel()} elements, the step needs {n}")
            return t.reshape(-1)[:n].view(*shape)

        self.q_a = take(Idx.Q, 1, s, a.q_lora_rank)
        self.kv = take(Idx.KV, 1, s, a.kv_lora_rank)
        self.ki = take(Idx.KI, 1, s, a.index_head_dim)
        self.idx_w = take(Idx.IDX_SCORES, 1, s, a.index_n_heads)
        self.q_nope = take(Idx.Q_NOPE_DOWN, 1, s, hl, a.qk_nope_head_dim)
        self.q_pe = take(Idx.Q_PE, 1, s, hl, a.qk_rope_head_dim)
        self.iq = take(Idx.IQ, 1, s, a.index_n_heads, a.index_head_dim)
        self.iq_rt = take(Idx.IQ_RT, 1, s, a.index_n_heads, a.index_head_dim)
        self.idx_logits = take(Idx.IDX_LOGITS, 1, s, cache_len)
        self.sel = take(Idx.IDX_SELECTS, 1, s, a.index_topk)
        self.q_lat = take(Idx.Q_NOPE, 1, s, hl, a.kv_lora_rank)
        self.o_lat = take(Idx.O, 1, s, hl, a.kv_lora_rank)
        self.o_acc = take(Idx.O_ACC, 1, s, hl, n_splits, a.kv_lora_rank)
        self.lse = take(Idx.O_LSE, 1, s, hl)
        self.lse_acc = take(Idx.O_LSE_ACC, 1, s, hl, n_splits)
        self.o = take(Idx.PROJ_O, 1, s, hl, a.v_head_dim)
        self.h = take(Idx.UNPROJ_O, 1, s, a.dim)
        self.h_norm = take(Idx.X_MLP_IN, 1, s, a.dim)
        self.outs = [take(Idx.EXP_OUT, 1, s, a.dim), take(Idx.X_TENSOR, 1, s, a.dim)]
        self.scores = take(Idx.SCORES, 1, s, a.n_routed_experts)
        self.probs = take(Idx.SEL_PROBS, 1, s, a.n_activated_experts)
        self.eidx = take(Idx.SEL_INDICES, 1, s, a.n_activated_experts)
        dev = tv[Idx.Q].device
        self.slot_ids = torch.zeros(s, n_slots, dtype=I32, device=dev)   # (no counterpart among the temp vars)
        self.slot_w = torch.zeros(s, n_slots, dtype=F32, device=dev)
        dense_local = a.inter_dim // world if a.n_dense_layers > 0 else 0
        self.ffn_flat = take(Idx.UP_GATE, s * max(n_slots * (a.moe_inter_dim // world), dense_local))
        return self


class DecoderLayer:
    """Caches, scratch tensors (its own, or a set shared with the model's other layers) and the operator
    sequence of one layer (one rank)."""

    def __init__(self, args: ModelArgs, weights: LayerWeights, device, cache_len: int, max_tokens: int = 1,
                 world: int = 1, comm: int | None = None, scratch: LayerScratch | None = None, out_slot: int = 0):
        a, dev, s = args, torch.device(device), max_tokens
        self.args, self.w, self.world, self.comm = a, weights, world, comm
        self.hl = a.n_heads // world
        self.cache_len = cache_len
        z = lambda *shape, dtype=BF16: torch.zeros(*shape, dtype=dtype, device=dev)  # noqa: E731
        self.kv_cache = z(1, cache_len, a.kv_lora_rank)
        self.pe_cache = z(1, cache_len, a.qk_rope_head_dim)
        self.ki_cache = z(1, cache_len, a.index_head_dim)
        sc = scratch if scratch is not None else LayerScratch(a, dev, cache_len, s, world)
        self.scratch = sc
        for name in ("q_a", "kv", "ki", "idx_w", "q_nope", "q_pe", "iq", "iq_rt", "idx_logits", "sel", "q_lat", "o_lat",
                     "o_acc", "lse", "lse_acc", "o", "h", "h_norm", "scores", "probs", "eidx", "slot_ids", "slot_w"):
            setattr(self, name, getattr(sc, name))
        self.out = sc.outs[out_slot & 1]
        self.mla_split = 64  # keys per attention split (a multiple of 64): splits x groups of 16 heads x tokens CTAs
        self.n_splits = (a.index_topk + 63) // 64
        if weights.dense:
            self.ffn_hidden = sc.ffn_flat[: s * weights.inter_local].view(1, s, weights.inter_local)
        else:
            n_slots = a.n_activated_experts + 1
            self.ffn_hidden = sc.ffn_flat[: s * n_slots * weights.inter_local].view(1, s, n_slots, weights.inter_local)
        self.forced_scores: torch.Tensor | None = None
        # When set ([1, S, topk] int32), replaces the indexer's selection before attention -- the role of
        # the reference's receive_selected_token_ids (ops/receive_selected_token_ids.py:10-35), used by
        # parity tests to separate the discrete selection from the floating-point path.
        self.injected_sel: torch.Tensor | None = None
        self.scale = softmax_scale(a)
        # The FP8 products of a step run one launch each (programmatic dependent launch overlaps their
        # boundaries), or, with TILERT_B200_CHAIN=1, as two chained persistent launches: measured, the single
        # launches are 4-6 % faster on one and two GPUs
        self.chained = os.environ.get("TILERT_B200_CHAIN", "0") == "1"
        # With single launches: the absorbed-q product beside the vector work and the indexer (two streams;
        # measured 6 us per layer step faster on one GPU; TILERT_B200_FORK=0 keeps everything on one stream)
        self.fork = os.environ.get("TILERT_B200_FORK", "1") != "0"
        # value up-projection inside the merge of the attention chunks (one launch less; TILERT_B200_FUSE_VPROJ=0:
        # the streaming product as a launch of its own)
        self.fuse_vproj = (os.environ.get("TILERT_B200_FUSE_VPROJ", "1") != "0" and a.kv_lora_rank == 512
                           and a.v_head_dim == 128)
        self._side = _side_stream(dev)  # (the attribute ``fork`` may be switched at any time between steps)
        self._ev_fork = torch.cuda.Event()
        self._ev_join = torch.cuda.Event()
        n_sm = ops.num_sms(dev)
        self._long_product_ctas = max(1, int(n_sm * FORK_LONG_PRODUCT_SHARE))
        self._long_select_ctas = max(1, n_sm - self._long_product_ctas)

    def inject_cache(self, ki: torch.Tensor, kv: torch.Tensor, pe: torch.Tensor, start_pos: int = 0) -> None:
        """Rows ``start_pos ..`` of the three caches from bf16 tensors [seq, 128 / 512 / 64] computed by an
        external prefill (one layer of DSAv32Generator.inject_cache, generator.py:419-484; the caches are
        replicated on every rank)."""
        n = ki.shape[0]
        if not (kv.shape[0] == pe.shape[0] == n) or start_pos < 0 or start_pos + n > self.cache_len:
            raise ValueError("inject_cache: the three tensors must hold the same rows and fit the caches")
        dev = self.kv_cache.device
        self.ki_cache[0, start_pos: start_pos + n].copy_(ki.to(dev, BF16))
        self.kv_cache[0, start_pos: start_pos + n].copy_(kv.to(dev, BF16))
        self.pe_cache[0, start_pos: start_pos + n].copy_(pe.to(dev, BF16))

    def inject_cache_fp8(self, kv_raw: torch.Tensor, pe_raw: torch.Tensor, ki_pages: torch.Tensor, seq_len: int,
                         start_pos: int = 0) -> None:
        """The same from the FP8 wire format (uint8 planes [seq, 528], [seq, 128], [pages, 8448];
        pd_vllm/profiles/mla_nsa.py:16-41), dequantised on the device in one launch."""
        dev = self.kv_cache.device
        ops.inject_cache_fp8(kv_raw.to(dev).contiguous(), pe_raw.to(dev).contiguous(), ki_pages.to(dev).contiguous(),
                             seq_len, start_pos, self.kv_cache, self.pe_cache, self.ki_cache)

    def _attn_prep_and_select(self, x, freqs, cur_pos, n_keys: int, s: int, chained: bool) -> None:
        a, w = self.args, self.w
        v = lambda t: t[:, :s]  # noqa: E731
        ops.attn_prep(x, w.in_norm, None if chained else w.wis, v(self.idx_w), v(self.kv), w.kv_norm, self.kv_cache,
                      v(self.q_pe), self.pe_cache, v(self.iq), v(self.iq_rt), v(self.ki), self.ki_cache, w.k_norm_w,
                      w.k_norm_b, freqs, cur_pos, eps=a.eps, rope=a.qk_rope_head_dim)
        ops.sparse_index_topk(v(self.iq_rt), self.ki_cache, v(self.idx_w), self.idx_logits, v(self.sel), cur_pos,
                              n_keys=n_keys)
        if self.injected_sel is not None:
            v(self.sel).copy_(self.injected_sel)

    def forward(self, x: torch.Tensor, cur_pos: torch.Tensor, freqs: torch.Tensor, n_keys: int) -> torch.Tensor:
        """``x`` [1, S, dim] bf16, ``cur_pos`` int32[1] (position of token 0), ``freqs`` f32 [S, rope/2, 2],
        ``n_keys`` = number of cache rows the indexer scans (>= cur_pos + S).  Returns [1, S, dim] bf16."""
        a, w = self.args, self.w
        s = x.shape[1]
        v = lambda t: t[:, :s]  # noqa: E731
        dev, chained = x.device, self.chained
        # Launch 1: the three FP8 products of the query path and the small per-token work between them
        # (indexer head weights, latent norm into the cache, RoPE, indexer rotations) as one persistent
        # kernel; with ``chained = False`` the same operators run as separate launches.
        fork = self.fork and not chained
        long_rows = n_keys > FORK_MAX_KEYS
        with ops.chain(dev, chained):
            ops.rmsnorm_projx_wqkva(x, w.in_norm, w.w_qkva, cur_pos, v(self.q_a), v(self.kv), self.pe_cache, v(self.ki),
                                    eps=a.eps)
            if chained:  # the indexer head weights as one more product of the stream (it waits for nothing)
                ops.rmsnorm_proj_rows2(x, w.in_norm, w.wis2, v(self.idx_w), eps=a.eps)
            ops.rmsnorm_proj_q(v(self.q_a), w.q_norm, w.w_qb, v(self.q_nope), v(self.q_pe), v(self.iq), eps=a.eps)
            if fork:
                # The absorbed-q product needs only q_nope; the per-token vector work and the indexer's scoring +
                # selection need only the rest of the q_b launch's outputs.  Run them side by side: the product on
                # this stream with a capped grid, the two small launches (whose thread blocks never wait on one
                # another, so they cannot starve the product's) on a second stream over the SMs left free.
                main = torch.cuda.current_stream(dev)
                self._ev_fork.record(main)
                self._side.wait_event(self._ev_fork)
                with torch.cuda.stream(self._side):
                    ops.set_grid_limit(dev, self._long_select_ctas if long_rows else 0)
                    try:
                        self._attn_prep_and_select(x, freqs, cur_pos, n_keys, s, chained)
                    finally:
                        ops.set_grid_limit(dev, 0)
                    self._ev_join.record(self._side)
                ops.set_grid_limit(dev, self._long_product_ctas if long_rows else FORK_PRODUCT_CTAS)
                try:
                    ops.projq_wqb(v(self.q_nope), w.w_absorb, None, v(self.q_lat))
                finally:
                    ops.set_grid_limit(dev, 0)
                main.wait_event(self._ev_join)
            else:
                ops.attn_prep(x, w.in_norm, None if chained else w.wis, v(self.idx_w), v(self.kv), w.kv_norm,
                              self.kv_cache, v(self.q_pe), self.pe_cache, v(self.iq), v(self.iq_rt), v(self.ki),
                              self.ki_cache, w.k_norm_w, w.k_norm_b, freqs, cur_pos, eps=a.eps, rope=a.qk_rope_head_dim)
                ops.projq_wqb(v(self.q_nope), w.w_absorb, None, v(self.q_lat))
        if not fork:
            ops.sparse_index_topk(v(self.iq_rt), self.ki_cache, v(self.idx_w), self.idx_logits, v(self.sel), cur_pos,
                                  n_keys=n_keys)
            if self.injected_sel is not None:
                v(self.sel).copy_(self.injected_sel)
        # With single launches the merge of the attention chunks also does the value up-projection of its head
        fuse_v = self.fuse_vproj and not chained
        ops.flash_sparse_mla(v(self.q_lat), v(self.q_pe), self.kv_cache, self.pe_cache, v(self.sel), cur_pos,
                             v(self.o_lat), softmax_scale=self.scale, split_size=self.mla_split, out_acc=self.o_acc,
                             lse=self.lse, lse_acc=self.lse_acc, w_v=w.w_v if fuse_v else None,
                             o_out=v(self.o) if fuse_v else None)
        # Launch 2: value up-projection, o_proj (+ all-reduce + residual), router, experts (or the dense FFN)
        with ops.chain(dev, chained):
            if not fuse_v:
                ops.projo_wkvb(v(self.o_lat), w.w_v, None, v(self.o))
            ops.unproj_o_allreduce(v(self.o), w.w_o, None, x, 0, v(self.h), comm=self.comm)
            if w.dense:
                ops.rmsnorm_up_gate_silu(v(self.h), w.post_norm, w.w_gu, v(self.ffn_hidden), eps=a.eps)
                ops.down_allreduce(v(self.ffn_hidden), w.w_down, None, v(self.h), 0, v(self.out), comm=self.comm)
            else:
                if chained and w.router2 is not None:
                    # router logits on the weight stream, ahead of the shared expert that covers the routing
                    ops.rmsnorm_proj_rows2(v(self.h), w.post_norm, w.router2, v(self.scores), eps=a.eps)
                else:
                    ops.rmsnorm_expert_proj(v(self.h), w.post_norm, w.router, v(self.scores),
                                            None if chained else v(self.h_norm), eps=a.eps)
                scores = v(self.scores) if self.forced_scores is None else self.forced_scores
                # chained: the products normalise the raw state themselves instead of waiting for the router's copy
                ops.expert_select_up_gate_silu(v(self.h) if chained else v(self.h_norm), scores, w.router_bias, w.w_gu,
                                               v(self.ffn_hidden), v(self.probs), v(self.eidx), dim=a.dim,
                                               n_groups=a.n_expert_groups, n_limited_groups=a.n_limited_groups,
                                               route_scale=a.route_scale, slot_ids=self.slot_ids, slot_w=self.slot_w,
                                               gamma=w.post_norm if chained else None, eps=a.eps)
                ops.expert_down_allreduce(v(self.ffn_hidden), w.w_down, None, v(self.eidx), v(self.probs), v(self.h), 0,
                                          v(self.out), slot_ids=self.slot_ids, slot_w=self.slot_w, comm=self.comm)
        return v(self.out)
