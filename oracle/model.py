"""Layer / model composition of the oracle (test infrastructure only).

The reference has no Python forward for a layer or a model: its module classes are
weight and buffer registries whose forwards raise (tilert/models/base.py:355-371) and the
real forward lives in the closed native library.  The composition below follows the
operator registration order of tilert/models/deepseek_v3_2/modules/mla_v2.py:44-63,127-161,
modules/moe.py:27-46 and modules/mlp.py:24-35, with the residual placement given by the
``x_in`` arguments of ``unproj_o_allreduce`` (ops/unproj_o_allreduce.py:23-58) and
``expert_down_allreduce`` (ops/expert_down_allreduce.py:23-63).  The embedding lookup and
the greedy arg-max are not stated anywhere in the reference; standard forms are used.
Parity unpinned for the composition itself (each operator inside it is pinned).
"""

from __future__ import annotations

from dataclasses import dataclass, replace

import torch

from . import ops
from .quant import quantize_weight_block128, weight_dequant

BF16 = torch.bfloat16


@dataclass
class Args:
    """Same fields and defaults as tilert/models/deepseek_v3_2/model_args.py:51-95."""

    vocab_size: int = 129280
    dim: int = 7168
    inter_dim: int = 18432
    moe_inter_dim: int = 2048
    n_layers: int = 61
    n_dense_layers: int = 3
    n_heads: int = 128
    n_routed_experts: int = 256
    n_shared_experts: int = 1
    n_activated_experts: int = 8
    n_expert_groups: int = 8
    n_limited_groups: int = 4
    route_scale: float = 2.5
    q_lora_rank: int = 1536
    kv_lora_rank: int = 512
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    original_seq_len: int = 4096
    rope_theta: float = 10000.0
    rope_factor: float | None = 40
    beta_fast: int = 32
    beta_slow: int = 1
    index_n_heads: int = 64
    index_head_dim: int = 128
    index_topk: int = 2048
    max_seq_len: int = 160 * 1024
    eps: float = 1e-6


def toy_args() -> Args:
    """The toy workload: 2 layers (one dense, one MoE), hidden 1024, vocab 4096."""
    return Args(
        vocab_size=4096, dim=1024, inter_dim=2048, moe_inter_dim=512, n_layers=2,
        n_dense_layers=1, n_heads=16, n_routed_experts=32, n_activated_experts=4,
        n_expert_groups=1, n_limited_groups=1, q_lora_rank=384, index_n_heads=16,
        index_topk=256, max_seq_len=2048,
    )


def full_layer_args(max_seq_len: int = 160 * 1024) -> Args:
    """One full-shape DeepSeek-V3.2 MoE layer."""
    return replace(Args(), n_layers=1, n_dense_layers=0, max_seq_len=max_seq_len)


# --------------------------------------------------------------------- weights
def _fp8_linear(gen, n, k, std, out, key):
    w = torch.randn(n, k, generator=gen, dtype=torch.float32) * std
    q, s = quantize_weight_block128(w)
    out[f"{key}.weight"] = q
    out[f"{key}.weight_scale_inv"] = s


def random_state_dict(args: Args, seed: int = 0, std: float = 0.02,
                      expert_ids: list[int] | None = None, with_mtp: bool = False) -> dict[str, torch.Tensor]:
    """HF-keyed random checkpoint: N(0, std) -> e4m3 + 128x128 f32 scales, norm gains 1,
    router bias 0.  ``expert_ids`` limits which routed experts are materialised (the full
    layer has 256 of them; a one-step check touches 8).  ``with_mtp`` appends the multi-token
    prediction layer under ``model.layers.{n_layers}`` (an MoE layer plus ``enorm``, ``hnorm``,
    ``eh_proj`` and ``shared_head.norm``; embedding and head are the main model's), drawn after
    everything else so that the other tensors do not depend on the switch."""
    gen = torch.Generator().manual_seed(seed)
    sd: dict[str, torch.Tensor] = {}
    a = args
    sd["model.embed_tokens.weight"] = (torch.randn(a.vocab_size, a.dim, generator=gen, dtype=torch.float32) * std).to(BF16)

    def layer(li: int, dense: bool) -> None:
        p = f"model.layers.{li}"
        sd[f"{p}.input_layernorm.weight"] = torch.ones(a.dim, dtype=torch.float32)
        sd[f"{p}.post_attention_layernorm.weight"] = torch.ones(a.dim, dtype=torch.float32)
        at = f"{p}.self_attn"
        _fp8_linear(gen, a.q_lora_rank, a.dim, std, sd, f"{at}.q_a_proj")
        sd[f"{at}.q_a_layernorm.weight"] = torch.ones(a.q_lora_rank, dtype=torch.float32)
        _fp8_linear(gen, a.n_heads * (a.qk_nope_head_dim + a.qk_rope_head_dim), a.q_lora_rank, std, sd,
                    f"{at}.q_b_proj")
        _fp8_linear(gen, a.kv_lora_rank + a.qk_rope_head_dim, a.dim, std, sd, f"{at}.kv_a_proj_with_mqa")
        sd[f"{at}.kv_a_layernorm.weight"] = torch.ones(a.kv_lora_rank, dtype=torch.float32)
        _fp8_linear(gen, a.n_heads * (a.qk_nope_head_dim + a.v_head_dim), a.kv_lora_rank, std, sd,
                    f"{at}.kv_b_proj")
        _fp8_linear(gen, a.dim, a.n_heads * a.v_head_dim, std, sd, f"{at}.o_proj")
        _fp8_linear(gen, a.index_n_heads * a.index_head_dim, a.q_lora_rank, std, sd, f"{at}.indexer.wq_b")
        _fp8_linear(gen, a.index_head_dim, a.dim, std, sd, f"{at}.indexer.wk")
        sd[f"{at}.indexer.k_norm.weight"] = torch.ones(a.index_head_dim, dtype=torch.float32)
        sd[f"{at}.indexer.k_norm.bias"] = torch.zeros(a.index_head_dim, dtype=torch.float32)
        sd[f"{at}.indexer.weights_proj.weight"] = (
            torch.randn(a.index_n_heads, a.dim, generator=gen, dtype=torch.float32) * std).to(BF16)
        m = f"{p}.mlp"
        if dense:
            _fp8_linear(gen, a.inter_dim, a.dim, std, sd, f"{m}.gate_proj")
            _fp8_linear(gen, a.inter_dim, a.dim, std, sd, f"{m}.up_proj")
            _fp8_linear(gen, a.dim, a.inter_dim, std, sd, f"{m}.down_proj")
        else:
            sd[f"{m}.gate.weight"] = (torch.randn(a.n_routed_experts, a.dim, generator=gen, dtype=torch.float32) * std).to(BF16)
            sd[f"{m}.gate.e_score_correction_bias"] = torch.zeros(a.n_routed_experts, dtype=torch.float32)
            names = ["shared_experts"] + [
                f"experts.{e}" for e in (range(a.n_routed_experts) if expert_ids is None else expert_ids)]
            for nm in names:
                _fp8_linear(gen, a.moe_inter_dim, a.dim, std, sd, f"{m}.{nm}.gate_proj")
                _fp8_linear(gen, a.moe_inter_dim, a.dim, std, sd, f"{m}.{nm}.up_proj")
                _fp8_linear(gen, a.dim, a.moe_inter_dim, std, sd, f"{m}.{nm}.down_proj")

    for li in range(a.n_layers):
        layer(li, li < a.n_dense_layers)
    sd["model.norm.weight"] = torch.ones(a.dim, dtype=torch.float32)
    sd["lm_head.weight"] = (torch.randn(a.vocab_size, a.dim, generator=gen, dtype=torch.float32) * std).to(BF16)
    if with_mtp:
        p = f"model.layers.{a.n_layers}"
        layer(a.n_layers, False)
        sd[f"{p}.enorm.weight"] = torch.ones(a.dim, dtype=torch.float32)
        sd[f"{p}.hnorm.weight"] = torch.ones(a.dim, dtype=torch.float32)
        sd[f"{p}.eh_proj.weight"] = (torch.randn(a.dim, 2 * a.dim, generator=gen, dtype=torch.float32) * std).to(BF16)
        sd[f"{p}.shared_head.norm.weight"] = torch.ones(a.dim, dtype=torch.float32)
    return sd


class LayerWeights:
    """bf16-dequantised weights of one layer, held as the reference goldens hold them."""

    def __init__(self, args: Args, sd: dict[str, torch.Tensor], li: int):
        a = args
        p = f"model.layers.{li}"
        at = f"{p}.self_attn"

        def dq(key):
            return weight_dequant(sd[f"{key}.weight"], sd[f"{key}.weight_scale_inv"])

        self.in_norm = sd[f"{p}.input_layernorm.weight"]
        self.post_norm = sd[f"{p}.post_attention_layernorm.weight"]
        self.wq_a = dq(f"{at}.q_a_proj")
        kv_a = dq(f"{at}.kv_a_proj_with_mqa")
        self.wkv_a, self.w_pe = kv_a[: a.kv_lora_rank], kv_a[a.kv_lora_rank:]
        self.q_norm = sd[f"{at}.q_a_layernorm.weight"]
        self.kv_norm = sd[f"{at}.kv_a_layernorm.weight"]
        self.wq_b = dq(f"{at}.q_b_proj")
        wkv_b = dq(f"{at}.kv_b_proj").view(a.n_heads, a.qk_nope_head_dim + a.v_head_dim, a.kv_lora_rank)
        self.wkv_b_nope = wkv_b[:, : a.qk_nope_head_dim].contiguous()
        self.wkv_b_v = wkv_b[:, a.qk_nope_head_dim:].contiguous()
        self.w_o = dq(f"{at}.o_proj")
        self.wqi = dq(f"{at}.indexer.wq_b")
        self.wki = dq(f"{at}.indexer.wk")
        self.k_norm_w = sd[f"{at}.indexer.k_norm.weight"]
        self.k_norm_b = sd[f"{at}.indexer.k_norm.bias"]
        self.wis = sd[f"{at}.indexer.weights_proj.weight"]
        m = f"{p}.mlp"
        self.dense = li < a.n_dense_layers
        self._sd, self._m = sd, m
        self._cache: dict[str, tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}
        if self.dense:
            self.w_gate, self.w_up, self.w_down = dq(f"{m}.gate_proj"), dq(f"{m}.up_proj"), dq(f"{m}.down_proj")
        else:
            self.router = sd[f"{m}.gate.weight"]
            self.router_bias = sd[f"{m}.gate.e_score_correction_bias"]

    def expert(self, name: str):
        """(gate, up, down) bf16 of one expert, dequantised on first use."""
        if name not in self._cache:
            k = f"{self._m}.{name}"
            sd = self._sd
            self._cache[name] = tuple(
                weight_dequant(sd[f"{k}.{w}.weight"], sd[f"{k}.{w}.weight_scale_inv"])
                for w in ("gate_proj", "up_proj", "down_proj"))
        return self._cache[name]


class Caches:
    """Per-layer latent caches [1, T, {512, 64, 128}] bf16 (modules/mla_v2.py:93-113)."""

    def __init__(self, args: Args, t: int):
        self.kv = torch.zeros(1, t, args.kv_lora_rank, dtype=BF16)
        self.pe = torch.zeros(1, t, args.qk_rope_head_dim, dtype=BF16)
        self.ki = torch.zeros(1, t, args.index_head_dim, dtype=BF16)


def layer_step(args: Args, w: LayerWeights, c: Caches, x: torch.Tensor, pos: int,
               freqs_cis: torch.Tensor, trace: dict | None = None,
               forced_router_scores: torch.Tensor | None = None) -> torch.Tensor:
    """One decode step of one layer.  ``x`` is [1, S, dim] bf16; the S tokens sit at
    positions ``pos .. pos+S-1``.  Returns the layer output [1, S, dim] bf16 and updates
    the caches in place.  ``trace`` (optional) collects every intermediate."""
    a = args
    s = x.size(1)
    fc = freqs_cis[pos: pos + s]
    tr = trace if trace is not None else {}

    q_a, kv, k_pe = ops.projx_wqkva(x, w.in_norm, w.wq_a, w.wkv_a, w.w_pe, a.eps)
    _, ki, idx_w = ops.projx_wqakis(x, w.in_norm, w.wq_a, w.wki, w.wis, a.eps)
    c.kv[:, pos: pos + s] = ops.rmsnorm_kv(kv, w.kv_norm, a.eps)
    q_nope, q_pe = ops.rmsnorm_projq_wqb(q_a, w.q_norm, w.wq_b, a.n_heads, a.qk_nope_head_dim,
                                         a.qk_rope_head_dim, a.eps)
    q_pe, k_rot = ops.qkv_rope(q_pe, k_pe, fc)
    c.pe[:, pos: pos + s] = k_rot
    iq = ops.rmsnorm_projq_wqi(q_a, w.q_norm, w.wqi, a.index_head_dim, a.eps)
    iq = ops.rotate(iq, fc, a.qk_rope_head_dim)
    c.ki[:, pos: pos + s] = ops.layernorm_rope_rotate(ki, w.k_norm_w, w.k_norm_b, fc, a.qk_rope_head_dim)
    n_valid = pos + s
    idx_logits = ops.indexer_logits(iq, c.ki[:, :n_valid], idx_w, n_valid)
    sel = ops.topk_indices(idx_logits, a.index_topk)
    q_lat = ops.projq_wqb_absorb(q_nope, w.wkv_b_nope)
    o_lat = ops.flash_sparse_mla(q_lat, q_pe, c.kv[:, :n_valid], c.pe[:, :n_valid], sel, pos,
                                 ops.softmax_scale(a))
    o = ops.projo_wkvb(o_lat, w.wkv_b_v)
    h = (ops.unproj_o(o, w.w_o).float() + x.float()).to(BF16)
    tr.update(q_a=q_a, kv=kv, k_pe=k_pe, ki=ki, idx_w=idx_w, q_nope=q_nope, q_pe=q_pe, iq=iq,
              idx_logits=idx_logits, sel=sel, q_lat=q_lat, o_lat=o_lat, o=o, attn_out=h)

    if w.dense:
        hid = ops.dense_up_gate_silu(h, w.post_norm, w.w_gate, w.w_up, a.eps, max(a.inter_dim // a.moe_inter_dim, 1))
        ffn = ops.dense_down(hid, w.w_down, a.inter_dim // a.moe_inter_dim)
        tr.update(ffn_hidden=hid)
    else:
        hn, scores = ops.rmsnorm_expert_proj(h, w.post_norm, w.router, a.eps)
        scores = scores.view(1, s, -1)
        if forced_router_scores is not None:
            scores = forced_router_scores
        probs, eidx = ops.expert_select_ds(scores, w.router_bias, a.n_expert_groups, a.n_limited_groups,
                                           a.n_activated_experts, a.route_scale)
        gl, ul, dl = [], [], []
        for si in range(s):
            names = ["shared_experts"] + [f"experts.{int(e)}" for e in eidx[0, si]]
            trip = [w.expert(nm) for nm in names]
            gl.append([t[0] for t in trip])
            ul.append([t[1] for t in trip])
            dl.append([t[2] for t in trip])
        hid = ops.expert_up_gate_silu(hn, gl, ul)
        ffn = ops.expert_down(hid, dl, probs)
        tr.update(router_scores=scores, probs=probs, eidx=eidx, ffn_hidden=hid, x_mlp_in=hn)
    out = (ffn.float() + h.float()).to(BF16)
    tr.update(ffn_out=ffn, out=out)
    return out


class Model:
    """Whole-model greedy decoder over ``layer_step`` (embedding -> layers -> head)."""

    def __init__(self, args: Args, sd: dict[str, torch.Tensor], cache_len: int | None = None):
        self.args = args
        self.embed = sd["model.embed_tokens.weight"]
        self.layers = [LayerWeights(args, sd, li) for li in range(args.n_layers)]
        self.final_norm = sd["model.norm.weight"]
        self.head = sd["lm_head.weight"]
        self.freqs_cis = ops.precompute_freqs_cis(args)
        t = cache_len or args.max_seq_len
        self.caches = [Caches(args, t) for _ in range(args.n_layers)]
        self.pos = 0

    def step(self, token: int, traces: list | None = None) -> tuple[int, torch.Tensor]:
        """Feed one token at the current position; returns (arg-max token, f32 logits)."""
        x = self.embed[token].view(1, 1, -1)
        for li, (w, c) in enumerate(zip(self.layers, self.caches)):
            tr = {} if traces is not None else None
            x = layer_step(self.args, w, c, x, self.pos, self.freqs_cis, tr)
            if traces is not None:
                traces.append(tr)
        logits = ops.rmsnorm_head_proj(x, self.final_norm, self.head, self.args.eps).view(-1)
        self.pos += 1
        return int(torch.argmax(logits)), logits

    def generate(self, prompt: list[int], n_new: int) -> tuple[list[int], list[torch.Tensor]]:
        """Token-by-token prefill (the reference feeds prompts one token at a time,
        generator.py:220-245) then ``n_new`` greedy steps.  Returns tokens and the logits
        of every generated position."""
        nxt = 0
        for tok in prompt:
            nxt, lg = self.step(tok)
        toks, lgs = [nxt], [lg]
        for _ in range(n_new - 1):
            nxt, lg = self.step(nxt)
            toks.append(nxt)
            lgs.append(lg)
        return toks, lgs


class MtpModel(Model):
    """Greedy speculative decoding with the multi-token-prediction layer drafting three tokens.

    The reference runs this inside its native library (``dsa_mtp_e2e_show_hands``); Python only
    sees the interface: a step takes four draft tokens at the current position and leaves
    ``PREDICTED_TOKENS``, ``ACCEPTED_TOKENS`` (1..4 of them) and ``NEXT_DRAFT_TOKENS``
    (tilert/models/deepseek_v3_2/modules/end2end.py:598-651), and the host loop advances the position
    by the accepted count (generator.py:336-375).  The rule inside is not stated anywhere in the
    reference, so the standard one is used and **parity is unpinned** for it:

    * ``draft[0]`` is the last known token, ``draft[1:4]`` are guesses.  The main model runs the four
      tokens at positions ``p .. p+3`` in one pass; ``predicted[j]`` is the arg-max after row ``j``.
    * accepted count ``n`` = 1 + the number of leading guesses with ``draft[j+1] == predicted[j]``;
      ``predicted[:n]`` are emitted.
    * The prediction layer pairs the hidden state of position ``q`` (the last block's output, before
      the final norm) with the embedding of the token at ``q+1``: ``eh_proj([enorm(e), hnorm(h)])``
      -> one MoE decoder layer with its own caches -> ``shared_head.norm`` -> the main head
      (modules/mtp_preprocess.py:197-229, modules/mtp.py:28-50).  One four-row pass at ``p .. p+3``
      with the tokens ``predicted[0:4]`` yields guess 1 from row ``n-1``; two single-row passes at
      ``p+n`` and ``p+n+1`` chain the layer's own hidden state and the previous guess into guesses 2, 3.
    * ``next_draft = [predicted[n-1], guess 1, guess 2, guess 3]``.  Rows written past ``p+n-1`` by
      either model hold rejected tokens; the next step starts at ``p+n`` and rewrites them first.
    """

    N_TOKENS = 4

    def __init__(self, args: Args, sd: dict[str, torch.Tensor], cache_len: int | None = None):
        super().__init__(args, sd, cache_len)
        p = f"model.layers.{args.n_layers}"
        self.mtp_w = LayerWeights(args, sd, args.n_layers)
        self.mtp_cache = Caches(args, cache_len or args.max_seq_len)
        self.enorm, self.hnorm = sd[f"{p}.enorm.weight"], sd[f"{p}.hnorm.weight"]
        self.w_eh = sd[f"{p}.eh_proj.weight"]
        self.mtp_norm = sd[f"{p}.shared_head.norm.weight"]

    def main_pass(self, tokens: list[int], pos: int) -> tuple[torch.Tensor, torch.Tensor]:
        """The main model over ``tokens`` at ``pos ..``: (hidden [1, S, dim] bf16, logits [S, vocab] f32)."""
        x = self.embed[torch.tensor(tokens)].view(1, len(tokens), -1)
        for w, c in zip(self.layers, self.caches):
            x = layer_step(self.args, w, c, x, pos, self.freqs_cis)
        return x, ops.rmsnorm_head_proj(x, self.final_norm, self.head, self.args.eps).view(len(tokens), -1)

    def mtp_pass(self, next_tokens: list[int], h: torch.Tensor, pos: int) -> tuple[torch.Tensor, torch.Tensor]:
        """The prediction layer over rows at ``pos ..``: row j pairs ``h[:, j]`` with the embedding of
        ``next_tokens[j]``.  Returns (its hidden [1, S, dim] bf16, logits [S, vocab] f32)."""
        e = self.embed[torch.tensor(next_tokens)].view(1, len(next_tokens), -1)
        _, _, x = ops.mtp_preprocess(e, h, self.enorm, self.hnorm, self.w_eh, self.args.eps)
        x = layer_step(self.args, self.mtp_w, self.mtp_cache, x, pos, self.freqs_cis)
        return x, ops.rmsnorm_head_proj(x, self.mtp_norm, self.head, self.args.eps).view(len(next_tokens), -1)

    def prefill_chunk(self, tokens: list[int], extra_token: int) -> None:
        """Four prompt tokens at the current position through both models; ``extra_token`` is the prompt
        token that follows the chunk (generator.py:297-328).  Does not move the position."""
        h, _ = self.main_pass(tokens, self.pos)
        self.mtp_pass(tokens[1:] + [extra_token], h, self.pos)

    def verify_step(self, draft: list[int]) -> dict:
        """One speculative step at the current position; advances it by the accepted count."""
        n_tok, p = self.N_TOKENS, self.pos
        assert len(draft) == n_tok
        h, logits = self.main_pass(draft, p)
        predicted = [int(t) for t in torch.argmax(logits, dim=-1)]
        n = 1
        while n < n_tok and draft[n] == predicted[n - 1]:
            n += 1
        mh, mlog = self.mtp_pass(predicted, h, p)
        guesses, glogits = [int(torch.argmax(mlog[n - 1]))], [mlog[n - 1]]
        hh = mh[:, n - 1: n]
        for i in range(1, n_tok - 1):
            hh, gl = self.mtp_pass([guesses[-1]], hh, p + n - 1 + i)
            guesses.append(int(torch.argmax(gl[0])))
            glogits.append(gl[0])
        self.pos = p + n
        return {"predicted": predicted, "n_accepted": n, "next_draft": [predicted[n - 1]] + guesses,
                "logits": logits, "guess_logits": torch.stack(glogits)}

    def generate_mtp(self, prompt: list[int], n_new: int) -> tuple[list[int], list[int]]:
        """Chunked prefill, then speculative steps until ``n_new`` tokens are out
        (generator.py:267-417).  Returns (tokens, accepted count of every step)."""
        n_tok, plen = self.N_TOKENS, len(prompt)
        self.pos = 0
        while self.pos < plen - 1:
            end = min(self.pos + n_tok, plen)
            chunk = prompt[self.pos: end]
            valid = len(chunk)
            chunk = chunk + [chunk[-1]] * (n_tok - valid)
            extra = prompt[self.pos + n_tok] if self.pos + n_tok < plen else prompt[end - 1]
            self.prefill_chunk(chunk, extra)
            self.pos += valid
        self.pos = plen - 1
        draft = [prompt[-1]] * n_tok
        out: list[int] = []
        counts: list[int] = []
        while len(out) < n_new:
            r = self.verify_step(draft)
            out += r["predicted"][: r["n_accepted"]]
            counts.append(r["n_accepted"])
            draft = r["next_draft"]
        return out[:n_new], counts
