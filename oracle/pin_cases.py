"""Seeded cases shared by the reference pin script and the fixture test (test
infrastructure only): the inputs, and the oracle's own result for every pinned case."""

from __future__ import annotations

import torch

from . import model as om
from . import ops as oo

BF16 = torch.bfloat16
POS = 37


def pin_inputs(seed: int = 1234) -> dict[str, torch.Tensor]:
    """Seeded toy-shape activations shared by this script and the fixture test."""
    a = om.toy_args()
    g = torch.Generator().manual_seed(seed)

    def rn(*shape, scale=1.0):
        return (torch.randn(*shape, generator=g, dtype=torch.float32) * scale).to(BF16)

    t = 320
    return {
        "x": rn(1, 1, a.dim),
        "x2": rn(1, 2, a.dim),
        "q_a": rn(1, 1, a.q_lora_rank),
        "kv": rn(1, 1, a.kv_lora_rank),
        "q_pe": rn(1, 1, a.n_heads, a.qk_rope_head_dim),
        "k_pe": rn(1, 1, a.qk_rope_head_dim),
        "iq": rn(1, 1, a.index_n_heads, a.index_head_dim),
        "ki": rn(1, 1, a.index_head_dim),
        "q_nope": rn(1, 1, a.n_heads, a.qk_nope_head_dim),
        "q_lat": rn(1, 1, a.n_heads, a.kv_lora_rank, scale=0.3),
        "kv_cache": rn(1, t, a.kv_lora_rank),
        "pe_cache": rn(1, t, a.qk_rope_head_dim),
        "o_lat": rn(1, 1, a.n_heads, a.kv_lora_rank),
        "o": rn(1, 1, a.n_heads, a.v_head_dim),
        "topk_logits": torch.randn(1, 1, t, generator=g, dtype=torch.float32),
        "sel": torch.sort(torch.randperm(t, generator=g)[:64])[0].view(1, 1, 64),
        "hidden": rn(1, 1, a.dim),
        "ffn_hidden": rn(1, 1, 1 + a.n_activated_experts, a.moe_inter_dim, scale=0.1),
        "dense_hidden": rn(1, 1, a.inter_dim, scale=0.1),
        "e_norm": rn(1, 2, a.dim),
        "h_norm": rn(1, 2, a.dim),
        "w_eh": rn(a.dim, 2 * a.dim, scale=0.03),
    }



def oracle_results(inp: dict[str, torch.Tensor] | None = None) -> dict[str, list[torch.Tensor]]:
    """The oracle's output for each case name used in ``tests/golden/ref_goldens.pt``."""
    a = om.toy_args()
    inp = inp or pin_inputs()
    sd = om.random_state_dict(a, seed=0)
    w0, w1 = om.LayerWeights(a, sd, 0), om.LayerWeights(a, sd, 1)
    fc = oo.precompute_freqs_cis(a)
    f1 = fc[POS: POS + 1]
    r: dict[str, list[torch.Tensor]] = {}
    r["freqs"] = [torch.view_as_real(fc[:128]).float()]
    r["wqkva"] = list(oo.projx_wqkva(inp["x"], w0.in_norm, w0.wq_a, w0.wkv_a, w0.w_pe, a.eps))
    r["wqakis"] = list(oo.projx_wqakis(inp["x"], w0.in_norm, w0.wq_a, w0.wki, w0.wis, a.eps))
    r["wqb"] = list(oo.rmsnorm_projq_wqb(inp["q_a"], w0.q_norm, w0.wq_b, a.n_heads, a.qk_nope_head_dim,
                                          a.qk_rope_head_dim, a.eps))
    r["wqi"] = [oo.rmsnorm_projq_wqi(inp["q_a"], w0.q_norm, w0.wqi, a.index_head_dim, a.eps)]
    r["kvnorm"] = [oo.rmsnorm_kv(inp["kv"], w0.kv_norm, a.eps)]
    r["rope"] = list(oo.qkv_rope(inp["q_pe"], inp["k_pe"], f1))
    r["rotate"] = [oo.rotate(inp["iq"], f1, a.qk_rope_head_dim)]
    r["lnrr"] = [oo.layernorm_rope_rotate(inp["ki"], w0.k_norm_w, w0.k_norm_b, f1, a.qk_rope_head_dim)]
    r["topk"] = [oo.topk_indices(inp["topk_logits"], 64)]
    r["absorb"] = [oo.projq_wqb_absorb(inp["q_nope"], w0.wkv_b_nope)]
    r["mla"] = [oo.flash_sparse_mla(inp["q_lat"], inp["q_pe"], inp["kv_cache"], inp["pe_cache"], inp["sel"],
                                    319, oo.softmax_scale(a))]
    r["vproj"] = [oo.projo_wkvb(inp["o_lat"], w0.wkv_b_v)]
    r["oproj"] = [oo.unproj_o(inp["o"], w0.w_o)]
    xn, scores = oo.rmsnorm_expert_proj(inp["hidden"], w1.post_norm, w1.router, a.eps)
    r["router"] = [xn, scores]
    scores = scores.view(1, 1, -1)
    probs, eidx = oo.expert_select_ds(scores, w1.router_bias, 1, 1, a.n_activated_experts, a.route_scale)
    names = ["shared_experts"] + [f"experts.{int(e)}" for e in eidx[0, 0]]
    trip = [w1.expert(n) for n in names]
    r["experts"] = [oo.expert_up_gate_silu(xn, [[t[0] for t in trip]], [[t[1] for t in trip]]),
                    probs.float(), eidx.to(torch.int32)]
    eidx2 = torch.tensor([[[3, 17, 8, 29]]])
    probs2 = torch.tensor([[[0.9, 0.7, 0.5, 0.4]]], dtype=torch.float32)
    names2 = ["shared_experts"] + [f"experts.{int(e)}" for e in eidx2[0, 0]]
    r["expert_down"] = [oo.expert_down(inp["ffn_hidden"], [[w1.expert(n)[2] for n in names2]], probs2)]
    r["dense_upgate"] = [oo.dense_up_gate_silu(inp["x2"], w0.post_norm, w0.w_gate, w0.w_up, a.eps, a.inter_dim // a.moe_inter_dim)]
    r["dense_down"] = [oo.dense_down(inp["dense_hidden"], w0.w_down, a.inter_dim // a.moe_inter_dim)]
    r["head"] = [oo.rmsnorm_head_proj(inp["hidden"], sd["model.norm.weight"], sd["lm_head.weight"], a.eps)]
    r["eh_proj"] = [oo.eh_proj(inp["e_norm"], inp["h_norm"], inp["w_eh"])]
    return r


def route_groups_result(scores: torch.Tensor, bias: torch.Tensor) -> list[torch.Tensor]:
    """Full-shape grouped routing (256 experts, 8 groups, keep 4, top-8, scale 2.5)."""
    w, i = oo.expert_select_ds(scores, bias, 8, 4, 8, 2.5)
    return [w.float(), i.to(torch.int32)]
