"""Seeded random-init checkpoints in the HF DeepSeek FP8 format (e4m3 ``weight`` + f32
``weight_scale_inv`` per 128x128 block), generated on any device.  Used where the reference would
load real weights (its ``--use-random-weights`` path, tilert/generate.py:106-110, does the same in
spirit): benchmarks and smoke runs have no checkpoint to read."""

from __future__ import annotations

import torch

from .models.deepseek_v3_2.model_args import ModelArgs

BF16 = torch.bfloat16


def quantize_block128(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """f32 [N, K] -> (e4m3 [N, K], f32 scales [ceil(N/128), ceil(K/128)]) with scale = amax / 448."""
    n, k = w.shape
    np_, kp = (n + 127) // 128 * 128, (k + 127) // 128 * 128
    wp = torch.zeros(np_, kp, dtype=torch.float32, device=w.device)
    wp[:n, :k] = w
    blk = wp.view(np_ // 128, 128, kp // 128, 128)
    scale = blk.abs().amax(dim=(1, 3)).clamp_min(1e-12) / 448.0
    q = (blk / scale[:, None, :, None]).clamp(-448, 448).view(np_, kp)[:n, :k].contiguous()
    return q.to(torch.float8_e4m3fn), scale.contiguous()


def random_layer_state_dict(args: ModelArgs, li: int, device, seed: int = 0, std: float = 0.02,
                            expert_ids=None) -> dict[str, torch.Tensor]:
    """One layer's tensors under their HF keys (``model.layers.{li}. ...``)."""
    a = args
    gen = torch.Generator(device=device).manual_seed(seed * 1000 + li)
    sd: dict[str, torch.Tensor] = {}

    def rnd(*shape):
        return torch.randn(*shape, generator=gen, dtype=torch.float32, device=device) * std

    def fp8(key, n, k):
        sd[f"{key}.weight"], sd[f"{key}.weight_scale_inv"] = quantize_block128(rnd(n, k))

    p = f"model.layers.{li}"
    at = f"{p}.self_attn"
    ones = lambda n: torch.ones(n, dtype=torch.float32, device=device)  # noqa: E731
    sd[f"{p}.input_layernorm.weight"] = ones(a.dim)
    sd[f"{p}.post_attention_layernorm.weight"] = ones(a.dim)
    fp8(f"{at}.q_a_proj", a.q_lora_rank, a.dim)
    sd[f"{at}.q_a_layernorm.weight"] = ones(a.q_lora_rank)
    fp8(f"{at}.q_b_proj", a.n_heads * (a.qk_nope_head_dim + a.qk_rope_head_dim), a.q_lora_rank)
    fp8(f"{at}.kv_a_proj_with_mqa", a.kv_lora_rank + a.qk_rope_head_dim, a.dim)
    sd[f"{at}.kv_a_layernorm.weight"] = ones(a.kv_lora_rank)
    fp8(f"{at}.kv_b_proj", a.n_heads * (a.qk_nope_head_dim + a.v_head_dim), a.kv_lora_rank)
    fp8(f"{at}.o_proj", a.dim, a.n_heads * a.v_head_dim)
    fp8(f"{at}.indexer.wq_b", a.index_n_heads * a.index_head_dim, a.q_lora_rank)
    fp8(f"{at}.indexer.wk", a.index_head_dim, a.dim)
    sd[f"{at}.indexer.k_norm.weight"] = ones(a.index_head_dim)
    sd[f"{at}.indexer.k_norm.bias"] = torch.zeros(a.index_head_dim, dtype=torch.float32, device=device)
    sd[f"{at}.indexer.weights_proj.weight"] = rnd(a.index_n_heads, a.dim).to(BF16)
    m = f"{p}.mlp"
    if li < a.n_dense_layers:
        fp8(f"{m}.gate_proj", a.inter_dim, a.dim)
        fp8(f"{m}.up_proj", a.inter_dim, a.dim)
        fp8(f"{m}.down_proj", a.dim, a.inter_dim)
    else:
        sd[f"{m}.gate.weight"] = rnd(a.n_routed_experts, a.dim).to(BF16)
        sd[f"{m}.gate.e_score_correction_bias"] = torch.zeros(a.n_routed_experts, dtype=torch.float32, device=device)
        ids = range(a.n_routed_experts) if expert_ids is None else expert_ids
        for nm in ["shared_experts"] + [f"experts.{e}" for e in ids]:
            fp8(f"{m}.{nm}.gate_proj", a.moe_inter_dim, a.dim)
            fp8(f"{m}.{nm}.up_proj", a.moe_inter_dim, a.dim)
            fp8(f"{m}.{nm}.down_proj", a.dim, a.moe_inter_dim)
    return sd


def random_model_state_dict(args: ModelArgs, device, seed: int = 0, std: float = 0.02, with_mtp: bool = False,
                            expert_ids=None) -> dict[str, torch.Tensor]:
    """A whole random-init model under HF keys: embedding, every decoder layer, final norm and head; with
    ``with_mtp`` also the multi-token-prediction layer under ``model.layers.{n_layers}`` (an MoE decoder layer
    plus ``enorm`` / ``hnorm`` / ``eh_proj`` / ``shared_head.norm``, the checkpoint layout the reference's
    converter reads, tilert/models/preprocess/weight_converter.py:243-537)."""
    a = args
    gen = torch.Generator(device=device).manual_seed(seed * 1000 + 999)
    sd: dict[str, torch.Tensor] = {}
    sd["model.embed_tokens.weight"] = (torch.randn(a.vocab_size, a.dim, generator=gen, dtype=torch.float32,
                                                   device=device) * std).to(BF16)
    for li in range(a.n_layers):
        sd.update(random_layer_state_dict(a, li, device, seed=seed, std=std, expert_ids=expert_ids))
    sd["model.norm.weight"] = torch.ones(a.dim, dtype=torch.float32, device=device)
    sd["lm_head.weight"] = (torch.randn(a.vocab_size, a.dim, generator=gen, dtype=torch.float32, device=device) * std).to(BF16)
    if with_mtp:
        li = a.n_layers
        from dataclasses import replace

        sd.update(random_layer_state_dict(replace(a, n_dense_layers=0), li, device, seed=seed, std=std, expert_ids=expert_ids))
        p = f"model.layers.{li}"
        sd[f"{p}.enorm.weight"] = torch.ones(a.dim, dtype=torch.float32, device=device)
        sd[f"{p}.hnorm.weight"] = torch.ones(a.dim, dtype=torch.float32, device=device)
        sd[f"{p}.eh_proj.weight"] = (torch.randn(a.dim, 2 * a.dim, generator=gen, dtype=torch.float32, device=device) * std).to(BF16)
        sd[f"{p}.shared_head.norm.weight"] = torch.ones(a.dim, dtype=torch.float32, device=device)
    return sd


def random_packed_layer(args: ModelArgs, li: int, device, world: int = 1, rank: int = 0, seed: int = 0):
    """One rank's ``LayerWeights`` of layer ``li`` drawn directly in the packed block format (random e4m3 bytes,
    one constant scale): what a 61-layer random-init model is built from when its HF-format tensors (84 GB per
    rank at eight ranks, 670 GB in all) are not worth materialising first.  Timing-equivalent to converted
    weights -- same tensors, same shapes, same bytes streamed -- but not derived from an HF-keyed state dict,
    so there is no CPU restatement to compare values with."""
    from . import pack
    from .models.deepseek_v3_2.layer import LayerWeights

    a, dev = args, torch.device(device)
    gen = torch.Generator(device=dev).manual_seed(seed * 100003 + li * 131 + rank + 1)  # this rank's shards
    gen_all = torch.Generator(device=dev).manual_seed(seed * 100003 + li * 131)         # tensors every rank replicates
    hl = a.n_heads // world

    def blocks(*lead, shared=False):
        g_ = gen_all if shared else gen
        t = torch.randint(0, 127, (*lead, pack.WBLK_BYTES), generator=g_, dtype=torch.uint8, device=dev)
        t[..., :16384] |= torch.randint(0, 2, (*lead, 16384), generator=g_, dtype=torch.uint8, device=dev) << 7
        t[..., 16384:] = 0
        t[..., 16384:].view(torch.float32).fill_(2.2e-4)  # random e4m3 codes have an rms near 90: weights of rms ~0.02
        return t

    ones = lambda n: torch.ones(n, dtype=torch.float32, device=dev)  # noqa: E731
    lw = LayerWeights.__new__(LayerWeights)
    lw.in_norm, lw.post_norm, lw.q_norm, lw.kv_norm = ones(a.dim), ones(a.dim), ones(a.q_lora_rank), ones(a.kv_lora_rank)
    lw.k_norm_w, lw.k_norm_b = ones(a.index_head_dim), torch.zeros(a.index_head_dim, dtype=torch.float32, device=dev)
    lw.wis = (torch.randn(a.index_n_heads, a.dim, generator=gen_all, device=dev) * 0.02).to(BF16)
    lw.wis2 = pack.pack_bf16_two_term(lw.wis)
    n_kb = a.dim // 128
    qkva_rows = a.q_lora_rank + a.kv_lora_rank + a.qk_rope_head_dim + a.index_head_dim
    lw.w_qkva = blocks((qkva_rows + 127) // 128, n_kb, shared=True)
    own_rows, idx_rows = hl * (a.qk_nope_head_dim + a.qk_rope_head_dim), a.index_n_heads * a.index_head_dim
    assert own_rows % 128 == 0 and idx_rows % 128 == 0
    lw.w_qb = torch.cat([blocks(own_rows // 128, a.q_lora_rank // 128),
                         blocks(idx_rows // 128, a.q_lora_rank // 128, shared=True)], dim=0)
    lw.w_absorb = blocks(hl * a.kv_lora_rank // 128, a.qk_nope_head_dim // 128)
    lw.w_v = blocks(hl * a.v_head_dim // 128, a.kv_lora_rank // 128)
    lw.w_o = blocks(a.dim // 128, hl * a.v_head_dim // 128)
    lw.dense = li < a.n_dense_layers
    if lw.dense:
        il = a.inter_dim // world
        lw.w_gu, lw.w_down = blocks(2 * il // 128, n_kb), blocks(a.dim // 128, il // 128)
    else:
        il = a.moe_inter_dim // world
        lw.router = (torch.randn(a.n_routed_experts, a.dim, generator=gen_all, device=dev) * 0.02).to(BF16)
        lw.router2 = pack.pack_bf16_two_term(lw.router)
        lw.router_bias = torch.zeros(a.n_routed_experts, dtype=torch.float32, device=dev)
        lw.w_gu = blocks(a.n_routed_experts + 1, 2 * il // 128, n_kb)
        lw.w_down = blocks(a.n_routed_experts + 1, a.dim // 128, il // 128)
    lw.inter_local = il
    return lw


def random_packed_model(args: ModelArgs, device, world: int = 1, rank: int = 0, seed: int = 0, with_mtp: bool = False) -> dict:
    """The ``packed`` dictionary ``DsaModel`` / ``MtpDsaModel`` take (as ``convert.load_model`` returns it), drawn
    at random on the device for one rank: every layer by ``random_packed_layer``, the embedding, the final norm
    and the rank's slice of the vocabulary head; with ``with_mtp`` also the prediction layer (one more MoE layer,
    its two input norms, ``eh_proj`` and the shared head's norm)."""
    a, dev = args, torch.device(device)
    gen = torch.Generator(device=dev).manual_seed(seed * 7919 + 17)  # same embedding on every rank
    v_l = a.vocab_size // world
    embed = (torch.randn(a.vocab_size, a.dim, generator=gen, device=dev) * 0.02).to(BF16)
    gen_r = torch.Generator(device=dev).manual_seed(seed * 7919 + 101 + rank)
    head = (torch.randn(v_l, a.dim, generator=gen_r, device=dev) * 0.02).to(BF16)
    ones = torch.ones(a.dim, dtype=torch.float32, device=dev)
    mtp = None
    if with_mtp:
        mtp = {"layer": random_packed_layer(a, a.n_layers, dev, world, rank, seed), "enorm": ones.clone(), "hnorm": ones.clone(),
               "w_eh": (torch.randn(a.dim, 2 * a.dim, generator=gen, device=dev) * 0.01).to(BF16), "norm": ones.clone()}
    return {"layers": [random_packed_layer(a, li, dev, world, rank, seed) for li in range(a.n_layers)], "world": world,
            "embed": embed, "final_norm": ones, "head": head, "mtp": mtp}
