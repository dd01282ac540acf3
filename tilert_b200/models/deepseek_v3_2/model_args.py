"""Hyper-parameters of a DeepSeek-V3.2-style model; field names and defaults follow
tilert/models/deepseek_v3_2/model_args.py:51-95 so configurations carry over unchanged."""

from __future__ import annotations

from dataclasses import dataclass, replace


@dataclass
class ModelArgs:
    arch_name: str = "deepseek_v3_2"
    max_batch_size: int = 1
    max_seq_len: int = 160 * 1024
    dtype: str = "fp8"
    scale_fmt: str | None = None
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
    score_func: str = "sigmoid"
    route_scale: float = 2.5
    q_lora_rank: int = 1536
    kv_lora_rank: int = 512
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    original_seq_len: int | None = 4096
    rope_theta: float = 10000.0
    rope_factor: float | None = 40
    beta_fast: int | None = 32
    beta_slow: int | None = 1
    mscale: float = 1.0
    index_n_heads: int = 64
    index_head_dim: int = 128
    index_topk: int = 2048
    kv_cache_pad: int = 8
    block_size: int = 128
    eps: float = 1e-6


def toy_model_args() -> ModelArgs:
    """The CPU-runnable toy workload: 2 layers (dense + MoE), hidden 1024, vocab 4096."""
    return ModelArgs(
        vocab_size=4096, dim=1024, inter_dim=2048, moe_inter_dim=512, n_layers=2, n_dense_layers=1,
        n_heads=16, n_routed_experts=32, n_activated_experts=4, n_expert_groups=1, n_limited_groups=1,
        q_lora_rank=384, index_n_heads=16, index_topk=256, max_seq_len=2048)


def full_layer_args(max_seq_len: int = 160 * 1024) -> ModelArgs:
    """One full-shape MoE decoder layer."""
    return replace(ModelArgs(), n_layers=1, n_dense_layers=0, max_seq_len=max_seq_len)
