"""Oracle (test infrastructure only): the FP8 wire format in which an external prefill hands the latent
caches to the decode side, restated from tilert/pd_vllm/profiles/mla_nsa.py.

Layout (mla_nsa.py:16-41): per token 512 e4m3 latent values + 4 f32 scales (one per 128 values) = 528
bytes; 64 bf16 rope values = 128 bytes; indexer keys in pages of 64 tokens, 64 x 128 e4m3 values followed
by 64 f32 scales = 8448 bytes.  The decode side dequantises to bf16 (``dequant_kv``, ``dequant_ki``) and
copies the rows into its caches (tilert/models/deepseek_v3_2/generator.py:419-484).

The two quantisers below only make test inputs (the producer is the prefill engine, which is not part of
the reference): scale = amax / 448 per 128 values, the usual rule of this format.
"""

from __future__ import annotations

import torch

from .ops import hadamard_matrix

KV_LORA_RANK, ROPE_DIM, INDEX_DIM, BLOCK, PAGE = 512, 64, 128, 128, 64
KV_BYTES = KV_LORA_RANK + KV_LORA_RANK // BLOCK * 4          # 528
PE_BYTES = ROPE_DIM * 2                                      # 128
KI_PAGE_BYTES = PAGE * INDEX_DIM + PAGE * INDEX_DIM // BLOCK * 4  # 8448


def dequant_kv(kv_raw: torch.Tensor, seq_len: int) -> torch.Tensor:
    """MlaNsaProfile._dequant_kv, mla_nsa.py:186-210: uint8 [seq, 528] -> bf16 [seq, 512]."""
    nblk = KV_LORA_RANK // BLOCK
    fp8 = kv_raw[:, :KV_LORA_RANK].reshape(-1).view(torch.float8_e4m3fn).reshape(seq_len, KV_LORA_RANK)
    scale = kv_raw[:, KV_LORA_RANK:].reshape(-1).contiguous().view(torch.float32).reshape(seq_len, nblk)
    deq = fp8.float().view(seq_len, nblk, BLOCK) * scale.unsqueeze(-1)
    return deq.view(seq_len, KV_LORA_RANK).to(torch.bfloat16)


def dequant_ki(ki_raw: torch.Tensor, seq_len: int) -> torch.Tensor:
    """MlaNsaProfile._dequant_ki, mla_nsa.py:212-232: uint8 [pages, 8448] -> bf16 [seq, 128], dequantised,
    rounded to bf16, then rotated by the Hadamard matrix scaled by 128^-1/2 (mla_nsa.py:48-62)."""
    npages = ki_raw.shape[0]
    nb = PAGE * INDEX_DIM
    fp8 = ki_raw[:, :nb].reshape(-1).view(torch.float8_e4m3fn).reshape(npages * PAGE, INDEX_DIM)
    scale = ki_raw[:, nb:].reshape(-1).contiguous().view(torch.float32).reshape(npages * PAGE, INDEX_DIM // BLOCK)
    deq = (fp8[:seq_len].float() * scale[:seq_len]).to(torch.bfloat16)
    h = hadamard_matrix(INDEX_DIM) * (INDEX_DIM ** -0.5)
    return (deq.float() @ h).to(torch.bfloat16)


def _quant_rows(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    rows, nblk = x.shape[0], x.shape[1] // BLOCK
    blocks = x.float().view(rows, nblk, BLOCK)
    scale = blocks.abs().amax(-1).clamp_min(1e-4) / 448.0
    q = (blocks / scale.unsqueeze(-1)).to(torch.float8_e4m3fn)
    return q.view(rows, nblk * BLOCK), scale


def quant_kv(kv: torch.Tensor) -> torch.Tensor:
    """Test-input maker: bf16 [seq, 512] -> uint8 [seq, 528]."""
    q, scale = _quant_rows(kv)
    return torch.cat([q.view(torch.uint8), scale.contiguous().view(torch.uint8).view(kv.shape[0], KV_BYTES - KV_LORA_RANK)], dim=1).contiguous()


def quant_ki_pages(ki_unrotated: torch.Tensor) -> torch.Tensor:
    """Test-input maker: bf16 [seq, 128] (keys BEFORE the Hadamard rotation) -> uint8 [pages, 8448]."""
    seq = ki_unrotated.shape[0]
    npages = (seq + PAGE - 1) // PAGE
    if npages == 0:
        return torch.zeros(0, KI_PAGE_BYTES, dtype=torch.uint8)
    padded = torch.zeros(npages * PAGE, INDEX_DIM, dtype=torch.bfloat16)
    padded[:seq] = ki_unrotated
    q, scale = _quant_rows(padded)
    pages = torch.zeros(npages, KI_PAGE_BYTES, dtype=torch.uint8)
    pages[:, : PAGE * INDEX_DIM] = q.view(torch.uint8).view(npages, PAGE * INDEX_DIM)
    pages[:, PAGE * INDEX_DIM:] = scale.contiguous().view(torch.uint8).view(npages, PAGE * 4)
    return pages
