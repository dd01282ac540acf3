"""FP8 block quantisation helpers of the oracle (test infrastructure only).

The HF DeepSeek FP8 checkpoint format stores ``weight`` as e4m3 and
``weight_scale_inv`` as one f32 per 128x128 block; the reference dequantises with
``w = fp8 * s[i // 128, j // 128]`` (tilert/models/deepseek_v3_2/refs/kernel.py:82-129).
"""

from __future__ import annotations

import torch

BLOCK = 128
FP8_MAX = 448.0


def weight_dequant(w_fp8: torch.Tensor, scale: torch.Tensor, block: int = BLOCK,
                   out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Block dequantisation, refs/kernel.py:82-94 (``_weight_dequant_torch``).

    The reference's CPU fallback needs both dimensions to be multiples of 128 and so
    fails on the 576-row ``kv_a_proj_with_mqa`` weight; its Triton kernel masks the
    ragged edge (refs/kernel.py:70-78).  This restatement pads like the masked kernel.
    The result is rounded to ``out_dtype`` exactly as the reference rounds to the
    default dtype (bf16 in every golden).
    """
    m, n = w_fp8.shape
    mp = (m + block - 1) // block * block
    np_ = (n + block - 1) // block * block
    w = torch.zeros(mp, np_, dtype=torch.float32)
    w[:m, :n] = w_fp8.float()
    w = w.reshape(mp // block, block, np_ // block, block) * scale.float()[:, None, :, None]
    return w.reshape(mp, np_)[:m, :n].to(out_dtype).contiguous()


def quantize_weight_block128(w: torch.Tensor, block: int = BLOCK) -> tuple[torch.Tensor, torch.Tensor]:
    """Quantise an f32 matrix to e4m3 with one f32 scale per 128x128 block.

    ``scale = amax / 448`` per block (the synthetic-weight recipe of the workload
    definitions; the inverse of ``weight_dequant``).  Ragged edges are handled by
    padding with zeros.
    """
    m, n = w.shape
    mp = (m + block - 1) // block * block
    np_ = (n + block - 1) // block * block
    wp = torch.zeros(mp, np_, dtype=torch.float32)
    wp[:m, :n] = w.float()
    blk = wp.reshape(mp // block, block, np_ // block, block)
    amax = blk.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = (amax / FP8_MAX).float()
    q = (blk / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX)
    q = q.reshape(mp, np_)[:m, :n].contiguous().to(torch.float8_e4m3fn)
    return q, scale.contiguous()


def act_quant(x: torch.Tensor, block: int = BLOCK) -> tuple[torch.Tensor, torch.Tensor]:
    """1x128 activation quantisation, refs/kernel.py:154-199.

    ``amax = max(|x|, 1e-4)``, ``s = amax / 448``, ``y = clamp(x / s, +-448)`` cast to
    e4m3 (the non-rounded-scale branch, ``scale_fmt is None``).
    """
    shp = x.shape
    xf = x.float().reshape(-1, shp[-1] // block, block)
    amax = xf.abs().amax(dim=-1).clamp_min(1e-4)
    s = amax / FP8_MAX
    y = (xf / s[..., None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return y.reshape(shp), s.reshape(*shp[:-1], shp[-1] // block)
