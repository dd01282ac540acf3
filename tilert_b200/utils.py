"""Parity metrics with the reference's definitions (tilert/utils.py:65-90)."""

import torch


def cosine_similarity(gt: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.cosine_similarity(gt.flatten().float(), out.flatten().float(), dim=-1)


def relative_l2_error(gt: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    gt, out = gt.float(), out.float()
    return torch.norm(gt - out) / torch.norm(gt)
