"""Host-side packers: HF-format FP8 tensors -> the library's weight-block format.

The reference's converters (``convert_to_*`` methods of the ops under
tilert/models/deepseek_v3_2/ops/) emit layouts private to its closed kernels; these emit the
layout of ``tilert_b200/csrc/formats.h``.  Inputs are what the reference's ``device_sharding``
methods hand to a converter: an e4m3 ``weight`` and its f32 ``weight_scale_inv`` (one scale per
128x128 block).  Pure tensor reshuffling; runs on whatever device the tensors live on.
"""

from __future__ import annotations

import torch

TILE = 128
KB = 128
WBLK_BYTES = 16448
XBLK_BYTES = 1056


def row_scales(scale: torch.Tensor, n_rows: int) -> torch.Tensor:
    """Expand block scales [ceil(N/128), K/128] to one row of scales per weight row [N, K/128]."""
    return scale.float().repeat_interleave(TILE, dim=0)[:n_rows].contiguous()


def pack_rows(w: torch.Tensor, rscale: torch.Tensor) -> torch.Tensor:
    """Pack weight rows into W blocks.

    ``w``      [N, K] e4m3 (or uint8 view), rows in the order the kernel should emit them;
    ``rscale`` [N, K/128] f32, the dequantisation scale of each row for each k block (every
               aligned group of 8 rows must share its scales).
    Returns uint8 [ceil(N/128), K/128, 16448].
    """
    w = w.view(torch.uint8)
    n, k = w.shape
    assert k % KB == 0 and rscale.shape == (n, k // KB)
    n_t, n_kb = (n + TILE - 1) // TILE, k // KB
    npad = n_t * TILE
    if npad != n:
        # padding rows are zero bytes; they repeat the last real row's scales, so that a ragged row count
        # (n not a multiple of 8) still has one scale per aligned group of 8 packed rows
        w = torch.cat([w, torch.zeros(npad - n, k, dtype=torch.uint8, device=w.device)], 0)
        rscale = torch.cat([rscale, rscale[-1:].expand(npad - n, n_kb)], 0)
    g8 = rscale.view(npad // 8, 8, n_kb)
    if not bool((g8 == g8[:, :1]).all()):
        raise ValueError("each aligned group of 8 packed rows must share one scale per k block")
    # rows: t, row group(16), r(8)      cols: kb, c(4), kc(2), b(16)   ->   t, kb, c, row group, kc, r, b
    v = w.view(n_t, 16, 8, n_kb, 4, 2, 16)
    data = v.permute(0, 3, 4, 1, 5, 2, 6).reshape(n_t, n_kb, 16384)
    sc = g8[:, 0].view(n_t, 16, n_kb).permute(0, 2, 1).contiguous().float()
    sc_bytes = sc.view(torch.uint8).view(n_t, n_kb, 64)
    return torch.cat([data, sc_bytes], dim=2).contiguous()


def pack_matrix(w: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """Pack a plain [N, K] FP8 linear weight (rows in natural order)."""
    return pack_rows(w, row_scales(scale, w.shape[0]))


def pack_concat(parts: list[tuple[torch.Tensor, torch.Tensor]]) -> torch.Tensor:
    """Pack several [N_i, K] FP8 weights as one row-concatenated matrix."""
    w = torch.cat([p[0].view(torch.uint8) for p in parts], 0)
    rs = torch.cat([row_scales(p[1], p[0].shape[0]) for p in parts], 0)
    return pack_rows(w, rs)


def pack_q_b(wq_b, sq_b, n_heads: int, nope: int, rope: int, wqi=None, sqi=None) -> torch.Tensor:
    """q_b_proj rows regrouped as [all heads' nope | all heads' rope | indexer wq_b]."""
    hd = nope + rope
    w = wq_b.view(torch.uint8).view(n_heads, hd, -1)
    rs = row_scales(sq_b, wq_b.shape[0]).view(n_heads, hd, -1)
    ws = [w[:, :nope].reshape(n_heads * nope, -1), w[:, nope:].reshape(n_heads * rope, -1)]
    rss = [rs[:, :nope].reshape(n_heads * nope, -1), rs[:, nope:].reshape(n_heads * rope, -1)]
    if wqi is not None:
        ws.append(wqi.view(torch.uint8))
        rss.append(row_scales(sqi, wqi.shape[0]))
    return pack_rows(torch.cat(ws, 0), torch.cat(rss, 0))


def pack_q_b_rows(w_rows, rs_rows, n_heads: int, nope: int, rope: int, wqi=None, sqi=None) -> torch.Tensor:
    """Same regrouping as ``pack_q_b`` for a head range whose rows and per-row scales were already
    sliced out of the full matrix (head boundaries are not multiples of the 128-row scale blocks)."""
    hd = nope + rope
    w = w_rows.view(torch.uint8).view(n_heads, hd, -1)
    rs = rs_rows.view(n_heads, hd, -1)
    ws = [w[:, :nope].reshape(n_heads * nope, -1), w[:, nope:].reshape(n_heads * rope, -1)]
    rss = [rs[:, :nope].reshape(n_heads * nope, -1), rs[:, nope:].reshape(n_heads * rope, -1)]
    if wqi is not None:
        ws.append(wqi.view(torch.uint8))
        rss.append(row_scales(sqi, wqi.shape[0]))
    return pack_rows(torch.cat(ws, 0), torch.cat(rss, 0))


def pack_kv_b_absorb(wkv_b, skv_b, n_heads: int, nope: int, v_dim: int) -> torch.Tensor:
    """W_kvb^nope transposed per head: rows (h, c), columns d  (q_lat[h, c] = sum_d q_nope[h, d] W[h, d, c])."""
    c_dim = wkv_b.shape[1]
    w = wkv_b.view(torch.uint8).view(n_heads, nope + v_dim, c_dim)[:, :nope]         # [h, d, c]
    wt = w.permute(0, 2, 1).reshape(n_heads * c_dim, nope).contiguous()                 # [(h, c), d]
    s = skv_b.float().view(n_heads, (nope + v_dim) // TILE, c_dim // TILE)[:, : nope // TILE]  # [h, d_blk, c_blk]
    rs = s.permute(0, 2, 1).repeat_interleave(TILE, dim=1).reshape(n_heads * c_dim, nope // TILE)
    return pack_rows(wt, rs.contiguous())


def pack_kv_b_v(wkv_b, skv_b, n_heads: int, nope: int, v_dim: int) -> torch.Tensor:
    """W_kvb^v per head: rows (h, d), columns c  (o[h, d] = sum_c o_lat[h, c] W[h, d, c])."""
    c_dim = wkv_b.shape[1]
    w = wkv_b.view(torch.uint8).view(n_heads, nope + v_dim, c_dim)[:, nope:].reshape(n_heads * v_dim, c_dim)
    rs = row_scales(skv_b, wkv_b.shape[0]).view(n_heads, nope + v_dim, -1)[:, nope:].reshape(n_heads * v_dim, -1)
    return pack_rows(w.contiguous(), rs.contiguous())


def pack_gate_up(w_gate, s_gate, w_up, s_up) -> torch.Tensor:
    """Gate and up rows interleaved in groups of 8, so one 16-row MMA tile holds (gate, up) pairs."""
    inter, k = w_gate.shape
    assert inter % 8 == 0
    g = w_gate.view(torch.uint8).view(inter // 8, 8, k)
    u = w_up.view(torch.uint8).view(inter // 8, 8, k)
    w = torch.stack([g, u], dim=1).reshape(2 * inter, k)
    rg = row_scales(s_gate, inter).view(inter // 8, 8, -1)
    ru = row_scales(s_up, inter).view(inter // 8, 8, -1)
    rs = torch.stack([rg, ru], dim=1).reshape(2 * inter, -1)
    return pack_rows(w, rs)


def pack_bf16_two_term(w: torch.Tensor) -> torch.Tensor:
    """A bf16 weight [N, K] (router gate, indexer head weights: bf16 in the checkpoint) as TWO e4m3 rows per
    source row, so that it can ride the FP8 weight stream: ``w = hi * s + lo * s / 16`` with a power-of-two
    scale ``s`` per (8 rows x 128 columns).  bf16 has 8 significant bits and e4m3 has 4, so the split is exact
    unless an element is more than ~2^13 times smaller than its group's largest (then it keeps fewer bits; the
    error is below 2^-22 of the group maximum).  Packed rows: for every group of 8 source rows, the 8 ``hi``
    rows followed by the 8 ``lo`` rows; the kernel's pair-add epilogue sums row l and row l + 8.
    Returns uint8 [ceil(2 N / 128), K / 128, 16448]."""
    n, k = w.shape
    assert k % KB == 0
    npad = (n + 7) // 8 * 8
    wf = torch.zeros(npad, k, dtype=torch.float32, device=w.device)
    wf[:n] = w.float()
    g = wf.view(npad // 8, 8, k // KB, KB)
    amax = g.abs().amax(dim=(1, 3), keepdim=True)
    s = torch.where(amax > 0, torch.exp2(torch.ceil(torch.log2(amax / 448.0))), torch.ones_like(amax))
    hi = (g / s).clamp(-448, 448).to(torch.float8_e4m3fn)
    r = g - hi.float() * s
    lo = (r / (s / 16)).clamp(-448, 448).to(torch.float8_e4m3fn)
    rows = torch.stack([hi.view(torch.uint8).reshape(npad // 8, 8, k), lo.view(torch.uint8).reshape(npad // 8, 8, k)], dim=1)
    sc = s.reshape(npad // 8, 1, k // KB)
    rs = torch.stack([sc.expand(-1, 8, -1), (sc / 16).expand(-1, 8, -1)], dim=1)
    return pack_rows(rows.reshape(2 * npad, k), rs.reshape(2 * npad, k // KB).contiguous())


def unpack_rows(packed: torch.Tensor, n: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Inverse of ``pack_rows`` (for round-trip tests): returns (uint8 [n, K], row scales [n/8.., ...])."""
    n_t, n_kb, _ = packed.shape
    data = packed[:, :, :16384].reshape(n_t, n_kb, 4, 16, 2, 8, 16)  # t kb c rg kc r b
    w = data.permute(0, 3, 5, 1, 2, 4, 6).reshape(n_t * TILE, n_kb * KB)
    sc = packed[:, :, 16384:].contiguous().view(torch.float32).view(n_t, n_kb, 16).permute(0, 2, 1)
    rs = sc.reshape(n_t * 16, n_kb).repeat_interleave(8, dim=0)
    return w[:n].contiguous(), rs[:n].contiguous()


def reference_xpack(x: torch.Tensor) -> torch.Tensor:
    """CPU model of the device activation packer (split mode) for tests of the format: returns the
    values hi*s_hi + lo*s_lo that the GEMM effectively multiplies with, shape of ``x``."""
    xf = x.float().reshape(-1, x.shape[-1] // KB, KB)
    amax = xf.abs().amax(-1, keepdim=True)
    s_hi = torch.where(amax > 0, torch.exp2(torch.ceil(torch.log2(amax / 448.0))), torch.ones_like(amax))
    hi = (xf / s_hi).clamp(-448, 448).to(torch.float8_e4m3fn).float()
    r = xf - hi * s_hi
    lo = (r / (s_hi / 16)).clamp(-448, 448).to(torch.float8_e4m3fn).float()
    return (hi * s_hi + lo * s_hi / 16).reshape(x.shape)
