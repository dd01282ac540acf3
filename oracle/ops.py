"""Per-operator CPU restatements of the reference goldens (test infrastructure only).

Every function cites the reference ``golden_forward`` it follows, by path inside the
reference project.  All tensors are CPU tensors; activations are bf16 unless noted and
weights arrive already dequantised to bf16 (``oracle.quant.weight_dequant``), exactly
as the reference's ``init_reference_weights`` methods hold them.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

BF16 = torch.bfloat16


# --------------------------------------------------------------------------- helpers
def rms_norm_f32(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    """``torch.nn.functional.rms_norm(x.float(), [dim], gamma, eps)`` kept in f32."""
    return F.rms_norm(x.float(), [x.size(-1)], gamma.float(), eps)


def precompute_freqs_cis(args) -> torch.Tensor:
    """YaRN rotary table, tilert/models/utils.py:17-118.  Returns complex64 [T, rope/2]."""
    dim = args.qk_rope_head_dim
    seqlen = args.max_seq_len
    base = args.rope_theta
    factor = args.rope_factor

    def corr_dim(num_rot: float) -> float:
        return dim * math.log(args.original_seq_len / (num_rot * 2 * math.pi)) / (2 * math.log(base))

    freqs = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    if factor is not None and seqlen > args.original_seq_len:
        low = max(math.floor(corr_dim(args.beta_fast)), 0)
        high = min(math.ceil(corr_dim(args.beta_slow)), dim - 1)
        lo, hi = float(low), float(high)
        if lo == hi:
            hi += 0.001
        ramp = torch.clamp((torch.arange(dim // 2, dtype=torch.float32) - lo) / (hi - lo), 0, 1)
        smooth = 1 - ramp
        freqs = freqs / factor * (1 - smooth) + freqs * smooth
    t = torch.arange(seqlen)
    ang = torch.outer(t, freqs)
    return torch.polar(torch.ones_like(ang), ang)


def apply_rotary_emb(x: torch.Tensor, freqs_cis: torch.Tensor, interleaved: bool = True) -> torch.Tensor:
    """tilert/models/utils.py:121-145.  ``x`` is [B, S, H, D]; ``freqs_cis`` is [S, D/2]."""
    dtype = x.dtype
    shape = x.shape
    if not interleaved:
        x = x.view(*shape[:-1], 2, -1).transpose(-1, -2).contiguous()
    xc = torch.view_as_complex(x.float().view(*shape[:-1], -1, 2))
    fc = freqs_cis.view(1, xc.size(1), 1, xc.size(-1))
    y = torch.view_as_real(xc * fc).flatten(3)
    if not interleaved:
        y = torch.cat([y[..., 0::2], y[..., 1::2]], dim=-1)
    return y.to(dtype)


def hadamard_matrix(n: int) -> torch.Tensor:
    """Sylvester Hadamard matrix (what scipy.linalg.hadamard returns), f32."""
    h = torch.ones(1, 1)
    while h.size(0) < n:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return h


def rotate_activation(x: torch.Tensor) -> torch.Tensor:
    """tilert/models/deepseek_v3_2/ops/rotate.py:27-49 (scipy fallback branch).

    ``F.linear(x_bf16, H_bf16) * dim**-0.5`` -- the matrix product and the scaling are
    both carried out in bf16 tensors, as the reference's fallback does.
    """
    assert x.dtype == BF16
    d = x.size(-1)
    h = hadamard_matrix(d).to(BF16)
    out = F.linear(x.reshape(-1, d), h) * d ** -0.5
    return out.reshape(x.shape)


# ------------------------------------------------------------------ MLA projections
def projx_wqkva(x, gamma, wq_a, wkv_a, w_pe, eps):
    """RMSNormProjxWqkva.golden_forward, ops/rmsnorm_projx_wqkva.py:450-471."""
    xn = rms_norm_f32(x, gamma, eps)
    q = xn @ wq_a.float().T
    kv = xn @ wkv_a.float().T
    pe = xn @ w_pe.float().T
    return q.to(BF16), kv.to(BF16), pe.to(BF16)


def projx_wqakis(x, gamma, wq_a, wki, wis, eps):
    """RMSNormProjxWqakis.golden_forward, ops/rmsnorm_projx_wqakis.py:279-299."""
    xn = rms_norm_f32(x, gamma, eps)
    q = xn @ wq_a.float().T
    ki = xn @ wki.float().T
    w = xn @ wis.to(BF16).float().T
    return q.to(BF16), ki.to(BF16), w.to(BF16)


def rmsnorm_projq_wqb(q, q_norm, wq_b, n_heads, nope, rope, eps):
    """RmsnormProjqWqb.golden_forward, ops/rmsnorm_projq_wqb.py:496-512."""
    b, s, _ = q.shape
    qr = rms_norm_f32(q, q_norm, eps).to(q.dtype)
    out = torch.matmul(qr, wq_b.T).view(b, s, n_heads, nope + rope)
    q_nope, q_pe = torch.split(out, [nope, rope], dim=-1)
    return q_nope.contiguous(), q_pe.contiguous()


def rmsnorm_projq_wqi(q, q_norm, wqi, head_dim, eps):
    """RmsnormProjqWqi.golden_forward, ops/rmsnorm_projq_wqi.py:301-314."""
    b, s, _ = q.shape
    qr = rms_norm_f32(q, q_norm, eps).to(q.dtype)
    return torch.matmul(qr, wqi.T).view(b, s, -1, head_dim)


def rmsnorm_kv(kv, gamma, eps):
    """KVRMSNorm.golden_forward, ops/rmsnorm_kv.py:172-181 (value written to the cache)."""
    return rms_norm_f32(kv, gamma, eps).to(kv.dtype)


def qkv_rope(q_pe, k_pe, freqs_cis):
    """QKVRoPE.golden_forward, ops/qkv_rope.py:137-152.  Returns (q_pe_rot, k_pe_rot)."""
    k_rot = apply_rotary_emb(k_pe.unsqueeze(2), freqs_cis).squeeze(2)
    return apply_rotary_emb(q_pe, freqs_cis), k_rot


def rotate(idx_q, freqs_cis, rope_dim):
    """Rotate.golden_forward, ops/rotate.py:201-213."""
    q_pe, q_nope = torch.split(idx_q, [rope_dim, idx_q.size(-1) - rope_dim], dim=-1)
    q_pe = apply_rotary_emb(q_pe, freqs_cis, interleaved=False)
    return rotate_activation(torch.cat([q_pe, q_nope], dim=-1))


def layernorm_rope_rotate(idx_k, weight, bias, freqs_cis, rope_dim):
    """LayerNormRoPERotate.golden_forward, ops/layernorm_rope_rotate.py:206-220."""
    d = idx_k.size(-1)
    k = F.layer_norm(idx_k.float(), (d,), weight.float(), bias.float(), 1e-6).to(idx_k.dtype)
    k_pe, k_nope = torch.split(k, [rope_dim, d - rope_dim], dim=-1)
    k_pe = apply_rotary_emb(k_pe.unsqueeze(2), freqs_cis, interleaved=False).squeeze(2)
    return rotate_activation(torch.cat([k_pe, k_nope], dim=-1))


# ------------------------------------------------------------- indexer and top-k
def indexer_logits(iq, ki_cache, weights, n_valid):
    """Lightning-indexer scores -- NO reference golden exists (ops/sparse_index.py:11-69
    only says "q * kv * weights"); parity unpinned for this function.

    DeepSeek-V3.2's published indexer: ``logit[s, t] = sum_h w[s, h] * relu(q[s, h] . k[t])``.
    ``iq`` [1, S, H, D] bf16, ``ki_cache`` [1, T, D] bf16, ``weights`` [1, S, H] bf16.
    Token ``s`` of the step sits at position ``n_valid - S + s`` and may see keys
    ``0 .. n_valid - S + s``; later keys get ``-inf`` (ops/topk.py:78-80 states the same
    valid lengths ``seq-k+1 .. seq``).  Returns f32 [1, S, T].
    """
    s_len = iq.size(1)
    t_len = ki_cache.size(1)
    dots = torch.einsum("bshd,btd->bsht", iq.float(), ki_cache.float())
    logits = (torch.relu(dots) * weights.float()[..., None]).sum(dim=2)
    pos = torch.arange(t_len)[None, None, :]
    last = (n_valid - s_len + torch.arange(s_len))[None, :, None]
    return logits.masked_fill(pos > last, float("-inf"))


def topk_indices(logits, k):
    """TopK.golden_forward, ops/topk.py:128-143: ``logits.topk(min(k, T))[1]``.

    ``torch.topk`` leaves ties unspecified; this oracle fixes the convention the CUDA
    path follows: larger value first, equal values by lower index first, -inf entries
    are never selected, and unused slots hold -1.  Returns int32 [..., k] sorted by
    index ascending (comparison is on the index *set*).
    """
    shp = logits.shape
    flat = logits.reshape(-1, shp[-1])
    out = torch.full((flat.size(0), k), -1, dtype=torch.int32)
    for r in range(flat.size(0)):
        row = flat[r]
        order = torch.sort(row, descending=True, stable=True)[1]
        order = order[torch.isfinite(row[order]) | (row[order] == float("inf"))][:k]
        sel = torch.sort(order)[0]
        out[r, : sel.numel()] = sel.to(torch.int32)
    return out.reshape(*shp[:-1], k)


# ------------------------------------------------------------- sparse MLA decode
def softmax_scale(args) -> float:
    """FlashSparseMLACombine.__init__, ops/flash_sparse_mla.py:125-130."""
    scale = (args.qk_nope_head_dim + args.qk_rope_head_dim) ** -0.5
    mscale = 1.0 if args.rope_factor is None else 0.1 * math.log(args.rope_factor) + 1.0
    return scale * mscale * mscale


def projq_wqb_absorb(q_nope, wkv_b_nope):
    """ProjqWqb.golden_forward, ops/projq_wqb.py:448-450.  ``wkv_b_nope`` is [h, d, c] bf16."""
    return torch.einsum("bshd,hdc->bshc", q_nope, wkv_b_nope)


def flash_sparse_mla(q_lat, q_pe, kv_cache, pe_cache, topk_idx, start_pos, scale):
    """FlashSparseMLACombine.golden_forward, ops/flash_sparse_mla.py:153-195.

    Entries of ``topk_idx`` equal to -1 are unused slots (the reference never produces
    them; they are dropped here before the scatter).
    """
    b, s, h, _ = q_lat.shape
    t = kv_cache.size(1)
    scores = (
        torch.einsum("bshc,btc->bsht", q_lat.float(), kv_cache.float())
        + torch.einsum("bshr,btr->bsht", q_pe.float(), pe_cache.float())
    ) * scale
    index_mask = torch.full((b, s, t + 1), float("-inf"))
    idx = topk_idx.long().clone()
    idx[idx < 0] = t
    index_mask.scatter_(-1, idx, 0.0)
    index_mask = index_mask[..., :t]
    if s > 1:
        index_mask = index_mask + torch.full((s, t), float("-inf")).triu_(start_pos + 1)
    scores = scores + index_mask.unsqueeze(2)
    probs = scores.softmax(dim=-1, dtype=torch.float32)
    return torch.einsum("bsht,btc->bshc", probs.to(BF16), kv_cache)


def projo_wkvb(o_lat, wkv_b_v):
    """ProjoWKVb.golden_forward, ops/projo_wkvb.py:465-467.  ``wkv_b_v`` is [h, d, c] bf16."""
    return torch.einsum("bshc,hdc->bshd", o_lat, wkv_b_v)


def unproj_o(o, w_o):
    """UnProjOAllReduce.golden_forward, ops/unproj_o_allreduce.py:480-498 (one shard's
    partial product; the kernel adds the all-reduce and the residual, :23-58)."""
    b, s = o.shape[:2]
    return (o.reshape(b, s, -1).float() @ w_o.float().T).to(BF16)


# ----------------------------------------------------------------------- MoE / FFN
def rmsnorm_bf16(x, gamma, eps, residual=None):
    """RMSNorm.forward, tilert/models/common.py:111-133."""
    if residual is None:
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        return (gamma.float() * xf).to(BF16)
    xf = x.float() + residual.float()
    res = xf
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (gamma.float() * xf).to(BF16), res.to(BF16)


def rmsnorm_expert_proj(x, gamma, w_gate, eps):
    """RMSNormExpertProj.golden_forward, ops/rmsnorm_expert_proj.py:142-149."""
    xn = rmsnorm_bf16(x, gamma, eps)
    scores = xn.view(-1, x.size(-1)).float() @ w_gate.float().T
    return xn, scores


def expert_select_ds(scores, bias, n_groups, n_limited_groups, top_k, route_scale):
    """``_ref_expert_select_ds`` -- defined only in the GLM fork of the op,
    tilert/models/glm_5/_dsa_v32/ops/expert_sel_up_gate_silu.py:714-737; the
    DeepSeek-V3.2 golden calls it (ops/expert_sel_up_gate_silu.py:665).

    ``torch.topk`` ties are resolved here as larger value first, lower index first.
    """
    n = scores.size(-1)
    flat = scores.reshape(-1, n).float().sigmoid()
    orig = flat
    sel_scores = flat + bias.float() if bias is not None else flat.clone()
    if n_groups > 1:
        g = sel_scores.view(-1, n_groups, n // n_groups)
        if bias is None:
            gs = g.amax(dim=-1)
        else:
            gs = g.topk(2, dim=-1)[0].sum(dim=-1)
        keep = torch.sort(gs, dim=-1, descending=True, stable=True)[1][:, :n_limited_groups]
        mask = torch.ones(g.size(0), n_groups, dtype=torch.bool).scatter_(1, keep, False)
        sel_scores = g.masked_fill(mask.unsqueeze(-1), float("-inf")).flatten(1)
    idx = torch.sort(sel_scores, dim=-1, descending=True, stable=True)[1][:, :top_k]
    w = orig.gather(-1, idx)
    w = w / w.sum(dim=-1, keepdim=True)
    w = w * route_scale
    shp = scores.shape[:-1]
    return w.view(*shp, top_k), idx.view(*shp, top_k)


def expert_up_gate_silu(x, gate_list, up_list):
    """ExpertSelectUpGateSiLU.golden_forward (the GEMV part), ops/expert_sel_up_gate_silu.py:654-692.

    ``gate_list`` / ``up_list`` hold, per token, the bf16 weights of the shared expert
    followed by the selected routed experts, in selection order.  Returns bf16
    [1, S, E, inter].
    """
    outs = []
    for s in range(x.size(1)):
        xs = x[0, s].float()
        w1 = torch.stack([xs @ g.float().T for g in gate_list[s]], dim=0)
        w3 = torch.stack([xs @ u.float().T for u in up_list[s]], dim=0)
        outs.append((F.silu(w1) * w3).to(BF16))
    return torch.stack(outs, dim=0)[None]


def expert_down(vec, down_list, probs):
    """ExpertDownAllReduce.golden_forward, ops/expert_down_allreduce.py:445-468.

    Each expert's product is cast to bf16 *before* the sum (:463-464).  ``probs`` is
    [1, S, E-1] f32 (the shared expert, slot 0, has weight 1).  Returns bf16 [1, S, dim].
    """
    outs = []
    for s in range(vec.size(1)):
        parts = [vec[0, s, 0].float() @ down_list[s][0].float().T]
        for i in range(1, vec.size(2)):
            parts.append((vec[0, s, i].float() @ down_list[s][i].float().T) * probs[0, s, i - 1])
        outs.append(torch.stack(parts, dim=0).to(BF16).sum(dim=0))
    return torch.stack(outs, dim=0)[None]


def dense_up_gate_silu(x, gamma, w_gate, w_up, eps, n_split=1):
    """RMSNormUpGateSiLU.golden_forward, ops/rmsnorm_up_gate_silu.py:318-347: the intermediate
    dimension is cut into ``n_split`` pseudo-experts and every token's normalised vector is
    multiplied with each slice on its own (f32), as the golden's loops do."""
    xn = rms_norm_f32(x, gamma, eps)
    chunk = w_gate.size(0) // n_split
    outs = []
    for s in range(x.size(1)):
        w1 = torch.stack([xn[0, s].float() @ w_gate[i * chunk:(i + 1) * chunk].float().T for i in range(n_split)], dim=0)
        w3 = torch.stack([xn[0, s].float() @ w_up[i * chunk:(i + 1) * chunk].float().T for i in range(n_split)], dim=0)
        outs.append((F.silu(w1.float()) * w3.float()).to(BF16).reshape(-1))
    return torch.stack(outs, dim=0)[None]


def dense_down(vec, w_down, n_split):
    """DownAllReduce.golden_forward, ops/down_allreduce.py:293-319: the intermediate
    dimension is cut into ``n_split`` equal pseudo-experts, each partial product is cast
    to bf16 and the bf16 partials are summed."""
    b, s, inter = vec.shape
    chunk = inter // n_split
    outs = []
    for si in range(s):
        parts = []
        for i in range(n_split):
            sl = slice(i * chunk, (i + 1) * chunk)
            parts.append(vec[0, si, sl].float() @ w_down[:, sl].float().T)
        outs.append(torch.stack(parts, dim=0).to(BF16).sum(dim=0))
    return torch.stack(outs, dim=0)[None]


def rmsnorm_head_proj(x, gamma, w_head, eps):
    """RMSNormHeadProj.golden_forward, ops/rmsnorm_head_proj.py:253-273.  f32 logits."""
    return rms_norm_f32(x, gamma, eps) @ w_head.float().T


def eh_proj(e_norm, h_norm, w_eh):
    """EHProjAllReduce.golden_forward, ops/eh_proj_allreduce.py:252-277, summed over devices: the
    concatenated normalised embedding and hidden state through eh_proj [dim, 2*dim] (bf16 in, bf16 out)."""
    cat = torch.cat([e_norm, h_norm], dim=-1)
    return cat @ w_eh.T  # a bf16 matmul, as in the reference


def mtp_preprocess(e, h, gamma_e, gamma_h, w_eh, eps=1e-6):
    """MTPPreprocessLayer.golden_forward, modules/mtp_preprocess.py:197-229: enorm(embedding),
    hnorm(previous hidden state), concatenate, eh_proj.  The reference golden keeps the two
    normalised vectors in f32 and multiplies them with the bf16 weight, which its own ``linear``
    rejects on CPU (dtype mismatch); its kernel path hands bf16 vectors to eh_proj_allreduce_op
    (ops/eh_proj_allreduce.py:40), and that is what is restated here.  Returns (e_norm, h_norm, out)."""
    e_norm = rmsnorm_bf16(e, gamma_e, eps)
    h_norm = rmsnorm_bf16(h, gamma_h, eps)
    return e_norm, h_norm, eh_proj(e_norm, h_norm, w_eh)


def sample_uniform(seed: int, step: int, tok: int) -> float:
    """The sampler's uniform number for (seed, step, token index): a splitmix64 finaliser, top 24 bits."""
    mask = (1 << 64) - 1
    z = (seed + 0x9E3779B97F4A7C15 * (step + 1) + 0xD1B54A32D192ED03 * (tok + 1)) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z ^= z >> 31
    return float(z >> 40) / 16777216.0


def sample_intervals(logits_row, temperature, top_p, top_k, use_top_p, n_candidates=1024):
    """Restatement of the sampling rule -- NO reference golden exists (the rule lives in the reference's
    binary; only its configuration and outputs are visible, modules/end2end.py:253-311, 665-703); parity
    unpinned.  Standard temperature / top-k / top-p sampling over the ``n_candidates`` largest logits:
    returns (token ids in sampling order, cumulative upper bounds in [0, 1] of each kept token,
    log-probabilities of the unscaled softmax for all candidates).  A uniform number u selects the first
    token whose bound exceeds u.  Computed in float64."""
    x = logits_row.double()
    order = torch.argsort(-x, stable=True)[:n_candidates]  # value descending, ties to the lower id
    vals = x[order]
    lse1 = torch.logsumexp(x, 0)
    logp = vals - lse1
    if temperature <= 0:
        return order[:1], torch.ones(1, dtype=torch.float64), logp
    pt = torch.exp((vals - x.max()) / temperature) / torch.exp((x - x.max()) / temperature).sum()
    k_eff = top_k if 1 <= top_k <= n_candidates else n_candidates
    k_eff = min(k_eff, order.numel())
    cum = torch.cumsum(pt[:k_eff], 0)
    n_keep = k_eff
    if use_top_p:
        reach = torch.nonzero(cum >= top_p)
        if reach.numel():
            n_keep = min(int(reach[0]) + 1, k_eff)
    return order[:n_keep], cum[:n_keep] / cum[n_keep - 1], logp

