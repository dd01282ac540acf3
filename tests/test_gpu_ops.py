"""GPU parity of every operator of the decode path against the CPU oracle, through the C ABI
(``tilert_b200.models.deepseek_v3_2.ops`` is a thin ctypes layer over ``include/tilert_b200.h``).

Tolerances: floating-point outputs must reach cosine >= 0.999 and relative L2 <= 2e-2 against the
oracle (the thresholds the workload definition states); integer outputs (top-k index sets, routed
expert ids) must be identical.
"""

import json
import os

import pytest
import torch

from oracle import model as om
from oracle import ops as oo
from oracle.quant import act_quant

pytestmark = pytest.mark.gpu

BF16, F32, I32 = torch.bfloat16, torch.float32, torch.int32
COS_MIN, L2_MAX = 0.999, 2e-2


def _metrics(name, ref, out):
    ref, out = ref.float().cpu().flatten(), out.float().cpu().flatten()
    cos = torch.nn.functional.cosine_similarity(ref, out, dim=0).item()
    l2 = (torch.norm(ref - out) / torch.norm(ref).clamp_min(1e-30)).item()
    path = os.environ.get("TB_METRICS")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps({"name": name, "cos": cos, "rel_l2": l2, "n": ref.numel()}) + "\n")
    return cos, l2


def close(name, ref, out, cos_min=COS_MIN, l2_max=L2_MAX):
    assert ref.shape == out.shape, (name, ref.shape, out.shape)
    cos, l2 = _metrics(name, ref, out)
    assert cos >= cos_min and l2 <= l2_max, f"{name}: cosine {cos:.6f}, rel-L2 {l2:.3e}"


@pytest.fixture(scope="module")
def env():
    import tilert_b200
    from tilert_b200.models.deepseek_v3_2 import layer as L
    from tilert_b200.models.deepseek_v3_2 import ops
    from tilert_b200.models.deepseek_v3_2.model_args import toy_model_args

    assert torch.cuda.is_available()
    tilert_b200.load_backend("deepseek_v3_2")
    tilert_b200.tilert_init(0)
    a = om.toy_args()
    sd = om.random_state_dict(a, seed=0)
    e = {
        "tb": tilert_b200, "ops": ops, "L": L, "a": a, "margs": toy_model_args(), "sd": sd,
        "w": [om.LayerWeights(a, sd, 0), om.LayerWeights(a, sd, 1)],
        "gw": [L.LayerWeights(toy_model_args(), sd, li, "cuda") for li in range(2)],
        "fc": oo.precompute_freqs_cis(a),
    }
    yield e
    assert tilert_b200.device_status(0) == 0, "a kernel gave up on a bounded wait"


def rn(gen, *shape, scale=1.0):
    return (torch.randn(*shape, generator=gen, dtype=torch.float32) * scale).to(BF16)


def decode_xpack(xp: torch.Tensor, n_kb: int, cols: int) -> torch.Tensor:
    """Host model of the X-block format: returns f32 [cols, n_kb*128] = e4m3 value * column scale."""
    blk = xp.cpu().view(n_kb, 1056)
    data = blk[:, :1024].reshape(n_kb, 4, 2, 8, 16)            # kb, c, kc, col, b
    vals = data.permute(3, 0, 1, 2, 4).reshape(8, n_kb, 128)     # col, kb, (c, kc, b)
    scales = blk[:, 1024:].contiguous().view(torch.float32).view(n_kb, 8).t()  # col, kb
    f = vals.contiguous().view(torch.float8_e4m3fn).float() * scales[:, :, None]
    return f.reshape(8, n_kb * 128)[:cols]


# ------------------------------------------------------------------------ activation packing
@pytest.mark.parametrize("tokens,dim", [(1, 1024), (2, 7168), (4, 2048)])
def test_act_pack_reproduces_bf16_exactly(env, tokens, dim):
    ops = env["ops"]
    g = torch.Generator().manual_seed(tokens * 1000 + dim)
    x = rn(g, 1, tokens, dim)
    x[0, 0, :128] = 0  # an all-zero block
    xp = ops.new_xpack(dim, "cuda")
    ops.act_pack(x.cuda(), xp)
    d = decode_xpack(xp, dim // 128, 2 * tokens)
    rec = d[0::2] + d[1::2]
    # exact wherever |x| >= 2^-6 of the block scale; below that the absolute error is < 2^-17 of the block maximum
    xf = x[0].float()
    amax = xf.view(tokens, -1, 128).abs().amax(-1, keepdim=True).clamp_min(1e-30)
    rel = ((rec - xf).view(tokens, -1, 128).abs() / amax)
    assert float(rel.max()) < 2 ** -17, float(rel.max())
    assert float((rec == xf).float().mean()) > 0.999


def test_rmsnorm_quant_outputs(env):
    ops, a = env["ops"], env["a"]
    g = torch.Generator().manual_seed(5)
    x = rn(g, 1, 2, a.dim)
    gamma = torch.rand(a.dim, generator=g) + 0.5
    out = torch.empty(1, 2, a.dim, dtype=BF16, device="cuda")
    q = torch.empty(1, 2, a.dim, dtype=torch.float8_e4m3fn, device="cuda")
    s = torch.empty(1, 2, a.dim // 128, dtype=F32, device="cuda")
    xp = ops.new_xpack(a.dim, "cuda")
    ops.rmsnorm_quant(x.cuda(), gamma.cuda(), out, q, s, eps=a.eps, xpack=xp)
    ref = oo.rmsnorm_bf16(x, gamma, a.eps)
    close("rmsnorm.out", ref, out, cos_min=0.99999, l2_max=4e-3)
    # the packed operand is exactly the bf16 output
    d = decode_xpack(xp, a.dim // 128, 4)
    of = out[0].float().cpu()
    amax = of.view(2, -1, 128).abs().amax(-1, keepdim=True)
    assert float((((d[0::2] + d[1::2]) - of).view(2, -1, 128).abs() / amax).max()) < 2 ** -17
    # reference-format 1x128 quantisation of that output
    rq, rs = act_quant(out.cpu())
    close("rmsnorm.qscale", rs, s, cos_min=0.999999, l2_max=1e-5)
    close("rmsnorm.q", rq.float() * rs.repeat_interleave(128, -1), q.float().cpu() * s.cpu().repeat_interleave(128, -1),
          cos_min=0.9999, l2_max=5e-3)


# ------------------------------------------------------------------------------ projections
@pytest.mark.parametrize("tokens", [1, 2])
def test_projx_wqkva_and_indexer_k(env, tokens):
    ops, a, w, gw = env["ops"], env["a"], env["w"][0], env["gw"][0]
    g = torch.Generator().manual_seed(11 + tokens)
    x = rn(g, 1, tokens, a.dim)
    pos = 37
    cur = torch.tensor([pos], dtype=I32, device="cuda")
    q = torch.zeros(1, tokens, a.q_lora_rank, dtype=BF16, device="cuda")
    kv = torch.zeros(1, tokens, a.kv_lora_rank, dtype=BF16, device="cuda")
    ki = torch.zeros(1, tokens, a.index_head_dim, dtype=BF16, device="cuda")
    pe = torch.zeros(1, 64, a.qk_rope_head_dim, dtype=BF16, device="cuda")
    ops.rmsnorm_projx_wqkva(x.cuda(), gw.in_norm, gw.w_qkva, cur, q, kv, pe, ki, eps=a.eps)
    rq, rkv, rpe = oo.projx_wqkva(x, w.in_norm, w.wq_a, w.wkv_a, w.w_pe, a.eps)
    _, rki, rw = oo.projx_wqakis(x, w.in_norm, w.wq_a, w.wki, w.wis, a.eps)
    close("wqkva.q", rq, q)
    close("wqkva.kv", rkv, kv)
    close("wqkva.pe", rpe, pe[:, pos: pos + tokens])
    close("wqkva.ki", rki, ki)
    assert float(pe[:, :pos].abs().max()) == 0 and float(pe[:, pos + tokens:].abs().max()) == 0
    iw = torch.zeros(1, tokens, a.index_n_heads, dtype=BF16, device="cuda")
    ops.projx_wis(x.cuda(), gw.wis, iw, gamma=gw.in_norm, eps=a.eps)
    close("wis", rw, iw)
    # the two-launch form (packed activations prepared by rmsnorm_quant) gives the same result
    xn = torch.empty(1, tokens, a.dim, dtype=BF16, device="cuda")
    xp = ops.new_xpack(a.dim, "cuda")
    ops.rmsnorm_quant(x.cuda(), gw.in_norm, xn, None, None, eps=a.eps, xpack=xp)
    q2, kv2 = torch.zeros_like(q), torch.zeros_like(kv)
    ops.projx_wqkva_packed(xp, 2, gw.w_qkva, tokens, a.dim, a.q_lora_rank, a.kv_lora_rank, a.qk_rope_head_dim,
                           a.index_head_dim, cur, q2, kv2, pe, None)
    close("wqkva.q.packed", rq, q2)
    close("wqkva.kv.packed", rkv, kv2)


def test_projx_wqkva_reference_format_input(env):
    """The reference operator signature: e4m3 activations + 1x128 scales (ops/projx_wqkva.py:22-48)."""
    ops, a, w, gw = env["ops"], env["a"], env["w"][0], env["gw"][0]
    g = torch.Generator().manual_seed(21)
    xn = rn(g, 1, 1, a.dim)
    xq, xs = act_quant(xn)
    q = torch.zeros(1, 1, a.q_lora_rank, dtype=BF16, device="cuda")
    kv = torch.zeros(1, 1, a.kv_lora_rank, dtype=BF16, device="cuda")
    pe = torch.zeros(1, 8, a.qk_rope_head_dim, dtype=BF16, device="cuda")
    cur = torch.tensor([3], dtype=I32, device="cuda")
    ops.projx_wqkva(xq.cuda(), xs.cuda(), gw.w_qkva, cur, q, kv, pe)
    xdq = (xq.float() * xs.repeat_interleave(128, -1))
    close("wqkva_q8.q", (xdq @ w.wq_a.float().T), q, l2_max=1e-2)
    close("wqkva_q8.kv", (xdq @ w.wkv_a.float().T), kv, l2_max=1e-2)
    close("wqkva_q8.pe", (xdq @ w.w_pe.float().T), pe[:, 3:4], l2_max=1e-2)


@pytest.mark.parametrize("tokens", [1, 4])
def test_rmsnorm_proj_q(env, tokens):
    ops, a, w, gw = env["ops"], env["a"], env["w"][0], env["gw"][0]
    g = torch.Generator().manual_seed(31 + tokens)
    qa = rn(g, 1, tokens, a.q_lora_rank)
    q_nope = torch.zeros(1, tokens, a.n_heads, a.qk_nope_head_dim, dtype=BF16, device="cuda")
    q_pe = torch.zeros(1, tokens, a.n_heads, a.qk_rope_head_dim, dtype=BF16, device="cuda")
    iq = torch.zeros(1, tokens, a.index_n_heads, a.index_head_dim, dtype=BF16, device="cuda")
    ops.rmsnorm_proj_q(qa.cuda(), gw.q_norm, gw.w_qb, q_nope, q_pe, iq, eps=a.eps)
    rn_, rp = oo.rmsnorm_projq_wqb(qa, w.q_norm, w.wq_b, a.n_heads, a.qk_nope_head_dim, a.qk_rope_head_dim, a.eps)
    ri = oo.rmsnorm_projq_wqi(qa, w.q_norm, w.wqi, a.index_head_dim, a.eps)
    close("wqb.q_nope", rn_, q_nope)
    close("wqb.q_pe", rp, q_pe)
    close("wqi.iq", ri, iq)


def test_vector_ops(env):
    ops, a, w, gw, fc = env["ops"], env["a"], env["w"][0], env["gw"][0], env["fc"]
    g = torch.Generator().manual_seed(41)
    tokens, pos = 2, 100
    cur = torch.tensor([pos], dtype=I32, device="cuda")
    fr = torch.view_as_real(fc[pos: pos + tokens]).contiguous().cuda()
    f_ref = fc[pos: pos + tokens]
    kv = rn(g, 1, tokens, a.kv_lora_rank)
    gamma = (torch.rand(a.kv_lora_rank, generator=g) + 0.5)
    cache = torch.zeros(1, 128, a.kv_lora_rank, dtype=BF16, device="cuda")
    ops.rmsnorm_kv(kv.cuda(), gamma.cuda(), cur, cache, eps=a.eps)
    close("kvnorm", oo.rmsnorm_kv(kv, gamma, a.eps), cache[:, pos: pos + tokens], cos_min=0.99999, l2_max=4e-3)

    q_pe = rn(g, 1, tokens, a.n_heads, a.qk_rope_head_dim)
    k_pe = rn(g, 1, tokens, a.qk_rope_head_dim)
    pe_cache = torch.zeros(1, 128, a.qk_rope_head_dim, dtype=BF16, device="cuda")
    pe_cache[:, pos: pos + tokens] = k_pe.cuda()
    q_dev = q_pe.cuda()
    ops.qkv_rope(q_dev, pe_cache, fr, cur)
    rq, rk = oo.qkv_rope(q_pe, k_pe, f_ref)
    close("rope.q", rq, q_dev, cos_min=0.99999, l2_max=4e-3)
    close("rope.k", rk, pe_cache[:, pos: pos + tokens], cos_min=0.99999, l2_max=4e-3)

    iq = rn(g, 1, tokens, a.index_n_heads, a.index_head_dim)
    out = torch.zeros_like(iq, device="cuda")
    ops.rotate(iq.cuda(), out, fr)
    close("rotate", oo.rotate(iq, f_ref, a.qk_rope_head_dim), out, cos_min=0.99999, l2_max=6e-3)

    ki = rn(g, 1, tokens, a.index_head_dim)
    lw = torch.rand(128, generator=g) + 0.5
    lb = torch.randn(128, generator=g) * 0.1
    kc = torch.zeros(1, 128, a.index_head_dim, dtype=BF16, device="cuda")
    ops.layernorm_rope_rotate(ki.cuda(), cur, kc, lw.cuda(), lb.cuda(), fr)
    close("lnrr", oo.layernorm_rope_rotate(ki, lw, lb, f_ref, a.qk_rope_head_dim), kc[:, pos: pos + tokens],
          cos_min=0.99999, l2_max=6e-3)


@pytest.mark.parametrize("tokens", [1, 2, 4])
def test_attn_prep_equals_the_separate_operators(env, tokens):
    """The fused launch must give bit-identical results to the five operators it replaces."""
    ops, a, fc = env["ops"], env["a"], env["fc"]
    g = torch.Generator().manual_seed(43 + tokens)
    pos = 77
    cur = torch.tensor([pos], dtype=I32, device="cuda")
    fr = torch.view_as_real(fc[pos: pos + tokens]).contiguous().cuda()
    x = rn(g, 1, tokens, a.dim).cuda()
    in_gamma = (torch.rand(a.dim, generator=g) + 0.5).cuda()
    w_is = (torch.randn(a.index_n_heads, a.dim, generator=g) * 0.05).to(BF16).cuda()
    kv = rn(g, 1, tokens, a.kv_lora_rank).cuda()
    kv_gamma = (torch.rand(a.kv_lora_rank, generator=g) + 0.5).cuda()
    q_pe = rn(g, 1, tokens, a.n_heads, a.qk_rope_head_dim).cuda()
    k_pe = rn(g, 1, tokens, a.qk_rope_head_dim).cuda()
    iq = rn(g, 1, tokens, a.index_n_heads, a.index_head_dim).cuda()
    ki = rn(g, 1, tokens, a.index_head_dim).cuda()
    lw = (torch.rand(128, generator=g) + 0.5).cuda()
    lb = (torch.randn(128, generator=g) * 0.1).cuda()

    def buffers():
        pe = torch.zeros(1, 128, a.qk_rope_head_dim, dtype=BF16, device="cuda")
        pe[:, pos: pos + tokens] = k_pe
        return dict(idx_w=torch.zeros(1, tokens, a.index_n_heads, dtype=BF16, device="cuda"),
                    kvc=torch.zeros(1, 128, a.kv_lora_rank, dtype=BF16, device="cuda"), q=q_pe.clone(), pe=pe,
                    iq_rt=torch.zeros_like(iq), kc=torch.zeros(1, 128, a.index_head_dim, dtype=BF16, device="cuda"))

    r = buffers()
    ops.projx_wis(x, w_is, r["idx_w"], gamma=in_gamma, eps=a.eps)
    ops.rmsnorm_kv(kv, kv_gamma, cur, r["kvc"], eps=a.eps)
    ops.qkv_rope(r["q"], r["pe"], fr, cur)
    ops.rotate(iq, r["iq_rt"], fr)
    ops.layernorm_rope_rotate(ki, cur, r["kc"], lw, lb, fr)
    f = buffers()
    ops.attn_prep(x, in_gamma, w_is, f["idx_w"], kv, kv_gamma, f["kvc"], f["q"], f["pe"], iq, f["iq_rt"], ki, f["kc"],
                  lw, lb, fr, cur, eps=a.eps)
    torch.cuda.synchronize()
    for k in r:
        assert torch.equal(r[k], f[k]), k
    assert r["idx_w"].float().abs().max() > 0


# ---------------------------------------------------------------------- indexer and top-k
@pytest.mark.parametrize("heads,t_len,tokens", [(16, 300, 1), (64, 1000, 2), (32, 64, 1)])
def test_indexer_logits(env, heads, t_len, tokens):
    ops = env["ops"]
    g = torch.Generator().manual_seed(heads + t_len)
    q = rn(g, 1, tokens, heads, 128)
    k = rn(g, 1, t_len, 128)
    w = rn(g, 1, tokens, heads, scale=0.5)
    n_valid = t_len - 5
    cur = torch.tensor([n_valid - tokens], dtype=I32, device="cuda")
    logits = torch.zeros(1, tokens, t_len + 8, dtype=F32, device="cuda")
    ops.sparse_index(q.cuda(), k.cuda(), w.cuda(), logits, cur, n_keys=t_len)
    ref = oo.indexer_logits(q, k[:, :t_len], w, n_valid)
    got = logits[..., :t_len].cpu()
    fin = torch.isfinite(ref)
    assert torch.equal(torch.isinf(got) & (got < 0), ~fin)
    close("indexer.logits", ref[fin], got[fin], cos_min=0.99999, l2_max=1e-3)


def _topk_case(env, logits, n, k):
    ops = env["ops"]
    got = ops.topk_accurate(logits.cuda().contiguous(), n, k).cpu()
    ref = oo.topk_indices(logits[..., :n], k).view(-1, k)
    assert torch.equal(got, ref), (got[0, :10], ref[0, :10])


def test_topk_exact_random(env):
    g = torch.Generator().manual_seed(7)
    _topk_case(env, torch.randn(1, 2, 5000, generator=g), 5000, 256)
    _topk_case(env, torch.randn(1, 1, 20000, generator=g), 19990, 2048)
    # row lengths on both sides of the register-resident kernels' limits (4096 and 8192 entries)
    for n in (4095, 4096, 4097, 8191, 8192, 8193):
        _topk_case(env, torch.randn(1, 2, n, generator=g), n, 2048)


def test_topk_ties_infs_and_short_rows(env):
    g = torch.Generator().manual_seed(8)
    x = torch.randint(0, 6, (1, 3, 3000), generator=g).float()          # heavy ties
    x[0, 1, 100:2000] = float("-inf")
    _topk_case(env, x, 3000, 512)
    y = torch.randn(1, 1, 300, generator=g)                               # fewer entries than k
    y[0, 0, 200:] = float("-inf")
    _topk_case(env, y, 300, 256)
    z = torch.full((1, 1, 4096), 1.5)                                     # all equal: lowest indices win
    _topk_case(env, z, 4096, 2048)
    neg = -torch.rand(1, 1, 4096, generator=g) - 1e-3                     # negative values and -0.0
    neg[0, 0, 5] = -0.0
    _topk_case(env, neg, 4096, 1024)


def test_indexer_plus_topk_matches_oracle_selection(env):
    ops = env["ops"]
    g = torch.Generator().manual_seed(9)
    q, k, w = rn(g, 1, 1, 16, 128), rn(g, 1, 1500, 128), rn(g, 1, 1, 16, scale=0.5)
    cur = torch.tensor([1499], dtype=I32, device="cuda")
    logits = torch.zeros(1, 1, 1536, dtype=F32, device="cuda")
    sel = torch.zeros(1, 1, 256, dtype=I32, device="cuda")
    ops.sparse_index_topk(q.cuda(), k.cuda(), w.cuda(), logits, sel, cur, n_keys=1500)
    # bit-exact given identical scores: select on the kernel's own logits with the oracle's rule
    ref = oo.topk_indices(logits[..., :1500].cpu(), 256)
    assert torch.equal(sel.cpu(), ref)


@pytest.mark.parametrize("heads,t_len,tokens,k,distinct", [
    (16, 300, 1, 256, 0), (32, 4096, 2, 2048, 0), (64, 5000, 4, 2048, 37), (64, 40000, 1, 2048, 0),
    (64, 40000, 3, 2048, 500), (16, 2048, 1, 2048, 0), (64, 37888, 8, 512, 3)])
def test_indexer_plus_topk_cooperative_selection(env, heads, t_len, tokens, k, distinct):
    """The one-launch scoring + selection on rows long enough for several thread blocks per token, with
    repeated key vectors (``distinct`` > 0: exact ties that straddle the blocks' key ranges, so the lowest
    positions must win across blocks), masked tails and several tokens; run twice back to back, because the
    launch clears its own histograms and counters for the next one."""
    ops = env["ops"]
    g = torch.Generator().manual_seed(heads * 7 + t_len + tokens)
    q, w = rn(g, 1, tokens, heads, 128), rn(g, 1, tokens, heads, scale=0.5)
    if distinct:
        base = rn(g, distinct, 128)
        kc = base[torch.randint(0, distinct, (t_len,), generator=g)][None]
    else:
        kc = rn(g, 1, t_len, 128)
    n_valid = t_len - 3                       # the newest token sees keys 0 .. n_valid - 1
    cur = torch.tensor([n_valid - tokens], dtype=I32, device="cuda")
    stride = (t_len + 8 + 3) // 4 * 4
    qd, kd, wd = q.cuda(), kc.cuda(), w.cuda()
    for _ in range(2):
        logits = torch.zeros(1, tokens, stride, dtype=F32, device="cuda")
        sel = torch.zeros(1, tokens, k, dtype=I32, device="cuda")
        ops.sparse_index_topk(qd, kd, wd, logits, sel, cur, n_keys=t_len)
        got_logits = logits[..., :t_len].cpu()
        ref_logits = oo.indexer_logits(q, kc, w, n_valid)
        fin = torch.isfinite(ref_logits)
        assert torch.equal(torch.isinf(got_logits) & (got_logits < 0), ~fin)
        close("indexer.coop.logits", ref_logits[fin], got_logits[fin], cos_min=0.99999, l2_max=1e-3)
        assert torch.equal(sel.cpu(), oo.topk_indices(got_logits, k))


def test_dsa_stress_128k_context(env):
    """Long-context stress case: one query against 131072 cached keys (64 indexer heads), exact
    top-2048, then sparse MLA over the selected rows.  Synthetic N(0,1) keys stand in for a real cache."""
    ops, a = env["ops"], env["a"]
    g = torch.Generator().manual_seed(131072)
    t_len, heads, topk = 131072, 64, 2048
    q, w = rn(g, 1, 1, heads, 128), rn(g, 1, 1, heads, scale=0.5)
    k = torch.randn(1, t_len, 128, generator=g, dtype=F32).to(BF16)
    cur = torch.tensor([t_len - 1], dtype=I32, device="cuda")
    logits = torch.zeros(1, 1, t_len + 8, dtype=F32, device="cuda")
    sel = torch.zeros(1, 1, topk, dtype=I32, device="cuda")
    ops.sparse_index_topk(q.cuda(), k.cuda(), w.cuda(), logits, sel, cur, n_keys=t_len)
    torch.cuda.synchronize()
    got_logits = logits[..., :t_len].cpu()
    ref_logits = oo.indexer_logits(q, k, w, t_len)
    close("c3.logits", ref_logits, got_logits, cos_min=0.99999, l2_max=1e-3)
    # integer part: bit-exact given identical scores; against the oracle's scores only near-ties may differ
    assert torch.equal(sel.cpu(), oo.topk_indices(got_logits, topk))
    ref_sel = oo.topk_indices(ref_logits, topk)
    overlap = len(set(sel.view(-1).tolist()) & set(ref_sel.view(-1).tolist())) / topk
    assert overlap >= 0.995, overlap
    # sparse attention over the device's selection (16 heads keep the CPU oracle to seconds)
    mh = 16
    ql, qp = rn(g, 1, 1, mh, 512, scale=0.3), rn(g, 1, 1, mh, 64)
    kvc = torch.randn(1, t_len, 512, generator=g, dtype=F32).to(BF16)
    pec = torch.randn(1, t_len, 64, generator=g, dtype=F32).to(BF16)
    o = torch.zeros(1, 1, mh, 512, dtype=BF16, device="cuda")
    ops.flash_sparse_mla(ql.cuda(), qp.cuda(), kvc.cuda(), pec.cuda(), sel, cur, o, softmax_scale=oo.softmax_scale(a))
    sel_cpu = sel.cpu()
    rows = sel_cpu.view(-1).long()
    # the oracle scores every cached row; restrict it to the selected rows (re-indexed) to keep it small
    sub_sel = torch.arange(topk, dtype=I32).view(1, 1, topk)
    ref = oo.flash_sparse_mla(ql, qp, kvc[:, rows], pec[:, rows], sub_sel, topk - 1, oo.softmax_scale(a))
    close("c3.mla", ref, o)


# ------------------------------------------------------------------ attention-side products
def test_absorb_attention_vproj_oproj(env):
    ops, a, w, gw = env["ops"], env["a"], env["w"][0], env["gw"][0]
    g = torch.Generator().manual_seed(51)
    tokens, t_len, pos = 2, 700, 650
    q_nope = rn(g, 1, tokens, a.n_heads, a.qk_nope_head_dim)
    q_lat = torch.zeros(1, tokens, a.n_heads, a.kv_lora_rank, dtype=BF16, device="cuda")
    ops.projq_wqb(q_nope.cuda(), gw.w_absorb, None, q_lat)
    close("absorb", oo.projq_wqb_absorb(q_nope, w.wkv_b_nope), q_lat)

    ql = rn(g, 1, tokens, a.n_heads, a.kv_lora_rank, scale=0.3)
    qp = rn(g, 1, tokens, a.n_heads, a.qk_rope_head_dim)
    kvc, pec = rn(g, 1, t_len, a.kv_lora_rank), rn(g, 1, t_len, a.qk_rope_head_dim)
    sel = torch.full((1, tokens, a.index_topk), -1, dtype=I32)
    for s in range(tokens):
        pick = torch.sort(torch.randperm(pos + s + 1, generator=g)[:200])[0]
        sel[0, s, :200] = pick.to(I32)
    cur = torch.tensor([pos], dtype=I32, device="cuda")
    o_lat = torch.zeros(1, tokens, a.n_heads, a.kv_lora_rank, dtype=BF16, device="cuda")
    ops.flash_sparse_mla(ql.cuda(), qp.cuda(), kvc.cuda(), pec.cuda(), sel.cuda(), cur, o_lat,
                         softmax_scale=oo.softmax_scale(a))
    ref = oo.flash_sparse_mla(ql, qp, kvc, pec, sel, pos, oo.softmax_scale(a))
    close("mla", ref, o_lat)

    ol = rn(g, 1, tokens, a.n_heads, a.kv_lora_rank)
    o = torch.zeros(1, tokens, a.n_heads, a.v_head_dim, dtype=BF16, device="cuda")
    ops.projo_wkvb(ol.cuda(), gw.w_v, None, o)
    close("vproj", oo.projo_wkvb(ol, w.wkv_b_v), o)

    ov = rn(g, 1, tokens, a.n_heads, a.v_head_dim)
    res = rn(g, 1, tokens, a.dim)
    h = torch.zeros(1, tokens, a.dim, dtype=BF16, device="cuda")
    ops.unproj_o_allreduce(ov.cuda(), gw.w_o, None, res.cuda(), 0, h)
    close("oproj+res", (oo.unproj_o(ov, w.w_o).float() + res.float()).to(BF16), h)


def test_mla_full_topk_and_masking(env):
    """2048 selected rows (32 chunks), indices beyond the causal limit and -1 padding are ignored."""
    ops, a = env["ops"], env["a"]
    g = torch.Generator().manual_seed(52)
    heads, t_len, pos, topk = 16, 4096, 3000, 2048
    ql, qp = rn(g, 1, 1, heads, 512, scale=0.3), rn(g, 1, 1, heads, 64)
    kvc, pec = rn(g, 1, t_len, 512), rn(g, 1, t_len, 64)
    sel = torch.sort(torch.randperm(t_len, generator=g)[:topk])[0].to(I32).view(1, 1, topk)
    cur = torch.tensor([pos], dtype=I32, device="cuda")
    o = torch.zeros(1, 1, heads, 512, dtype=BF16, device="cuda")
    ops.flash_sparse_mla(ql.cuda(), qp.cuda(), kvc.cuda(), pec.cuda(), sel.cuda(), cur, o,
                         softmax_scale=oo.softmax_scale(a))
    sel_ref = sel.clone()
    sel_ref[sel_ref > pos] = -1
    close("mla.2048", oo.flash_sparse_mla(ql, qp, kvc, pec, sel_ref, pos, oo.softmax_scale(a)), o)


@pytest.mark.parametrize("heads,topk,tokens", [(16, 384, 1), (32, 320, 2), (16, 64, 1), (128, 2048, 1), (48, 1024, 4)])
def test_mla_chunk_counts_head_groups_and_tokens(env, heads, topk, tokens):
    """Odd and even chunk counts (6, 5, 1, 32, 16 chunks of 64 rows), several head groups and tokens, padding inside
    the last chunk, the log-sum-exp output; run twice."""
    ops, a = env["ops"], env["a"]
    g = torch.Generator().manual_seed(heads + topk + tokens)
    t_len = 3000
    pos = t_len - tokens
    ql, qp = rn(g, 1, tokens, heads, 512, scale=0.3), rn(g, 1, tokens, heads, 64)
    kvc, pec = rn(g, 1, t_len, 512), rn(g, 1, t_len, 64)
    sel = torch.stack([torch.sort(torch.randperm(pos + 1, generator=g)[:topk])[0] for _ in range(tokens)]).to(I32)
    sel = sel.view(1, tokens, topk)
    sel[0, 0, -7:] = -1                                   # padding inside the last chunk
    cur = torch.tensor([pos], dtype=I32, device="cuda")
    ref = oo.flash_sparse_mla(ql, qp, kvc, pec, sel, pos, oo.softmax_scale(a))
    for _ in range(2):
        o = torch.zeros(1, tokens, heads, 512, dtype=BF16, device="cuda")
        lse = torch.zeros(1, tokens, heads, dtype=F32, device="cuda")
        ops.flash_sparse_mla(ql.cuda(), qp.cuda(), kvc.cuda(), pec.cuda(), sel.cuda(), cur, o,
                             softmax_scale=oo.softmax_scale(a), lse=lse)
        close(f"mla.{heads}.{topk}", ref, o)
        assert torch.isfinite(lse).all()


# ------------------------------------------------------------------------------- MoE / FFN
def test_router_and_expert_path(env):
    ops, a, w, gw = env["ops"], env["a"], env["w"][1], env["gw"][1]
    g = torch.Generator().manual_seed(61)
    tokens = 2
    h = rn(g, 1, tokens, a.dim)
    hn = torch.zeros(1, tokens, a.dim, dtype=BF16, device="cuda")
    scores = torch.zeros(1, tokens, a.n_routed_experts, dtype=F32, device="cuda")
    ops.rmsnorm_expert_proj(h.cuda(), gw.post_norm, gw.router, scores, hn, eps=a.eps)
    rhn, rsc = oo.rmsnorm_expert_proj(h, w.post_norm, w.router, a.eps)
    close("router.hn", rhn, hn, cos_min=0.99999, l2_max=4e-3)
    close("router.scores", rsc.view(1, tokens, -1), scores, cos_min=0.9999, l2_max=5e-3)

    n_slots = a.n_activated_experts + 1
    hid = torch.zeros(1, tokens, n_slots, a.moe_inter_dim, dtype=BF16, device="cuda")
    probs = torch.zeros(1, tokens, a.n_activated_experts, dtype=F32, device="cuda")
    eidx = torch.zeros(1, tokens, a.n_activated_experts, dtype=I32, device="cuda")
    slot_ids = torch.zeros(tokens, n_slots, dtype=I32, device="cuda")
    slot_w = torch.zeros(tokens, n_slots, dtype=F32, device="cuda")
    ops.expert_select_up_gate_silu(hn, scores, gw.router_bias, gw.w_gu, hid, probs, eidx, dim=a.dim, n_groups=1,
                                   n_limited_groups=1, route_scale=a.route_scale, slot_ids=slot_ids, slot_w=slot_w)
    rp, ri = oo.expert_select_ds(scores.cpu(), w.router_bias, 1, 1, a.n_activated_experts, a.route_scale)
    assert torch.equal(ri.to(I32), eidx.cpu())
    close("route.probs", rp, probs, cos_min=0.999999, l2_max=1e-5)
    gl, ul, dl = [], [], []
    for s in range(tokens):
        trip = [w.expert(n) for n in ["shared_experts"] + [f"experts.{int(e)}" for e in ri[0, s]]]
        gl.append([t[0] for t in trip]); ul.append([t[1] for t in trip]); dl.append([t[2] for t in trip])
    rhid = oo.expert_up_gate_silu(hn.cpu(), gl, ul)
    close("experts.hidden", rhid, hid)

    out = torch.zeros(1, tokens, a.dim, dtype=BF16, device="cuda")
    ops.expert_down_allreduce(hid, gw.w_down, None, eidx, probs, h.cuda(), 0, out, slot_ids=slot_ids, slot_w=slot_w)
    rdown = oo.expert_down(hid.cpu(), dl, probs.cpu())
    close("experts.down+res", (rdown.float() + h.float()).to(BF16), out)

    # the same pair through the reference's dispatcher names and argument order: identical bytes; the down
    # product rebuilds the slot table from the routed indices and weights the reference passes
    from tilert_b200 import torch_ops

    torch_ops.register()
    hid2, probs2, eidx2, out2 = torch.zeros_like(hid), torch.zeros_like(probs), torch.zeros_like(eidx), torch.zeros_like(out)
    torch.ops.tilert.expert_select_up_gate_silu_op(hn, scores, gw.router_bias, gw.w_gu, hid2, probs2, eidx2, None,
                                                   "deepseek_v3_2", "fp8mma", 1, 1, a.route_scale)
    assert torch.equal(hid, hid2) and torch.equal(eidx, eidx2) and torch.equal(probs, probs2)
    torch.ops.tilert.expert_down_allreduce_op(hid2, gw.w_down, None, eidx2, probs2, h.cuda(), 0, out2, None,
                                              "deepseek_v3_2", "fp8mma")
    assert torch.equal(out, out2)


def test_grouped_routing_full_shape(env):
    """256 experts in 8 groups, 4 groups kept, top-8 -- checked through the up/gate operator with a
    weight stack of zeros (only the routing outputs are compared)."""
    ops = env["ops"]
    g = torch.Generator().manual_seed(62)
    tokens, dim, inter = 3, 256, 64
    scores = torch.randn(1, tokens, 256, generator=g)
    bias = torch.randn(256, generator=g) * 0.1
    w = torch.zeros(257, 1, dim // 128, 16448, dtype=torch.uint8, device="cuda")
    xp = torch.zeros(1, tokens, dim, dtype=BF16, device="cuda")
    hid = torch.zeros(1, tokens, 9, inter, dtype=BF16, device="cuda")
    probs = torch.zeros(1, tokens, 8, dtype=F32, device="cuda")
    eidx = torch.zeros(1, tokens, 8, dtype=I32, device="cuda")
    ops.expert_select_up_gate_silu(xp, scores.cuda(), bias.cuda(), w, hid, probs, eidx, dim=dim, n_groups=8,
                                   n_limited_groups=4, route_scale=2.5)
    rp, ri = oo.expert_select_ds(scores, bias, 8, 4, 8, 2.5)
    assert torch.equal(ri.to(I32), eidx.cpu())
    close("route8.probs", rp, probs, cos_min=0.999999, l2_max=1e-5)


def test_dense_ffn(env):
    ops, a, w, gw = env["ops"], env["a"], env["w"][0], env["gw"][0]
    g = torch.Generator().manual_seed(71)
    h = rn(g, 1, 1, a.dim)
    hid = torch.zeros(1, 1, a.inter_dim, dtype=BF16, device="cuda")
    ops.rmsnorm_up_gate_silu(h.cuda(), gw.post_norm, gw.w_gu, hid, eps=a.eps)
    rh = oo.dense_up_gate_silu(h, w.post_norm, w.w_gate, w.w_up, a.eps)
    close("dense.hidden", rh, hid)
    out = torch.zeros(1, 1, a.dim, dtype=BF16, device="cuda")
    ops.down_allreduce(hid, gw.w_down, None, h.cuda(), 0, out)
    rd = oo.dense_down(hid.cpu(), w.w_down, a.inter_dim // a.moe_inter_dim)
    close("dense.down+res", (rd.float() + h.float()).to(BF16), out)


def test_head(env):
    ops, a, sd = env["ops"], env["a"], env["sd"]
    g = torch.Generator().manual_seed(81)
    x = rn(g, 1, 2, a.dim)
    logits = torch.zeros(1, 2, a.vocab_size, dtype=F32, device="cuda")
    ops.rmsnorm_head_proj(x.cuda(), sd["model.norm.weight"].cuda(), sd["lm_head.weight"].cuda(), None, logits,
                          eps=a.eps)
    close("head", oo.rmsnorm_head_proj(x, sd["model.norm.weight"], sd["lm_head.weight"], a.eps), logits,
          cos_min=0.99999, l2_max=2e-3)


@pytest.mark.parametrize("tokens", [1, 2, 4])
def test_mtp_preprocess_and_eh_proj(env, tokens):
    ops, a = env["ops"], env["a"]
    g = torch.Generator().manual_seed(91 + tokens)
    e, h = rn(g, 1, tokens, a.dim), rn(g, 1, tokens, a.dim, scale=2.0)
    ge, gh = torch.rand(a.dim, generator=g) + 0.5, torch.rand(a.dim, generator=g) + 0.5
    w = rn(g, a.dim, 2 * a.dim, scale=0.03)
    e_ref, h_ref, out_ref = oo.mtp_preprocess(e, h, ge, gh, w, a.eps)
    out = torch.zeros(1, tokens, a.dim, dtype=BF16, device="cuda")
    en, hn = torch.zeros_like(out), torch.zeros_like(out)
    ops.mtp_preprocess(e.cuda(), h.cuda(), ge.cuda(), gh.cuda(), w.cuda(), out, eps=a.eps, e_norm_out=en, h_norm_out=hn)
    close("mtp.enorm", e_ref, en, cos_min=0.99999, l2_max=4e-3)
    close("mtp.hnorm", h_ref, hn, cos_min=0.99999, l2_max=4e-3)
    close("mtp.out", out_ref, out, cos_min=0.9999, l2_max=8e-3)
    out2 = torch.zeros_like(out)
    ops.eh_proj_allreduce(e_ref.cuda(), h_ref.cuda(), w.cuda(), 0, out2)
    close("eh_proj", oo.eh_proj(e_ref, h_ref, w), out2, cos_min=0.9999, l2_max=8e-3)


def test_padded_allreduce_add_single_rank(env):
    """Without a communicator the stand-alone all-reduce + residual add is partial + x_in, through the C ABI wrapper
    and through the reference's dispatcher name."""
    ops = env["ops"]
    g = torch.Generator().manual_seed(77)
    for tokens in (1, 4):
        part, x = rn(g, 1, tokens, 7168), rn(g, 1, tokens, 7168, scale=2.0)
        out = torch.zeros(1, tokens, 7168, dtype=BF16, device="cuda")
        ops.padded_allreduce_add(part.cuda(), x.cuda(), 0, out)
        ref = (part.float() + x.float()).to(BF16)
        assert torch.equal(out.cpu(), ref)
        from tilert_b200 import torch_ops

        torch_ops.register()
        out2 = torch.zeros_like(out)
        torch.ops.tilert.padded_allreduce_add_op(part.cuda(), x.cuda(), 0, out2, None, "deepseek_v3_2", "bf16")
        assert torch.equal(out2.cpu(), ref)


def test_torch_ops_namespace_calls_reach_the_kernels(env):
    """A reference-style call through torch.ops.tilert gives the same bytes as the direct wrapper."""
    from tilert_b200 import torch_ops

    torch_ops.register()
    ops, a = env["ops"], env["a"]
    g = torch.Generator().manual_seed(77)
    cur = torch.tensor([5], dtype=I32, device="cuda")
    kv = rn(g, 1, 2, a.kv_lora_rank).cuda()
    gamma = (torch.rand(a.kv_lora_rank, generator=g) + 0.5).cuda()
    c1 = torch.zeros(1, 16, a.kv_lora_rank, dtype=BF16, device="cuda")
    c2 = torch.zeros_like(c1)
    ops.rmsnorm_kv(kv, gamma, cur, c1, eps=1e-6)
    torch.ops.tilert.rmsnorm_kv_op(kv, gamma, cur, c2, "deepseek_v3_2", "bf16", None)
    assert torch.equal(c1, c2) and c1.float().abs().max() > 0
    logits = torch.randn(1, 1, 3000, generator=g).cuda()
    idx = torch.zeros(1, 256, dtype=I32, device="cuda")
    torch.ops.tilert.topk_accurate_op(logits, idx, 3000, None, "deepseek_v3_2", "bf16", None, 1)
    assert torch.equal(idx.cpu(), oo.topk_indices(logits.cpu(), 256).view(1, 256))


def test_sampling_matches_the_restated_rule(env):
    """Greedy, top-k, top-p and plain temperature sampling over a vocabulary-sized row: the kernel's
    token must be the one the float64 restatement assigns to the same uniform number (a token whose
    cumulative interval the number misses by less than 1e-4 is accepted: f32 vs f64 sums)."""
    ops = env["ops"]
    g = torch.Generator().manual_seed(404)
    vocab, tokens = 129280, 3
    logits = (torch.randn(tokens, vocab, generator=g) * 2.5)
    logits[0, 777] = 30.0                                  # a dominant token
    logits[1, 5] = logits[1, 9] = logits[1].max() + 1.0    # an exact tie at the top
    dev_logits = logits.cuda()
    tok = torch.zeros(tokens, dtype=I32, device="cuda")
    lp = torch.zeros(tokens, dtype=F32, device="cuda")
    tn_lp = torch.zeros(tokens, 256, dtype=F32, device="cuda")
    tn_ix = torch.zeros(tokens, 256, dtype=I32, device="cuda")
    for cfg, seed, step in [((0.0, 1.0, 0.0, 0.0), 1, 0), ((1.0, 1.0, 50.0, 0.0), 2, 3), ((0.7, 0.9, 0.0, 1.0), 3, 11),
                            ((1.3, 0.5, 40.0, 1.0), 4, 12345), ((1.0, 1.0, 0.0, 0.0), 5, 7)]:
        config = torch.tensor(cfg, dtype=F32, device="cuda")
        ops.sample(dev_logits, config, tok, seed=seed, step_value=step, token_logprob=lp, topn_logprobs=tn_lp,
                   topn_indices=tn_ix)
        torch.cuda.synchronize()
        for t in range(tokens):
            ids, bounds, logp = oo.sample_intervals(logits[t], cfg[0], cfg[1], int(cfg[2]), cfg[3] != 0)
            got = int(tok[t])
            if cfg[0] == 0.0:
                assert got == int(ids[0]), (cfg, t)
            else:
                u = oo.sample_uniform(seed, step, t)
                pos = (ids == got).nonzero()
                assert pos.numel() == 1, (cfg, t, got)
                j = int(pos[0])
                lo = float(bounds[j - 1]) if j > 0 else 0.0
                assert lo - 1e-4 <= u < float(bounds[j]) + 1e-4, (cfg, t, got, u, lo, float(bounds[j]))
            order = torch.argsort(-logits[t].double(), stable=True)
            assert torch.equal(tn_ix[t].cpu().long(), order[:256])
            assert torch.allclose(tn_lp[t].cpu().double(), logp[:256], atol=2e-4)
            assert abs(float(lp[t]) - float(logp[(order[:1024] == got).nonzero()[0]])) < 2e-4
    # a device step counter makes identical launches draw different numbers (what a replayed graph needs)
    step = torch.zeros(2, dtype=torch.int64, device="cuda")
    config = torch.tensor((1.0, 1.0, 0.0, 0.0), dtype=F32, device="cuda")
    flat = torch.zeros(1, 4096, dtype=F32, device="cuda")  # uniform distribution: the token tracks u
    seen = set()
    one = torch.zeros(1, dtype=I32, device="cuda")
    for i in range(6):
        ops.sample(flat, config, one, seed=9, step=step)
        torch.cuda.synchronize()
        assert int(step[0]) == i + 1 and int(step[1]) == 0
        expect = int(oo.sample_uniform(9, i, 0) * 1024)  # candidates = ids 0..1023, each 1/1024
        assert abs(int(one[0]) - expect) <= 1
        seen.add(int(one[0]))
    assert len(seen) >= 5


def test_argmax_exchange_single_rank_is_exact(env):
    """Without a communicator the exchange operator is a plain arg-max: exact, lowest index on ties,
    offset added (the cross-rank part is checked by the multi-GPU run)."""
    ops = env["ops"]
    g = torch.Generator().manual_seed(91)
    for vocab, tokens in ((4096, 1), (129280, 4), (1000, 2)):
        logits = torch.randn(1, tokens, vocab, generator=g, dtype=F32)
        logits[0, 0, 17] = logits[0, 0, vocab - 5] = 9.5          # a tie at the maximum
        tok = torch.zeros(tokens, dtype=torch.int64, device="cuda")
        val = torch.zeros(tokens, dtype=F32, device="cuda")
        ops.argmax_exchange(logits.cuda(), 1000, tok, val)
        ref = torch.argmax(logits[0], dim=-1)
        assert tok.cpu().tolist() == (ref + 1000).tolist() and int(tok[0]) == 1017
        assert torch.equal(val.cpu(), logits[0].max(dim=-1).values)


def test_inject_cache_fp8_wire_format(env):
    """Caches injected from the FP8 wire format: the latent rows are bit-exact against the oracle (and so
    against the reference's dequantiser, which the oracle is pinned to), the rope rows are copied, the
    indexer keys match after the Hadamard rotation (f32 butterfly here, f32 matrix product there); rows
    outside [start_pos, start_pos + seq) stay untouched; ragged lengths and an empty injection work."""
    from oracle import cache_format as cf

    ops = env["ops"]
    g = torch.Generator().manual_seed(33)
    for seq, start in ((150, 0), (64, 7), (1, 300), (0, 5)):
        kv = (torch.randn(seq, 512, generator=g) * 1.7).to(BF16)
        pe = torch.randn(seq, 64, generator=g).to(BF16)
        ki = torch.randn(seq, 128, generator=g).to(BF16)
        kv_raw, ki_pages = cf.quant_kv(kv), cf.quant_ki_pages(ki)
        pe_raw = pe.contiguous().view(torch.uint8).view(seq, 128)
        rows = 512
        kc = torch.full((1, rows, 512), 3.0, dtype=BF16, device="cuda")
        pc = torch.full((1, rows, 64), 3.0, dtype=BF16, device="cuda")
        ic = torch.full((1, rows, 128), 3.0, dtype=BF16, device="cuda")
        ops.inject_cache_fp8(kv_raw.cuda(), pe_raw.cuda(), ki_pages.cuda(), seq, start, kc, pc, ic)
        torch.cuda.synchronize()
        if seq:
            assert torch.equal(kc[0, start: start + seq].cpu().view(torch.int16), cf.dequant_kv(kv_raw, seq).view(torch.int16))
            assert torch.equal(pc[0, start: start + seq].cpu().view(torch.int16), pe.view(torch.int16))
            ref_ki = cf.dequant_ki(ki_pages, seq).float()
            got_ki = ic[0, start: start + seq].float().cpu()
            assert (got_ki - ref_ki).abs().max() <= 2.0 ** -7 * ref_ki.abs().max()
        for c in (kc, pc, ic):
            assert (c[0, :start] == 3.0).all() and (c[0, start + seq:] == 3.0).all()
    with pytest.raises(env["tb"].TilertError):
        ops.inject_cache_fp8(torch.zeros(4, 528, dtype=torch.uint8, device="cuda"), None, None, 4, 510,
                             torch.zeros(1, 512, 512, dtype=BF16, device="cuda"), None, None)


def test_cache_row_past_the_cache_is_not_written(env):
    """The position is device-resident, so the kernels themselves check it against the cache's rows: a row
    at or past the end is not stored and the status word reports a bad argument (4)."""
    ops, a, w = env["ops"], env["a"], env["gw"][0]
    g = torch.Generator().manual_seed(77)
    rows = 16
    kv = rn(g, 1, 1, a.kv_lora_rank).cuda()
    cache = torch.zeros(1, rows, a.kv_lora_rank, dtype=BF16, device="cuda")
    guard = torch.zeros(1, 4, a.kv_lora_rank, dtype=BF16, device="cuda")  # what an unchecked store at row 16.. would hit
    # a view of a larger buffer, so that the row just past the cache is memory this test owns
    buf = torch.zeros(1, rows + 4, a.kv_lora_rank, dtype=BF16, device="cuda")
    cache = buf[:, :rows]
    for pos, want_status in ((rows - 1, 0), (rows, 4), (rows + 2, 4)):
        buf.zero_()
        cur = torch.tensor([pos], dtype=I32, device="cuda")
        ops.rmsnorm_kv(kv, w.kv_norm, cur, cache, eps=a.eps)
        torch.cuda.synchronize()
        assert env["tb"].device_status(0) == want_status
        written = buf[0].float().abs().sum(dim=-1).nonzero().flatten().tolist()
        assert written == ([pos] if want_status == 0 else []), (pos, written)
    del guard


def test_bad_arguments_raise(env):
    ops = env["ops"]
    with pytest.raises(ValueError):
        ops.rotate(torch.zeros(1, 1, 4, 64, dtype=BF16, device="cuda"), torch.zeros(1, 1, 4, 64, dtype=BF16, device="cuda"),
                   torch.zeros(1, 32, 2, device="cuda"))
    with pytest.raises(ValueError):
        ops.topk_accurate(torch.zeros(1, 1, 100, dtype=BF16, device="cuda"), 100, 16)
    with pytest.raises(ValueError):
        ops.rmsnorm_kv(torch.zeros(1, 1, 512), torch.ones(512), torch.zeros(1, dtype=I32), torch.zeros(1, 8, 512))
    with pytest.raises(env["tb"].TilertError):
        ops.flash_sparse_mla(torch.zeros(1, 1, 16, 512, dtype=BF16, device="cuda"),
                             torch.zeros(1, 1, 16, 64, dtype=BF16, device="cuda"),
                             torch.zeros(1, 64, 512, dtype=BF16, device="cuda"),
                             torch.zeros(1, 64, 64, dtype=BF16, device="cuda"),
                             torch.zeros(1, 1, 64, dtype=I32, device="cuda"), torch.zeros(1, dtype=I32, device="cuda"),
                             torch.zeros(1, 1, 16, 512, dtype=BF16, device="cuda"), softmax_scale=0.1, split_size=48)
