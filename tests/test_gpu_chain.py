"""Chained launches (``ops.chain``): several dependent FP8 products recorded and run as the phases of
one persistent kernel must give what the same operators give as separate launches -- bit for bit
where the arithmetic is the same (the streaming products keep their partition and summation order),
within 1e-6 where a bf16 row product runs as a hook with another K split."""

import pytest
import torch

from oracle import model as om
from oracle import ops as oo

pytestmark = pytest.mark.gpu
BF16, F32, I32 = torch.bfloat16, torch.float32, torch.int32


@pytest.fixture(scope="module")
def tb():
    import tilert_b200

    tilert_b200.load_backend("deepseek_v3_2")
    tilert_b200.tilert_init(0)
    yield tilert_b200
    assert tilert_b200.device_status(0) == 0, "a kernel gave up on a bounded wait"


def _rand_packed(gen, n, k):
    """Random packed weight [n/128, k/128, 16448]: e4m3 bytes (finite codes) and small positive scales."""
    w = torch.randint(0, 120, (n // 128, k // 128, 16448), generator=gen, dtype=torch.uint8, device="cuda")
    sign = torch.randint(0, 2, (n // 128, k // 128, 16384), generator=gen, dtype=torch.uint8, device="cuda") * 128
    w[:, :, :16384] += sign
    w[:, :, 16384:] = 0
    w[:, :, 16384:].view(F32).copy_(torch.rand(n // 128, k // 128, 16, generator=gen, device="cuda") * 2e-3 + 1e-3)
    return w


@pytest.mark.parametrize("tokens", [1, 4])
@pytest.mark.parametrize("shape", [(1024, 2304, 1024), (4096, 7168, 2048), (512, 128, 256)])
def test_three_chained_products_equal_separate_launches(tb, shape, tokens):
    """x -> RMSNorm -> A -> RMSNorm -> B (+ residual x) -> C: whole tiles, split tiles, products with fewer
    units than CTAs, shared X blocks (K = 7168) and the ring's first pass all occur."""
    from tilert_b200.models.deepseek_v3_2 import ops

    d0, d1, d2 = shape
    g = torch.Generator(device="cuda").manual_seed(d0 + tokens)
    wa, wb, wc = _rand_packed(g, d1, d0), _rand_packed(g, d0, d1), _rand_packed(g, d2, d0)
    x = torch.randn(1, tokens, d0, generator=g, device="cuda").to(BF16)
    g0 = (torch.rand(d0, generator=g, device="cuda") + 0.5).float()
    g1 = (torch.rand(d1, generator=g, device="cuda") + 0.5).float()

    def run(chained):
        y = torch.zeros(1, tokens, d1, dtype=BF16, device="cuda")
        z = torch.zeros(1, tokens, d0, dtype=BF16, device="cuda")
        o = torch.zeros(1, tokens, d2, dtype=BF16, device="cuda")
        with ops.chain("cuda:0", chained):
            ops.rmsnorm_proj_q(x, g0, wa, y.view(1, tokens, 1, d1), None, None, eps=1e-6)
            ops.rmsnorm_proj_q(y, g1, wb, z.view(1, tokens, 1, d0), None, None, eps=1e-6)
            ops.unproj_o_allreduce(z, wc, None, None, 0, o)
        torch.cuda.synchronize()
        return y, z, o

    ref, got = run(False), run(True)
    for name, r, c in zip("yzo", ref, got):
        assert torch.isfinite(r.float()).all(), name
        assert torch.equal(r, c), (name, (r.float() - c.float()).abs().max().item())
    # a second chained launch right behind the first (signals and X epoch restart by themselves)
    again = run(True)
    assert all(torch.equal(r, c) for r, c in zip(ref, again))


@pytest.mark.parametrize("li,tokens", [(0, 1), (1, 1), (1, 2), (1, 4)])
def test_toy_layer_chained_equals_separate_launches(tb, li, tokens):
    """Both toy layers through DecoderLayer.forward with chained and with separate launches.  Router
    scores are forced and the key selection injected, so the two runs take identical discrete decisions;
    every streaming product is then bit-identical, and the two bf16 row products (indexer head weights,
    router logits), which the chained step runs as two-term FP8 products, agree to rounding."""
    from tilert_b200.models.deepseek_v3_2 import layer as L
    from tilert_b200.models.deepseek_v3_2.model_args import toy_model_args

    a, margs = om.toy_args(), toy_model_args()
    sd = om.random_state_dict(a, seed=0)
    g = torch.Generator().manual_seed(7 + li)
    t_ctx, cache_len = 500, 1024
    caches = [torch.randn(1, cache_len, d, generator=g).to(BF16) for d in (a.kv_lora_rank, a.qk_rope_head_dim, a.index_head_dim)]
    x = torch.randn(1, tokens, a.dim, generator=g).to(BF16).cuda()
    fc = oo.precompute_freqs_cis(a)
    fr = torch.view_as_real(fc[t_ctx: t_ctx + tokens]).contiguous().cuda()
    cur = torch.tensor([t_ctx], dtype=I32, device="cuda")
    weights = L.LayerWeights(margs, sd, li, "cuda")
    sel = torch.stack([torch.randperm(t_ctx, generator=g)[: a.index_topk].sort().values for _ in range(tokens)])
    sel = sel.view(1, tokens, -1).to(I32).cuda()
    fs = torch.randn(1, tokens, a.n_routed_experts, generator=g).float().cuda()

    outs = {}
    for chained in (False, True):
        gl = L.DecoderLayer(margs, weights, "cuda", cache_len, max_tokens=tokens)
        gl.chained = chained
        gl.fuse_vproj = False  # the value up-projection as the streaming product in both runs (same bits)
        for dst, src in zip((gl.kv_cache, gl.pe_cache, gl.ki_cache), caches):
            dst.copy_(src)
        gl.injected_sel = sel
        if not weights.dense:
            gl.forced_scores = fs
        out = gl.forward(x, cur, fr, n_keys=t_ctx + tokens).clone()
        torch.cuda.synchronize()
        outs[chained] = (gl, out)
    (ga, oa), (gb, ob) = outs[False], outs[True]
    for name in ("q_a", "kv", "ki", "q_nope", "q_pe", "iq", "iq_rt", "q_lat", "o_lat", "o", "h"):
        ra, rb = getattr(ga, name), getattr(gb, name)
        assert torch.equal(ra, rb), (name, (ra.float() - rb.float()).abs().max().item())

    def near(ra, rb):
        # The chained expert gate/up product is split into a shared-expert and a routed phase, so its row
        # tiles are cut between CTAs at other k blocks and their f32 partial sums are added in another
        # grouping: bf16 results may differ in the last bit.
        d = (ra.float() - rb.float()).norm() / ra.float().norm().clamp_min(1e-20)
        return d.item() <= 2e-3

    if weights.dense:
        assert torch.equal(ga.ffn_hidden, gb.ffn_hidden)
    else:
        assert near(ga.ffn_hidden, gb.ffn_hidden)
    for name in ("kv_cache", "pe_cache", "ki_cache"):
        assert torch.equal(getattr(ga, name), getattr(gb, name)), name
    # (the chained product rounds the normalised activations to bf16 before the product, the row kernel does not)
    assert (ga.idx_w.float() - gb.idx_w.float()).abs().max() <= 1e-2 * ga.idx_w.float().abs().max()
    if not weights.dense:
        assert torch.equal(ga.eidx, gb.eidx) and torch.equal(ga.probs, gb.probs)
        # router logits: bf16 row product (separate launches) vs the two-e4m3-term product on the weight stream
        assert torch.allclose(ga.scores, gb.scores, rtol=1e-3, atol=1e-4), (ga.scores - gb.scores).abs().max().item()
    if weights.dense:
        assert torch.equal(oa, ob), (oa.float() - ob.float()).abs().max().item()
    else:
        assert near(oa, ob)
    # the chained step is two launches + indexer, top-k, attention, combine
    n0 = tb.lib().tilert_b200_launch_count()
    gb.forward(x, cur, fr, n_keys=t_ctx + tokens)
    torch.cuda.synchronize()
    assert tb.lib().tilert_b200_launch_count() - n0 <= 5


@pytest.mark.parametrize("tokens", [1, 4])
def test_value_projection_inside_the_attention_merge(tb, tokens):
    """The merge of the attention chunks fused with the value up-projection (f32 multiply-adds on the bf16 latent
    vector) against the streaming product on the same vector (two e4m3 terms on the tensor core): the same
    numbers up to the order of f32 additions."""
    from tilert_b200.models.deepseek_v3_2 import layer as L
    from tilert_b200.models.deepseek_v3_2.model_args import toy_model_args

    a, margs = om.toy_args(), toy_model_args()
    sd = om.random_state_dict(a, seed=0)
    g = torch.Generator().manual_seed(17 + tokens)
    t_ctx, cache_len = 500, 1024
    caches = [torch.randn(1, cache_len, d, generator=g).to(BF16) for d in (a.kv_lora_rank, a.qk_rope_head_dim, a.index_head_dim)]
    x = torch.randn(1, tokens, a.dim, generator=g).to(BF16).cuda()
    fr = torch.view_as_real(oo.precompute_freqs_cis(a)[t_ctx: t_ctx + tokens]).contiguous().cuda()
    cur = torch.tensor([t_ctx], dtype=I32, device="cuda")
    weights = L.LayerWeights(margs, sd, 1, "cuda")
    res = {}
    for fused in (False, True):
        gl = L.DecoderLayer(margs, weights, "cuda", cache_len, max_tokens=tokens)
        gl.fuse_vproj = fused
        for dst, src in zip((gl.kv_cache, gl.pe_cache, gl.ki_cache), caches):
            dst.copy_(src)
        out = gl.forward(x, cur, fr, n_keys=t_ctx + tokens).clone()
        torch.cuda.synchronize()
        res[fused] = (gl.o_lat.clone(), gl.o.clone(), gl.lse.clone(), out)
    assert torch.equal(res[False][0], res[True][0])      # the merged latent vector: identical
    assert torch.equal(res[False][2], res[True][2])
    d = (res[False][1].float() - res[True][1].float()).norm() / res[False][1].float().norm()
    assert d.item() <= 1e-3, d.item()
    d = (res[False][3].float() - res[True][3].float()).norm() / res[False][3].float().norm()
    assert d.item() <= 2e-3, d.item()
    assert tb.device_status(0) == 0


def test_chain_rejects_what_it_cannot_hold(tb):
    from tilert_b200.models.deepseek_v3_2 import ops

    x = torch.zeros(1, 1, 256, dtype=BF16, device="cuda")
    gamma = torch.ones(256, dtype=F32, device="cuda")
    w = torch.zeros(8, 256, dtype=BF16, device="cuda")
    out = torch.zeros(1, 1, 8, dtype=BF16, device="cuda")
    # a bf16 row product is not chainable (its two-term packed form is)
    with pytest.raises(tb.TilertError):
        with ops.chain("cuda:0"):
            ops.projx_wis(x, w, out, gamma=gamma)
    # operators outside the recordable set refuse while a chain is open
    with pytest.raises(tb.TilertError):
        with ops.chain("cuda:0"):
            ops.rmsnorm(x, gamma, torch.zeros_like(x))
    # the context is usable afterwards
    ops.rmsnorm(x, gamma, torch.zeros_like(x))
    torch.cuda.synchronize()
