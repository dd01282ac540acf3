"""GPU parity of whole decoder layers and of the toy model's greedy decoding against the CPU
oracle: per-layer cosine >= 0.999, logits relative L2 <= 2e-2, greedy tokens identical."""

import json
import os

import pytest
import torch

from oracle import model as om
from oracle import ops as oo

pytestmark = pytest.mark.gpu
BF16, F32, I32 = torch.bfloat16, torch.float32, torch.int32


def _m(ref, out):
    ref, out = ref.float().cpu().flatten(), out.float().cpu().flatten()
    cos = torch.nn.functional.cosine_similarity(ref, out, dim=0).item()
    l2 = (torch.norm(ref - out) / torch.norm(ref).clamp_min(1e-30)).item()
    return cos, l2


def _log(rec):
    path = os.environ.get("TB_METRICS")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps(rec) + "\n")


@pytest.fixture(scope="module")
def tb():
    import tilert_b200

    tilert_b200.load_backend("deepseek_v3_2")
    tilert_b200.tilert_init(0)
    yield tilert_b200
    assert tilert_b200.device_status(0) == 0


@pytest.mark.parametrize("li,tokens", [(0, 1), (1, 1), (1, 2)])
def test_toy_layer_step_matches_oracle(tb, li, tokens):
    from tilert_b200.models.deepseek_v3_2 import layer as L
    from tilert_b200.models.deepseek_v3_2.model_args import toy_model_args

    a, margs = om.toy_args(), toy_model_args()
    sd = om.random_state_dict(a, seed=0)
    g = torch.Generator().manual_seed(100 + li)
    t_ctx, cache_len = 600, 1024
    ow, oc = om.LayerWeights(a, sd, li), om.Caches(a, cache_len)
    for c in (oc.kv, oc.pe, oc.ki):
        c[:, :t_ctx] = (torch.randn(1, t_ctx, c.size(-1), generator=g, dtype=torch.float32)).to(BF16)
    x = (torch.randn(1, tokens, a.dim, generator=g, dtype=torch.float32)).to(BF16)
    fc = oo.precompute_freqs_cis(a)

    gl = L.DecoderLayer(margs, L.LayerWeights(margs, sd, li, "cuda"), "cuda", cache_len, max_tokens=tokens)
    gl.kv_cache.copy_(oc.kv); gl.pe_cache.copy_(oc.pe); gl.ki_cache.copy_(oc.ki)
    cur = torch.tensor([t_ctx], dtype=I32, device="cuda")
    fr = torch.view_as_real(fc[t_ctx: t_ctx + tokens]).contiguous().cuda()
    out = gl.forward(x.cuda(), cur, fr, n_keys=t_ctx + tokens)
    torch.cuda.synchronize()

    trace = {}
    ref = om.layer_step(a, ow, oc, x, t_ctx, fc, trace)
    pairs = {"q_a": gl.q_a, "kv": gl.kv, "ki": gl.ki, "idx_w": gl.idx_w, "q_nope": gl.q_nope, "q_pe": gl.q_pe,
             "iq": gl.iq_rt, "q_lat": gl.q_lat, "o_lat": gl.o_lat, "o": gl.o, "attn_out": gl.h,
             "ffn_hidden": gl.ffn_hidden, "out": gl.out}
    worst = 1.0
    for name, dev_t in pairs.items():
        r = trace[name]
        cos, l2 = _m(r, dev_t.view(r.shape))
        _log({"name": f"layer{li}.s{tokens}.{name}", "cos": cos, "rel_l2": l2})
        worst = min(worst, cos)
    # caches written at the new positions
    for name, rc, dc in (("kv", oc.kv, gl.kv_cache), ("pe", oc.pe, gl.pe_cache), ("ki", oc.ki, gl.ki_cache)):
        cos, l2 = _m(rc[:, t_ctx: t_ctx + tokens], dc[:, t_ctx: t_ctx + tokens])
        _log({"name": f"layer{li}.s{tokens}.cache_{name}", "cos": cos, "rel_l2": l2})
        assert cos >= 0.999, (name, cos)
    # selected key sets: identical up to near-ties at the k-th score
    sel_ref, sel_dev = set(trace["sel"][0, 0].tolist()), set(gl.sel[0, 0].cpu().tolist())
    overlap = len(sel_ref & sel_dev) / max(len(sel_ref), 1)
    _log({"name": f"layer{li}.s{tokens}.sel_overlap", "overlap": overlap})
    assert overlap >= 0.97
    if not ow.dense:
        assert torch.equal(trace["eidx"].to(I32), gl.eidx.cpu()[:, :tokens])
    cos, l2 = _m(ref, out)
    assert cos >= 0.999 and l2 <= 2e-2, (cos, l2)
    assert worst >= 0.999, worst


def test_toy_model_greedy_decode_matches_oracle(tb):
    """The toy workload: 1024 random prompt ids (seed 1), 64 greedy steps.  Prompt length is cut by
    TB_TOY_PROMPT (default 1024) to bound the oracle's CPU time if needed."""
    from tilert_b200.models.deepseek_v3_2.model import DsaModel
    from tilert_b200.models.deepseek_v3_2.model_args import toy_model_args

    a, margs = om.toy_args(), toy_model_args()
    sd = om.random_state_dict(a, seed=0)
    n_prompt, n_new = int(os.environ.get("TB_TOY_PROMPT", "1024")), 64
    prompt = torch.randint(0, a.vocab_size, (n_prompt,), generator=torch.Generator().manual_seed(1)).tolist()

    dev = DsaModel(margs, sd, "cuda", cache_len=n_prompt + n_new + 8)
    toks, lgs = dev.generate(prompt, n_new, collect_logits=True)
    torch.cuda.synchronize()

    ref = om.Model(a, sd, cache_len=n_prompt + n_new + 8)
    rtoks, rlgs = ref.generate(prompt, n_new)
    l2s = [_m(r, d)[1] for r, d in zip(rlgs, lgs)]
    n_same = sum(int(x == y) for x, y in zip(rtoks, toks))
    first_div = next((i for i, (x, y) in enumerate(zip(rtoks, toks)) if x != y), n_new)
    _log({"name": "toy.generate", "tokens_equal": n_same, "first_divergence": first_div,
          "logits_rel_l2_first": l2s[0], "logits_rel_l2_max_before_div": max(l2s[: max(first_div, 1)])})
    # logits of the first generated position depend only on the (identical) prompt
    assert l2s[0] <= 2e-2, l2s[0]
    assert max(l2s[: max(first_div, 1)]) <= 2e-2
    assert rtoks == toks, (first_div, rtoks[:8], toks[:8])
