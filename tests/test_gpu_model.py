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
    # The selected key set can differ from the oracle's by a key or two at the k-th score (the
    # scores agree to ~5e-3), and attention over random caches is sensitive to single keys.  The
    # attention output is therefore checked against the oracle run on the DEVICE's selection.
    o_lat_dev_sel = oo.flash_sparse_mla(trace["q_lat"], trace["q_pe"], oc.kv[:, : t_ctx + tokens],
                                        oc.pe[:, : t_ctx + tokens], gl.sel.cpu()[:, :tokens], t_ctx,
                                        oo.softmax_scale(a))
    trace["o_lat"] = o_lat_dev_sel
    trace["o"] = oo.projo_wkvb(o_lat_dev_sel, ow.wkv_b_v)
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


@pytest.mark.parametrize("use_graph", [False, True])
def test_toy_model_first_steps(tb, use_graph):
    """A short sequence from position 0: logits of every step against the oracle, with and without
    CUDA-graph replay."""
    from tilert_b200.models.deepseek_v3_2.model import DsaModel
    from tilert_b200.models.deepseek_v3_2.model_args import toy_model_args

    a, margs = om.toy_args(), toy_model_args()
    sd = om.random_state_dict(a, seed=0)
    toks = torch.randint(0, a.vocab_size, (12,), generator=torch.Generator().manual_seed(3)).tolist()
    dev = DsaModel(margs, sd, "cuda", cache_len=512, use_graph=use_graph)
    ref = om.Model(a, sd, cache_len=512)
    dev.reset_sequence()
    for pos, t in enumerate(toks):
        dev.forward(t, pos)
        torch.cuda.synchronize()
        _, rl = ref.step(t)
        cos, l2 = _m(rl, dev.logits.view(-1))
        _log({"name": f"toy.first_steps.graph{int(use_graph)}.pos{pos}", "cos": cos, "rel_l2": l2,
              "argmax_equal": int(int(torch.argmax(rl)) == int(dev.token_out))})
        assert l2 <= 2e-2, (pos, cos, l2)


def test_toy_model_greedy_decode_matches_oracle(tb):
    """The toy workload: 1024 random prompt ids (seed 1), 64 greedy steps.

    Three discrete decisions sit on the path -- the indexer's top-256 key selection, the router's
    top-4 expert choice and the arg-max over the vocabulary -- and all amplify last-bit differences between two correct bf16 pipelines: with
    random weights one swapped key at the 256th score changes the attention output by several per
    cent, and the top-2 logit margin is often smaller than the logits' numerical noise.  The check is
    therefore split the way the workload definition splits it:
      * floating-point path: the device model is fed the oracle's tokens, selected key sets and router
        scores (the device then routes on identical scores); at each of the 64 generated positions its logits must be within rel-L2 2e-2 of the
        oracle's, every layer output must reach cosine 0.999, and its arg-max must equal the oracle's
        token unless the oracle's top-2 margin is below the measured logit error (a numerical tie);
      * selection: given identical scores the top-k is bit-exact (tests/test_gpu_ops.py); here the
        free-running device model's own selections must overlap the oracle's by >= 90 % on average.
    The free-running greedy continuation is logged (tokens equal, first divergence) for the record."""
    from tilert_b200.models.deepseek_v3_2.model import DsaModel
    from tilert_b200.models.deepseek_v3_2.model_args import toy_model_args

    a, margs = om.toy_args(), toy_model_args()
    sd = om.random_state_dict(a, seed=0)
    n_prompt, n_new = int(os.environ.get("TB_TOY_PROMPT", "1024")), 64
    prompt = torch.randint(0, a.vocab_size, (n_prompt,), generator=torch.Generator().manual_seed(1)).tolist()
    cache_len = n_prompt + n_new + 8

    # oracle, free running, keeping each step's selections and layer outputs
    ref = om.Model(a, sd, cache_len=cache_len)
    fed, sels, routes, outs, rlogits, rtoks = list(prompt), [], [], [], [], []
    i = 0
    while i < len(fed):
        traces = []
        nxt, lg = ref.step(fed[i], traces)
        sels.append([t["sel"].clone() for t in traces])
        routes.append([t.get("router_scores") for t in traces])
        if i >= n_prompt - 1:
            outs.append([t["out"].clone() for t in traces])
            rlogits.append(lg)
            rtoks.append(nxt)
            if len(rtoks) < n_new:
                fed.append(nxt)
        i += 1
    assert len(rtoks) == n_new and len(fed) == n_prompt + n_new - 1

    # device, teacher-forced tokens, injected selections, eager launches
    dev = DsaModel(margs, sd, "cuda", cache_len=cache_len, use_graph=False)
    dev.reset_sequence()
    worst_l2, worst_cos, mismatches, ties = 0.0, 1.0, 0, 0
    overlaps = []
    for pos, tok in enumerate(fed):
        for li, layer in enumerate(dev.layers):
            layer.injected_sel = sels[pos][li].cuda()
            if routes[pos][li] is not None:
                layer.forced_scores = routes[pos][li].float().cuda()
        dev.forward(tok, pos)
        if pos >= n_prompt - 1:
            torch.cuda.synchronize()
            j = pos - (n_prompt - 1)
            dl = dev.logits.view(-1).float().cpu()
            cos, l2 = _m(rlogits[j], dl)
            worst_l2 = max(worst_l2, l2)
            for li, layer in enumerate(dev.layers):
                worst_cos = min(worst_cos, _m(outs[j][li], layer.out[:, :1])[0])
            if int(torch.argmax(dl)) != rtoks[j]:
                mismatches += 1
                top2 = torch.topk(rlogits[j], 2)[0]
                err = float((dl - rlogits[j]).abs().max())
                assert float(top2[0] - top2[1]) <= 2.0 * err, (j, float(top2[0] - top2[1]), err)
                ties += 1
    _log({"name": "toy.generate.forced", "logits_rel_l2_max": worst_l2, "layer_cos_min": worst_cos,
          "argmax_mismatches": mismatches, "all_mismatches_are_numerical_ties": int(mismatches == ties)})
    assert worst_l2 <= 2e-2, worst_l2
    assert worst_cos >= 0.999, worst_cos

    # device, free running under CUDA-graph replay: its own key selections, its own routing, its own tokens.
    # Wherever its token differs from the oracle's, the difference must be a numerical tie (the oracle's
    # top-2 margin below twice the measured logit error of that step); the sequence is then re-synchronised
    # to the oracle's token, so that one tie cannot hide a later real regression.
    free = DsaModel(margs, sd, "cuda", cache_len=cache_len, use_graph=True)
    free.reset_sequence()
    n_same, first_div, tie_count, not_ties = 0, n_new, 0, []
    for pos, tok in enumerate(fed):
        free.forward(tok, pos)
        if pos >= n_prompt - 1:
            torch.cuda.synchronize()
            j = pos - (n_prompt - 1)
            dl = free.logits.view(-1).float().cpu()
            if int(free.token_out) == rtoks[j]:
                n_same += 1
                continue
            first_div = min(first_div, j)
            top2 = torch.topk(rlogits[j], 2)[0]
            margin, err = float(top2[0] - top2[1]), float((dl - rlogits[j]).abs().max())
            if margin <= 2.0 * err:
                tie_count += 1
            else:
                not_ties.append((j, margin, err))
    _log({"name": "toy.generate.free", "tokens_equal": n_same, "first_divergence": first_div, "ties": tie_count,
          "not_ties": len(not_ties)})
    assert not not_ties, not_ties
    assert n_same + tie_count == n_new


def test_toy_selection_overlap_during_prefill(tb):
    """Free-running device model vs oracle over a 600-token prompt: the per-step selected key sets
    (top-256 of up to 600 keys) overlap by >= 90 % on average in the first layer, whose inputs are
    identical on both sides (token embeddings)."""
    from tilert_b200.models.deepseek_v3_2.model import DsaModel
    from tilert_b200.models.deepseek_v3_2.model_args import toy_model_args

    a, margs = om.toy_args(), toy_model_args()
    sd = om.random_state_dict(a, seed=0)
    prompt = torch.randint(0, a.vocab_size, (600,), generator=torch.Generator().manual_seed(4)).tolist()
    ref = om.Model(a, sd, cache_len=640)
    dev = DsaModel(margs, sd, "cuda", cache_len=640, use_graph=False)
    dev.reset_sequence()
    overlaps = []
    for pos, tok in enumerate(prompt):
        traces = []
        ref.step(tok, traces)
        dev.forward(tok, pos)
        if pos >= 300 and pos % 10 == 0:
            torch.cuda.synchronize()
            r = set(traces[0]["sel"][0, 0].tolist()) - {-1}
            d = set(dev.layers[0].sel[0, 0].cpu().tolist()) - {-1}
            overlaps.append(len(r & d) / len(r))
    mean = sum(overlaps) / len(overlaps)
    _log({"name": "toy.sel_overlap.layer0", "mean": mean, "min": min(overlaps)})
    assert mean >= 0.9, (mean, min(overlaps))


def test_full_shape_moe_layer_matches_oracle(tb):
    """The full-shape workload: hidden 7168, 128 heads, 256 experts (8 forced hot experts + shared),
    indexer 64x128 top-2048, one decode step at the end of a 4096-row N(0,1) cache."""
    from tilert_b200.models.deepseek_v3_2 import layer as L
    from tilert_b200.models.deepseek_v3_2.model_args import full_layer_args

    cache_len = 4096
    a, margs = om.full_layer_args(max_seq_len=cache_len), full_layer_args(max_seq_len=cache_len)
    hot = [0, 16, 64, 80, 128, 144, 192, 208]
    sd = om.random_state_dict(a, seed=0, expert_ids=hot)
    ow, oc = om.LayerWeights(a, sd, 0), om.Caches(a, cache_len)
    g = torch.Generator().manual_seed(2)
    for c in (oc.kv, oc.pe, oc.ki):
        c.copy_(torch.randn(c.shape, generator=g, dtype=torch.float32).to(BF16))
    x = torch.randn(1, 1, a.dim, generator=g, dtype=torch.float32).to(BF16)
    fs = torch.full((1, 1, a.n_routed_experts), -8.0)
    fs[0, 0, hot] = 4.0
    fc = oo.precompute_freqs_cis(a)
    pos = cache_len - 1

    gl = L.DecoderLayer(margs, L.LayerWeights(margs, sd, 0, "cuda", expert_ids=hot), "cuda", cache_len)
    gl.kv_cache.copy_(oc.kv); gl.pe_cache.copy_(oc.pe); gl.ki_cache.copy_(oc.ki)
    gl.forced_scores = fs.cuda()
    cur = torch.tensor([pos], dtype=I32, device="cuda")
    fr = torch.view_as_real(fc[pos: pos + 1]).contiguous().cuda()
    out = gl.forward(x.cuda(), cur, fr, n_keys=cache_len)
    torch.cuda.synchronize()

    trace = {}
    ref = om.layer_step(a, ow, oc, x, pos, fc, trace, forced_router_scores=fs)
    assert sorted(trace["eidx"][0, 0].tolist()) == hot and sorted(gl.eidx[0, 0].cpu().tolist()) == hot
    sel_ref, sel_dev = set(trace["sel"][0, 0].tolist()), set(gl.sel[0, 0].cpu().tolist())
    _log({"name": "full.sel_overlap", "overlap": len(sel_ref & sel_dev) / len(sel_ref)})
    o_lat_dev_sel = oo.flash_sparse_mla(trace["q_lat"], trace["q_pe"], oc.kv, oc.pe, gl.sel.cpu(), pos, oo.softmax_scale(a))
    for name, r, d in (("q_a", trace["q_a"], gl.q_a), ("q_nope", trace["q_nope"], gl.q_nope), ("iq", trace["iq"], gl.iq_rt),
                       ("q_lat", trace["q_lat"], gl.q_lat), ("o_lat", o_lat_dev_sel, gl.o_lat),
                       ("attn_out", trace["attn_out"], gl.h), ("ffn_hidden", trace["ffn_hidden"], gl.ffn_hidden),
                       ("out", ref, out)):
        cos, l2 = _m(r, d.view(r.shape))
        _log({"name": f"full.{name}", "cos": cos, "rel_l2": l2})
        assert cos >= 0.999 and l2 <= 2e-2, (name, cos, l2)


def test_model_driver_sampling(tb):
    """The driver's sampling switch: temperature 0 reproduces greedy decoding through the sampling
    operator; a seeded temperature-1 run is reproducible, and the reported log-probability is the
    log-softmax of the step's logits at the sampled token."""
    from tilert_b200.models.deepseek_v3_2.model import DsaModel
    from tilert_b200.models.deepseek_v3_2.model_args import toy_model_args

    a = om.toy_args()
    sd = om.random_state_dict(a, seed=0)
    prompt = torch.randint(0, a.vocab_size, (9,), generator=torch.Generator().manual_seed(4)).tolist()
    dev = DsaModel(toy_model_args(), sd, "cuda", cache_len=256)
    greedy = dev.generate(prompt, 8)
    dev.set_sampling(temperature=0.0)
    assert dev.generate(prompt, 8) == greedy

    def run(seed):
        dev.set_sampling(temperature=1.0, top_p=0.95, top_k=64, use_top_p=True, seed=seed)
        dev.sample_step.zero_()
        return dev.generate(prompt, 8)

    first, again, other = run(7), run(7), run(8)
    assert first == again
    assert first != greedy or other != greedy  # 64 candidates at temperature 1: sampling moves off the arg-max
    # after the last step: logits and the sampled token of that step
    lp = torch.log_softmax(dev.logits.view(-1).double(), dim=-1)
    assert abs(float(lp[int(dev.token_out)]) - float(dev.token_logprob)) < 2e-4
    assert torch.equal(dev.topn_indices[0].long().cpu(), torch.argsort(-dev.logits.view(-1).double(), stable=True)[:256].cpu())


def test_positions_past_the_caches_are_refused_on_the_host(tb):
    """The driver keeps a host copy of the device-resident position: a step at or past the end of the
    caches, a ``pos`` that differs from the device position, or a ``set_cur_pos`` outside the caches
    raises before anything is launched."""
    from tilert_b200.models.deepseek_v3_2.model import DsaModel
    from tilert_b200.models.deepseek_v3_2.model_args import toy_model_args

    a = om.toy_args()
    sd = om.random_state_dict(a, seed=0)
    dev = DsaModel(toy_model_args(), sd, "cuda", cache_len=8, use_graph=False)
    with pytest.raises(ValueError):
        dev.set_cur_pos(8)
    with pytest.raises(ValueError):
        dev.forward(1, 3)  # the device position is 0
    n0 = tb.lib().tilert_b200_launch_count()
    for pos in range(8):
        dev.forward(pos + 1, pos)
    with pytest.raises(ValueError):
        dev.forward(1, 8)
    with pytest.raises(ValueError):
        dev.generate([1, 2, 3, 4, 5], 8)  # 5 + 8 steps do not fit 8 rows: raises at position 8
    torch.cuda.synchronize()
    assert tb.lib().tilert_b200_launch_count() > n0
    assert tb.device_status(0) == 0


def test_injected_caches_continue_a_sequence(tb):
    """Prefill/decode disaggregation: a model that receives the caches of a prompt (bf16, as
    DSAv32Generator.inject_cache takes them) continues exactly like the model that computed them itself;
    through the FP8 wire format the continuation's logits stay within the format's quantisation error."""
    from oracle import cache_format as cf
    from tilert_b200.models.deepseek_v3_2.model import DsaModel
    from tilert_b200.models.deepseek_v3_2.model_args import toy_model_args

    a = om.toy_args()
    sd = om.random_state_dict(a, seed=0)
    prompt = torch.randint(0, a.vocab_size, (40,), generator=torch.Generator().manual_seed(6)).tolist()
    src = DsaModel(toy_model_args(), sd, "cuda", cache_len=256)
    src.reset_sequence()
    for pos, t in enumerate(prompt[:-1]):
        src.forward(t, pos)
    n = len(prompt) - 1
    caches = [(ly.ki_cache[0, :n].clone(), ly.kv_cache[0, :n].clone(), ly.pe_cache[0, :n].clone()) for ly in src.layers]
    src.forward(prompt[-1], n)
    torch.cuda.synchronize()
    want = src.logits.view(-1).clone()

    dst = DsaModel(toy_model_args(), sd, "cuda", cache_len=256)
    dst.inject_cache(caches, start_pos=0)
    dst.set_cur_pos(n)
    dst.forward(prompt[-1], n)
    torch.cuda.synchronize()
    assert torch.equal(dst.logits.view(-1), want)

    # FP8 wire format.  The indexer keys travel un-rotated (the receiver applies the Hadamard rotation, which
    # is its own inverse up to the scale): rotate the cache rows back to make the wire input.
    h = oo.hadamard_matrix(128) * 128 ** -0.5
    planes = []
    for ki, kv, pe in caches:
        ki_plain = (ki.float().cpu() @ h).to(BF16)
        planes.append((cf.quant_kv(kv.cpu()), pe.cpu().contiguous().view(torch.uint8).view(n, 128), cf.quant_ki_pages(ki_plain)))
    dq = DsaModel(toy_model_args(), sd, "cuda", cache_len=256)
    dq.inject_cache(planes, start_pos=0, end_pos=n)
    dq.set_cur_pos(n)
    dq.forward(prompt[-1], n)
    torch.cuda.synchronize()
    cos, l2 = _m(want, dq.logits.view(-1))
    _log({"name": "inject.fp8.logits", "cos": cos, "rel_l2": l2})
    assert cos >= 0.95, (cos, l2)  # e4m3 caches: per cent-level noise, and room for one router near-tie
    for (ki, kv, pe), ly in zip(caches, dq.layers):
        c, _ = _m(kv, ly.kv_cache[0, :n])
        assert c >= 0.999, c
        c, _ = _m(ki, ly.ki_cache[0, :n])
        assert c >= 0.998, c


@pytest.mark.parametrize("t_ctx,cache_len", [(400, 512), (9000, 9216)])
def test_two_stream_step_equals_one_stream_step(t_ctx, cache_len):
    """The layer step on two streams (absorbed-q product beside the vector launch and the indexer's scoring +
    selection; long rows: the cooperative selection on its share of the SMs) gives the same bytes as the step on one
    stream, eagerly and from a captured graph, with one and with four rows."""
    import tilert_b200
    from tilert_b200.models.deepseek_v3_2 import layer as L
    from tilert_b200.models.deepseek_v3_2.model_args import toy_model_args

    tilert_b200.load_backend("deepseek_v3_2")
    tilert_b200.tilert_init(0)
    margs = toy_model_args()
    from dataclasses import replace

    margs = replace(margs, max_seq_len=max(margs.max_seq_len, cache_len))
    a = om.toy_args()
    sd = om.random_state_dict(a, seed=0)
    g = torch.Generator().manual_seed(t_ctx)
    for tokens in (1, 4):
        gl = L.DecoderLayer(margs, L.LayerWeights(margs, sd, 1, "cuda"), "cuda", cache_len, tokens)
        for c in (gl.kv_cache, gl.pe_cache, gl.ki_cache):
            c[:, :t_ctx].copy_(torch.randn(1, t_ctx, c.shape[-1], generator=g).to(torch.bfloat16))
        x = torch.randn(1, tokens, a.dim, generator=g).to(torch.bfloat16).cuda()
        cur = torch.tensor([t_ctx], dtype=torch.int32, device="cuda")
        fr = L.precompute_freqs(margs)[t_ctx: t_ctx + tokens].contiguous().cuda()
        n_keys = (t_ctx + tokens + 255) // 256 * 256
        outs = {}
        for fork in (False, True):
            gl.fork = fork
            outs[fork, "eager"] = gl.forward(x, cur, fr, n_keys).clone()
            sel_eager = gl.sel.clone()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                y = gl.forward(x, cur, fr, n_keys)
            graph.replay()
            torch.cuda.synchronize()
            outs[fork, "graph"] = y.clone()
            assert torch.equal(sel_eager, gl.sel)
        ref = outs[False, "eager"]
        assert torch.isfinite(ref.float()).all()
        for key, val in outs.items():
            assert torch.equal(ref, val), key
    assert tilert_b200.device_status(0) == 0
