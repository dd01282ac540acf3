"""Single operators at the real model's shapes (the toy-shape cases live in test_gpu_ops.py): the dense
FFN with intermediate 18432 (one rank's view and the 1/8 slice an eight-way split gives a rank), the
vocabulary head on a 16160-row slice of the 129280-row vocabulary (what one of eight ranks holds), and
``eh_proj`` at 7168 x 14336.  Same bounds as everywhere: cosine >= 0.999 and rel-L2 <= 2e-2 against the CPU
restatement of the reference's golden_forward (tighter where the operator has no FP8 weight).
"""

import pytest
import torch

from oracle import ops as oo
from oracle.quant import quantize_weight_block128, weight_dequant

pytestmark = pytest.mark.gpu

BF16, F32 = torch.bfloat16, torch.float32
DIM, INTER, VOCAB = 7168, 18432, 129280


def close(name, ref, out, cos_min=0.999, l2_max=2e-2):
    ref, out = ref.float().cpu().flatten(), out.float().cpu().flatten()
    assert ref.shape == out.shape, (name, ref.shape, out.shape)
    cos = torch.nn.functional.cosine_similarity(ref, out, dim=0).item()
    l2 = (torch.norm(ref - out) / torch.norm(ref).clamp_min(1e-30)).item()
    assert cos >= cos_min and l2 <= l2_max, f"{name}: cosine {cos:.6f}, rel-L2 {l2:.3e}"


@pytest.fixture(scope="module")
def ops():
    import tilert_b200
    from tilert_b200.models.deepseek_v3_2 import ops as _ops

    tilert_b200.load_backend("deepseek_v3_2")
    tilert_b200.tilert_init(0)
    yield _ops
    assert tilert_b200.device_status(0) == 0, "a kernel gave up on a bounded wait"


def fp8(gen, n, k, std=0.02):
    return quantize_weight_block128(torch.randn(n, k, generator=gen, dtype=F32) * std)


@pytest.mark.parametrize("world", [1, 8])
def test_dense_ffn_full_shape(ops, world):
    """Layers 0-2 of the model: gate/up 7168 -> 18432 with SiLU * mul, then down 18432 -> 7168 plus the
    residual.  ``world`` = 8 checks the slice one of eight ranks computes (2304 intermediate rows, i.e.
    18 scale blocks: not a multiple of the kernel's eight-CTA split)."""
    from tilert_b200 import pack

    g = torch.Generator().manual_seed(1843 + world)
    il = INTER // world
    (wg, sg), (wu, su), (wd, sdn) = fp8(g, il, DIM), fp8(g, il, DIM), fp8(g, DIM, il)
    gamma = torch.rand(DIM, generator=g) + 0.5
    x = (torch.randn(1, 1, DIM, generator=g) * 1.5).to(BF16)
    w_gu = pack.pack_gate_up(wg.cuda(), sg.cuda(), wu.cuda(), su.cuda())
    w_down = pack.pack_matrix(wd.cuda(), sdn.cuda())
    hid = torch.zeros(1, 1, il, dtype=BF16, device="cuda")
    ops.rmsnorm_up_gate_silu(x.cuda(), gamma.cuda(), w_gu, hid, eps=1e-6)
    n_split = 9  # the golden cuts the intermediate into nine pseudo-experts (2048 rows each; 256 on one of eight ranks)
    ref_h = oo.dense_up_gate_silu(x, gamma, weight_dequant(wg, sg), weight_dequant(wu, su), 1e-6, n_split)
    close("dense18432.hidden", ref_h, hid)
    out = torch.zeros(1, 1, DIM, dtype=BF16, device="cuda")
    ops.down_allreduce(hid, w_down, None, x.cuda(), 0, out)
    ref_d = oo.dense_down(hid.cpu(), weight_dequant(wd, sdn), n_split)
    close("dense18432.down+res", (ref_d.float() + x.float()).to(BF16), out)


@pytest.mark.parametrize("tokens", [1, 4])
def test_head_vocab_slice_of_eight(ops, tokens):
    """The vocabulary head as one of eight ranks runs it: 16160 of the 129280 rows (bf16), RMSNorm fused,
    f32 logits; and the arg-max over the slice is the restatement's."""
    g = torch.Generator().manual_seed(12928 + tokens)
    rows = VOCAB // 8
    w = (torch.randn(rows, DIM, generator=g) * 0.02).to(BF16)
    gamma = torch.rand(DIM, generator=g) + 0.5
    x = (torch.randn(1, tokens, DIM, generator=g) * 2.0).to(BF16)
    logits = torch.zeros(1, tokens, rows, dtype=F32, device="cuda")
    ops.rmsnorm_head_proj(x.cuda(), gamma.cuda(), w.cuda(), None, logits, eps=1e-6)
    ref = oo.rmsnorm_head_proj(x, gamma, w, 1e-6)
    close("head16160", ref, logits, cos_min=0.99999, l2_max=2e-3)
    got = logits.cpu()
    for t in range(tokens):
        top = int(torch.argmax(ref[0, t]))
        mine = int(torch.argmax(got[0, t]))
        # an arg-max may differ from the restatement's only where the two candidates tie within the tolerance
        assert mine == top or abs(float(ref[0, t, mine] - ref[0, t, top])) <= 2e-3 * float(ref[0, t].abs().max())


@pytest.mark.parametrize("tokens", [1, 4])
def test_eh_proj_full_shape(ops, tokens):
    """The speculative layer's input projection: [e_norm | h_norm] (2 x 7168) through eh_proj 7168 x 14336, bf16."""
    g = torch.Generator().manual_seed(14336 + tokens)
    e = (torch.randn(1, tokens, DIM, generator=g)).to(BF16)
    h = (torch.randn(1, tokens, DIM, generator=g) * 2.0).to(BF16)
    ge, gh = torch.rand(DIM, generator=g) + 0.5, torch.rand(DIM, generator=g) + 0.5
    w = (torch.randn(DIM, 2 * DIM, generator=g) * 0.01).to(BF16)
    e_ref, h_ref, out_ref = oo.mtp_preprocess(e, h, ge, gh, w, 1e-6)
    out = torch.zeros(1, tokens, DIM, dtype=BF16, device="cuda")
    en, hn = torch.zeros_like(out), torch.zeros_like(out)
    ops.mtp_preprocess(e.cuda(), h.cuda(), ge.cuda(), gh.cuda(), w.cuda(), out, eps=1e-6, e_norm_out=en, h_norm_out=hn)
    close("mtp7168.enorm", e_ref, en, cos_min=0.99999, l2_max=4e-3)
    close("mtp7168.hnorm", h_ref, hn, cos_min=0.99999, l2_max=4e-3)
    close("mtp7168.out", out_ref, out, cos_min=0.9999, l2_max=8e-3)
    out2 = torch.zeros_like(out)
    ops.eh_proj_allreduce(e_ref.cuda(), h_ref.cuda(), w.cuda(), 0, out2)
    close("eh_proj7168", oo.eh_proj(e_ref, h_ref, w), out2, cos_min=0.9999, l2_max=8e-3)
