"""The driver surface the reference's generator runs on -- ``dsa_show_hands*``, ``ShowHandsDSALayer``,
``DSAv32Generator``, the generate command line -- on the toy model: tokens come out of
``temp_vars[Idx.TOKEN_OUT]``, and they are the tokens the model classes give directly."""

import subprocess
import sys
from pathlib import Path

import pytest
import torch

from oracle import model as om

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def tb():
    import tilert_b200

    tilert_b200.load_backend("deepseek_v3_2")
    tilert_b200.tilert_init(0)
    yield tilert_b200
    assert tilert_b200.device_status(0) == 0


def _toy(with_mtp=False):
    from tilert_b200.models.deepseek_v3_2.model_args import toy_model_args

    a = om.toy_args()
    return toy_model_args(), om.random_state_dict(a, seed=0, with_mtp=with_mtp), a


def test_show_hands_calls_drive_the_toy_model(tb):
    from tilert_b200.models.deepseek_v3_2 import end2end as e2e
    from tilert_b200.models.deepseek_v3_2.model import DsaModel
    from tilert_b200.models.deepseek_v3_2.temp_var_indices import Idx

    margs, sd, a = _toy()
    toks = torch.randint(0, a.vocab_size, (10,), generator=torch.Generator().manual_seed(11)).tolist()
    direct = DsaModel(margs, sd, "cuda", cache_len=128)
    want_tok, want_logits = [], []
    for pos, t in enumerate(toks):
        direct.forward(t, pos)
        torch.cuda.synchronize()
        want_tok.append(int(direct.token_out))
        want_logits.append(direct.logits.view(-1).clone())

    params = e2e.StepParams(margs, sd)
    tv = e2e.get_temp_vars(margs, "cuda:0")
    caches = [torch.zeros(1, 128, d, dtype=torch.bfloat16, device="cuda")
              for _ in range(margs.n_layers) for d in (margs.index_head_dim, margs.kv_lora_rank, margs.qk_rope_head_dim)]
    e2e.dsa_show_hands_prepare_money(params, tv, caches, None, 128)
    try:
        for pos, t in enumerate(toks):
            e2e.dsa_show_hands(torch.tensor([t]))  # a CPU tensor, as the reference passes it
            torch.cuda.synchronize()
            assert int(tv[Idx.TOKEN_OUT].view(-1)[0]) == want_tok[pos]
            assert torch.equal(tv[Idx.LOGITS_OUT].view(-1), want_logits[pos])
            assert int(tv[Idx.CUR_POS][0]) == pos + 1
        # the caches handed in are the ones the step writes
        assert float(caches[1][0, : len(toks)].float().abs().sum()) > 0
        # reset, then set_cur_pos: the sequence can be resumed at a position
        e2e.dsa_show_hands_reset()
        e2e.dsa_show_hands(torch.tensor([toks[0]]))
        torch.cuda.synchronize()
        assert int(tv[Idx.TOKEN_OUT].view(-1)[0]) == want_tok[0]
        e2e.dsa_show_hands_set_cur_pos(5)
        e2e.dsa_show_hands(torch.tensor([toks[5]]))
        torch.cuda.synchronize()
        assert int(tv[Idx.CUR_POS][0]) == 6
    finally:
        e2e.dsa_show_hands_go_home()
    with pytest.raises(RuntimeError):
        e2e.dsa_show_hands(torch.tensor([1]))


def test_dispatcher_names_drive_the_toy_model(tb):
    """Only ``torch.ops.tilert.*`` calls, after the registration library has been loaded the way the reference
    loads its own (``torch.ops.load_library``): prepare_money, one show_hands per token, the token read from
    ``temp_vars[Idx.TOKEN_OUT]``; plus one per-operator name served by the same library."""
    from tilert_b200 import torch_ops
    from tilert_b200.models.deepseek_v3_2 import end2end as e2e
    from tilert_b200.models.deepseek_v3_2.model import DsaModel
    from tilert_b200.models.deepseek_v3_2.temp_var_indices import Idx

    torch_ops.register()
    T = torch.ops.tilert
    assert T.dsa_temp_vars_size() == 56
    margs, sd, a = _toy()
    toks = torch.randint(0, a.vocab_size, (8,), generator=torch.Generator().manual_seed(21)).tolist()
    direct = DsaModel(margs, sd, "cuda", cache_len=64)
    want = []
    for pos, t in enumerate(toks):
        direct.forward(t, pos)
        want.append(int(direct.token_out))
    params = e2e.StepParams(margs, sd)
    tv = e2e.get_temp_vars(margs, "cuda:0")
    caches = [torch.zeros(1, 64, d, dtype=torch.bfloat16, device="cuda")
              for _ in range(margs.n_layers) for d in (margs.index_head_dim, margs.kv_lora_rank, margs.qk_rope_head_dim)]
    torch_ops.bind_params(params)
    T.dsa_show_hands_prepare_money(list(params), tv, caches, None, 64)
    try:
        got = []
        for t in toks:
            T.dsa_show_hands(torch.tensor([t]))
            got.append(int(tv[Idx.TOKEN_OUT].view(-1)[0]))
        assert got == want
        T.dsa_show_hands_reset()
        T.dsa_show_hands_set_cur_pos(3)
        T.dsa_show_hands_set_sampling_seed(5)
    finally:
        T.dsa_show_hands_go_home()
    # a per-operator name of the same library: C++ registration -> C ABI -> kernel
    x = torch.randn(1, 2, margs.dim, device="cuda").to(torch.bfloat16)
    gamma = torch.rand(margs.dim, device="cuda") + 0.5
    out = torch.zeros_like(x)
    T.rmsnorm_op(x, gamma, out, "deepseek_v3_2", "bf16", None)
    ref = torch.nn.functional.rms_norm(x.float(), [margs.dim], gamma, 1e-6)
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)
    with pytest.raises(RuntimeError):
        T.rmsnorm_op(x.float(), gamma, out, "deepseek_v3_2", "bf16", None)  # dtype checked like the reference's wrappers


@pytest.mark.parametrize("with_mtp", [False, True])
def test_generator_matches_the_model_classes(tb, with_mtp):
    from tilert_b200.models.deepseek_v3_2.generator import DSAv32Generator
    from tilert_b200.models.deepseek_v3_2.model import DsaModel
    from tilert_b200.models.deepseek_v3_2.mtp import MtpDsaModel

    margs, sd, a = _toy(with_mtp)
    prompt = torch.randint(0, a.vocab_size, (9,), generator=torch.Generator().manual_seed(12)).tolist()
    n_new = 12
    if with_mtp:
        want, want_counts = MtpDsaModel(margs, sd, "cuda", cache_len=256).generate(prompt, n_new)
    else:
        want, want_counts = DsaModel(margs, sd, "cuda", cache_len=256).generate(prompt, n_new), []
    gen = DSAv32Generator(margs, max_new_tokens=n_new, with_mtp=with_mtp, max_seq_len=256)
    gen.from_state_dict(sd)
    try:
        text, times, counts, plen = gen.generate("", print_log=False, prompt_tokens=prompt)
    finally:
        gen.cleanup()
    got = [int(t) for t in text.split()]
    assert plen == len(prompt) and got == want
    if with_mtp:
        assert counts[: len(want_counts)] == want_counts[: len(counts)] and all(1 <= c <= 4 for c in counts)
    else:
        assert counts == [] and len(times) == len(prompt) + n_new - 1


def test_model_from_converted_files_equals_the_model_from_the_checkpoint(tb, tmp_path):
    from tilert_b200 import convert
    from tilert_b200.models.deepseek_v3_2.model import DsaModel

    margs, sd, a = _toy()
    convert.convert(sd, tmp_path, margs, world=1)
    toks = torch.randint(0, a.vocab_size, (8,), generator=torch.Generator().manual_seed(13)).tolist()
    ref = DsaModel(margs, sd, "cuda", cache_len=64)
    got = DsaModel.from_converted(margs, tmp_path, "cuda", cache_len=64)
    for pos, t in enumerate(toks):
        ref.forward(t, pos)
        got.forward(t, pos)
        torch.cuda.synchronize()
        assert torch.equal(ref.logits, got.logits), pos


def test_generate_command_line_runs_with_random_weights(tb):
    out = subprocess.run([sys.executable, "-m", "tilert_b200.generate", "--model", "toy", "--use-random-weights",
                          "--max-new-tokens", "8", "--prompt-len", "6", "--max-seq-len", "128"], cwd=ROOT,
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "tokens/s" in out.stdout
