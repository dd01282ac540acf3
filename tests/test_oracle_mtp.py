"""CPU checks of the oracle's speculative-decoding restatement (oracle/model.py::MtpModel): greedy
verification is lossless against plain greedy decoding, and the accepted count follows the drafts."""

import torch

from oracle import model as om


def _setup(n_prompt=21, seed=11):
    a = om.toy_args()
    sd = om.random_state_dict(a, seed=0, with_mtp=True)
    prompt = torch.randint(0, a.vocab_size, (n_prompt,), generator=torch.Generator().manual_seed(seed)).tolist()
    return a, sd, prompt


def test_mtp_layer_keys_do_not_disturb_the_main_model():
    a = om.toy_args()
    sd0, sd1 = om.random_state_dict(a, seed=0), om.random_state_dict(a, seed=0, with_mtp=True)
    for k, v in sd0.items():
        assert torch.equal(v.view(torch.uint8), sd1[k].view(torch.uint8)), k
    assert f"model.layers.{a.n_layers}.eh_proj.weight" in sd1


def test_speculative_decoding_is_lossless_up_to_numerical_ties():
    a, sd, prompt = _setup()
    n_new = 12
    plain, plain_logits = om.Model(a, sd, cache_len=128).generate(prompt, n_new)
    spec, counts = om.MtpModel(a, sd, cache_len=128).generate_mtp(prompt, n_new)
    assert all(1 <= c <= 4 for c in counts) and sum(counts) >= n_new
    for i, (p, s) in enumerate(zip(plain, spec)):
        if p != s:
            # a four-row pass and four one-row passes may round differently: only a tie may flip
            top2 = torch.topk(plain_logits[i], 2).values
            assert (top2[0] - top2[1]) <= 2e-2 * plain_logits[i].abs().max(), (i, p, s)
            break


def test_true_continuation_is_accepted_in_full():
    a, sd, prompt = _setup()
    plain, _ = om.Model(a, sd, cache_len=128).generate(prompt, 5)
    m = om.MtpModel(a, sd, cache_len=128)
    # caches of both models up to the last prompt token
    m.generate_mtp(prompt, 0)
    assert m.pos == len(prompt) - 1
    r = m.verify_step([prompt[-1]] + plain[:3])
    assert r["predicted"][:3] == plain[:3]
    assert r["n_accepted"] == 4 and m.pos == len(prompt) + 3
    assert r["next_draft"][0] == r["predicted"][3] and len(r["next_draft"]) == 4
    # a wrong second guess cuts the acceptance after two tokens
    m2 = om.MtpModel(a, sd, cache_len=128)
    m2.generate_mtp(prompt, 0)
    wrong = (plain[1] + 1) % a.vocab_size
    r2 = m2.verify_step([prompt[-1], plain[0], wrong, plain[2]])
    assert r2["n_accepted"] == 2 and r2["next_draft"][0] == r2["predicted"][1] == plain[1]
