"""The oracle must reproduce, bit for bit, the outputs that the reference's own
``golden_forward`` code produced for the seeded cases (fixture written by
``oracle/pin_reference.py``)."""

from pathlib import Path

import pytest
import torch

from oracle import pin_cases

FIXTURE = Path(__file__).parent / "golden" / "ref_goldens.pt"
GOLD = torch.load(FIXTURE, weights_only=False)
RESULTS = pin_cases.oracle_results()


def test_every_case_was_pinned():
    bad = [line for line in GOLD["__report__"] if "NOT PINNED" in line]
    assert not bad, bad


@pytest.mark.parametrize("name", sorted(RESULTS))
def test_oracle_matches_reference_golden(name):
    for i, mine in enumerate(RESULTS[name]):
        ref = GOLD[f"{name}.{i}"]
        assert ref.shape == mine.shape, (name, i, ref.shape, mine.shape)
        assert torch.equal(ref.float(), mine.float()), (name, i, (ref.float() - mine.float()).abs().max())


def test_grouped_routing_matches_reference():
    mine = pin_cases.route_groups_result(GOLD["route_groups.scores"], GOLD["route_groups.bias"])
    for i, m in enumerate(mine):
        assert torch.equal(GOLD[f"route_groups.{i}"].float(), m.float())


def test_cache_wire_format_matches_reference():
    """The FP8 cache wire format: the oracle's dequantisers against the reference's own outputs
    (fixture made by oracle/pin_cache_format.py from tilert/pd_vllm/profiles/mla_nsa.py)."""
    from pathlib import Path

    import torch

    from oracle import cache_format as cf

    fx = torch.load(Path(__file__).parent / "golden" / "ref_cache_format.pt")
    seq = fx["seq_len"]
    assert fx["kv_raw"].shape == (seq, cf.KV_BYTES) and fx["ki_pages"].shape == ((seq + 63) // 64, cf.KI_PAGE_BYTES)
    assert torch.equal(cf.dequant_kv(fx["kv_raw"], seq).view(torch.int16), fx["kv"].view(torch.int16))
    assert torch.equal(cf.dequant_ki(fx["ki_pages"], seq).view(torch.int16), fx["ki"].view(torch.int16))
    # the test-input quantisers round-trip within e4m3 precision
    g = torch.Generator().manual_seed(5)
    kv = torch.randn(70, 512, generator=g).to(torch.bfloat16)
    back = cf.dequant_kv(cf.quant_kv(kv), 70).float()
    assert (back - kv.float()).abs().max() <= 0.07 * kv.float().abs().max()
