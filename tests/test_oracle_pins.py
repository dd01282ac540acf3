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
