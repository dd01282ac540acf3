"""Makes tests/golden/ref_cache_format.pt: outputs of the REFERENCE's own ``_dequant_kv`` / ``_dequant_ki``
(tilert/pd_vllm/profiles/mla_nsa.py) on seeded wire-format inputs.  Needs the reference checkout:

    PYTHONPATH=/path/to/TileRT python oracle/pin_cache_format.py

The fixture travels with the repository; tests/test_oracle_pins.py re-checks the oracle against it.
"""

import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from oracle import cache_format as cf  # noqa: E402


def inputs(seq_len: int = 150, seed: int = 21):
    g = torch.Generator().manual_seed(seed)
    kv = (torch.randn(seq_len, cf.KV_LORA_RANK, generator=g) * 1.7).to(torch.bfloat16)
    ki = torch.randn(seq_len, cf.INDEX_DIM, generator=g).to(torch.bfloat16)
    return cf.quant_kv(kv), cf.quant_ki_pages(ki), seq_len


def main() -> None:
    from tilert.pd_vllm.profiles.mla_nsa import MlaNsaProfile

    kv_raw, ki_pages, seq = inputs()
    out = {"seq_len": seq, "kv_raw": kv_raw, "ki_pages": ki_pages,
           "kv": MlaNsaProfile._dequant_kv(kv_raw, seq), "ki": MlaNsaProfile._dequant_ki(ki_pages, seq)}
    path = ROOT / "tests" / "golden" / "ref_cache_format.pt"
    torch.save(out, path)
    print(path, {k: (tuple(v.shape), str(v.dtype)) for k, v in out.items() if hasattr(v, "shape")})


if __name__ == "__main__":
    main()
