"""Checkpoint conversion: HF DeepSeek-V3.2 FP8 checkpoint -> per-rank packed weight files.

The role of the reference's ``tilert/models/preprocess/weight_converter.py:243-537`` together with
each operator's ``device_sharding``: read the HF tensors (e4m3 ``weight`` + f32 ``weight_scale_inv`` per
128x128 block, sharded ``*.safetensors`` with ``model.safetensors.index.json``), shard them for
``world`` ranks and write, for every rank, one safetensors file per layer holding the tensors exactly
as the kernels stream them (``tilert_b200.pack`` formats), plus one file with the embedding, the final
norm and the rank's slice of the vocabulary head.  A checkpoint that carries the multi-token-prediction
layer (``model.layers.{n_layers}``) also gets that layer's decoder weights and a small ``mtp.safetensors``.

    python -m tilert_b200.convert --hf /path/to/DeepSeek-V3.2 --out /path/to/packed --world 8

``load_layer`` / ``load_head`` read the files back into the objects the model code uses.
"""

from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch

from .models.deepseek_v3_2.layer import LayerWeights
from .models.deepseek_v3_2.model_args import ModelArgs, full_layer_args, toy_model_args

FORMAT = "tilert_b200.packed.v1"
_COMMON = ("in_norm", "post_norm", "q_norm", "kv_norm", "k_norm_w", "k_norm_b", "wis", "wis2", "w_qkva", "w_qb",
           "w_absorb", "w_v", "w_o", "w_gu", "w_down")
_MOE_ONLY = ("router", "router_bias", "router2")


class HFCheckpoint:
    """Lazy key -> tensor view of an HF safetensors checkpoint directory (sharded or single file)."""

    def __init__(self, root: str | os.PathLike):
        from safetensors import safe_open

        self._open = safe_open
        self.root = Path(root)
        index = self.root / "model.safetensors.index.json"
        if index.exists():
            self.weight_map: dict[str, str] = json.loads(index.read_text())["weight_map"]
        else:
            self.weight_map = {}
            for f in sorted(self.root.glob("*.safetensors")):
                with safe_open(str(f), framework="pt") as h:
                    for k in h.keys():
                        self.weight_map[k] = f.name
        if not self.weight_map:
            raise FileNotFoundError(f"no safetensors weights under {self.root}")
        self._handles: dict[str, object] = {}

    def __contains__(self, key: str) -> bool:
        return key in self.weight_map

    def keys(self):
        return self.weight_map.keys()

    def __getitem__(self, key: str) -> torch.Tensor:
        if key not in self.weight_map:
            raise KeyError(key)
        fname = self.weight_map[key]
        if fname not in self._handles:
            self._handles[fname] = self._open(str(self.root / fname), framework="pt")
        return self._handles[fname].get_tensor(key)


def save_layer(lw: LayerWeights, path: str | os.PathLike) -> None:
    from safetensors.torch import save_file

    names = _COMMON + (() if lw.dense else _MOE_ONLY)
    tensors = {n: getattr(lw, n).detach().cpu().contiguous() for n in names if getattr(lw, n, None) is not None}
    meta = {"format": FORMAT, "dense": str(int(lw.dense)), "inter_local": str(int(lw.inter_local))}
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    save_file(tensors, str(path), metadata=meta)


def load_layer(path: str | os.PathLike, device) -> LayerWeights:
    from safetensors import safe_open

    lw = LayerWeights.__new__(LayerWeights)
    with safe_open(str(path), framework="pt") as h:
        meta = h.metadata() or {}
        if meta.get("format") != FORMAT:
            raise ValueError(f"{path}: not a {FORMAT} file")
        lw.dense = bool(int(meta["dense"]))
        lw.inter_local = int(meta["inter_local"])
        lw.router2 = None  # an f32 router gate has no two-term form
        for n in h.keys():
            setattr(lw, n, h.get_tensor(n).to(device))
    return lw


def load_model(out_dir: str | os.PathLike, device, rank: int = 0) -> dict:
    """Everything ``DsaModel`` needs from a converted directory, for one rank: ``{"layers": [LayerWeights...],
    "embed", "final_norm", "head", "world", "mtp": {...} or None}``."""
    root = Path(out_dir)
    manifest = json.loads((root / "manifest.json").read_text())
    if manifest.get("format") != FORMAT:
        raise ValueError(f"{root}: not a {FORMAT} directory")
    rdir = root / f"rank{rank}"
    main_layers = [li for li in manifest["layers"] if li != manifest.get("mtp_layer")]
    out = {"layers": [load_layer(rdir / f"layer_{li:03d}.safetensors", device) for li in main_layers],
           "world": int(manifest["world"]), "mtp": None}
    out.update(load_head(rdir / "head.safetensors", device))
    if manifest.get("mtp_layer") is not None:
        out["mtp"] = load_mtp(rdir / "mtp.safetensors", device)
        out["mtp"]["layer"] = load_layer(rdir / f"layer_{manifest['mtp_layer']:03d}.safetensors", device)
    return out


def save_head(sd, args: ModelArgs, world: int, rank: int, path: str | os.PathLike) -> None:
    from safetensors.torch import save_file

    v_l = args.vocab_size // world
    tensors = {
        "embed": sd["model.embed_tokens.weight"].to(torch.bfloat16).contiguous(),
        "final_norm": sd["model.norm.weight"].to(torch.float32).contiguous(),
        "head": sd["lm_head.weight"][rank * v_l:(rank + 1) * v_l].to(torch.bfloat16).contiguous(),
    }
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    save_file(tensors, str(path), metadata={"format": FORMAT, "vocab_begin": str(rank * v_l)})


def load_head(path: str | os.PathLike, device) -> dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    return {k: v.to(device) for k, v in load_file(str(path)).items()}


_MTP_KEYS = {"enorm": "enorm.weight", "hnorm": "hnorm.weight", "eh_proj": "eh_proj.weight",
             "shared_head_norm": "shared_head.norm.weight"}


def has_mtp_layer(ckpt, args: ModelArgs) -> bool:
    """True when the checkpoint carries the multi-token-prediction layer (``model.layers.{n_layers}``)."""
    return f"model.layers.{args.n_layers}.eh_proj.weight" in ckpt


def save_mtp(sd, args: ModelArgs, path: str | os.PathLike) -> None:
    """The prediction layer's own small tensors (the role of ``transform_mtp`` in the reference's converter,
    tilert/models/preprocess/weight_converter.py:405-435): enorm / hnorm / shared_head.norm gains in f32 and
    eh_proj in bf16, replicated on every rank.  Its decoder layer is written like any other layer; its
    embedding and head are the main model's."""
    from safetensors.torch import save_file

    p = f"model.layers.{args.n_layers}"
    tensors = {name: sd[f"{p}.{key}"].to(torch.bfloat16 if name == "eh_proj" else torch.float32).contiguous()
               for name, key in _MTP_KEYS.items()}
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    save_file(tensors, str(path), metadata={"format": FORMAT, "layer": str(args.n_layers)})


def load_mtp(path: str | os.PathLike, device) -> dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    return {k: v.to(device) for k, v in load_file(str(path)).items()}


def convert(hf_dir, out_dir, args: ModelArgs, world: int = 1, layers: list[int] | None = None, device="cpu",
            with_head: bool = True) -> list[str]:
    """Convert ``layers`` (default: all of ``args.n_layers``) for every rank; returns the files written."""
    ckpt = hf_dir if isinstance(hf_dir, (dict, HFCheckpoint)) else HFCheckpoint(hf_dir)
    out = Path(out_dir)
    written: list[str] = []
    layer_ids = list(range(args.n_layers)) if layers is None else layers
    mtp = has_mtp_layer(ckpt, args) and (layers is None or args.n_layers in layers)
    if mtp and args.n_layers not in layer_ids:
        layer_ids = layer_ids + [args.n_layers]  # the prediction layer's decoder layer
    for rank in range(world):
        for li in layer_ids:
            lw = LayerWeights(args, ckpt, li, device, world, rank)
            path = out / f"rank{rank}" / f"layer_{li:03d}.safetensors"
            save_layer(lw, path)
            written.append(str(path))
            del lw
        if mtp:
            path = out / f"rank{rank}" / "mtp.safetensors"
            save_mtp(ckpt, args, path)
            written.append(str(path))
        if with_head and "lm_head.weight" in ckpt:
            path = out / f"rank{rank}" / "head.safetensors"
            save_head(ckpt, args, world, rank, path)
            written.append(str(path))
    manifest = {"format": FORMAT, "world": world, "layers": layer_ids, "mtp_layer": args.n_layers if mtp else None, "dim": args.dim, "n_heads": args.n_heads,
                "n_routed_experts": args.n_routed_experts}
    (out / "manifest.json").write_text(json.dumps(manifest, indent=1))
    return written


def _parse_layers(spec: str | None) -> list[int] | None:
    if not spec:
        return None
    ids: list[int] = []
    for part in spec.split(","):
        if "-" in part:
            a, b = part.split("-")
            ids.extend(range(int(a), int(b) + 1))
        else:
            ids.append(int(part))
    return ids


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--hf", required=True, help="HF checkpoint directory (safetensors)")
    ap.add_argument("--out", required=True, help="output directory")
    ap.add_argument("--world", type=int, default=1, help="number of ranks to shard for")
    ap.add_argument("--layers", default=None, help="e.g. 0-2,5 (default: all)")
    ap.add_argument("--shape", default="full", choices=["full", "toy"], help="model arguments preset")
    ap.add_argument("--device", default="cpu", help="where to pack (cpu or cuda:N)")
    ns = ap.parse_args()
    args = full_layer_args() if ns.shape == "full" else toy_model_args()
    cfg = Path(ns.hf) / "config.json"
    if cfg.exists():  # take the layer count from the checkpoint when it says so
        n = json.loads(cfg.read_text()).get("num_hidden_layers")
        if n:
            args.n_layers = int(n)
    files = convert(ns.hf, ns.out, args, ns.world, _parse_layers(ns.layers), ns.device)
    print(f"wrote {len(files)} files under {ns.out}")


if __name__ == "__main__":
    main()
