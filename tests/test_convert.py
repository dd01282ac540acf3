"""Checkpoint converter: an HF-format FP8 safetensors checkpoint -> per-rank packed files (CPU only)."""

import json

import torch

from tilert_b200 import convert, synthetic
from tilert_b200.models.deepseek_v3_2.layer import LayerWeights
from tilert_b200.models.deepseek_v3_2.model_args import toy_model_args


def _toy_checkpoint(tmp_path, a):
    """Two-shard HF-style checkpoint of toy layers 0 (dense) and 1 (MoE) with an index file."""
    from safetensors.torch import save_file

    sd = {}
    for li in (0, 1):
        sd.update(synthetic.random_layer_state_dict(a, li, "cpu", seed=3))
    g = torch.Generator().manual_seed(5)
    sd["model.embed_tokens.weight"] = torch.randn(a.vocab_size, a.dim, generator=g).to(torch.bfloat16)
    sd["model.norm.weight"] = torch.rand(a.dim, generator=g) + 0.5
    sd["lm_head.weight"] = torch.randn(a.vocab_size, a.dim, generator=g).to(torch.bfloat16)
    keys = sorted(sd)
    shards = {"model-00001-of-00002.safetensors": keys[: len(keys) // 2],
              "model-00002-of-00002.safetensors": keys[len(keys) // 2:]}
    weight_map = {}
    for fname, ks in shards.items():
        save_file({k: sd[k].contiguous() for k in ks}, str(tmp_path / fname))
        weight_map.update({k: fname for k in ks})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    return sd


def test_convert_round_trip_matches_direct_packing(tmp_path):
    a = toy_model_args()
    hf = tmp_path / "hf"
    hf.mkdir()
    sd = _toy_checkpoint(hf, a)
    out = tmp_path / "packed"
    files = convert.convert(str(hf), str(out), a, world=2, layers=[0, 1])
    assert len(files) == 2 * 3 and (out / "manifest.json").exists()
    for rank in (0, 1):
        for li in (0, 1):
            direct = LayerWeights(a, sd, li, "cpu", 2, rank)
            loaded = convert.load_layer(out / f"rank{rank}" / f"layer_{li:03d}.safetensors", "cpu")
            assert loaded.dense == direct.dense and loaded.inter_local == direct.inter_local
            names = convert._COMMON + (() if direct.dense else convert._MOE_ONLY)
            for n in names:
                x, y = getattr(direct, n), getattr(loaded, n)
                assert x.dtype == y.dtype and x.shape == y.shape, n
                assert torch.equal(x.view(torch.uint8) if x.dtype == torch.uint8 else x, y), n
        head = convert.load_head(out / f"rank{rank}" / "head.safetensors", "cpu")
        v_l = a.vocab_size // 2
        assert torch.equal(head["head"], sd["lm_head.weight"][rank * v_l:(rank + 1) * v_l])
        assert torch.equal(head["embed"], sd["model.embed_tokens.weight"])


def test_lazy_checkpoint_reader(tmp_path):
    a = toy_model_args()
    sd = _toy_checkpoint(tmp_path, a)
    ck = convert.HFCheckpoint(tmp_path)
    k = "model.layers.1.self_attn.o_proj.weight"
    assert k in ck and torch.equal(ck[k].view(torch.uint8), sd[k].view(torch.uint8))
    try:
        ck["missing.key"]
    except KeyError:
        pass
    else:
        raise AssertionError("KeyError expected")


def test_convert_writes_the_prediction_layer(tmp_path):
    """A checkpoint with the multi-token-prediction layer: its decoder layer is packed like the others and its
    norms / eh_proj land in mtp.safetensors on every rank."""
    from safetensors.torch import save_file

    a = toy_model_args()
    hf = tmp_path / "hf"
    hf.mkdir()
    sd = _toy_checkpoint(hf, a)
    li = a.n_layers
    extra = synthetic.random_layer_state_dict(a, li, "cpu", seed=4)
    g = torch.Generator().manual_seed(6)
    p = f"model.layers.{li}"
    extra[f"{p}.enorm.weight"] = torch.rand(a.dim, generator=g) + 0.5
    extra[f"{p}.hnorm.weight"] = torch.rand(a.dim, generator=g) + 0.5
    extra[f"{p}.shared_head.norm.weight"] = torch.rand(a.dim, generator=g) + 0.5
    extra[f"{p}.eh_proj.weight"] = torch.randn(a.dim, 2 * a.dim, generator=g).to(torch.bfloat16)
    save_file({k: v.contiguous() for k, v in extra.items()}, str(hf / "model-mtp.safetensors"))
    index = json.loads((hf / "model.safetensors.index.json").read_text())
    index["weight_map"].update({k: "model-mtp.safetensors" for k in extra})
    (hf / "model.safetensors.index.json").write_text(json.dumps(index))
    sd.update(extra)

    out = tmp_path / "packed"
    files = convert.convert(str(hf), str(out), a, world=2)
    assert len(files) == 2 * (3 + 1 + 1)  # three decoder layers, mtp.safetensors, head per rank
    assert json.loads((out / "manifest.json").read_text())["mtp_layer"] == li
    for rank in (0, 1):
        small = convert.load_mtp(out / f"rank{rank}" / "mtp.safetensors", "cpu")
        assert torch.equal(small["eh_proj"], sd[f"{p}.eh_proj.weight"]) and small["enorm"].dtype == torch.float32
        assert torch.equal(small["shared_head_norm"], sd[f"{p}.shared_head.norm.weight"])
        direct = LayerWeights(a, sd, li, "cpu", 2, rank)
        loaded = convert.load_layer(out / f"rank{rank}" / f"layer_{li:03d}.safetensors", "cpu")
        assert not loaded.dense and torch.equal(loaded.w_o, direct.w_o) and torch.equal(loaded.w_gu, direct.w_gu)
    # asking for specific layers leaves the prediction layer out unless it is named
    files = convert.convert(str(hf), str(tmp_path / "some"), a, world=1, layers=[0], with_head=False)
    assert len(files) == 1


def test_pack_rows_ragged_row_count_round_trips():
    """A weight whose row count is neither a multiple of 128 nor of 8 (1001 rows) packs: the padding rows are
    zero bytes that repeat the last real row's scales, and unpacking returns the bytes and row scales."""
    from tilert_b200 import pack

    g = torch.Generator().manual_seed(1001)
    n, k = 1001, 384
    w = torch.randint(0, 255, (n, k), generator=g, dtype=torch.uint8)
    scale = torch.rand((n + 127) // 128, k // 128, generator=g) + 0.5
    packed = pack.pack_matrix(w, scale)
    assert packed.shape == (8, 3, pack.WBLK_BYTES)
    w2, rs2 = pack.unpack_rows(packed, n)
    assert torch.equal(w2, w)
    assert torch.equal(rs2, pack.row_scales(scale, n))
    two = pack.pack_bf16_two_term((torch.randn(70, 256, generator=g) * 0.02).to(torch.bfloat16))  # 70 rows: padded to 72
    assert two.shape == (2, 2, pack.WBLK_BYTES)
