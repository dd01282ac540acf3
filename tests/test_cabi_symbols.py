"""CPU tier: the built library loads and exports every function ``include/tilert_b200.h``
declares; host-side packers round-trip.  No kernel is launched."""

import torch

import tilert_b200
from tilert_b200 import _cabi, build, pack


def test_library_builds_and_exports_every_declared_symbol():
    path = build.build()
    assert path.exists()
    lib = tilert_b200.load_backend("deepseek_v3_2")
    protos = _cabi.parse_header()
    assert len(protos) >= 35
    for name in protos:
        assert hasattr(lib, name), name
    assert lib.tilert_b200_dsa_temp_vars_size() == 56
    assert lib.tilert_b200_xpack_bytes(7168) == 56 * 1056
    assert lib.tilert_b200_launch_count() == 0


def test_unknown_backend_raises():
    import pytest

    with pytest.raises(ValueError):
        tilert_b200.load_backend("glm5")


def test_temp_var_indices_match_native():
    from tilert_b200.models.deepseek_v3_2.temp_var_indices import Idx, validate_temp_vars_layout

    validate_temp_vars_layout()
    assert Idx.TOKEN_OUT == 25 and Idx.IDX_SEL_WS == 42


def test_ops_refuse_cpu_tensors():
    import pytest
    from tilert_b200.models.deepseek_v3_2 import ops

    with pytest.raises(ValueError):
        ops.rmsnorm_kv(torch.zeros(1, 1, 512, dtype=torch.bfloat16), torch.ones(512), torch.zeros(1, dtype=torch.int32),
                       torch.zeros(1, 8, 512, dtype=torch.bfloat16))


def test_weight_pack_round_trip_and_byte_map():
    g = torch.Generator().manual_seed(0)
    w = torch.randint(0, 255, (576, 1024), generator=g, dtype=torch.uint8)
    s = torch.rand(5, 8, generator=g) + 0.1
    p = pack.pack_matrix(w, s)
    assert p.shape == (5, 8, pack.WBLK_BYTES)
    w2, rs = pack.unpack_rows(p, 576)
    assert torch.equal(w2, w) and torch.equal(rs, pack.row_scales(s, 576))
    # the documented byte map of a W block (tilert_b200/csrc/formats.h)
    for t, kb, c, rg, kc, r, b in [(0, 0, 0, 0, 0, 0, 0), (4, 7, 3, 9, 1, 5, 13), (2, 5, 2, 15, 0, 7, 3)]:
        row = t * 128 + rg * 8 + r
        col = kb * 128 + 32 * c + 16 * kc + b
        exp = int(w[row, col]) if row < 576 else 0
        assert int(p[t, kb, c * 4096 + rg * 256 + kc * 128 + r * 16 + b]) == exp


def test_gate_up_interleave_and_absorb_transpose():
    g = torch.Generator().manual_seed(1)
    gate = torch.randint(0, 255, (256, 256), generator=g, dtype=torch.uint8)
    up = torch.randint(0, 255, (256, 256), generator=g, dtype=torch.uint8)
    sg, su = torch.rand(2, 2, generator=g) + 0.1, torch.rand(2, 2, generator=g) + 0.1
    w, rs = pack.unpack_rows(pack.pack_gate_up(gate, sg, up, su), 512)
    assert torch.equal(w[0:8], gate[0:8]) and torch.equal(w[8:16], up[0:8]) and torch.equal(w[16:24], gate[8:16])
    assert torch.equal(rs[8:16], pack.row_scales(su, 256)[0:8])
    heads, nope, v, c = 2, 128, 128, 256
    wkv = torch.randint(0, 255, (heads * (nope + v), c), generator=g, dtype=torch.uint8)
    skv = torch.rand(heads * 2, c // 128, generator=g) + 0.1
    wa, rsa = pack.unpack_rows(pack.pack_kv_b_absorb(wkv, skv, heads, nope, v), heads * c)
    assert int(wa[1 * c + 37, 5]) == int(wkv[1 * 256 + 5, 37])            # A[(h, c), d] = W[h, d, c]
    assert float(rsa[1 * c + 200, 0]) == float(skv[2, 1])                  # block (2h, c // 128)
    wv_, rsv = pack.unpack_rows(pack.pack_kv_b_v(wkv, skv, heads, nope, v), heads * v)
    assert torch.equal(wv_[v:2 * v], wkv[256 + 128: 512]) and float(rsv[v, 1]) == float(skv[3, 1])


def test_activation_split_is_exact_for_bf16():
    g = torch.Generator().manual_seed(2)
    x = (torch.randn(4, 2048, generator=g) * torch.logspace(-3, 3, 2048)).to(torch.bfloat16)
    rec = pack.reference_xpack(x)
    rel = (rec - x.float()).abs() / x.float().abs().amax(-1, keepdim=True)
    assert float(rel.max()) < 2 ** -18


def test_torch_ops_namespace_registers_reference_names():
    """The dispatcher names the reference's wrappers call exist after register() (no GPU work here)."""
    import torch

    from tilert_b200 import torch_ops

    torch_ops.register()
    torch_ops.register()  # idempotent
    for name in torch_ops.op_names():
        assert hasattr(torch.ops.tilert, name), name
    assert torch.ops.tilert.dsa_temp_vars_size() == 56
    schema = str(torch.ops.tilert.rmsnorm_kv_op.default._schema)
    assert schema.startswith("tilert::rmsnorm_kv_op(Tensor kv, Tensor gamma, Tensor cur_pos, Tensor(a!) kv_cache")

