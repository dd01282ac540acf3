"""The allocation-free product entry point (``tilert_b200_matvec_fp8_static``).

Some hosts of this library may not allocate device memory at call time -- a plug-in inside a
runtime that owns the GPU memory pool, or a serving loop whose memory budget is frozen -- so one
entry point keeps its scratch in a fixed array inside the library instead of a context.  It must
give exactly what the context-based operator gives, on repeated calls (the array keeps the previous
call's contents), and must refuse sizes its array cannot cover.  Collected last on purpose.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def test_static_scratch_product_matches_context_operator_twice():
    import tilert_b200
    from tilert_b200 import pack
    from tilert_b200.models.deepseek_v3_2 import ops

    lib = tilert_b200.load_backend("deepseek_v3_2")
    tilert_b200.tilert_init(0)
    g = torch.Generator().manual_seed(123)
    n, k, tokens = 1000, 2048, 2      # 8 row tiles (the last one ragged), 16 k blocks: tiles split across thread blocks
    w = (torch.randn(n, k, generator=g) * 0.05).clamp(-400, 400).to(torch.float8_e4m3fn)
    scale = torch.rand((n + 127) // 128, k // 128, generator=g) * 0.01 + 0.001
    wp = pack.pack_matrix(w.cuda(), scale.cuda())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):
        x = (torch.randn(1, tokens, k, generator=g)).to(BF16).cuda()
        res = (torch.randn(1, tokens, n, generator=g)).to(BF16).cuda()
        want = torch.zeros(1, tokens, n, dtype=BF16, device="cuda")
        ops.unproj_o_allreduce(x, wp, None, res, 0, want)
        got = torch.full((1, tokens, n), 7.0, dtype=BF16, device="cuda")
        status = torch.full((1,), -1, dtype=torch.int32, device="cuda")
        mem_before = torch.cuda.memory_allocated()
        rc = lib.tilert_b200_matvec_fp8_static(_p(x), _p(wp), _p(res), tokens, k, n, _p(got), _p(status), stream)
        assert rc == 0, lib.tilert_b200_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == mem_before
        assert int(status) == 0
        ref = (x.float().cpu() @ (w.float() * scale.repeat_interleave(128, 0)[:n].repeat_interleave(128, 1)).T
               + res.float().cpu())
        cos = torch.nn.functional.cosine_similarity(ref.flatten(), got.float().cpu().flatten(), dim=0).item()
        assert cos >= 0.999, (call, cos)
        assert torch.equal(got, want), (call, (got.float() - want.float()).abs().max().item())
    assert tilert_b200.device_status(0) == 0


def test_static_scratch_shared_activation_blocks_three_calls_back_to_back():
    """A product with more units per thread block than ring slots (n = 4096, k = 8192: 2048 units), so the
    thread blocks share the activation conversion through the X-block part of the static array and its
    ready flags; three calls are queued on one stream without a host synchronisation in between, each with
    new activations, so every call must find the flags and their epoch cleared by its own start."""
    import tilert_b200
    from tilert_b200.models.deepseek_v3_2 import ops

    lib = tilert_b200.load_backend("deepseek_v3_2")
    tilert_b200.tilert_init(0)
    n, k, tokens = 4096, 8192, 1
    g = torch.Generator(device="cuda").manual_seed(5)
    wp = torch.randint(0, 120, (n // 128, k // 128, 16448), generator=g, dtype=torch.uint8, device="cuda")
    wp[:, :, 16384:] = 0
    wp[:, :, 16384:].view(torch.float32).copy_(torch.rand(n // 128, k // 128, 16, generator=g, device="cuda") * 1e-3 + 1e-3)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    xs = [torch.randn(1, tokens, k, generator=g, device="cuda").to(BF16) for _ in range(3)]
    res = torch.randn(1, tokens, n, generator=g, device="cuda").to(BF16)
    wants = []
    for x in xs:
        w_ = torch.zeros(1, tokens, n, dtype=BF16, device="cuda")
        ops.unproj_o_allreduce(x, wp, None, res, 0, w_)
        wants.append(w_)
    torch.cuda.synchronize()
    gots = [torch.full((1, tokens, n), 7.0, dtype=BF16, device="cuda") for _ in range(3)]
    stats = [torch.full((1,), -1, dtype=torch.int32, device="cuda") for _ in range(3)]
    for x, got, st in zip(xs, gots, stats):
        rc = lib.tilert_b200_matvec_fp8_static(_p(x), _p(wp), _p(res), tokens, k, n, _p(got), _p(st), stream)
        assert rc == 0, lib.tilert_b200_last_error()
    torch.cuda.synchronize()
    for i, (got, want, st) in enumerate(zip(gots, wants, stats)):
        assert int(st) == 0, i
        assert torch.isfinite(want.float()).all() and want.float().abs().max() > 0
        assert torch.equal(got, want), (i, (got.float() - want.float()).abs().max().item())
    assert not torch.equal(wants[0], wants[1])


def test_static_scratch_product_rejects_oversized_problems():
    import tilert_b200

    lib = tilert_b200.load_backend("deepseek_v3_2")
    dummy = torch.zeros(16, dtype=torch.uint8, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.tilert_b200_matvec_fp8_static(_p(dummy), _p(dummy), None, 1, 128, 131072 + 128, _p(dummy), None, stream)
    assert rc != 0 and b"static scratch" in lib.tilert_b200_last_error()
    rc = lib.tilert_b200_matvec_fp8_static(_p(dummy), _p(dummy), None, 5, 128, 128, _p(dummy), None, stream)
    assert rc != 0
