"""What the kernels do when a bounded wait runs out: they return, leave a status code for the host and the
context stays usable.  The failure is made on the host side only -- a "peer" that never sends (a second local
buffer nobody writes) and a short wait budget -- never by faulting, trapping or hanging the GPU."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def test_all_reduce_gives_up_on_a_silent_peer_and_the_context_recovers():
    import tilert_b200
    from tilert_b200.models.deepseek_v3_2 import ops

    lib = tilert_b200.load_backend("deepseek_v3_2")
    ctx = ctypes.c_void_p(tilert_b200.tilert_init(0))
    assert tilert_b200.device_status(0) == 0
    n, k = 512, 1024
    g = torch.Generator(device="cuda").manual_seed(9)
    wp = torch.randint(0, 120, (n // 128, k // 128, 16448), generator=g, dtype=torch.uint8, device="cuda")
    wp[:, :, 16384:] = 0
    wp[:, :, 16384:].view(torch.float32).fill_(1e-3)
    x = torch.randn(1, 1, k, generator=g, device="cuda").to(BF16)
    res = torch.randn(1, 1, n, generator=g, device="cuda").to(BF16)

    # a communicator of two "ranks" in one process: rank 0 is real, rank 1's buffer is memory nobody writes
    nbytes = lib.tilert_b200_comm_buffer_bytes(2, n)
    bufs = (ctypes.c_void_p * 2)()
    for i in range(2):
        ptr = ctypes.c_void_p()
        tilert_b200.check(lib.tilert_b200_dev_alloc(nbytes, ctypes.byref(ptr)))
        bufs[i] = ptr.value
    comm = ctypes.c_void_p()
    tilert_b200.check(lib.tilert_b200_comm_create(ctx, 2, 0, bufs, n, ctypes.byref(comm)))
    try:
        tilert_b200.set_wait_budget(4_000_000)  # ~2 ms
        out = torch.full((1, 1, n), 7.0, dtype=BF16, device="cuda")
        ops.unproj_o_allreduce(x, wp, None, res, 0, out, comm=comm.value)
        torch.cuda.synchronize()  # the kernel RETURNS
        assert tilert_b200.device_status(0) == 3  # ST_PEER_TIMEOUT, read and cleared
        assert tilert_b200.device_status(0) == 0
        assert bool((out == 7.0).all()), "rows whose peer partial never arrived must not be written"
    finally:
        tilert_b200.set_wait_budget(0)
        lib.tilert_b200_comm_destroy(comm)
        for i in range(2):
            lib.tilert_b200_dev_free(ctypes.c_void_p(bufs[i]))
    # the context is still good: the same product without a communicator
    want = torch.zeros(1, 1, n, dtype=BF16, device="cuda")
    ops.unproj_o_allreduce(x, wp, None, res, 0, want)
    again = torch.zeros_like(want)
    with ops.chain("cuda:0"):
        ops.unproj_o_allreduce(x, wp, None, res, 0, again)
    torch.cuda.synchronize()
    assert tilert_b200.device_status(0) == 0
    assert torch.isfinite(want.float()).all() and torch.equal(want, again)


def test_chained_launch_gives_up_when_a_signal_never_completes():
    """A chained launch whose second product waits for a peer that never sends: the first phase's all-reduce
    runs out of its budget, the CTAs skip the rest, every thread-block barrier is still executed and the
    kernel returns with a status code; the signal counters are clean again for the next chained launch."""
    import tilert_b200
    from tilert_b200.models.deepseek_v3_2 import ops

    lib = tilert_b200.load_backend("deepseek_v3_2")
    ctx = ctypes.c_void_p(tilert_b200.tilert_init(0))
    n, k = 512, 512
    g = torch.Generator(device="cuda").manual_seed(10)
    wp = torch.randint(0, 120, (n // 128, k // 128, 16448), generator=g, dtype=torch.uint8, device="cuda")
    wp[:, :, 16384:] = 0
    wp[:, :, 16384:].view(torch.float32).fill_(1e-3)
    x = torch.randn(1, 1, k, generator=g, device="cuda").to(BF16)
    nbytes = lib.tilert_b200_comm_buffer_bytes(2, n)
    bufs = (ctypes.c_void_p * 2)()
    for i in range(2):
        ptr = ctypes.c_void_p()
        tilert_b200.check(lib.tilert_b200_dev_alloc(nbytes, ctypes.byref(ptr)))
        bufs[i] = ptr.value
    comm = ctypes.c_void_p()
    tilert_b200.check(lib.tilert_b200_comm_create(ctx, 2, 0, bufs, n, ctypes.byref(comm)))
    y = torch.zeros(1, 1, n, dtype=BF16, device="cuda")
    z = torch.full((1, 1, n), 7.0, dtype=BF16, device="cuda")
    try:
        tilert_b200.set_wait_budget(4_000_000)
        with ops.chain("cuda:0"):
            ops.unproj_o_allreduce(x, wp, None, None, 0, y, comm=comm.value)  # waits for the silent peer
            ops.unproj_o_allreduce(y, wp, None, None, 0, z)                   # depends on it
        torch.cuda.synchronize()
        assert tilert_b200.device_status(0) != 0
        assert bool((z == 7.0).all())
    finally:
        tilert_b200.set_wait_budget(0)
        lib.tilert_b200_comm_destroy(comm)
        for i in range(2):
            lib.tilert_b200_dev_free(ctypes.c_void_p(bufs[i]))
    a = torch.zeros(1, 1, n, dtype=BF16, device="cuda")
    b = torch.zeros(1, 1, n, dtype=BF16, device="cuda")
    ops.unproj_o_allreduce(x, wp, None, None, 0, a)
    with ops.chain("cuda:0"):
        ops.unproj_o_allreduce(x, wp, None, None, 0, b)
    torch.cuda.synchronize()
    assert tilert_b200.device_status(0) == 0 and torch.equal(a, b)
