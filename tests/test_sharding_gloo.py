"""CPU tier, two gloo ranks: the per-rank weight shards that ``LayerWeights`` packs for tensor
parallelism reproduce the unsharded oracle products once the row-parallel partials are summed.

The products are evaluated on the CPU straight from the packed blocks (``pack.unpack_rows`` inverts
the device layout), so this checks the host logic -- head / expert-slice selection, scale slicing,
row regrouping -- and the all-reduce contract (sum of partials + residual), with no GPU."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import model as om
from oracle import ops as oo
from tilert_b200 import pack
from tilert_b200.models.deepseek_v3_2 import layer as L
from tilert_b200.models.deepseek_v3_2.model_args import toy_model_args


def dense_from_packed(packed: torch.Tensor, n_rows: int) -> torch.Tensor:
    """f32 matrix [n_rows, K] a packed weight represents (e4m3 value * its row scale)."""
    w, rs = pack.unpack_rows(packed, n_rows)
    return w.view(torch.float8_e4m3fn).float() * rs.repeat_interleave(128, dim=1)


def _worker(rank: int, world: int, port: int, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        a, margs = om.toy_args(), toy_model_args()
        sd = om.random_state_dict(a, seed=0)
        g = torch.Generator().manual_seed(9)
        hl = a.n_heads // world
        errs = {}
        for li in (0, 1):
            ow = om.LayerWeights(a, sd, li)
            gw = L.LayerWeights(margs, sd, li, "cpu", world, rank)
            # o_proj: this rank's heads, summed over ranks, plus the residual
            o = (torch.randn(1, 1, a.n_heads, a.v_head_dim, generator=g)).to(torch.bfloat16)
            res = torch.randn(1, 1, a.dim, generator=g).to(torch.bfloat16)
            part = o[:, :, rank * hl:(rank + 1) * hl].reshape(1, -1).float() @ dense_from_packed(gw.w_o, a.dim).T
            dist.all_reduce(part)
            ref = oo.unproj_o(o, ow.w_o).float().view(1, -1)
            errs[f"l{li}.o_proj"] = float((part - ref).norm() / ref.norm())
            # q_b rows of this rank: [nope of local heads | rope of local heads | indexer (replicated)]
            q_a = torch.randn(1, 1, a.q_lora_rank, generator=g).to(torch.bfloat16)
            qr = oo.rms_norm_f32(q_a, ow.q_norm, a.eps).to(torch.bfloat16).float().view(-1)
            rows = hl * (a.qk_nope_head_dim + a.qk_rope_head_dim) + a.index_n_heads * a.index_head_dim
            y = dense_from_packed(gw.w_qb, rows) @ qr
            rn, rp = oo.rmsnorm_projq_wqb(q_a, ow.q_norm, ow.wq_b, a.n_heads, a.qk_nope_head_dim, a.qk_rope_head_dim, a.eps)
            want = torch.cat([rn[0, 0, rank * hl:(rank + 1) * hl].reshape(-1), rp[0, 0, rank * hl:(rank + 1) * hl].reshape(-1),
                              oo.rmsnorm_projq_wqi(q_a, ow.q_norm, ow.wqi, a.index_head_dim, a.eps).reshape(-1)]).float()
            errs[f"l{li}.q_b"] = float((y - want).norm() / want.norm())
            if ow.dense:
                h = torch.randn(1, 1, a.dim, generator=g).to(torch.bfloat16)
                xn = oo.rms_norm_f32(h, ow.post_norm, a.eps).view(-1)
                il = a.inter_dim // world
                gu = dense_from_packed(gw.w_gu, 2 * il) @ xn                      # rows interleaved (8 gate, 8 up)
                gu = gu.view(il // 8, 2, 8)
                hid = (torch.nn.functional.silu(gu[:, 0]) * gu[:, 1]).reshape(-1).to(torch.bfloat16)
                ref_hid = oo.dense_up_gate_silu(h, ow.post_norm, ow.w_gate, ow.w_up, a.eps).view(-1)[rank * il:(rank + 1) * il]
                errs["l0.gate_up"] = float((hid.float() - ref_hid.float()).norm() / ref_hid.float().norm())
                full_hid = oo.dense_up_gate_silu(h, ow.post_norm, ow.w_gate, ow.w_up, a.eps)
                part = full_hid.view(-1)[rank * il:(rank + 1) * il].float() @ dense_from_packed(gw.w_down, a.dim).T
                dist.all_reduce(part)
                ref = full_hid.view(-1).float() @ ow.w_down.float().T
                errs["l0.down"] = float((part - ref).norm() / ref.norm())
            else:
                il = a.moe_inter_dim // world
                e = 5
                hvec = torch.randn(a.moe_inter_dim, generator=g).to(torch.bfloat16)
                part = hvec[rank * il:(rank + 1) * il].float() @ dense_from_packed(gw.w_down[e], a.dim).T
                dist.all_reduce(part)
                ref = hvec.float() @ ow.expert(f"experts.{e}")[2].float().T
                errs["l1.expert_down"] = float((part - ref).norm() / ref.norm())
                assert gw.w_gu.shape[0] == a.n_routed_experts + 1     # shared expert in the last slot
        if rank == 0:
            out_q.put(errs)
    finally:
        dist.destroy_process_group()


def test_two_rank_shards_sum_to_the_unsharded_products():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 200
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    errs = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # the goldens round dequantised weights to bf16; the packed path keeps fp8 * scale exact
    for name, e in errs.items():
        assert e < 5e-3, (name, e)
