#!/usr/bin/env python
"""Benchmark of the batch-1 FP8 decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: one full-shape DeepSeek-V3.2 MoE decoder layer (hidden 7168, 128 heads, 256 routed
experts top-8 + 1 shared, indexer 64x128 top-2048), batch 1, one decode step at position 4095 of
a 4096-row latent cache filled from N(0,1); random-init FP8 weights; router logits forced so the
eight routed experts are fixed (two in each of four expert groups).  A "step" is one pass of the layer over one token.
With N > 1 (launched by torch.distributed.run, one rank per GPU) the layer is tensor-parallel
over N GPUs and the two row-parallel products reduce inside their kernels over peer memory.

Prints ONE JSON line (rank 0).  ``--impl reference`` times the CPU restatement of the reference's
PyTorch path (the reference's fast path is a closed binary that is not in its source tree) on the
host cores, on the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

METRIC = "batch1_decode_layer_tokens_per_s"
UNIT = "tokens/s"
CACHE_LEN = 4096
WORKLOAD = ("C1: one full-shape DeepSeek-V3.2 MoE decoder layer, batch 1, 1 token/step, 4096-row latent KV "
            "cache, FP8 e4m3 weights with 128x128 block scales")


# DRAM traffic per algorithmic byte of the streaming kernel, from one ncu capture of
# `bench.py --profile-gemv` (dram__bytes_read.sum + dram__bytes_write.sum = 239.50 MB for 235.80 MB of weights).
NCU_TRAFFIC_RATIO = 239.50 / 235.80


def forced_scores(n_experts: int, top_k: int) -> torch.Tensor:
    """Router logits with `top_k` hot experts spread evenly: two in every other group of 32 (the
    group-limited routing keeps 4 of the 8 groups, so the hot experts must sit in 4 groups)."""
    s = torch.full((1, 1, n_experts), -8.0)
    s[0, 0, hot_experts(n_experts, top_k)] = 4.0
    return s


def hot_experts(n_experts: int, top_k: int) -> list[int]:
    group = n_experts // 8
    return sorted(g * group + j * (group // 2) for g in range(0, 8, 2) for j in range(top_k // 4))


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows: list[list[str]] = []
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def workload_inputs(S: int, cache_len: int):
    """The seeded synthetic workload, generated on the host so that every rank -- and the CPU checker --
    sees the same bytes: an HF-keyed FP8 state dict of the layer (only the hot experts are materialised;
    the forced router logits never select another), the three caches, the token's hidden state."""
    from tilert_b200 import synthetic
    from tilert_b200.models.deepseek_v3_2.model_args import full_layer_args

    a = full_layer_args(max_seq_len=cache_len)
    hot = hot_experts(a.n_routed_experts, a.n_activated_experts)
    sd = synthetic.random_layer_state_dict(a, 0, "cpu", seed=0, expert_ids=hot)
    g = torch.Generator().manual_seed(2)
    caches = [torch.randn(1, cache_len, d, generator=g, dtype=torch.float32).to(torch.bfloat16)
              for d in (a.kv_lora_rank, a.qk_rope_head_dim, a.index_head_dim)]
    x = torch.randn(1, S, a.dim, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    return a, hot, sd, caches, x


class CpuChecker:
    """The CPU restatement of the reference's PyTorch path (``oracle/``) on the bench's own workload: the
    checker of the GPU result (outside every timed region) and the reported CPU baseline."""

    def __init__(self, sd, caches, x, S: int, cache_len: int):
        from oracle import model as om
        from oracle import ops as oo

        torch.set_num_threads(os.cpu_count() or 1)  # torch.distributed.run exports OMP_NUM_THREADS=1
        self.om = om
        self.a = om.full_layer_args(max_seq_len=cache_len)
        self.w = om.LayerWeights(self.a, sd, 0)
        self.c = om.Caches(self.a, cache_len)
        for dst, src in zip((self.c.kv, self.c.pe, self.c.ki), caches):
            dst.copy_(src)
        self.x, self.pos = x, cache_len - S
        self.fc = oo.precompute_freqs_cis(self.a)
        self.fs = forced_scores(self.a.n_routed_experts, self.a.n_activated_experts).expand(1, S, -1).contiguous()

    def step(self) -> torch.Tensor:
        return self.om.layer_step(self.a, self.w, self.c, self.x, self.pos, self.fc, forced_router_scores=self.fs)

    def timed(self, n_steps: int, warmup: int) -> tuple[float, dict]:
        for _ in range(max(warmup, 1)):  # the first step also dequantises the nine active experts
            self.step()
        t0 = time.perf_counter()
        for _ in range(n_steps):
            self.step()
        dt = (time.perf_counter() - t0) / n_steps
        desc = {"kind": "port", "cores": torch.get_num_threads(),
                "sample": f"{n_steps} decode step(s) of the same layer (weights dequantised to bf16 once, outside the "
                          "timed region, as the reference goldens hold them)"}
        return dt, desc


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    _, _, sd, caches, x = workload_inputs(1, CACHE_LEN)
    chk = CpuChecker(sd, caches, x, 1, CACHE_LEN)
    steps, warmup = max(args.steps, 1), max(args.warmup, 1)
    dt, desc = chk.timed(steps, warmup)
    val = 1.0 / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp8_e4m3 weights (dequantised to bf16), f32 accumulate", "data": "synthetic",
        "config": {"workload": WORKLOAD, "parallelism": f"tp{args.gpus}", "cache_rows": CACHE_LEN, "tokens_per_step": 1},
        "note": "CPU restatement of the reference's golden_forward path on the host cores; the reference's GPU path "
                "is a closed binary absent from its source tree",
        "cpu_baseline": {"value": val, "unit": UNIT, **desc},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_ours(args) -> None:
    import torch.distributed as dist

    import tilert_b200
    from tilert_b200.models.deepseek_v3_2 import layer as L
    from tilert_b200.models.deepseek_v3_2 import ops
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the decode path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    tilert_b200.load_backend("deepseek_v3_2")
    tilert_b200.tilert_init(local)
    lib = tilert_b200.lib()

    # --tokens 4 --cache-rows 16384: the speculative-decoding verify step (four rows per pass) instead
    # of the headline workload
    S, cache_len = args.tokens, args.cache_rows
    workload = WORKLOAD if (S, cache_len) == (1, CACHE_LEN) else (
        f"C4-style verify step: one full-shape DeepSeek-V3.2 MoE decoder layer, batch 1, {S} tokens/step, "
        f"{cache_len}-row latent KV cache, FP8 e4m3 weights with 128x128 block scales")
    a, hot, sd, caches, x_cpu = workload_inputs(S, cache_len)
    comm = None
    if world > 1:
        from tilert_b200.comm import Comm

        comm = Comm(a.dim, local)
    weights = L.LayerWeights(a, sd, 0, dev, world, rank, expert_ids=hot)
    torch.cuda.empty_cache()
    layer = L.DecoderLayer(a, weights, dev, cache_len, S, world, None if comm is None else comm.handle)
    if args.mla_split:
        layer.mla_split = args.mla_split
    for dst, src in zip((layer.kv_cache, layer.pe_cache, layer.ki_cache), caches):
        dst.copy_(src)
    layer.forced_scores = forced_scores(a.n_routed_experts, a.n_activated_experts).expand(1, S, -1).contiguous().to(dev)
    x_host = x_cpu.pin_memory()
    out_host = torch.empty(1, S, a.dim, dtype=torch.bfloat16).pin_memory()
    x = x_host.to(dev)
    cur = torch.tensor([cache_len - S], dtype=torch.int32, device=dev)
    freqs = L.precompute_freqs(a)[cache_len - S: cache_len].contiguous().to(dev)

    def step():
        return layer.forward(x, cur, freqs, cache_len)

    # warm-up outside capture, then capture one step in a CUDA graph
    step()
    torch.cuda.synchronize()
    n0 = lib.tilert_b200_launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = step()
    launches_per_step = lib.tilert_b200_launch_count() - n0
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > L2 (126 MB)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        graph.replay()
    barrier()

    if args.trace_step:
        # one eager step with every streaming launch traced into its own record
        import ctypes
        n_rec = 16
        trace = torch.zeros(n_rec, 256, 16, dtype=torch.int64, device=dev)
        ctx = ctypes.c_void_p(tilert_b200.tilert_init(local))
        flush.fill_(1)
        torch.cuda.synchronize()
        tilert_b200.check(lib.tilert_b200_set_profile_ring(ctx, ctypes.c_void_p(trace.data_ptr()), n_rec))
        step()
        torch.cuda.synchronize()
        tilert_b200.check(lib.tilert_b200_set_profile(ctx, None))
        tr = trace.cpu().double()
        tr = tr[:, :148]
        used = [r for r in range(n_rec) if tr[r, :, 0].max() > 0]
        t_step0 = min(tr[r, :, 0][tr[r, :, 0] > 0].min() for r in used)
        rows = []
        for r in used:
            m = tr[r, :, 0] > 0
            ent, rdy, fd, lu, td, ex = (tr[r, m, i] for i in (0, 1, 2, 3, 4, 7))
            fc = tr[r, m, 5]
            nd = tr[r, m, 13]
            k0 = ent.min()
            rows.append({"launch": r, "ctas": int(m.sum()), "start_us": round(float(k0 - t_step0) / 1e3, 2),
                         "entry_max": round(float((ent - k0).max()) / 1e3, 2),
                         "ready_med": round(float((rdy - k0).median()) / 1e3, 2),
                         "norm_done_med": round(float((nd[nd > 0] - k0).median()) / 1e3, 2) if (nd > 0).any() else None,
                         "first_convert_med": round(float((fc[fc > 0] - k0).median()) / 1e3, 2) if (fc > 0).any() else None,
                         "first_data_med": round(float((fd - k0).median()) / 1e3, 2),
                         "tiles_done_max": round(float((td - k0).max()) / 1e3, 2),
                         "last_unit_min_med_max": [round(float(v) / 1e3, 2) for v in
                                                   ((lu - k0).min(), (lu - k0).median(), (lu - k0).max())],
                         "exit_max": round(float((ex - k0).max()) / 1e3, 2)})
        print(json.dumps({"mode": "trace-step", "launches": rows}), flush=True)
        if comm is not None:
            comm.close()
        return

    # ---- device-timed steps: L2 flushed (untimed) before each step ----
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    for i in range(args.steps):
        flush.fill_(i & 0xff)
        if world > 1:
            dist.barrier()
        starts[i].record()
        graph.replay()
        ends[i].record()
    barrier()
    dev_ms = sum(s.elapsed_time(e) for s, e in zip(starts, ends))
    # keep sampling clocks through a longer loaded stretch (about a second) so the median is meaningful.
    # Every rank must replay the step the SAME number of times -- a rank that did one more would wait
    # for partial sums nobody sends -- so the count is agreed on, not decided by each rank's clock.
    reps = torch.tensor([0 if args.profile else int(1000.0 * args.steps / max(dev_ms, 1e-3))], dtype=torch.int64,
                        device=dev)
    if world > 1:
        dist.all_reduce(reps, op=dist.ReduceOp.MIN)
    for _ in range(int(reps.item())):
        graph.replay()
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None

    def phase_status(name: str) -> int:
        """Device status word after a phase, worst over ranks (0 = every wait in every kernel was met)."""
        st = torch.tensor([tilert_b200.device_status(local)], dtype=torch.int64, device=dev)
        if world > 1:
            dist.all_reduce(st, op=dist.ReduceOp.MAX)
        if rank == 0 and int(st.item()) != 0:
            print(f"bench: device status {int(st.item())} after {name}", file=sys.stderr, flush=True)
        return int(st.item())

    healthy = phase_status("the timed steps and the load loop") == 0

    # ---- the same layer four times per replay, each pass fed by the previous one: what a layer costs
    # inside a model, where its first launch overlaps the previous layer's tail instead of a cold start
    # (the weights are 4-8x the L2, so every pass still streams them from HBM) ----
    n_chain = 4
    chain_ms = None
    if not args.profile and healthy:
        def chain():
            y = x
            for _ in range(n_chain):
                y = layer.forward(y, cur, freqs, cache_len)
            return y
        chain()
        torch.cuda.synchronize()
        g4 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g4):
            chain()
        c0 = [torch.cuda.Event(enable_timing=True) for _ in range(10)]
        c1 = [torch.cuda.Event(enable_timing=True) for _ in range(10)]
        barrier()
        for i in range(10):
            flush.fill_(i & 0xff)
            if world > 1:
                dist.barrier()
            c0[i].record()
            g4.replay()
            c1[i].record()
        barrier()
        chain_ms = sum(a_.elapsed_time(b_) for a_, b_ in zip(c0, c1)) / 10 / n_chain
        phase_status("the chained passes")

    # ---- end to end: host buffers, H2D + step + D2H inside the timed region ----
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        x.copy_(x_host, non_blocking=True)
        graph.replay()
        out_host.copy_(out, non_blocking=True)
        torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()

    # ---- dominant kernel alone: the routed+shared expert up/gate product (9 experts x 29.4 MB) ----
    n_slots = a.n_activated_experts + 1
    k_iters = 2 if args.profile else 20
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def upgate():
        ops.expert_select_up_gate_silu(layer.h_norm, layer.forced_scores, weights.router_bias, weights.w_gu,
                                       layer.ffn_hidden, layer.probs, layer.eidx, dim=a.dim,
                                       n_groups=a.n_expert_groups, n_limited_groups=a.n_limited_groups,
                                       route_scale=a.route_scale, slot_ids=layer.slot_ids, slot_w=layer.slot_w)
    g2 = torch.cuda.CUDAGraph()
    upgate()
    torch.cuda.synchronize()
    with torch.cuda.graph(g2):
        for _ in range(k_iters):
            upgate()
    g2.replay()
    torch.cuda.synchronize()
    flush.fill_(1)
    ev0.record()
    g2.replay()
    ev1.record()
    torch.cuda.synchronize()
    # each iteration = 1 routing launch (a few us, one warp) + 1 streaming launch; subtract nothing, report as is
    upgate_ms = ev0.elapsed_time(ev1) / k_iters
    upgate_bytes = n_slots * weights.w_gu[0].numel()

    # ---- output check, outside every timed region: all ranks' results bit-identical, and rank 0's result
    # against the CPU restatement of the reference on the same seeded inputs ----
    graph.replay()
    torch.cuda.synchronize()
    result = out.clone()
    ranks_identical = True
    if world > 1:
        gathered = [torch.empty_like(result) for _ in range(world)]
        dist.all_gather(gathered, result)
        ranks_identical = all(torch.equal(gathered[0], g_) for g_ in gathered[1:])
    parity, checker = None, None
    if rank == 0 and not args.profile:
        checker = CpuChecker(sd, caches, x_cpu, S, cache_len)
        ref = checker.step().float().flatten()
        got = result.float().cpu().flatten()
        cos = torch.nn.functional.cosine_similarity(ref, got, dim=0).item()
        rel = (torch.norm(ref - got) / torch.norm(ref)).item()
        parity = {"cos": cos, "rel_l2": rel, "ranks_identical": bool(ranks_identical),
                  "checker": "CPU restatement of the reference's golden_forward path, same seeded weights, caches and input",
                  "bounds": {"cos_min": 0.999, "rel_l2_max": 2e-2}}
        parity["ok"] = bool(cos >= 0.999 and rel <= 2e-2 and ranks_identical)

    status = tilert_b200.device_status(local)
    t = torch.tensor([dev_ms, e2e_s, float(status), chain_ms or 0.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_s, status, chain_ms = t.tolist()

    peaks = {}
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        peaks = json.loads(pk.read_text())
    peak_gbs = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "fallback 6650 GB/s"

    if rank == 0:
        ms_per_step = dev_ms / args.steps
        step_bytes = weights.weight_bytes(a) + a.index_topk * (a.kv_lora_rank + a.qk_rope_head_dim) * 2 \
            + cache_len * a.index_head_dim * 2
        achieved = upgate_bytes / (upgate_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": 1000.0 * S / ms_per_step, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "fp8_e4m3 (weights and activations as two e4m3 terms), f32 accumulate", "data": "synthetic",
            "config": {"workload": workload, "parallelism": f"tp{world}", "cache_rows": cache_len, "tokens_per_step": S,
                       "l2": "256 MB buffer written before every timed step (untimed); per-step weights (>=75 MB "
                             "per GPU) are streamed with an evict-first policy",
                       "timing": "CUDA events around each CUDA-graph replay of the step, summed over steps, max over ranks"},
            "e2e": {"value": args.steps * S / e2e_s, "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * 2,
                    "d2h_bytes_per_step": out_host.numel() * 2},
            "gpu_launches": int(launches_per_step * args.steps),
            "launches_per_step": int(launches_per_step),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "wstream_gemv_kernel (expert up/gate launch, 9 experts)",
                         "achieved": achieved, "peak": peak_gbs, "unit": "GB/s", "frac": achieved / peak_gbs,
                         "peak_source": peak_src, "traffic": upgate_bytes * NCU_TRAFFIC_RATIO,
                         "traffic_source": "ncu dram read+write of the same kernel on a 235.8 MB weight "
                                           "(239.5 MB per launch), scaled by bytes streamed",
                         "bytes_per_launch": upgate_bytes, "launch_ms": upgate_ms},
            "step_roofline": {"bytes_per_step_this_gpu": step_bytes, "achieved": step_bytes / (ms_per_step * 1e-3) / 1e9,
                              "frac": step_bytes / (ms_per_step * 1e-3) / 1e9 / peak_gbs, "unit": "GB/s"},
            "device_status": int(status),
            "parity": parity,
        }
        if chain_ms:
            line["chained_layers"] = {"passes_per_replay": n_chain, "ms_per_layer": chain_ms,
                                      "step_roofline_frac": step_bytes / (chain_ms * 1e-3) / 1e9 / peak_gbs}
        if S > 1:
            # every row is verified; on average `accept` of them are emitted per step
            line["speculative"] = {"rows_per_step": S, "assumed_mean_accepted": 3.2,
                                   "emitted_tokens_per_s": 1000.0 * min(3.2, S) / ms_per_step}
        if world == 1 and S == 1 and not args.no_cpu_baseline and checker is not None:
            try:
                dt, desc = checker.timed(20, 2)
                line["cpu_baseline"] = {"value": 1.0 / dt, "unit": UNIT, **desc}
            except Exception as e:  # noqa: BLE001  (report the GPU numbers even if the CPU leg fails)
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "error": f"{type(e).__name__}: {e}"}
        print(json.dumps(line), flush=True)
    failed = torch.tensor([1 if (rank == 0 and parity is not None and not parity["ok"]) or status != 0 else 0], device=dev)
    if world > 1:
        dist.all_reduce(failed, op=dist.ReduceOp.MAX)
    if comm is not None:
        comm.close()
    if world > 1:
        dist.destroy_process_group()
    if int(failed.item()):
        print("bench: the output check or the device status failed (see \"parity\" / \"device_status\")", file=sys.stderr)
        sys.exit(1)


def _peak_gbs() -> tuple[float, str]:
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        return float(json.loads(pk.read_text()).get("hbm_gbs", 6650.0)), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback 6650 GB/s"


def run_c2(args) -> None:
    """Workload C2: the whole model -- ``--layers`` decoder layers of the full shape (61 in the real model, the
    first three dense), vocabulary 129280 -- tensor-parallel over the ranks, greedy decoding from contexts of
    ``--ctx`` tokens (a comma-separated list: the model is built once) whose caches are filled with N(0, 1).
    Weights are drawn at random per rank directly in the packed block format on the device.  Prints one JSON
    line per context (and per launch mode with ``--chain both``): the time per output token (CUDA events around
    every step: graph replay of layers, head and greedy token exchange), its median, tokens/s and the fraction
    of the HBM roofline.  ``--with-mtp`` times speculative steps (four rows verified, three drafted)."""
    import torch.distributed as dist

    import tilert_b200
    from dataclasses import replace
    from tilert_b200 import synthetic
    from tilert_b200.models.deepseek_v3_2.model import DsaModel
    from tilert_b200.models.deepseek_v3_2.model_args import ModelArgs

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    tilert_b200.load_backend("deepseek_v3_2")
    tilert_b200.tilert_init(local)
    n_new, n_warm = args.steps, max(args.warmup, 3)
    contexts = [int(c) for c in str(args.ctx).split(",")]
    rows = 4 if args.with_mtp else 1
    cache_len = (max(contexts) + rows * (n_new + n_warm) * 2 + 16 + 255) // 256 * 256
    a = replace(ModelArgs(), n_layers=args.layers, n_dense_layers=min(3, max(args.layers - 1, 0)), max_seq_len=cache_len)
    comm = None
    if world > 1:
        from tilert_b200.comm import Comm

        comm = Comm(a.dim, local)
    t0 = time.perf_counter()
    packed = synthetic.random_packed_model(a, dev, world, rank, seed=0, with_mtp=args.with_mtp)
    handle = None if comm is None else comm.handle
    if args.with_mtp:
        from tilert_b200.models.deepseek_v3_2.mtp import MtpDsaModel

        model = MtpDsaModel(a, packed, dev, cache_len=cache_len, world=world, rank=rank, comm=handle)
        layers = model.layers + [model.mtp_layer]
    else:
        model = DsaModel(a, packed, dev, cache_len=cache_len, world=world, rank=rank, comm=handle, share_scratch=True)
        layers = model.layers
    g = torch.Generator(device=dev).manual_seed(5)  # the same cache contents on every rank
    for layer in layers:
        for t in (layer.kv_cache, layer.pe_cache, layer.ki_cache):
            t[:, : max(contexts)].copy_(torch.randn(1, max(contexts), t.shape[-1], generator=g, device=dev).to(torch.bfloat16))
    torch.cuda.synchronize()
    build_s = time.perf_counter() - t0
    weight_bytes = sum(l.w.weight_bytes(a) for l in model.layers) + model.head.numel() * 2
    peak, peak_src = _peak_gbs()
    modes = {"both": [True, False], "on": [True], "off": [False], "default": [None]}[args.chain]

    for ctx_len in contexts:
        for chained in modes:
            if chained is not None:
                for layer in layers:
                    layer.chained = chained
            model._graphs.clear()
            model.set_cur_pos(ctx_len)
            accepted = []
            if args.with_mtp:
                draft = torch.ones(4, dtype=torch.int64, device=dev)

                def step(_i):
                    nonlocal draft
                    model.forward(draft)
                    accepted.append(model.get_num_accepted())  # one host read per step, as in the reference's loop
                    draft = model.next_draft.clone()
            else:
                tok = torch.tensor([1], dtype=torch.int64, device=dev)

                def step(i):
                    nonlocal tok
                    model.forward(tok, ctx_len + i)
                    tok = model.token_out  # the device feeds the next step: no host read in the loop
            for i in range(n_warm):  # also captures the graph of this scan-length bucket
                step(i)
            accepted.clear()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            sampler = ClockSampler(local)
            if rank == 0:
                sampler.start()
            ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_new)]
            for i in range(n_new):
                ev[i][0].record()
                step(n_warm + i)
                ev[i][1].record()
            torch.cuda.synchronize()
            clocks = sampler.stop() if rank == 0 else None
            times = torch.tensor([s_.elapsed_time(e_) for s_, e_ in ev], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(times, op=dist.ReduceOp.MAX)
            status = torch.tensor([tilert_b200.device_status(local)], dtype=torch.int64, device=dev)
            if world > 1:
                dist.all_reduce(status, op=dist.ReduceOp.MAX)
            if rank != 0:
                continue
            ts = sorted(times.tolist())
            med = ts[len(ts) // 2]
            kv_bytes = a.n_layers * (a.index_topk * (a.kv_lora_rank + a.qk_rope_head_dim) * 2 + ctx_len * a.index_head_dim * 2)
            bytes_gpu = weight_bytes + kv_bytes
            line = {
                "metric": "batch1_decode_tpot_ms", "value": med, "unit": "ms", "n_gpus": world, "steps": n_new,
                "warmup": n_warm, "ms_per_step": sum(ts) / len(ts), "higher_is_better": False, "scaling": "strong",
                "vs_baseline": None, "tokens_per_s": 1000.0 / med, "dtype": "fp8_e4m3 weights, f32 accumulate",
                "data": "synthetic",
                "config": {"workload": f"C2: {a.n_layers}-layer DeepSeek-V3.2-shape model ({a.n_dense_layers} dense), vocab "
                                       f"{a.vocab_size}, batch 1 greedy decode after a {ctx_len}-token context",
                           "parallelism": f"tp{world}", "context": ctx_len, "with_mtp": bool(args.with_mtp),
                           "chained_launches": layers[0].chained,
                           "weights": "random e4m3 blocks drawn per rank in the packed format on the device",
                           "timing": "CUDA events around every step (graph replay of layers + head + token exchange), "
                                     "max over ranks"},
                "tpot_ms": {"median": med, "min": ts[0], "p90": ts[int(len(ts) * 0.9)]},
                "speculative": None if not args.with_mtp else {
                    "rows_per_step": 4, "mean_accepted": sum(accepted) / max(len(accepted), 1),
                    "note": "value is the time of one speculative step (four rows verified, three drafted); with random "
                            "weights the drafts are almost never accepted, so tokens/s here is the floor: multiply by the "
                            "mean accepted length of a trained model",
                    "tokens_per_s_at_accept": {str(n): n * 1000.0 / med for n in (1, 2, 3, 4)}},
                "step_roofline": {"bytes_per_step_this_gpu": bytes_gpu, "achieved": bytes_gpu / (med * 1e-3) / 1e9,
                                  "frac": bytes_gpu / (med * 1e-3) / 1e9 / peak, "unit": "GB/s", "peak": peak,
                                  "peak_source": peak_src,
                                  "note": "bytes of one single-row pass; a speculative step streams more (four rows route "
                                          "to more experts, three more passes of the prediction layer and the head)"},
                "reference_published": {"tokens_per_s": 600, "source": "reference README: DeepSeek-V3.2 on 8x B200, best case"},
                "build_seconds": build_s, "clocks": clocks, "device_status": int(status.item()),
            }
            print(json.dumps(line), flush=True)
    if comm is not None:
        comm.close()
    if world > 1:
        dist.destroy_process_group()


def run_c3(args) -> None:
    """Workload C3: the long-context indexer stress at the full layer shape -- ``--ctx`` (131072) cached keys
    drawn from N(0, 1), one query token, exact top-2048, then sparse MLA over the selected latent rows.  Reports
    the microseconds of scoring + selection (one launch) and of attention (+ combine), the key-scan rate against
    the HBM peak, and the checks: indices identical to a CPU selection on the device's own scores, attention
    within cosine 0.999 of the CPU restatement on the same selection."""
    import tilert_b200
    from tilert_b200.models.deepseek_v3_2 import ops
    from tilert_b200.models.deepseek_v3_2.layer import softmax_scale
    from tilert_b200.models.deepseek_v3_2.model_args import full_layer_args

    tilert_b200.load_backend("deepseek_v3_2")
    tilert_b200.tilert_init(0)
    dev = torch.device("cuda", 0)
    T = args.ctx
    a = full_layer_args(max_seq_len=T)
    H, k = a.index_n_heads, a.index_topk
    g = torch.Generator(device=dev).manual_seed(7)
    rn = lambda *s, sc=1.0: (torch.randn(*s, generator=g, device=dev) * sc).to(torch.bfloat16)  # noqa: E731
    ki, kv, pe = rn(1, T, 128), rn(1, T, a.kv_lora_rank), rn(1, T, a.qk_rope_head_dim)
    iq, w = rn(1, 1, H, 128), rn(1, 1, H, sc=0.3)
    q_lat, q_pe = rn(1, 1, a.n_heads, a.kv_lora_rank, sc=0.3), rn(1, 1, a.n_heads, a.qk_rope_head_dim, sc=0.3)
    logits = torch.zeros(1, 1, T, dtype=torch.float32, device=dev)
    sel = torch.zeros(1, 1, k, dtype=torch.int32, device=dev)
    cur = torch.tensor([T - 1], dtype=torch.int32, device=dev)
    out = torch.zeros(1, 1, a.n_heads, a.kv_lora_rank, dtype=torch.bfloat16, device=dev)
    n_splits = k // 64
    o_acc = torch.zeros(1, 1, a.n_heads, n_splits, a.kv_lora_rank, dtype=torch.float32, device=dev)
    lse_acc = torch.zeros(1, 1, a.n_heads, n_splits, dtype=torch.float32, device=dev)
    lse = torch.zeros(1, 1, a.n_heads, dtype=torch.float32, device=dev)
    scale = softmax_scale(a)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def select():
        ops.sparse_index_topk(iq, ki, w, logits, sel, cur, n_keys=T)

    def attend():
        ops.flash_sparse_mla(q_lat, q_pe, kv, pe, sel, cur, out, softmax_scale=scale, split_size=64, out_acc=o_acc, lse=lse,
                             lse_acc=lse_acc)

    def timed(fn, n):
        ts = []
        for i in range(n):
            flush.fill_(i & 255)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return sorted(ts)[len(ts) // 2]

    for _ in range(max(args.warmup, 3)):
        select(); attend()
    torch.cuda.synchronize()
    us_sel, us_att = timed(select, args.steps), timed(attend, args.steps)
    # checks (outside the timed regions)
    lg = logits[0, 0, :T].float().cpu()
    kk = min(k, T)
    want = torch.sort(torch.topk(lg, kk, sorted=False).indices).values
    thr = torch.topk(lg, kk).values.min()
    got = sel[0, 0].cpu().long()
    got = torch.sort(got[got >= 0]).values
    if int((lg == thr).sum()) == 1:  # no tie at the threshold: the index set is unique
        idx_exact = bool(torch.equal(want, got))
    else:
        idx_exact = bool(got.numel() == kk and set(got.tolist()) >= set(torch.nonzero(lg > thr).flatten().tolist()))
    s_idx = sel[0, 0].long()
    s_idx = s_idx[s_idx >= 0]
    kq = torch.cat([kv[0, s_idx].float(), pe[0, s_idx].float()], dim=-1)                      # [k, 576]
    qq = torch.cat([q_lat[0, 0].float(), q_pe[0, 0].float()], dim=-1)                         # [h, 576]
    p_ = torch.softmax(qq @ kq.T * scale, dim=-1).to(torch.bfloat16).float()
    ref = (p_ @ kv[0, s_idx].float())
    cos = torch.nn.functional.cosine_similarity(ref.flatten(), out[0, 0].float().flatten(), dim=0).item()
    peak, peak_src = _peak_gbs()
    scan_bytes = T * 256
    line = {
        "metric": "dsa_stress_select_plus_attention_us", "value": us_sel + us_att, "unit": "us", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": (us_sel + us_att) * 1e-3, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16 keys and latent rows, f32 scores", "data": "synthetic",
        "config": {"workload": f"C3: DSA long-context stress, {T} keys, 1 query token, indexer {H}x128, top-{k}, sparse MLA over "
                               f"{a.n_heads} heads", "l2": "256 MB buffer written before every timed launch"},
        "select_us": us_sel, "attention_us": us_att,
        "roofline": {"bound": "hbm", "kernel": "indexer_topk_kernel (key scan + selection)", "achieved": scan_bytes / us_sel / 1e3,
                     "peak": peak, "unit": "GB/s", "frac": scan_bytes / us_sel / 1e3 / peak, "peak_source": peak_src,
                     "bytes_per_launch": scan_bytes, "traffic": None},
        "parity": {"indices_exact_on_device_scores": idx_exact, "attention_cos": cos, "ok": bool(idx_exact and cos >= 0.999)},
        "device_status": tilert_b200.device_status(0),
    }
    print(json.dumps(line), flush=True)
    if not line["parity"]["ok"]:
        sys.exit(1)


def run_profile_gemv(args) -> None:
    """One weight-streaming product alone: N = 7168 rows, K = 32768 (235 MB of FP8 weights, larger
    than L2), a few launches.  Small device footprint, meant to be captured by a profiler."""
    import tilert_b200
    from tilert_b200.models.deepseek_v3_2 import ops

    tilert_b200.load_backend("deepseek_v3_2")
    tilert_b200.tilert_init(0)
    dev = torch.device("cuda", 0)
    n, k = 7168, args.gemv_k
    g = torch.Generator(device=dev).manual_seed(0)
    w = torch.randint(0, 120, (n // 128, k // 128, 16448), generator=g, dtype=torch.uint8, device=dev)
    w[:, :, 16384:] = 0
    w[:, :, 16384:].view(torch.float32).fill_(1e-3)
    vec = torch.randn(1, 1, k, generator=g, device=dev).to(torch.bfloat16)
    res = torch.randn(1, 1, n, generator=g, device=dev).to(torch.bfloat16)
    out = torch.zeros(1, 1, n, dtype=torch.bfloat16, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.gemv_packed:
        xp = ops.new_xpack(k, dev)
        ops.act_pack(vec, xp)

        def launch():
            ops.projx_wqkva_packed(xp, 2, w, 1, k, n, 0, 0, 0, None, out, None, None, None)
    else:
        def launch():
            ops.unproj_o_allreduce(vec, w, None, res, 0, out)
    for _ in range(max(args.warmup, 1)):
        launch()
    torch.cuda.synchronize()
    # back-to-back launches replayed from a CUDA graph: no host launch overhead in the timed region
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(args.steps):
            launch()
    graph.replay()
    torch.cuda.synchronize()
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    # calibration: a plain read-only pass over 1 GiB with a library reduction
    big = torch.empty(1 << 28, dtype=torch.int32, device=dev).fill_(1)
    big.sum()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(5):
        big.sum()
    e1.record()
    torch.cuda.synchronize()
    read_gbs = 5 * big.numel() * 4 / (e0.elapsed_time(e1) * 1e-3) / 1e9
    # per-CTA phase stamps of one traced launch
    import ctypes
    trace = torch.zeros(256, 16, dtype=torch.int64, device=dev)
    ctx = ctypes.c_void_p(tilert_b200.tilert_init(0))
    tilert_b200.check(tilert_b200.lib().tilert_b200_set_profile(ctx, ctypes.c_void_p(trace.data_ptr())))
    launch()
    torch.cuda.synchronize()
    tilert_b200.check(tilert_b200.lib().tilert_b200_set_profile(ctx, None))
    if os.environ.get("TB_TIMELINE_OUT"):
        torch.save(trace.cpu(), os.environ["TB_TIMELINE_OUT"])
    tr = trace[:148].cpu().double()
    t0 = tr[:, 0].min()
    rel = (tr[:, :8] - t0) / 1e3
    names = ["entry", "ready", "first_data", "last_unit", "tiles_done", "first_convert", "issued", "exit"]
    phases = {nm: [round(float(rel[:, i].min()), 2), round(float(rel[:, i].median()), 2), round(float(rel[:, i].max()), 2)]
              for i, nm in enumerate(names)}
    units = tr[:, 10].clamp_min(1)
    phases["wait_cycles_per_unit"] = round(float((tr[:, 8] / units).median()), 1)
    phases["math_cycles_per_unit"] = round(float((tr[:, 9] / units).median()), 1)
    for idx, nm in ((11, "mma0_wait_full_x2"), (12, "mma0_issue_x2"), (14, "prod0_wait_empty_x4"),
                    (15, "conv0_cycles_x2")):
        phases[nm + "_per_unit"] = round(float((tr[:, idx] / units).median()), 1)
    print(json.dumps({"trace_us_min_med_max": phases}))
    print(json.dumps({"mode": "profile-gemv", "n": n, "k": k, "weight_bytes": w.numel(), "ms_per_launch": ms,
                      "gbs": w.numel() / ms / 1e6, "torch_sum_read_gbs": read_gbs,
                      "status": tilert_b200.device_status(0)}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=1, choices=[1, 2, 4],
                    help="rows per step (4 = the speculative-decoding verify step); default 1, the headline workload")
    ap.add_argument("--cache-rows", type=int, default=CACHE_LEN, help="rows of the latent caches (context length)")
    ap.add_argument("--mla-split", type=int, default=0, help="keys per attention split (multiple of 64); 0 = the layer's choice")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile", action="store_true",
                    help="short run for a profiler: no clock-sampling loop, no CPU baseline")
    ap.add_argument("--trace-step", action="store_true",
                    help="print the per-launch phase stamps of the streaming products of one step")
    ap.add_argument("--config", default="c1", choices=["c1", "c2", "c3"],
                    help="c1: the headline layer step; c2: whole-model decode (time per output token); c3: long-context "
                         "indexer + sparse attention stress")
    ap.add_argument("--ctx", default=None, help="c2: context length(s), comma separated (default 1024); c3: cached keys "
                                                "(default 131072)")
    ap.add_argument("--chain", default="default", choices=["default", "on", "off", "both"],
                    help="c2: run the layers' products as chained launches, as single launches, or time both")
    ap.add_argument("--with-mtp", action="store_true", help="c2: speculative decoding steps with the prediction layer")
    ap.add_argument("--layers", type=int, default=61, help="c2: decoder layers (61 = the real model; needs 8 GPUs)")
    ap.add_argument("--gemv-k", type=int, default=32768)
    ap.add_argument("--gemv-packed", action="store_true", help="profile-gemv: activations packed beforehand")
    ap.add_argument("--profile-gemv", action="store_true",
                    help="run only the weight-streaming product on a 235 MB weight (small footprint for ncu)")
    args = ap.parse_args()
    if args.profile:
        args.no_cpu_baseline = True
    if args.config == "c2" and args.impl == "ours":
        args.ctx = args.ctx or 1024
        run_c2(args)
    elif args.config == "c3" and args.impl == "ours":
        args.ctx = int(args.ctx or 131072)
        run_c3(args)
    elif args.profile_gemv:
        run_profile_gemv(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
