"""Tensor-parallel parity check, run as one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 tests/multi_gpu_check.py

Every rank runs its shard of both toy layers (heads / N, expert intermediate / N) with the fused
peer-memory all-reduce, then the whole toy model with the vocabulary head split across ranks and the
greedy token exchanged over peer memory; every rank's output must match the CPU oracle's unsharded layer (cosine
>= 0.999, rel-L2 <= 2e-2) and all ranks must hold bit-identical results.  Several steps are run
back to back so that both halves of the receive buffers and the epoch bookkeeping are exercised.
"""

import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch
import torch.distributed as dist

from oracle import model as om
from oracle import ops as oo


def main() -> int:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import tilert_b200
    from tilert_b200.comm import Comm
    from tilert_b200.models.deepseek_v3_2 import layer as L
    from tilert_b200.models.deepseek_v3_2.model_args import toy_model_args

    tilert_b200.load_backend("deepseek_v3_2")
    tilert_b200.tilert_init(local)
    a, margs = om.toy_args(), toy_model_args()
    sd = om.random_state_dict(a, seed=0)
    comm = Comm(a.dim, local)
    fc = oo.precompute_freqs_cis(a)
    failures = []
    # The stand-alone all-reduce + residual add (the reference's padded_allreduce_add_op): every rank contributes a
    # vector of its own; all ranks must hold the f32 sum in rank order plus the residual, bit for bit, on every call
    # (three calls: both halves of the receive buffers, and the call number shared with the fused all-reduces).
    from tilert_b200.models.deepseek_v3_2 import ops as _ops
    for call, tokens in enumerate((1, 4, 2)):
        gens = [torch.Generator().manual_seed(900 + 10 * call + r) for r in range(world)]
        parts = [torch.randn(1, tokens, a.dim, generator=gr).to(torch.bfloat16) for gr in gens]
        resid = torch.randn(1, tokens, a.dim, generator=torch.Generator().manual_seed(800 + call)).to(torch.bfloat16)
        got = torch.zeros(1, tokens, a.dim, dtype=torch.bfloat16, device=dev)
        _ops.padded_allreduce_add(parts[rank].to(dev), resid.to(dev), 0, got, comm=comm.handle)
        torch.cuda.synchronize()
        acc = torch.zeros(1, tokens, a.dim, dtype=torch.float32)
        for pt in parts:
            acc += pt.float()
        want = (acc + resid.float()).to(torch.bfloat16)
        ok_here = torch.equal(got.cpu(), want)
        if rank == 0:
            print(f"allreduce_add call {call} tokens {tokens}: exact {ok_here}", flush=True)
        if not ok_here:
            failures.append(("allreduce_add", call, tokens))
    # The toy model shards only as far as its smallest dimension allows (expert intermediate 512: 128-row scale blocks
    # give at most 4 ranks); with more ranks only the full-shape layer at the end is checked.
    toy_ok = (a.moe_inter_dim % (128 * world) == 0 and a.inter_dim % (128 * world) == 0 and a.n_heads % world == 0
              and a.vocab_size % world == 0)
    if not toy_ok and rank == 0:
        print(f"toy layers, toy model, sampling and speculative steps skipped: the toy shapes do not shard {world} ways",
              flush=True)
    for li in ((0, 1) if toy_ok else ()):
        for tokens in (1, 2):
            g = torch.Generator().manual_seed(300 + li + tokens)
            t_ctx, cache_len, n_steps = 400, 512, 3
            ow, oc = om.LayerWeights(a, sd, li), om.Caches(a, cache_len)
            for c in (oc.kv, oc.pe, oc.ki):
                c[:, :t_ctx] = torch.randn(1, t_ctx, c.size(-1), generator=g, dtype=torch.float32).to(torch.bfloat16)
            gl = L.DecoderLayer(margs, L.LayerWeights(margs, sd, li, dev, world, rank), dev, cache_len, tokens, world,
                                comm.handle)
            gl.kv_cache.copy_(oc.kv); gl.pe_cache.copy_(oc.pe); gl.ki_cache.copy_(oc.ki)
            for step in range(n_steps):
                pos = t_ctx + step * tokens
                x = torch.randn(1, tokens, a.dim, generator=g, dtype=torch.float32).to(torch.bfloat16)
                cur = torch.tensor([pos], dtype=torch.int32, device=dev)
                fr = torch.view_as_real(fc[pos: pos + tokens]).contiguous().to(dev)
                trace = {}
                ref = om.layer_step(a, ow, oc, x, pos, fc, trace)
                gl.injected_sel = trace["sel"].to(dev)      # identical selections on every rank and in the oracle
                if "router_scores" in trace:
                    gl.forced_scores = trace["router_scores"].float().to(dev)
                out = gl.forward(x.to(dev), cur, fr, n_keys=pos + tokens).clone()
                torch.cuda.synchronize()
                o = out.float().cpu()
                cos = torch.nn.functional.cosine_similarity(ref.float().flatten(), o.flatten(), dim=0).item()
                l2 = (torch.norm(ref.float() - o) / torch.norm(ref.float())).item()
                gathered = [torch.empty_like(out) for _ in range(world)]
                dist.all_gather(gathered, out)
                same = all(torch.equal(gathered[0], t) for t in gathered)
                if rank == 0:
                    print(f"layer {li} tokens {tokens} step {step}: cos {cos:.6f} rel_l2 {l2:.3e} ranks_identical {same}",
                          flush=True)
                if not (cos >= 0.999 and l2 <= 2e-2 and same):
                    failures.append((li, tokens, step, cos, l2, same))
    if toy_ok:
        # The whole toy model with the vocabulary head split across ranks: the greedy token comes from the
        # (value, index) exchange over peer memory and must be the arg-max of the gathered logits on every
        # rank; graph replay is on, so the exchange's device-resident epoch is exercised too.
        from tilert_b200.models.deepseek_v3_2.model import DsaModel
        toks = torch.randint(0, a.vocab_size, (10,), generator=torch.Generator().manual_seed(3)).tolist()
        dm = DsaModel(margs, sd, dev, cache_len=256, world=world, rank=rank, comm=comm.handle)
        ref = om.Model(a, sd, cache_len=256)
        for pos, t in enumerate(toks):
            dm.forward(t, pos)
            torch.cuda.synchronize()
            _, rl = ref.step(t)
            parts = [torch.empty_like(dm.logits) for _ in range(world)]
            dist.all_gather(parts, dm.logits)
            full = torch.cat([p.view(-1) for p in parts]).float().cpu()
            l2 = (torch.norm(rl.float() - full) / torch.norm(rl.float())).item()
            picked = [torch.empty_like(dm.token_out) for _ in range(world)]
            dist.all_gather(picked, dm.token_out)
            picked = [int(p) for p in picked]
            expected = int(torch.argmax(full))
            if rank == 0:
                print(f"model pos {pos}: logits rel_l2 {l2:.3e} token {picked} expected {expected}", flush=True)
            if not (l2 <= 2e-2 and all(p == expected for p in picked)):
                failures.append(("model", pos, l2, picked, expected))
        # Sampling with the head split across ranks: the slices are gathered, every rank draws with the same seed and
        # step counter, so all ranks must hold the same token, and it must be one of the top_k of the gathered logits.
        dm.set_sampling(temperature=0.8, top_p=0.95, top_k=20, use_top_p=True, seed=7)
        pos = len(toks)
        tok = toks[-1]
        for _ in range(4):
            dm.forward(tok, pos)
            torch.cuda.synchronize()
            picked = [torch.empty_like(dm.token_out) for _ in range(world)]
            dist.all_gather(picked, dm.token_out)
            picked = [int(p) for p in picked]
            top = torch.topk(dm.full_logits, 20).indices.tolist()
            if rank == 0:
                print(f"sampled pos {pos}: tokens {picked} in top-20 {picked[0] in top}", flush=True)
            if not (all(p == picked[0] for p in picked) and picked[0] in top):
                failures.append(("sampling", pos, picked))
            tok, pos = picked[0], pos + 1
        dm.set_sampling(temperature=0.0)
        # Speculative decoding across ranks: chunked prefill, then verify steps fed with the oracle's drafts
        # (the second one with the true continuation, so several drafts are accepted).  The four rows' logits,
        # gathered over the vocabulary slices, must match the oracle's; the predicted tokens must be the arg-max
        # of the gathered logits and, like the accepted count and the next drafts, the same on every rank.
        from tilert_b200.models.deepseek_v3_2.mtp import MtpDsaModel
        sd_mtp = om.random_state_dict(a, seed=0, with_mtp=True)
        prompt = torch.randint(0, a.vocab_size, (21,), generator=torch.Generator().manual_seed(11)).tolist()
        plain, _ = om.Model(a, sd_mtp, cache_len=256).generate(prompt, 8)
        ref = om.MtpModel(a, sd_mtp, cache_len=256)
        ref.generate_mtp(prompt, 0)
        spec = MtpDsaModel(margs, sd_mtp, dev, cache_len=256, world=world, rank=rank, comm=comm.handle)
        spec.generate(prompt, 0)
        draft = [prompt[-1]] * 4
        for step in range(3):
            if step == 1:
                k = ref.pos - (len(prompt) - 1)
                draft = [draft[0]] + plain[k: k + 3]
            r = ref.verify_step(list(draft))
            spec.forward(draft)
            torch.cuda.synchronize()
            parts = [torch.empty_like(spec.logits) for _ in range(world)]
            dist.all_gather(parts, spec.logits)
            full = torch.cat(parts, dim=-1)[0].float().cpu()
            l2 = (torch.norm(r["logits"] - full) / torch.norm(r["logits"])).item()
            mine = torch.cat([spec.predicted, spec.n_accepted, spec.next_draft])
            everyone = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(everyone, mine)
            same = all(torch.equal(everyone[0], t) for t in everyone)
            pred = spec.predicted.cpu().tolist()
            exact = pred == torch.argmax(full, dim=-1).tolist()
            n_dev = spec.get_num_accepted()
            if rank == 0:
                print(f"speculative step {step}: logits rel_l2 {l2:.3e} predicted {pred} oracle {r['predicted']} "
                      f"accepted {n_dev} oracle {r['n_accepted']} ranks_identical {same}", flush=True)
            if not (l2 <= 2e-2 and same and exact):
                failures.append(("speculative", step, l2, same, exact))
            if pred != r["predicted"]:
                break  # an arg-max tie fell the other way: the sequences part ways here
            if n_dev != r["n_accepted"] or (step == 1 and n_dev < 2):
                failures.append(("speculative accepted", step, n_dev, r["n_accepted"]))
            draft = r["next_draft"]
    # The full-shape MoE layer of the benchmark (hidden 7168, 128 heads, 256 experts of which eight are forced
    # hot, indexer 64 x 128, top-2048, 4096-row caches), sharded over the ranks exactly as bench.py times it:
    # rank 0 compares with the CPU restatement of the reference's unsharded layer, all ranks must agree bit for bit.
    if os.environ.get("TB_MG_FULL", "1") != "0":
        import bench

        fa, hot, fsd, fcaches, fx = bench.workload_inputs(1, bench.CACHE_LEN)
        fcomm = Comm(fa.dim, local)
        flayer = L.DecoderLayer(fa, L.LayerWeights(fa, fsd, 0, dev, world, rank, expert_ids=hot), dev, bench.CACHE_LEN, 1,
                                world, fcomm.handle)
        for dst, src in zip((flayer.kv_cache, flayer.pe_cache, flayer.ki_cache), fcaches):
            dst.copy_(src)
        flayer.forced_scores = bench.forced_scores(fa.n_routed_experts, fa.n_activated_experts).to(dev)
        cur = torch.tensor([bench.CACHE_LEN - 1], dtype=torch.int32, device=dev)
        fr = L.precompute_freqs(fa)[bench.CACHE_LEN - 1: bench.CACHE_LEN].contiguous().to(dev)
        for step in range(2):  # twice: both halves of the receive buffers
            fout = flayer.forward(fx.to(dev), cur, fr, bench.CACHE_LEN).clone()
            torch.cuda.synchronize()
        gathered = [torch.empty_like(fout) for _ in range(world)]
        dist.all_gather(gathered, fout)
        same = all(torch.equal(gathered[0], t) for t in gathered)
        ok_flag = torch.ones(1, device=dev)
        if rank == 0:
            ref = bench.CpuChecker(fsd, fcaches, fx, 1, bench.CACHE_LEN).step().float().flatten()
            got = fout.float().cpu().flatten()
            cos = torch.nn.functional.cosine_similarity(ref, got, dim=0).item()
            l2 = (torch.norm(ref - got) / torch.norm(ref)).item()
            print(f"full-shape layer, {world} ranks: cos {cos:.6f} rel_l2 {l2:.3e} ranks_identical {same}", flush=True)
            if not (cos >= 0.999 and l2 <= 2e-2 and same):
                failures.append(("full", cos, l2, same))
        elif not same:
            failures.append(("full", same))
        dist.barrier()
        fcomm.close()
    status = tilert_b200.device_status(local)
    if status != 0:
        failures.append(("device_status", status))
    comm.close()
    dist.destroy_process_group()
    if failures:
        print(f"rank {rank} FAILURES: {failures}", flush=True)
        return 1
    if rank == 0:
        print("multi_gpu_check: OK", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
