"""``python -m tilert_b200.generate``: the reference's text-generation entry (tilert/generate.py:75-150) for
this backend.  No checkpoint or tokenizer ships with the repository, so the runnable form is
``--use-random-weights`` with a seeded random prompt of ``--prompt-len`` token ids (the reference's own
``prompt_tokens=`` path, generator.py:160,195).

    python -m tilert_b200.generate --model toy --use-random-weights --max-new-tokens 32 [--with-mtp]
"""

from __future__ import annotations

import argparse
import statistics

import torch


def parse_args():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="toy", choices=["toy", "deepseek_v3_2"],
                    help="toy: the 2-layer test model; deepseek_v3_2: the full shape with --layers layers")
    ap.add_argument("--layers", type=int, default=2, help="decoder layers of the full-shape model (61 in the real one)")
    ap.add_argument("--use-random-weights", action="store_true")
    ap.add_argument("--model-weights-dir", default=None, help="directory written by python -m tilert_b200.convert")
    ap.add_argument("--with-mtp", action="store_true")
    ap.add_argument("--max-new-tokens", type=int, default=32)
    ap.add_argument("--prompt-len", type=int, default=16)
    ap.add_argument("--max-seq-len", type=int, default=1024)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    return ap.parse_args()


def main() -> None:
    args = parse_args()
    import tilert_b200
    from tilert_b200.models.deepseek_v3_2.generator import DSAv32Generator
    from tilert_b200.models.deepseek_v3_2.model_args import ModelArgs, toy_model_args
    from dataclasses import replace

    if not torch.cuda.is_available():
        raise SystemExit("tilert_b200.generate needs a CUDA device (sm_100a); there is no CPU path")
    tilert_b200.load_backend("deepseek_v3_2")
    tilert_b200.tilert_init(0)
    if args.model == "toy":
        margs = replace(toy_model_args(), max_seq_len=args.max_seq_len)
    else:
        margs = replace(ModelArgs(), n_layers=args.layers, n_dense_layers=min(3, args.layers - 1), max_seq_len=args.max_seq_len)
    gen = DSAv32Generator(margs, max_new_tokens=args.max_new_tokens, with_mtp=args.with_mtp, sampling_seed=args.seed,
                          max_seq_len=args.max_seq_len)
    if args.use_random_weights or args.model_weights_dir is None:
        gen.init_random_weights(args.seed)
    else:
        from tilert_b200 import convert

        gen.from_state_dict(convert.load_state_dict(args.model_weights_dir))
    if args.temperature > 0:
        gen.update_sampling_config(args.temperature, args.top_p, args.top_k, args.top_p < 1.0)
    g = torch.Generator().manual_seed(args.seed + 1)
    prompt = torch.randint(0, margs.vocab_size, (args.prompt_len,), generator=g).tolist()
    text, times, accepted, plen = gen.generate("", print_log=True, prompt_tokens=prompt)
    decode = times[plen:] if not args.with_mtp else times[-len(accepted):]
    if decode:
        per_step = statistics.median(decode)
        toks = (sum(accepted) / len(accepted)) if accepted else 1.0
        print(f"prompt {plen} tokens, {len(decode)} decode steps, median {per_step * 1e3:.3f} ms per step, "
              f"{toks / per_step:.1f} tokens/s" + (f", mean accepted {toks:.2f}" if accepted else ""))
    gen.cleanup()


if __name__ == "__main__":
    main()
