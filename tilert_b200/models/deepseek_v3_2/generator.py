"""Single-sequence generation on top of ``ShowHandsDSALayer``: the reference's ``DSAv32Generator``
(tilert/models/deepseek_v3_2/generator.py:45-540) -- token-by-token prefill then decode, with or without
multi-token prediction, per-token wall-clock times, and the synthetic-workload entry ``prompt_tokens=``.
A tokenizer is optional (none ships with this repository): without one, prompts are token id lists and the
returned text is the space-joined ids."""

from __future__ import annotations

import time

import torch

from .end2end import ShowHandsDSALayer
from .model_args import ModelArgs
from .mtp import N_TOKENS
from .temp_var_indices import Idx


class DSAv32Generator:
    def __init__(self, model_args: ModelArgs, max_new_tokens: int = 100, device="cuda:0", with_mtp: bool = False,
                 tokenizer=None, eos_id: int = -1, sampling_seed: int = 0, max_seq_len: int | None = None):
        self.config, self.max_new_tokens, self.with_mtp = model_args, max_new_tokens, with_mtp
        self.tokenizer, self.eos_id, self.sampling_seed = tokenizer, eos_id, sampling_seed
        self.default_device = torch.device(device)
        self.decode_layer = ShowHandsDSALayer(model_args, device, max_seq_len or model_args.max_seq_len, with_mtp)

    # -- weights (generator.py:90-150) --
    def init_random_weights(self, seed: int = 0) -> None:
        self.decode_layer.init_random_weights(seed)

    def from_state_dict(self, sd) -> None:
        self.decode_layer.from_state_dict(sd)

    def update_sampling_config(self, temperature=0.0, top_p=1.0, top_k=0, use_topp=False) -> None:
        self.decode_layer.update_sampling_config(temperature=temperature, top_p=top_p, top_k=top_k, use_topp=use_topp)

    def _tokens_of(self, prompt, prompt_tokens):
        if prompt_tokens is not None:
            return list(prompt_tokens)
        if self.tokenizer is None:
            raise ValueError("no tokenizer: pass prompt_tokens=[...]")
        return self.tokenizer.apply_chat_template([{"role": "user", "content": prompt}], add_generation_prompt=True)

    def _text_of(self, toks: list[int]) -> str:
        if self.tokenizer is not None:
            return self.tokenizer.decode(toks, skip_special_tokens=True)
        return " ".join(str(t) for t in toks)

    @torch.inference_mode()
    def generate(self, prompt: str = "", print_log: bool = True, with_mtp: bool | None = None,
                 prompt_tokens: list[int] | None = None) -> tuple[str, list[float], list[int], int]:
        """generator.py:155-185: returns (text, per-step seconds, accepted counts (MTP only), prompt length)."""
        active_mtp = self.with_mtp if with_mtp is None else with_mtp
        if active_mtp and not self.with_mtp:
            raise ValueError("Cannot use MTP mode: MTP weights were not loaded")
        self.decode_layer.set_sampling_seed(self.sampling_seed)
        toks = self._tokens_of(prompt, prompt_tokens)
        if active_mtp:
            return self._generate_with_mtp(toks, print_log)
        return self._generate_without_mtp(toks, print_log)

    def _generate_without_mtp(self, prompt_tokens: list[int], print_log: bool):
        """generator.py:187-265."""
        prompt_len = len(prompt_tokens)
        total_len = min(self.decode_layer.max_seq_len, self.max_new_tokens + prompt_len)
        tokens = list(prompt_tokens) + [-1] * (total_len - prompt_len)
        time_list: list[float] = []
        for cur in range(1, total_len):
            t0 = time.time()
            intermediates, *_ = self.decode_layer.forward(tokens[cur - 1])[0]
            nxt = int(intermediates[Idx.TOKEN_OUT].view(-1)[0])  # the read synchronises, as the reference's does
            time_list.append(time.time() - t0)
            if cur >= prompt_len:
                tokens[cur] = nxt
                if print_log:
                    print(self._text_of([nxt]), end=" ", flush=True)
                if nxt == self.eos_id:
                    tokens = tokens[: cur + 1]
                    break
        self.decode_layer.reset_sequence()
        out = [t for t in tokens[prompt_len:] if t != -1]
        if self.eos_id in out:
            out = out[: out.index(self.eos_id)]
        if print_log:
            print()
        return self._text_of(out) + "\n", time_list, [], prompt_len

    def _generate_with_mtp(self, prompt_tokens: list[int], print_log: bool):
        """generator.py:267-417: chunked prefill of four, then draft / verify / accept steps."""
        from . import end2end as e2e

        s, plen = N_TOKENS, len(prompt_tokens)
        layer, tv = self.decode_layer, self.decode_layer.temp_vars
        time_list: list[float] = []
        pos = 0
        while pos < plen - 1:
            end = min(pos + s, plen)
            chunk = prompt_tokens[pos:end]
            valid = len(chunk)
            chunk = chunk + [chunk[-1]] * (s - valid)
            extra = prompt_tokens[pos + s] if pos + s < plen else prompt_tokens[end - 1]
            e2e.dsa_mtp_e2e_show_hands_set_prefill_mtp_extra_token(extra)
            e2e.dsa_mtp_e2e_show_hands_set_prefill_valid_tokens(valid)
            t0 = time.time()
            layer.forward(chunk)
            torch.cuda.synchronize()
            time_list.append(time.time() - t0)
            pos += valid
        e2e.dsa_show_hands_set_cur_pos(plen - 1)
        e2e.dsa_mtp_e2e_show_hands_set_prefill_valid_tokens(0)
        draft = [prompt_tokens[-1]] * s
        out: list[int] = []
        counts: list[int] = []
        budget = min(self.max_new_tokens, self.decode_layer.max_seq_len - plen - 2 * s)
        while len(out) < budget:
            t0 = time.time()
            layer.forward(draft)
            n = int(tv[Idx.ACCEPTED_TOKENS].view(-1)[0])
            time_list.append(time.time() - t0)
            new = [int(t) for t in tv[Idx.PREDICTED_TOKENS].view(-1)[:n].cpu()]
            out += new
            counts.append(n)
            draft = [int(t) for t in tv[Idx.NEXT_DRAFT_TOKENS].view(-1)[:s].cpu()]
            if print_log:
                print(self._text_of(new), end=" ", flush=True)
            if self.eos_id in new:
                out = out[: out.index(self.eos_id)]
                break
        layer.reset_sequence()
        if print_log:
            print()
        return self._text_of(out[:budget]) + "\n", time_list, counts, plen

    def cleanup(self) -> None:
        self.decode_layer.cleanup()
