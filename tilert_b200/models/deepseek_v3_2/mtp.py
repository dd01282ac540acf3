"""Speculative decoding with the multi-token-prediction layer: four tokens verified per step, three
drafted for the next one -- the role of the reference's ``dsa_mtp_e2e_show_hands`` native call
(tilert/models/deepseek_v3_2/modules/end2end.py:79-163,598-651) and of the host loop around it
(generator.py:267-417).

A step takes ``draft[4]`` at the current position ``p``: ``draft[0]`` is the last known token, the
rest are guesses.  The main model runs the four rows in one pass (every FP8 product streams its
weights once for all four); ``predicted[j]`` is the arg-max after row ``j``; the accepted count ``n``
is 1 + the number of leading guesses with ``draft[j+1] == predicted[j]``.  The prediction layer
(enorm / hnorm / eh_proj -> one MoE decoder layer with caches of its own -> shared_head.norm -> the
main head; modules/mtp_preprocess.py:197-229, modules/mtp.py:28-50) pairs the hidden state of
position ``q`` with the embedding of the token at ``q+1``: one four-row pass at ``p .. p+3`` over
``predicted[0:4]`` gives guess 1 from row ``n-1``, two single-row passes at ``p+n`` and ``p+n+1`` chain
the layer's own hidden state into guesses 2 and 3.  Rows either model wrote past ``p+n-1`` belong to
rejected tokens; the next step starts at ``p+n`` and rewrites them before anything reads them.

Everything up to the accepted count stays on the device (the count selects rows through index
tensors), so a step is one CUDA-graph replay; the host reads the count once per step, as the
reference's loop does.
"""

from __future__ import annotations

import torch

from . import ops
from .layer import DecoderLayer, LayerWeights, precompute_freqs
from .model_args import ModelArgs

BF16 = torch.bfloat16
F32 = torch.float32
I32 = torch.int32
I64 = torch.int64

N_TOKENS = 4  # rows per step: the reference's ``forward_max_seq_len`` (end2end.py:188-189)


class MtpDsaModel:
    """Main model + prediction layer on one rank of ``world`` (tensor parallel like ``DsaModel``: heads,
    expert slices and vocabulary rows per rank, fused all-reduces, ``comm`` from ``tilert_b200.comm``).
    ``sd`` is an HF-keyed FP8 state dict whose prediction layer sits under ``model.layers.{n_layers}``, or a
    dictionary of packed per-rank weights with an ``"mtp"`` entry (``synthetic.random_packed_model``)."""

    def __init__(self, args: ModelArgs, sd: dict[str, torch.Tensor], device="cuda", cache_len: int | None = None,
                 use_graph: bool = True, world: int = 1, rank: int = 0, comm: int | None = None):
        self.args, self.device = args, torch.device(device)
        self.world, self.rank, self.comm = world, rank, comm
        dev, s = self.device, N_TOKENS
        self.cache_len = cache_len or args.max_seq_len
        v_l = args.vocab_size // world
        packed = sd if isinstance(sd, dict) and "layers" in sd else None  # converted or randomly drawn packed weights
        if packed is not None:
            if packed["world"] != world or packed.get("mtp") is None:
                raise ValueError("the packed weights are for another number of ranks or lack the prediction layer")
            m = packed["mtp"]
            self.embed, self.final_norm, self.head = packed["embed"], packed["final_norm"], packed["head"]
            self.enorm, self.hnorm, self.w_eh, self.mtp_norm = m["enorm"], m["hnorm"], m["w_eh"], m["norm"]
            main_w, mtp_w = packed["layers"], m["layer"]
        else:
            p = f"model.layers.{args.n_layers}"
            self.embed = sd["model.embed_tokens.weight"].to(dev, BF16)
            self.final_norm = sd["model.norm.weight"].to(dev, F32)
            # with several ranks every rank holds vocab / world rows of the head (shared by both models) and
            # the greedy tokens come from the (value, index) exchange over peer memory
            self.head = sd["lm_head.weight"][rank * v_l:(rank + 1) * v_l].to(dev, BF16).contiguous()
            self.enorm = sd[f"{p}.enorm.weight"].to(dev, F32)
            self.hnorm = sd[f"{p}.hnorm.weight"].to(dev, F32)
            self.w_eh = sd[f"{p}.eh_proj.weight"].to(dev, BF16).contiguous()
            self.mtp_norm = sd[f"{p}.shared_head.norm.weight"].to(dev, F32)
            main_w = [LayerWeights(args, sd, li, dev, world, rank) for li in range(args.n_layers)]
            mtp_w = LayerWeights(args, sd, args.n_layers, dev, world, rank)
        self.layers = [DecoderLayer(args, main_w[li], dev, self.cache_len, s, world, comm) for li in range(args.n_layers)]
        self.mtp_layer = DecoderLayer(args, mtp_w, dev, self.cache_len, s, world, comm)
        self.freqs = precompute_freqs(args).to(dev)
        z = lambda *shape, dtype: torch.zeros(*shape, dtype=dtype, device=dev)  # noqa: E731
        self.cur_pos = z(1, dtype=I32)
        self.rows = torch.arange(s, dtype=I64, device=dev)
        # step inputs
        self.draft = z(s, dtype=I64)
        self.extra_token = z(1, dtype=I64)      # prefill only: the prompt token after the chunk
        self.valid = z(1, dtype=I32)            # prefill only: rows of the chunk that are real
        # step results (the reference's PREDICTED_TOKENS / ACCEPTED_TOKENS / NEXT_DRAFT_TOKENS)
        self.logits = z(1, s, v_l, dtype=F32)                  # this rank's slice of the vocabulary
        self.predicted = z(s, dtype=I64)
        self.n_accepted = z(1, dtype=I64)
        self.next_draft = z(s, dtype=I64)
        self.guess_logits = z(s - 1, v_l, dtype=F32)
        # scratch
        self.mtp_in = z(1, s, args.dim, dtype=BF16)
        self.eh_part = z(1, s, args.dim, dtype=BF16)  # this rank's rows of eh_proj's output, zero elsewhere
        self.mtp_logits = z(1, s, v_l, dtype=F32)
        self.chain_pos = z(1, dtype=I32)
        self.chain_in = z(1, 1, args.dim, dtype=BF16)
        self.chain_logits = z(1, 1, v_l, dtype=F32)
        self.guess = z(1, dtype=I64)
        self.use_graph = use_graph
        self._graphs: dict[tuple[str, int], torch.cuda.CUDAGraph] = {}
        self.pos = 0  # host copy of the position

    # -- controls with the reference driver's names (end2end.py:551-577, 137-163) --
    def reset_sequence(self) -> None:
        self.set_cur_pos(0)

    def set_cur_pos(self, pos: int) -> None:
        self.pos = pos
        self.cur_pos.fill_(pos)

    def set_prefill_valid_tokens(self, n: int) -> None:
        self.valid.fill_(n)

    def set_prefill_mtp_extra_token(self, token: int) -> None:
        self.extra_token.fill_(token)

    def get_num_accepted(self) -> int:
        return int(self.n_accepted.item())

    def get_predicted_tokens(self) -> torch.Tensor:
        return self.predicted

    def get_next_draft_tokens(self) -> torch.Tensor:
        return self.next_draft

    def _argmax(self, logits: torch.Tensor, out: torch.Tensor) -> None:
        """Greedy tokens of ``logits`` [1, S, vocab / world] into ``out`` int64 [S], the same on every rank."""
        if self.world > 1:
            ops.argmax_exchange(logits, self.rank * logits.shape[-1], out, comm=self.comm)
        else:
            out.copy_(torch.argmax(logits.view(out.numel(), -1), dim=-1))

    # -- the passes --
    def _main_pass(self, tokens: torch.Tensor, n_keys: int) -> torch.Tensor:
        s = tokens.numel()
        x = self.embed[tokens].view(1, s, -1)
        fr = self.freqs[self.cur_pos.long() + self.rows[:s]]
        for layer in self.layers:
            x = layer.forward(x, self.cur_pos, fr, n_keys)
        ops.rmsnorm_head_proj(x, self.final_norm, self.head, None, self.logits[:, :s], eps=self.args.eps)
        return x

    def _mtp_pass(self, next_tokens: torch.Tensor, h: torch.Tensor, pos: torch.Tensor, n_keys: int,
                  x_in: torch.Tensor, logits_out: torch.Tensor) -> torch.Tensor:
        s = next_tokens.numel()
        e = self.embed[next_tokens].view(1, s, -1)
        if self.world > 1 and self.args.dim % self.world == 0:
            # every rank streams dim / world rows of eh_proj into its zero-padded buffer; the stand-alone all-reduce
            # assembles the vector on all ranks (adding zeros: the same bits as the unsharded product)
            rows = self.args.dim // self.world
            part = self.eh_part[:, :s]
            ops.mtp_preprocess_rows(e, h, self.enorm, self.hnorm, self.w_eh, part, self.rank * rows, rows, eps=self.args.eps)
            ops.padded_allreduce_add(part, None, 0, x_in, comm=self.comm)
        else:
            ops.mtp_preprocess(e, h, self.enorm, self.hnorm, self.w_eh, x_in, eps=self.args.eps)
        fr = self.freqs[pos.long() + self.rows[:s]]
        x = self.mtp_layer.forward(x_in, pos, fr, n_keys)
        ops.rmsnorm_head_proj(x, self.mtp_norm, self.head, None, logits_out, eps=self.args.eps)
        return x

    def _prefill_ops(self, n_keys: int) -> None:
        h = self._main_pass(self.draft, n_keys)
        nxt = torch.cat([self.draft[1:], self.extra_token])
        self._mtp_pass(nxt, h, self.cur_pos, n_keys, self.mtp_in, self.mtp_logits)
        self.cur_pos += self.valid

    def _verify_ops(self, n_keys: int) -> None:
        s = N_TOKENS
        h = self._main_pass(self.draft, n_keys)
        self._argmax(self.logits, self.predicted)
        match = (self.draft[1:] == self.predicted[:-1]).to(I64)
        self.n_accepted.copy_(1 + torch.cumprod(match, 0).sum().view(1))
        last = self.n_accepted - 1                                   # row of the last accepted token
        mh = self._mtp_pass(self.predicted, h, self.cur_pos, n_keys, self.mtp_in, self.mtp_logits)
        self.guess_logits[0].copy_(self.mtp_logits.view(s, -1).index_select(0, last).view(-1))
        self._argmax(self.guess_logits[0].view(1, 1, -1), self.guess)
        self.next_draft[0:1].copy_(self.predicted.index_select(0, last))
        self.next_draft[1:2].copy_(self.guess)
        hh = mh.index_select(1, last).clone()
        for i in range(1, s - 1):
            self.chain_pos.copy_(self.cur_pos + (last + i).to(I32))
            hh = self._mtp_pass(self.guess, hh, self.chain_pos, n_keys, self.chain_in, self.chain_logits).clone()
            self.guess_logits[i].copy_(self.chain_logits.view(-1))
            self._argmax(self.guess_logits[i].view(1, 1, -1), self.guess)
            self.next_draft[i + 1: i + 2].copy_(self.guess)
        self.cur_pos += self.n_accepted.to(I32)

    def _bucket(self) -> int:
        """Indexer scan length covering every row a step may touch (the four rows and the two chained
        ones), rounded up to a multiple of 256 so that graphs are reused."""
        need = self.pos + 2 * N_TOKENS
        return min(self.cache_len, (need // 256 + 1) * 256)

    def _run(self, kind: str) -> None:
        n_keys = self._bucket()
        fn = self._verify_ops if kind == "verify" else self._prefill_ops
        if not self.use_graph:
            fn(n_keys)
            return
        key = (kind, n_keys)
        if key not in self._graphs:
            saved = self.cur_pos.clone()
            fn(n_keys)  # warm-up outside the capture; the rows it wrote are rewritten by the real run
            torch.cuda.synchronize()
            self.cur_pos.copy_(saved)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn(n_keys)
            self.cur_pos.copy_(saved)
            self._graphs[key] = g
        self._graphs[key].replay()

    def forward(self, draft_tokens: torch.Tensor | list[int], with_mtp: bool = True) -> None:
        """One speculative step for ``draft_tokens`` [4] at the current position (or one prefill chunk
        when ``set_prefill_valid_tokens`` was given a non-zero count), as ``ShowHandsDSALayer.forward``
        (end2end.py:551-558).  Results: ``get_num_accepted`` / ``get_predicted_tokens`` /
        ``get_next_draft_tokens``."""
        if not with_mtp:
            raise ValueError("MtpDsaModel only runs the speculative path; use DsaModel for plain decoding")
        t = torch.as_tensor(draft_tokens).view(-1).to(self.device, I64)
        if t.numel() != N_TOKENS:
            raise ValueError(f"draft_tokens must hold {N_TOKENS} tokens")
        if self.pos + 2 * N_TOKENS > self.cache_len:
            raise ValueError("position too close to the end of the caches")
        self.draft.copy_(t)
        valid = int(self.valid.item())
        if valid > 0:
            self._run("prefill")
            self.pos += valid
        else:
            self._run("verify")
            self.pos += self.get_num_accepted()

    @torch.no_grad()
    def generate(self, prompt: list[int], n_new: int) -> tuple[list[int], list[int]]:
        """Chunked prefill, then speculative steps until ``n_new`` tokens are out
        (generator.py:267-417).  Returns (tokens, accepted count of every step)."""
        s, plen = N_TOKENS, len(prompt)
        self.reset_sequence()
        while self.pos < plen - 1:
            end = min(self.pos + s, plen)
            chunk = prompt[self.pos: end]
            valid = len(chunk)
            chunk = chunk + [chunk[-1]] * (s - valid)
            extra = prompt[self.pos + s] if self.pos + s < plen else prompt[end - 1]
            self.set_prefill_mtp_extra_token(extra)
            self.set_prefill_valid_tokens(valid)
            self.forward(chunk)
        self.set_cur_pos(plen - 1)
        self.set_prefill_valid_tokens(0)
        draft: torch.Tensor | list[int] = [prompt[-1]] * s
        out: list[int] = []
        counts: list[int] = []
        while len(out) < n_new:
            self.forward(draft)
            n = self.get_num_accepted()
            out += [int(t) for t in self.predicted[:n].cpu()]
            counts.append(n)
            draft = self.next_draft.clone()
        return out[:n_new], counts
