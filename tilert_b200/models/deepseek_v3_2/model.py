"""Whole-model driver for batch-1 greedy decoding: embedding lookup, the decoder layers, the
vocabulary head and arg-max -- the role of the reference's ``ShowHandsDSALayer``
(tilert/models/deepseek_v3_2/modules/end2end.py:166-703) whose forward is one native call per
token.  Here a step is the layers' operator sequence, replayed from a CUDA graph."""

from __future__ import annotations

import torch

from . import ops
from .layer import DecoderLayer, LayerWeights, precompute_freqs
from .model_args import ModelArgs

BF16 = torch.bfloat16
F32 = torch.float32
I32 = torch.int32


class DsaModel:
    def __init__(self, args: ModelArgs, sd: dict[str, torch.Tensor], device="cuda", cache_len: int | None = None,
                 world: int = 1, rank: int = 0, comm: int | None = None, use_graph: bool = True):
        self.args, self.device = args, torch.device(device)
        self.world, self.rank, self.comm = world, rank, comm
        dev = self.device
        self.cache_len = cache_len or args.max_seq_len
        self.embed = sd["model.embed_tokens.weight"].to(dev, BF16)
        self.final_norm = sd["model.norm.weight"].to(dev, F32)
        v_l = args.vocab_size // world
        self.head = sd["lm_head.weight"][rank * v_l:(rank + 1) * v_l].to(dev, BF16).contiguous()
        self.layers = [
            DecoderLayer(args, LayerWeights(args, sd, li, dev, world, rank), dev, self.cache_len, 1, world, comm)
            for li in range(args.n_layers)
        ]
        self.freqs = precompute_freqs(args).to(dev)
        self.cur_pos = torch.zeros(1, dtype=I32, device=dev)
        self.token = torch.zeros(1, dtype=torch.int64, device=dev)
        self.logits = torch.zeros(1, 1, v_l, dtype=F32, device=dev)
        self.token_out = torch.zeros(1, dtype=torch.int64, device=dev)
        self.use_graph = use_graph
        self._graphs: dict[int, torch.cuda.CUDAGraph] = {}

    # -- reference driver controls (end2end.py:551-577) --
    def reset_sequence(self) -> None:
        self.cur_pos.zero_()

    def set_cur_pos(self, pos: int) -> None:
        self.cur_pos.fill_(pos)

    def _step_ops(self, n_keys: int) -> None:
        x = self.embed[self.token].view(1, 1, -1)
        fr = self.freqs[self.cur_pos.long()]
        for layer in self.layers:
            x = layer.forward(x, self.cur_pos, fr, n_keys)
        ops.rmsnorm_head_proj(x, self.final_norm, self.head, None, self.logits, eps=self.args.eps)
        if self.world > 1:
            # every rank holds vocab / world rows of the head: exchange (value, index) pairs over peer memory
            ops.argmax_exchange(self.logits, self.rank * self.logits.shape[-1], self.token_out, comm=self.comm)
        else:
            self.token_out.copy_(torch.argmax(self.logits.view(-1)))
        self.cur_pos += 1

    def _bucket(self, pos: int) -> int:
        """Indexer scan length: next multiple of 256 above the position, so graphs are reused."""
        return min(self.cache_len, (pos // 256 + 1) * 256)

    def forward(self, token: int | torch.Tensor, pos: int) -> None:
        """Run one decode step for ``token`` at position ``pos`` (asynchronous; results in
        ``self.logits`` / ``self.token_out``)."""
        if isinstance(token, int):
            self.token.fill_(token)
        else:
            self.token.copy_(token.view(-1)[:1])
        n_keys = self._bucket(pos)
        if not self.use_graph:
            self._step_ops(n_keys)
            return
        if n_keys not in self._graphs:
            saved = self.cur_pos.clone()
            for ly in self.layers:  # warm-up outside capture (lazy function attributes, allocator)
                pass
            self._step_ops(n_keys)
            torch.cuda.synchronize()
            self.cur_pos.copy_(saved)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._step_ops(n_keys)
            self.cur_pos.copy_(saved)
            self._graphs[n_keys] = g
        self._graphs[n_keys].replay()

    @torch.no_grad()
    def generate(self, prompt: list[int], n_new: int, collect_logits: bool = False):
        """Token-by-token prefill then greedy decoding (tilert/models/deepseek_v3_2/generator.py:187-265).
        Returns the generated tokens (and the f32 logits of each generated position)."""
        self.reset_sequence()
        pos = 0
        for tok in prompt:
            self.forward(tok, pos)
            pos += 1
        toks, lgs = [], []
        for _ in range(n_new):
            if collect_logits:
                lgs.append(self.logits.view(-1).clone())
            nxt = self.token_out.clone()
            toks.append(nxt)
            self.forward(nxt, pos)
            pos += 1
        toks = [int(t) for t in torch.cat(toks).cpu()]
        return (toks, lgs) if collect_logits else toks
