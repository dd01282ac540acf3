"""Whole-model driver for batch-1 greedy decoding: embedding lookup, the decoder layers, the
vocabulary head and arg-max -- the role of the reference's ``ShowHandsDSALayer``
(tilert/models/deepseek_v3_2/modules/end2end.py:166-703) whose forward is one native call per
token.  Here a step is the layers' operator sequence, replayed from a CUDA graph."""

from __future__ import annotations

import torch

from . import ops
from .layer import DecoderLayer, LayerScratch, LayerWeights, precompute_freqs
from .model_args import ModelArgs

BF16 = torch.bfloat16
F32 = torch.float32
I32 = torch.int32


class DsaModel:
    def __init__(self, args: ModelArgs, sd: dict[str, torch.Tensor], device="cuda", cache_len: int | None = None,
                 world: int = 1, rank: int = 0, comm: int | None = None, use_graph: bool = True,
                 share_scratch: bool | None = None, temp_vars: list[torch.Tensor] | None = None):
        """``share_scratch``: one scratch set for all layers instead of one per layer (default: when the model
        has more than four layers).  ``temp_vars``: the reference driver's list of 56 scratch tensors
        (``DsaTempVarIdx``); the layers' scratch, the logits and the output token then live in it."""
        self.args, self.device = args, torch.device(device)
        self.world, self.rank, self.comm = world, rank, comm
        dev = self.device
        self.cache_len = cache_len or args.max_seq_len
        v_l = args.vocab_size // world
        if args.vocab_size % world != 0:
            raise ValueError(f"vocab_size {args.vocab_size} does not divide over {world} ranks")
        packed = sd if isinstance(sd, dict) and "layers" in sd else None  # a converted model (convert.load_model)
        if packed is not None:
            if packed["world"] != world:
                raise ValueError(f"the converted weights were sharded for {packed['world']} ranks, not {world}")
            self.embed, self.final_norm, self.head = packed["embed"], packed["final_norm"], packed["head"]
            layer_weights = packed["layers"]
        else:
            self.embed = sd["model.embed_tokens.weight"].to(dev, BF16)
            self.final_norm = sd["model.norm.weight"].to(dev, F32)
            self.head = sd["lm_head.weight"][rank * v_l:(rank + 1) * v_l].to(dev, BF16).contiguous()
            layer_weights = None
        if share_scratch is None:
            share_scratch = args.n_layers > 4 or temp_vars is not None
        scratch = None
        if temp_vars is not None:
            scratch = LayerScratch.from_temp_vars(args, temp_vars, self.cache_len, 1, world)
        elif share_scratch:
            scratch = LayerScratch(args, dev, self.cache_len, 1, world)
        self.layers = [
            DecoderLayer(args, layer_weights[li] if layer_weights is not None else LayerWeights(args, sd, li, dev, world, rank),
                         dev, self.cache_len, 1, world, comm, scratch=scratch, out_slot=li)
            for li in range(args.n_layers)
        ]
        self.freqs = precompute_freqs(args).to(dev)
        self.cur_pos = torch.zeros(1, dtype=I32, device=dev)
        self.token = torch.zeros(1, dtype=torch.int64, device=dev)
        self.logits = torch.zeros(1, 1, v_l, dtype=F32, device=dev)
        self.token_out = torch.zeros(1, dtype=torch.int64, device=dev)
        self.temp_vars = temp_vars
        if temp_vars is not None:
            from .temp_var_indices import Idx

            self.logits = temp_vars[Idx.LOGITS_OUT].reshape(-1)[:v_l].view(1, 1, v_l)
            self.cur_pos = temp_vars[Idx.CUR_POS].reshape(-1)[:1]
        self.use_graph = use_graph
        self._graphs: dict[int, torch.cuda.CUDAGraph] = {}
        # Host copy of the device-resident position: the kernels write cache row ``cur_pos`` and mask on it,
        # while the host picks the indexer's scan length from ``pos``; the two must not drift, and a position
        # past the caches or the rotary table must be refused before anything is launched.
        self._pos = 0
        # sampling state (the reference's SAMPLING_CONFIG / TOP_P_SCORES / TOP_N_LOG_PROBS / TOP_N_INDICES
        # temp vars, temp_var_indices.py:64-73): greedy until set_sampling is called
        self.sampling_config = torch.tensor([0.0, 1.0, 0.0, 0.0], dtype=F32, device=dev)  # temperature, top_p, top_k, use_top_p
        self.sampling_seed = 0
        self.sampling = False
        self.sample_step = torch.zeros(2, dtype=torch.int64, device=dev)  # advanced by every launch (graph replay safe)
        self.sampled = torch.zeros(1, dtype=I32, device=dev)
        self.full_logits: torch.Tensor | None = None  # world > 1 and sampling: every rank's slice, gathered
        self.token_logprob = torch.zeros(1, dtype=F32, device=dev)
        self.topn_logprobs = torch.zeros(1, 256, dtype=F32, device=dev)
        self.topn_indices = torch.zeros(1, 256, dtype=I32, device=dev)

    @classmethod
    def from_converted(cls, args: ModelArgs, out_dir, device="cuda", rank: int = 0, **kw) -> "DsaModel":
        """A model on the per-rank packed files that ``python -m tilert_b200.convert`` wrote."""
        from tilert_b200 import convert

        packed = convert.load_model(out_dir, device, rank)
        return cls(args, packed, device, world=packed["world"], rank=rank, **kw)

    # -- reference driver controls (end2end.py:551-577) --
    def reset_sequence(self) -> None:
        self.cur_pos.zero_()
        self._pos = 0

    def set_cur_pos(self, pos: int) -> None:
        if not 0 <= pos < min(self.cache_len, self.freqs.shape[0]):
            raise ValueError(f"set_cur_pos({pos}): the caches hold {self.cache_len} rows, the rotary table "
                             f"{self.freqs.shape[0]} positions")
        self.cur_pos.fill_(pos)
        self._pos = pos

    def set_sampling(self, temperature: float = 0.0, top_p: float = 1.0, top_k: int = 0, use_top_p: bool = False,
                     seed: int | None = None) -> None:
        """Sample the next token instead of taking the arg-max (end2end.py:253-311: temperature, top-p, top-k
        per request; ``set_sampling_seed``).  Temperature 0 with no seed change returns to greedy decoding.
        The token's log-probability and the top-256 log-probabilities / ids are left in ``token_logprob``,
        ``topn_logprobs`` and ``topn_indices`` after every step."""
        if self.world > 1:
            import torch.distributed as dist

            if not (dist.is_available() and dist.is_initialized()):
                raise ValueError("sampling over a vocabulary split across ranks gathers the logits with "
                                 "torch.distributed: initialise the default process group first")
            if self.full_logits is None:
                self.full_logits = torch.zeros(self.args.vocab_size, dtype=F32, device=self.device)
        self.sampling_config.copy_(torch.tensor([temperature, top_p, float(top_k), 1.0 if use_top_p else 0.0]))
        if seed is not None and seed != self.sampling_seed:
            self.sampling_seed = seed
            self._graphs.clear()  # the seed is a launch argument
        if not self.sampling:
            self.sampling = True
            self._graphs.clear()

    def set_sampling_seed(self, seed: int) -> None:
        """end2end.py:120-134."""
        if seed != self.sampling_seed:
            self.sampling_seed = seed
            self._graphs.clear()

    def inject_cache(self, layer_caches, start_pos: int = 0, end_pos: int | None = None) -> None:
        """``layer_caches``: one (ki, kv, pe) bf16 triple per layer from an external prefill
        (DSAv32Generator.inject_cache, generator.py:419-484); follow with ``set_cur_pos``.  A triple of
        uint8 planes (kv_raw [seq, 528], pe_raw [seq, 128], ki_pages [pages, 8448]) is taken as the FP8 wire
        format of pd_vllm/profiles/mla_nsa.py and needs ``end_pos`` (the pages do not tell the length)."""
        for layer, (c0, c1, c2) in zip(self.layers, layer_caches):
            if c0.dtype == torch.uint8:
                if end_pos is None:
                    raise ValueError("inject_cache: end_pos is needed with FP8 planes")
                layer.inject_cache_fp8(c0, c1, c2, end_pos - start_pos, start_pos)
            else:
                n = c0.shape[0] if end_pos is None else end_pos - start_pos
                layer.inject_cache(c0[:n], c1[:n], c2[:n], start_pos)

    def _step_ops(self, n_keys: int) -> None:
        x = self.embed[self.token].view(1, 1, -1)
        fr = self.freqs[self.cur_pos.long()]
        for layer in self.layers:
            x = layer.forward(x, self.cur_pos, fr, n_keys)
        ops.rmsnorm_head_proj(x, self.final_norm, self.head, None, self.logits, eps=self.args.eps)
        if self.world > 1 and self.sampling:
            # every rank gathers all slices of the logits (517 KB) and draws the same token: same seed, same step
            import torch.distributed as dist

            dist.all_gather_into_tensor(self.full_logits, self.logits.view(-1))
            ops.sample(self.full_logits.view(1, -1), self.sampling_config, self.sampled, seed=self.sampling_seed,
                       step=self.sample_step, token_logprob=self.token_logprob, topn_logprobs=self.topn_logprobs,
                       topn_indices=self.topn_indices)
            self.token_out.copy_(self.sampled)
        elif self.world > 1:
            # every rank holds vocab / world rows of the head: exchange (value, index) pairs over peer memory
            ops.argmax_exchange(self.logits, self.rank * self.logits.shape[-1], self.token_out, comm=self.comm)
        elif self.sampling:
            ops.sample(self.logits.view(1, -1), self.sampling_config, self.sampled, seed=self.sampling_seed,
                       step=self.sample_step, token_logprob=self.token_logprob, topn_logprobs=self.topn_logprobs,
                       topn_indices=self.topn_indices)
            self.token_out.copy_(self.sampled)
        else:
            self.token_out.copy_(torch.argmax(self.logits.view(-1)))
        if self.temp_vars is not None:
            from .temp_var_indices import Idx

            self.temp_vars[Idx.TOKEN_OUT].view(-1)[:1].copy_(self.token_out)
            self.temp_vars[Idx.TOKEN_ID].view(-1)[:1].copy_(self.token)
        self.cur_pos += 1

    def _bucket(self, pos: int) -> int:
        """Indexer scan length: next multiple of 256 above the position, so graphs are reused."""
        return min(self.cache_len, (pos // 256 + 1) * 256)

    def forward(self, token: int | torch.Tensor, pos: int) -> None:
        """Run one decode step for ``token`` at position ``pos`` (asynchronous; results in
        ``self.logits`` / ``self.token_out``)."""
        if pos != self._pos:
            raise ValueError(f"forward(pos={pos}): the device position is {self._pos} (use set_cur_pos to move it)")
        if pos >= self.cache_len or pos >= self.freqs.shape[0]:
            raise ValueError(f"forward(pos={pos}): past the end of the caches ({self.cache_len} rows) or of the rotary "
                             f"table ({self.freqs.shape[0]} positions)")
        if isinstance(token, int):
            self.token.fill_(token)
        else:
            self.token.copy_(token.view(-1)[:1])
        self._pos = pos + 1
        n_keys = self._bucket(pos)
        if not self.use_graph or (self.sampling and self.world > 1):  # the gather is a library collective: not captured
            self._step_ops(n_keys)
            return
        if n_keys not in self._graphs:
            saved, saved_step = self.cur_pos.clone(), self.sample_step.clone()
            self._step_ops(n_keys)  # warm-up outside capture (lazy function attributes, allocator)
            torch.cuda.synchronize()
            self.cur_pos.copy_(saved)
            self.sample_step.copy_(saved_step)  # the warm-up drew a number: give it back
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
