"""The decode driver behind the reference's names: the ``dsa[_mtp_e2e]_show_hands*`` calls and
``ShowHandsDSALayer`` (tilert/models/deepseek_v3_2/modules/end2end.py:79-163, 166-703).

The reference hands its native library three tensor lists -- ``params`` (the packed weights), ``temp_vars``
(the 56 scratch tensors of ``DsaTempVarIdx``) and ``caches`` ([ki, kv, pe] per layer) -- with
``prepare_money``, then makes ONE call per token (``show_hands``) with the token id in a CPU tensor and
reads the results out of ``temp_vars``.  The same calls exist here; behind them a ``DsaModel`` /
``MtpDsaModel`` replays the step from a CUDA graph.  ``params`` is this library's own packed form
(``StepParams``): the reference's packed layouts are private to its binary.
"""

from __future__ import annotations

import torch

from .model import DsaModel
from .model_args import ModelArgs
from .mtp import N_TOKENS, MtpDsaModel
from .temp_var_indices import Idx, TEMP_VARS_SIZE, validate_temp_vars_layout

BF16, F32, I32, I64 = torch.bfloat16, torch.float32, torch.int32, torch.int64


class StepParams(list):
    """``params`` of ``prepare_money``: a list of tensors (as the reference passes) that also remembers the
    HF-keyed state dict and the model arguments it was made from."""

    def __init__(self, args: ModelArgs, sd: dict[str, torch.Tensor]):
        super().__init__(sd.values())
        self.args, self.sd = args, sd


def get_temp_vars(args: ModelArgs, device, seq_len: int = 1, world: int = 1, temperature: float = 0.0,
                  top_p: float = 1.0, top_k: int = 0, use_topp: bool = False) -> list[torch.Tensor]:
    """The 56 scratch tensors, shaped as Dsa.get_temp_vars shapes them (modules/dsa.py:105-229)."""
    a, dev, bs = args, torch.device(device), (1, seq_len)
    hl, vocab = a.n_heads // world, a.vocab_size // world
    z = lambda *shape, dtype=BF16: torch.zeros(*shape, dtype=dtype, device=dev)  # noqa: E731
    tv: list[torch.Tensor | None] = [None] * TEMP_VARS_SIZE
    n_total = a.n_activated_experts + a.n_shared_experts
    ffn = max(n_total * (a.moe_inter_dim // world), (a.inter_dim // world) if a.n_dense_layers else 0)
    tv[Idx.Q] = z(*bs, a.q_lora_rank)
    tv[Idx.KV] = z(*bs, a.kv_lora_rank)
    tv[Idx.KI] = z(*bs, a.index_head_dim)
    tv[Idx.Q_NOPE_DOWN] = z(*bs, hl, a.qk_nope_head_dim)
    tv[Idx.Q_PE] = z(*bs, hl, a.qk_rope_head_dim)
    tv[Idx.IQ] = z(*bs, a.index_n_heads, a.index_head_dim)
    tv[Idx.IQ_RT] = z(*bs, a.index_n_heads, a.index_head_dim)
    tv[Idx.IDX_SCORES] = z(*bs, a.index_n_heads)
    tv[Idx.IDX_LOGITS] = z(*bs, a.max_seq_len + 8, dtype=F32)
    tv[Idx.IDX_SELECTS] = z(*bs, a.index_topk, dtype=I32)
    tv[Idx.Q_NOPE] = z(*bs, hl, a.kv_lora_rank)
    tv[Idx.O] = z(*bs, hl, a.kv_lora_rank)
    tv[Idx.O_ACC] = z(*bs, hl, 32, a.kv_lora_rank, dtype=F32)
    tv[Idx.O_LSE] = z(*bs, hl, dtype=F32)
    tv[Idx.O_LSE_ACC] = z(*bs, hl, 32, dtype=F32)
    tv[Idx.PROJ_O] = z(*bs, hl, a.v_head_dim)
    tv[Idx.UNPROJ_O] = z(*bs, a.dim)
    tv[Idx.SCORES] = z(*bs, a.n_routed_experts, dtype=F32)
    tv[Idx.X_MLP_IN] = z(*bs, a.dim)
    tv[Idx.UP_GATE] = z(*bs, ffn)
    tv[Idx.SEL_PROBS] = z(*bs, a.n_activated_experts, dtype=F32)
    tv[Idx.SEL_INDICES] = z(*bs, a.n_activated_experts, dtype=I32)
    tv[Idx.EXP_OUT] = z(*bs, a.dim)
    tv[Idx.X_RMSNORM] = z(*bs, a.dim)
    tv[Idx.LOGITS_OUT] = z(*bs, vocab, dtype=F32)
    tv[Idx.TOKEN_OUT] = z(*bs, 1, dtype=I32)
    for i in (Idx.EMBEDDING_RMSNORM, Idx.HIDDEN_RMSNORM, Idx.EH_PROJ, Idx.X_TENSOR, Idx.LAST_HIDDEN_STATES,
              Idx.PREDICTED_HIDDEN, Idx.MTP0_EXP_OUT):
        tv[i] = z(*bs, a.dim)
    tv[Idx.ROPE_FREQS] = z(*bs, a.qk_rope_head_dim, dtype=F32)
    tv[Idx.CUR_POS] = z(1, dtype=I32)
    tv[Idx.TOKEN_ID] = z(*bs, 1, dtype=I32)
    tv[Idx.DRAFT_TOKENS] = z(*bs, dtype=I32)
    tv[Idx.PREDICTED_TOKENS] = z(*bs, 1, dtype=I32)
    tv[Idx.ACCEPTED_TOKENS] = z(1, dtype=I32)
    tv[Idx.NEXT_DRAFT_TOKENS] = z(*bs, dtype=I32)
    tv[Idx.X_QUANT] = torch.zeros(*bs, a.dim, dtype=torch.float8_e4m3fn, device=dev)
    tv[Idx.X_SCALE] = z(*bs, a.dim // 128, dtype=F32)
    tv[Idx.MOE_UP_GATE] = z(*bs, ffn)
    tv[Idx.IDX_SEL_WS] = z(1, dtype=I32)  # (the reference's selection workspace; this library's top-k needs none)
    tv[Idx.MTP0_TOKEN_OUT] = z(*bs, 1, dtype=I32)
    tv[Idx.MTP1_TOKEN_OUT] = z(*bs, 1, dtype=I32)
    tv[Idx.SAMPLING_SEED] = z(*bs, dtype=I64)
    tv[Idx.SAMPLING_POSITIONS] = z(*bs, dtype=I64)
    tv[Idx.SAMPLING_CONFIG] = torch.tensor([temperature, top_p, float(top_k), 1.0 if use_topp else 0.0], dtype=F32,
                                           device=dev)
    tv[Idx.TOP_P_SCORES] = z(*bs, dtype=F32)
    tv[Idx.TOP_P_DEBUG] = z(1, dtype=F32)
    tv[Idx.LORA_SLOT_ID] = z(1, dtype=I32)
    tv[Idx.LORA_RANK] = z(1, dtype=I32)
    tv[Idx.TOP_N_LOG_PROBS] = z(*bs, 256, dtype=F32)
    tv[Idx.TOP_N_INDICES] = z(*bs, 256, dtype=I32)
    tv[Idx.LOGPROBS_FLAG] = z(1, dtype=I32)
    assert all(t is not None for t in tv)
    return tv  # type: ignore[return-value]


class _Driver:
    """What ``prepare_money`` captures: the model behind the ``show_hands`` calls of this process."""

    def __init__(self, params, temp_vars, caches, with_mtp: bool, max_seq_len: int):
        if not isinstance(params, StepParams):
            raise TypeError("params must be a StepParams list (this library's packed form of the weights)")
        validate_temp_vars_layout()
        if len(temp_vars) != TEMP_VARS_SIZE:
            raise RuntimeError(f"temp_vars must hold {TEMP_VARS_SIZE} tensors, got {len(temp_vars)}")
        a = params.args
        dev = temp_vars[Idx.Q].device
        self.with_mtp, self.tv = with_mtp, temp_vars
        if with_mtp:
            self.model = MtpDsaModel(a, params.sd, dev, cache_len=max_seq_len)
        else:
            self.model = DsaModel(a, params.sd, dev, cache_len=max_seq_len, temp_vars=temp_vars)
            self.model.sampling_config = temp_vars[Idx.SAMPLING_CONFIG]
            self.model.topn_logprobs = temp_vars[Idx.TOP_N_LOG_PROBS].view(-1, 256)[:1]
            self.model.topn_indices = temp_vars[Idx.TOP_N_INDICES].view(-1, 256)[:1]
        # the caller's cache tensors become the layers' caches ([ki, kv, pe] per layer, generator.py:474-482)
        layers = list(self.model.layers) + ([self.model.mtp_layer] if with_mtp else [])
        if caches:
            if len(caches) != 3 * len(layers):
                raise RuntimeError(f"caches must hold [ki, kv, pe] for each of the {len(layers)} layers")
            for li, layer in enumerate(layers):
                ki, kv, pe = caches[3 * li: 3 * li + 3]
                layer.ki_cache, layer.kv_cache, layer.pe_cache = ki.view(1, -1, ki.shape[-1]), kv.view(1, -1, kv.shape[-1]), \
                    pe.view(1, -1, pe.shape[-1])
        self.pos = 0

    def step(self, token_id: torch.Tensor) -> None:
        toks = token_id.reshape(-1).tolist()  # a CPU tensor, as the reference's call takes it
        if not self.with_mtp:
            self.model.forward(int(toks[0]), self.pos)
            self.pos += 1
            return
        m = self.model
        m.forward(toks + [0] * (N_TOKENS - len(toks)))
        tv = self.tv
        tv[Idx.PREDICTED_TOKENS].view(-1)[:N_TOKENS].copy_(m.predicted)
        tv[Idx.ACCEPTED_TOKENS].view(-1)[:1].copy_(m.n_accepted)
        tv[Idx.NEXT_DRAFT_TOKENS].view(-1)[:N_TOKENS].copy_(m.next_draft)
        tv[Idx.LOGITS_OUT].view(-1)[: m.logits[0, 0].numel()].copy_(m.logits[0, 0])

    def reset(self) -> None:
        self.model.reset_sequence()
        self.pos = 0

    def set_cur_pos(self, pos: int) -> None:
        self.model.set_cur_pos(pos)
        self.pos = pos


_driver: _Driver | None = None


def _need_driver() -> _Driver:
    if _driver is None:
        raise RuntimeError("dsa_show_hands_prepare_money has not been called")
    return _driver


def dsa_show_hands_prepare_money(params, temp_vars, cache_vars, profile_logs=None, forward_max_seq_len: int = 0,
                                 with_mtp: bool = False, is_glm5: bool = False) -> None:
    """end2end.py:79-96: hand the weights, scratch tensors and caches to the driver."""
    global _driver
    if is_glm5:
        raise ValueError("only model_arch 'deepseek_v3_2' is built")
    max_len = forward_max_seq_len or (cache_vars[0].shape[-2] if cache_vars else params.args.max_seq_len)
    _driver = _Driver(params, temp_vars, cache_vars, with_mtp, max_len)


def dsa_show_hands(token_id: torch.Tensor, with_mtp: bool = False, is_glm5: bool = False) -> None:
    """end2end.py:99-104: one decode step (asynchronous; results in ``temp_vars``)."""
    d = _need_driver()
    if with_mtp != d.with_mtp:
        raise RuntimeError("the driver was prepared for the other mode (with / without MTP)")
    d.step(token_id)


def dsa_show_hands_reset(with_mtp: bool = False, is_glm5: bool = False) -> None:
    """end2end.py:107-112."""
    _need_driver().reset()


def dsa_show_hands_go_home(with_mtp: bool = False, is_glm5: bool = False) -> None:
    """end2end.py:115-120: release the driver."""
    global _driver
    if _driver is not None:
        torch.cuda.synchronize()
    _driver = None


def dsa_show_hands_set_sampling_seed(seed: int, with_mtp: bool = False, is_glm5: bool = False) -> None:
    """end2end.py:123-134."""
    d = _need_driver()
    if not d.with_mtp:
        d.model.set_sampling_seed(seed)


def dsa_show_hands_set_cur_pos(pos: int) -> None:
    """generator.py:508."""
    _need_driver().set_cur_pos(pos)


def dsa_mtp_e2e_show_hands_set_prefill_valid_tokens(num_valid_tokens: int, is_glm5: bool = False) -> None:
    """end2end.py:137-151."""
    _need_driver().model.set_prefill_valid_tokens(num_valid_tokens)


def dsa_mtp_e2e_show_hands_set_prefill_mtp_extra_token(token: int, is_glm5: bool = False) -> None:
    """end2end.py:154-163."""
    _need_driver().model.set_prefill_mtp_extra_token(token)


class ShowHandsDSALayer:
    """end2end.py:166-703: owns the three tensor lists and drives the step through the calls above."""

    def __init__(self, model_args: ModelArgs, device="cuda:0", max_seq_len: int | None = None, with_mtp: bool = False):
        self.model_args, self.device, self.with_mtp = model_args, torch.device(device), with_mtp
        self.max_seq_len = max_seq_len or model_args.max_seq_len
        self.params: StepParams | None = None
        self.temp_vars: list[torch.Tensor] | None = None
        self.caches: list[torch.Tensor] = []
        self.sampling = {"temperature": 0.0, "top_p": 1.0, "top_k": 0, "use_topp": False}

    # -- weights --
    def from_state_dict(self, sd: dict[str, torch.Tensor]) -> None:
        """HF-keyed FP8 state dict (the reference's ``from_pretrained`` / ``init_random_weights`` roles)."""
        a = self.model_args
        self.params = StepParams(a, sd)
        self.temp_vars = get_temp_vars(a, self.device, N_TOKENS if self.with_mtp else 1, **self.sampling)
        n_layers = a.n_layers + (1 if self.with_mtp else 0)
        z = lambda d: torch.zeros(1, self.max_seq_len, d, dtype=BF16, device=self.device)  # noqa: E731
        self.caches = [t for _ in range(n_layers) for t in (z(a.index_head_dim), z(a.kv_lora_rank), z(a.qk_rope_head_dim))]
        dsa_show_hands_prepare_money(self.params, self.temp_vars, self.caches, None, self.max_seq_len, self.with_mtp)

    def init_random_weights(self, seed: int = 0) -> None:
        """tilert/generate.py:106-110 (``--use-random-weights``)."""
        from tilert_b200 import synthetic

        self.from_state_dict(synthetic.random_model_state_dict(self.model_args, self.device, seed=seed,
                                                               with_mtp=self.with_mtp))

    # -- the step --
    def forward(self, token, with_mtp: bool | None = None):
        """end2end.py:551-558.  Returns ``[(temp_vars,)]`` -- one entry per device of this process."""
        t = token if isinstance(token, torch.Tensor) else torch.tensor(token)
        dsa_show_hands(t.detach().to("cpu", torch.int64), with_mtp=self.with_mtp)
        return [(self.temp_vars,)]

    def reset_sequence(self) -> None:
        dsa_show_hands_reset(self.with_mtp)

    def set_sampling_seed(self, seed: int, with_mtp: bool | None = None) -> None:
        dsa_show_hands_set_sampling_seed(seed, self.with_mtp)

    def update_sampling_config(self, temperature: float = 0.0, top_p: float = 1.0, top_k: int = 0,
                               use_topp: bool = False) -> None:
        """end2end.py:253-311."""
        self.sampling = {"temperature": temperature, "top_p": top_p, "top_k": top_k, "use_topp": use_topp}
        d = _need_driver()
        if not d.with_mtp:
            d.model.set_sampling(temperature, top_p, top_k, use_topp)

    def get_logits(self) -> torch.Tensor:
        """end2end.py:653-663: the last step's logits."""
        return self.temp_vars[Idx.LOGITS_OUT]

    def get_top_n_logprobs(self, n: int = 256) -> tuple[torch.Tensor, torch.Tensor]:
        """end2end.py:665-692."""
        return self.temp_vars[Idx.TOP_N_LOG_PROBS][..., :n], self.temp_vars[Idx.TOP_N_INDICES][..., :n]

    def cleanup(self) -> None:
        dsa_show_hands_go_home(self.with_mtp)
