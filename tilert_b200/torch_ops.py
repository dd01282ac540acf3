"""``torch.ops.tilert.*``: the dispatcher names and argument orders the reference's Python wrappers and
driver call (tilert/models/deepseek_v3_2/ops/*.py, modules/end2end.py:79-163).

The per-operator names are registered by the native library itself -- ``tilert_b200/libtilert_dsv32.so``, a
``TORCH_LIBRARY(tilert, ...)`` translation unit (csrc/torch_binding.cpp) that forwards every operator to the
C ABI of ``libtilert_b200.so`` -- and ``register()`` loads it the way the reference loads its own library
(``ctypes.CDLL`` + ``torch.ops.load_library``, tilert/__init__.py:68-77).  The driver calls
(``dsa[_mtp_e2e]_show_hands*``) are added to the same namespace from Python: their implementation is the
Python driver in ``models/deepseek_v3_2/end2end.py``.

Weight operands are this library's packed tensors (``tilert_b200.pack``): the reference's own packed layouts
are private to its binary.  Every operator writes into caller-allocated outputs and returns nothing.
"""

from __future__ import annotations

from pathlib import Path

import torch

_FRAGMENT: torch.library.Library | None = None

NATIVE_OPS = [
    "tilert_init_op", "tilert_force_init_op", "dsa_temp_vars_size", "alloc_misc_ws", "rmsnorm_op", "rmsnorm_quant_op",
    "projx_wqkva_op", "proj_w_op", "rmsnorm_proj_qb_op", "rmsnorm_kv_op", "qkv_rope_op", "rotate_op",
    "layernorm_rope_rotate_op", "sparse_index_op", "sparse_index_topk_dsv32_op", "topk_accurate_op", "topk_approximate_op",
    "projq_wqb_op", "flash_sparse_mla_op", "projo_wkvb_op", "unproj_o_allreduce_op", "down_allreduce_op", "padded_allreduce_add_op",
    "rmsnorm_expert_proj_op", "expert_select_up_gate_silu_op", "expert_down_allreduce_op", "rmsnorm_up_gate_silu_op",
    "rmsnorm_head_proj_op", "eh_proj_allreduce_op",
]
DRIVER_OPS = [
    "dsa_show_hands_prepare_money", "dsa_show_hands", "dsa_show_hands_reset", "dsa_show_hands_go_home",
    "dsa_show_hands_set_sampling_seed", "dsa_show_hands_set_cur_pos", "dsa_mtp_e2e_show_hands_prepare_money",
    "dsa_mtp_e2e_show_hands", "dsa_mtp_e2e_show_hands_reset", "dsa_mtp_e2e_show_hands_go_home",
    "dsa_mtp_e2e_show_hands_set_sampling_seed", "dsa_mtp_e2e_show_hands_set_prefill_valid_tokens",
    "dsa_mtp_e2e_show_hands_set_prefill_mtp_extra_token",
]


def library_path() -> Path:
    return Path(__file__).resolve().parent / "libtilert_dsv32.so"


def op_names() -> list[str]:
    """Names available under ``torch.ops.tilert`` after :func:`register`."""
    return [*NATIVE_OPS, *DRIVER_OPS]


# ``prepare_money`` receives plain tensor lists through the dispatcher; the weights' state dict and model
# arguments travel beside them (the reference's native side knows its own packed layout instead).
_pending_params = None


def bind_params(params) -> None:
    """Tell the next ``torch.ops.tilert.dsa*_show_hands_prepare_money`` call which ``StepParams`` its ``params``
    tensor list belongs to (a dispatcher call cannot carry the Python object itself)."""
    global _pending_params
    _pending_params = params


def register() -> None:
    """Load the registration library and add the driver calls (once per process; a second call is a no-op).

    Raises ``RuntimeError`` if the library is missing, or if another library has already defined the
    namespace (the reference's own ``libtilert*.so`` in the same process): the two backends cannot be mixed."""
    global _FRAGMENT
    if _FRAGMENT is not None:
        return
    import tilert_b200 as tb

    tb.load_backend("deepseek_v3_2")  # libtilert_b200.so first (RTLD_GLOBAL): the registration library links to it
    path = library_path()
    if not path.exists():
        raise RuntimeError(f"{path} not found: build it with `python -m tilert_b200.build`")
    torch.ops.load_library(str(path))

    from .models.deepseek_v3_2 import end2end as e2e

    lib = torch.library.Library("tilert", "FRAGMENT")

    def prepare(with_mtp):
        def fn(params, temp_vars, cache_vars, profile_logs=None, forward_max_seq_len=0):
            global _pending_params
            sp, _pending_params = _pending_params, None
            if sp is None or len(sp) != len(params):
                raise RuntimeError("call tilert_b200.torch_ops.bind_params(step_params) before prepare_money")
            e2e.dsa_show_hands_prepare_money(sp, list(temp_vars), list(cache_vars), profile_logs, forward_max_seq_len, with_mtp)
        return fn

    for mtp, flag in ((False, ""), (True, "_mtp_e2e")):
        pre = f"dsa{flag}_show_hands"
        lib.define(f"{pre}_prepare_money(Tensor[] params, Tensor(a!)[] temp_vars, Tensor(b!)[] cache_vars, "
                   "Tensor? profile_logs=None, int forward_max_seq_len=0) -> ()")
        lib.impl(f"{pre}_prepare_money", prepare(mtp), "CompositeExplicitAutograd")
        lib.define(f"{pre}(Tensor token_id) -> ()")
        lib.impl(pre, (lambda m: lambda token_id: e2e.dsa_show_hands(token_id, with_mtp=m))(mtp), "CompositeExplicitAutograd")
        lib.define(f"{pre}_reset() -> ()")
        lib.impl(f"{pre}_reset", (lambda m: lambda: e2e.dsa_show_hands_reset(m))(mtp), "CompositeExplicitAutograd")
        lib.define(f"{pre}_go_home() -> ()")
        lib.impl(f"{pre}_go_home", (lambda m: lambda: e2e.dsa_show_hands_go_home(m))(mtp), "CompositeExplicitAutograd")
        lib.define(f"{pre}_set_sampling_seed(int seed) -> ()")
        lib.impl(f"{pre}_set_sampling_seed", (lambda m: lambda seed: e2e.dsa_show_hands_set_sampling_seed(seed, m))(mtp),
                 "CompositeExplicitAutograd")
    lib.define("dsa_show_hands_set_cur_pos(int pos) -> ()")
    lib.impl("dsa_show_hands_set_cur_pos", e2e.dsa_show_hands_set_cur_pos, "CompositeExplicitAutograd")
    lib.define("dsa_mtp_e2e_show_hands_set_prefill_valid_tokens(int num_valid_tokens) -> ()")
    lib.impl("dsa_mtp_e2e_show_hands_set_prefill_valid_tokens", e2e.dsa_mtp_e2e_show_hands_set_prefill_valid_tokens,
             "CompositeExplicitAutograd")
    lib.define("dsa_mtp_e2e_show_hands_set_prefill_mtp_extra_token(int token) -> ()")
    lib.impl("dsa_mtp_e2e_show_hands_set_prefill_mtp_extra_token", e2e.dsa_mtp_e2e_show_hands_set_prefill_mtp_extra_token,
             "CompositeExplicitAutograd")
    _FRAGMENT = lib
