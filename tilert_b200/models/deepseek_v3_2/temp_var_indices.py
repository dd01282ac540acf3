"""Names of the decode step's scratch tensors, in the order the driver and Python share them.

The numbering is an ABI: it must match tilert/models/deepseek_v3_2/temp_var_indices.py:15-76 so
that code indexing ``intermediates[Idx.TOKEN_OUT]`` keeps working.  ``validate_temp_vars_layout``
checks the count against the native library like the reference does (:81-118).
"""

from enum import IntEnum

_NAMES = (
    "Q",
    "KV",
    "KI",
    "Q_NOPE_DOWN",
    "Q_PE",
    "IQ",
    "IQ_RT",
    "IDX_SCORES",
    "IDX_LOGITS",
    "IDX_SELECTS",
    "Q_NOPE",
    "O",
    "O_ACC",
    "O_LSE",
    "O_LSE_ACC",
    "PROJ_O",
    "UNPROJ_O",
    "SCORES",
    "X_MLP_IN",
    "UP_GATE",
    "SEL_PROBS",
    "SEL_INDICES",
    "EXP_OUT",
    "X_RMSNORM",
    "LOGITS_OUT",
    "TOKEN_OUT",
    "EMBEDDING_RMSNORM",
    "HIDDEN_RMSNORM",
    "EH_PROJ",
    "X_TENSOR",
    "ROPE_FREQS",
    "CUR_POS",
    "TOKEN_ID",
    "LAST_HIDDEN_STATES",
    "DRAFT_TOKENS",
    "PREDICTED_TOKENS",
    "PREDICTED_HIDDEN",
    "ACCEPTED_TOKENS",
    "NEXT_DRAFT_TOKENS",
    "X_QUANT",
    "X_SCALE",
    "MOE_UP_GATE",
    "IDX_SEL_WS",
    "MTP0_TOKEN_OUT",
    "MTP1_TOKEN_OUT",
    "MTP0_EXP_OUT",
    "SAMPLING_SEED",
    "SAMPLING_POSITIONS",
    "SAMPLING_CONFIG",
    "TOP_P_SCORES",
    "TOP_P_DEBUG",
    "LORA_SLOT_ID",
    "LORA_RANK",
    "TOP_N_LOG_PROBS",
    "TOP_N_INDICES",
    "LOGPROBS_FLAG",
)

DsaTempVarIdx = IntEnum("DsaTempVarIdx", {name: i for i, name in enumerate(_NAMES)})
Idx = DsaTempVarIdx
TEMP_VARS_SIZE = len(_NAMES)


def validate_temp_vars_layout() -> None:
    """Raise if the native library disagrees on the number of scratch tensors."""
    from tilert_b200 import lib

    native = lib().tilert_b200_dsa_temp_vars_size()
    if native != TEMP_VARS_SIZE:
        raise RuntimeError(f"temp-var layout mismatch: python {TEMP_VARS_SIZE}, native {native}")
