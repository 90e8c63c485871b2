"""Generation config types, mirroring the reference's Go structs.

GenerateConfig      <- model/generate.go:13-20 (fields, zero-value meanings)
default_generate_config / greedy_config
                    <- model/generate.go:23-42
QwenGenerateConfig  <- model/qwen/generate.go:13-29
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

# Which of the reference's two top-p routines a row follows.
MODE_A = 0  # model/generate.go:184-228: trim the tail until mass <= 1.5*p
MODE_B = 1  # model/qwen/generate.go:123-153: shortest descending prefix with mass >= p

# Per-row device record, 16 bytes: {float T; int32 k; float p; int32 mode}.
CFG_DTYPE = np.dtype(
    [("temperature", "<f4"), ("top_k", "<i4"), ("top_p", "<f4"), ("topp_mode", "<i4")]
)

# out_flags bits written per row by the sampling kernels.
FLAG_BOUNDARY = 1 << 0      # uniform within 1e-6 of an edge of the chosen CDF interval
FLAG_FALLBACK = 1 << 1      # walk fell through: id = V-1 (model/generate.go:239)
FLAG_NONFINITE = 1 << 2     # NaN / +-Inf poisoned the softmax: id = V-1 as in the reference
FLAG_TIE_CUT = 1 << 3       # mode B: the cut separates equal probabilities (order unpinned upstream)
FLAG_TOPP_EDGE = 1 << 5     # top-p stop test decided within 1e-12 of its threshold
FLAG_GENERAL_PATH = 1 << 6  # row took the full-row path (informational)
FLAG_INTERNAL = 1 << 7      # an internal invariant failed; the id is unreliable
FLAG_BAD_CFG = 1 << 8       # temperature negative, NaN or infinite; id = -1

DTYPE_F32 = 0
DTYPE_BF16 = 1


@dataclass
class GenerateConfig:
    """model/generate.go:13-20. Temperature 0 => greedy; TopK 0 => off; TopP 0 =>
    off (and >= 1 is inert, generate.go:184); StopToken -1 => off."""
    max_new_tokens: int = 50
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.0
    stop_token: int = -1
    use_kv_cache: bool = False

    topp_mode: int = MODE_A

    def row_cfg(self) -> np.ndarray:
        rec = np.zeros(1, dtype=CFG_DTYPE)
        rec[0] = (self.temperature, self.top_k, self.top_p, self.topp_mode)
        return rec


def default_generate_config() -> GenerateConfig:
    """model/generate.go:23-31."""
    return GenerateConfig(max_new_tokens=50, temperature=0.8, top_k=40, top_p=0.0, stop_token=-1)


def greedy_config(max_tokens: int) -> GenerateConfig:
    """model/generate.go:34-42."""
    return GenerateConfig(max_new_tokens=max_tokens, temperature=0.0, top_k=0, top_p=0.0,
                          stop_token=-1)


@dataclass
class QwenGenerateConfig:
    """model/qwen/generate.go:13-20: no UseKVCache (always cached), a list of
    stop tokens, and a seed for the host-side uniform stream."""
    max_new_tokens: int = 0
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 0.0
    stop_tokens: list = field(default_factory=list)
    seed: int = 0

    topp_mode: int = MODE_B

    def row_cfg(self) -> np.ndarray:
        rec = np.zeros(1, dtype=CFG_DTYPE)
        rec[0] = (self.temperature, self.top_k, self.top_p, self.topp_mode)
        return rec


def qwen_greedy(max_new_tokens: int) -> QwenGenerateConfig:
    """model/qwen/generate.go:24-29 (ChatML stop tokens)."""
    return QwenGenerateConfig(max_new_tokens=max_new_tokens, stop_tokens=[151645, 151643])
