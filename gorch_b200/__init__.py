"""gorch_b200: the decode-time token-sampling step of gorch (greedy, temperature,
top-k, top-p, inverse-CDF draw) as hand-written sm_100a CUDA kernels behind a C ABI.

The package holds only that path and its nearest neighbours: csrc/ (kernels + the
C ABI of libgorchcuda.so), the ctypes binding, a host-side mirror of the
reference's sampling interface (sampling.py), the generate loops with their control
on the device (generate.py), the tensor-level TopK / Multinomial and the row
softmax / cross-entropy ops (sampling.py, row_ops.py), row and vocab sharding
(distributed.py), and the seeded synthetic workloads used for measurement.
"""
from .config import (CFG_DTYPE, FLAG_BAD_CFG, FLAG_BOUNDARY, FLAG_FALLBACK, FLAG_GENERAL_PATH,
                     FLAG_INTERNAL, FLAG_NONFINITE, FLAG_TIE_CUT, FLAG_TOPP_EDGE,
                     MODE_A, MODE_B, GenerateConfig, QwenGenerateConfig, default_generate_config,
                     greedy_config, qwen_greedy)

__all__ = [
    "CFG_DTYPE", "MODE_A", "MODE_B", "GenerateConfig", "QwenGenerateConfig",
    "default_generate_config", "greedy_config", "qwen_greedy",
    "FLAG_BOUNDARY", "FLAG_FALLBACK", "FLAG_NONFINITE", "FLAG_TIE_CUT",
    "FLAG_TOPP_EDGE", "FLAG_GENERAL_PATH", "FLAG_INTERNAL", "FLAG_BAD_CFG",
]
