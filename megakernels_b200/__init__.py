"""B200-native low-latency Llama decode engine.

Host side (Python/PyTorch) mirrors the operator surface of the reference
``megakernels`` package for its latency hot path: the instruction set, the
DAG -> per-SM scheduler, the generators/dispatch entry points and
``scripts/generate.py mode=mk``.  The device side is one persistent sm_100a
CUDA kernel reached through a C-ABI shared library (``native/libmkb200.so``).
There is no CPU fallback: every interpret call goes to the CUDA library and
fails loudly when it is missing.
"""

__version__ = "0.1.0"
