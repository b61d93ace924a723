"""flydsl_b200 — B200 (sm_100a) implementation of FlyDSL's FP8 block-scale GEMM / MoE hot path.

Python entry points keep the reference's names and call signatures; all compute happens in
``lib/libflyb200.so`` (hand-written CUDA, C ABI declared in ``include/flyb200.h``).
"""
__version__ = "0.1.0"

from . import compiler  # noqa: F401
from .compiler import compile  # noqa: F401,A001
