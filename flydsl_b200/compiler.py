"""Call-site pre-binding, the counterpart of ``flydsl.compiler.compile`` (``flyc.compile``,
python/flydsl/compiler/jit_function.py:895-954 of the reference).

In the reference ``flyc.compile(fn, *args)`` JIT-compiles for the argument types and returns a fast
positional-only callable. Here nothing is compiled at run time, so ``compile`` validates the example
arguments once (device, contiguity, dtype per position) and returns the launcher itself wrapped in
a thin callable that skips those checks afterwards. As in the reference, only ``data_ptr()`` of each
tensor is read per call; a tensor must keep the dtype it was bound with.
"""
from __future__ import annotations

import torch


class CompiledFunction:
    """Positional-only callable bound to one launcher and one per-position dtype signature."""

    def __init__(self, fn, dtypes):
        self._fn = fn
        self._dtypes = dtypes

    def __call__(self, *args):
        return self._fn(*args)

    def check(self, *args):
        """Re-validate a full argument list against the bound signature (debug aid)."""
        _validate(args, self._dtypes)


def _validate(args, dtypes=None):
    got = []
    for i, a in enumerate(args):
        if isinstance(a, torch.Tensor):
            if not a.is_cuda:
                raise ValueError(f"argument {i}: tensor must live on a CUDA device")
            if not a.is_contiguous():
                raise ValueError(f"argument {i}: tensor must be contiguous")
            got.append(a.dtype)
        else:
            got.append(type(a))
    if dtypes is not None and tuple(got) != tuple(dtypes):
        raise TypeError(f"argument types {got} do not match the bound signature {list(dtypes)}")
    return tuple(got)


def compile(fn, *args):  # noqa: A001 - name mirrors the reference API
    """Bind ``fn`` (a launcher from ``flydsl_b200.kernels``) to the types of ``args`` and run it once,
    as the reference does on first call. Returns the fast callable."""
    dtypes = _validate(args)
    fn(*args)
    return CompiledFunction(fn, dtypes)
