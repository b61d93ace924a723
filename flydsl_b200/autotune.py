"""Tile-configuration autotuner with a persistent cache for the dense block-scale GEMM.

Plays the part of the reference's autotuner (python/flydsl/autotune.py:91-268: benchmark a list of
configurations per key, keep the best, persist it as JSON) and of ``select_tile_config`` in its
dense test. A configuration here is what the C ABI's ``flyb200_gemm_cfg`` exposes: MMA width
``block_n``, kernel ``path`` (tiled / decode) and ``split_k``. The key is the shape with M rounded
up to a power-of-two bucket, the output type and the device name.

    tuner = GemmAutotuner()                       # cache: $FLYB200_AUTOTUNE_CACHE_DIR or ~/.flyb200
    fn = tuner.tuned_gemm(M=4096, N=7168, K=2048) # benchmarks once per key, then reads the cache
    fn(c, a, b_shuffled, scale_a_t, scale_b, M, N, stream)
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Callable, Dict, Iterable, List, Optional


class Config:
    """One candidate: keyword arguments of ``compile_blockscale_preshuffle_gemm``."""

    def __init__(self, *, block_n: Optional[int] = None, path: str = "auto", split_k: Optional[int] = None):
        self.block_n, self.path, self.split_k = block_n, path, split_k

    def kwargs(self) -> dict:
        return {"block_n": self.block_n, "path": self.path, "split_k": self.split_k}

    def to_dict(self) -> dict:
        return self.kwargs()

    @classmethod
    def from_dict(cls, d: dict) -> "Config":
        return cls(block_n=d.get("block_n"), path=d.get("path", "auto"), split_k=d.get("split_k"))

    def __repr__(self) -> str:
        return f"Config(block_n={self.block_n}, path={self.path!r}, split_k={self.split_k})"

    def __eq__(self, other) -> bool:
        return isinstance(other, Config) and self.to_dict() == other.to_dict()


def do_bench(fn: Callable[[], None], warmup: int = 5, rep: int = 25, flush=None) -> float:
    """Median milliseconds of ``fn`` by CUDA events on the current stream; ``flush`` (a tensor larger
    than L2) is zeroed before every timed call so operands come from HBM."""
    import torch

    for _ in range(warmup):
        fn()
    times = []
    for _ in range(rep):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2]


def m_bucket(m: int) -> int:
    """Power-of-two bucket of the row count (1, 2, 4, ... ): shapes in a bucket share a configuration."""
    b = 1
    while b < m:
        b <<= 1
    return b


def default_configs(M: int, N: int, K: int) -> List[Config]:
    cands = [Config()]                                                  # the library heuristic
    for bn in (256, 128, 64, 32):
        if bn <= max(32, N):
            cands.append(Config(block_n=bn, path="tiled"))
    if M <= 64:
        for s in (None, 1, 2, 4, 8):
            if s is None or (K // 128) % s == 0:
                cands.append(Config(path="decode", split_k=s))
    return cands


class GemmAutotuner:
    def __init__(self, cache_dir: Optional[str] = None, warmup: int = 5, rep: int = 25,
                 do_bench_fn: Optional[Callable] = None, device_name: Optional[str] = None):
        root = cache_dir or os.environ.get("FLYB200_AUTOTUNE_CACHE_DIR") or os.path.expanduser("~/.flyb200/autotune")
        self._cache_file = Path(root) / "blockscale_gemm.json"
        self.warmup, self.rep = warmup, rep
        self._do_bench = do_bench_fn or do_bench
        self._device_name = device_name
        self.cache: Dict[str, Config] = {}
        self.timings: Dict[str, Dict[str, float]] = {}
        self._load()

    # ---- cache ----
    def _load(self) -> None:
        try:
            raw = json.loads(self._cache_file.read_text())
        except (OSError, ValueError):
            return
        for key, d in raw.items():
            try:
                self.cache[key] = Config.from_dict(d)
            except (TypeError, AttributeError):
                continue

    def _save(self) -> None:
        try:
            self._cache_file.parent.mkdir(parents=True, exist_ok=True)
            tmp = self._cache_file.with_suffix(".tmp")
            tmp.write_text(json.dumps({k: c.to_dict() for k, c in sorted(self.cache.items())}, indent=1))
            os.replace(tmp, self._cache_file)
        except OSError:
            pass  # a read-only home directory must not break the GEMM

    def key(self, M: int, N: int, K: int, out_dtype: str = "bf16") -> str:
        name = self._device_name
        if name is None:
            import torch

            name = torch.cuda.get_device_name() if torch.cuda.is_available() else "nodevice"
            self._device_name = name
        return f"{name}|m{m_bucket(M)}|n{N}|k{K}|{out_dtype}"

    # ---- tuning ----
    def tune(self, M: int, N: int, K: int, out_dtype: str = "bf16",
             configs: Optional[Iterable[Config]] = None, make_call: Optional[Callable] = None) -> Config:
        """Best configuration for the shape (cached). ``make_call(config) -> callable`` may be supplied
        (tests do, to stay off the GPU); by default synthetic operands are built on the current device."""
        key = self.key(M, N, K, out_dtype)
        if key in self.cache:
            return self.cache[key]
        cands = list(configs) if configs is not None else default_configs(M, N, K)
        flush = None
        if make_call is None:
            make_call, flush = self._synthetic_problem(M, N, K, out_dtype)
        best, best_ms, seen = None, float("inf"), {}
        for cfg in cands:
            try:
                call = make_call(cfg)
                ms = self._do_bench(call, warmup=self.warmup, rep=self.rep, flush=flush) if flush is not None \
                    else self._do_bench(call, warmup=self.warmup, rep=self.rep)
            except (ValueError, RuntimeError):
                continue                      # configuration not valid for this shape
            seen[repr(cfg)] = ms
            if ms < best_ms:
                best, best_ms = cfg, ms
        if best is None:
            raise RuntimeError(f"no configuration ran for M={M} N={N} K={K}")
        self.cache[key], self.timings[key] = best, seen
        self._save()
        return best

    @staticmethod
    def _synthetic_problem(M, N, K, out_dtype):
        import torch

        from .kernels import compile_blockscale_preshuffle_gemm
        from .utils import FP8_DTYPE, shuffle_weight

        dev = torch.device("cuda", torch.cuda.current_device())
        a = torch.randn(M, K, device=dev).to(FP8_DTYPE)
        b = shuffle_weight((torch.randn(N, K, device=dev) * 0.5).to(FP8_DTYPE))
        sa = torch.rand(K // 128, M, device=dev)
        sb = torch.rand((N + 127) // 128, K // 128, device=dev)
        c = torch.empty(M, N, dtype=torch.bfloat16 if out_dtype == "bf16" else torch.float16, device=dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

        def make_call(cfg: Config):
            fn = compile_blockscale_preshuffle_gemm(M=M, N=N, K=K, tile_m=64, tile_n=128, tile_k=128,
                                                    out_dtype=out_dtype, **cfg.kwargs())
            fn(c, a, b, sa, sb, M, N, None)      # raises here if the configuration is invalid
            return lambda: fn(c, a, b, sa, sb, M, N, None)

        return make_call, flush

    def tuned_gemm(self, *, M: int, N: int, K: int, out_dtype: str = "bf16", **factory_kwargs):
        """Launcher of ``compile_blockscale_preshuffle_gemm`` with the tuned configuration."""
        from .kernels import compile_blockscale_preshuffle_gemm

        cfg = self.tune(M, N, K, out_dtype)
        kw = dict(tile_m=64, tile_n=128, tile_k=128)
        kw.update(factory_kwargs)
        return compile_blockscale_preshuffle_gemm(M=M, N=N, K=K, out_dtype=out_dtype, **kw, **cfg.kwargs())
