"""Shape-keyed backend dispatcher.

Same contract as the reference's tritonix/dispatcher.py:38-175: implementations are registered
under names, the first call for a new tuning key times every backend, the fastest is cached in
``.cache`` (its timings in ``.timings``) and, optionally, on disk.  In this package the only
backend registered for the contraction ops is ``"cuda"``; the class itself stays general.

Disk layout: ``<cache dir>/<sha256(op - sorted backends - key)>/backend_dispatch.json`` holding
``{"op", "key", "winner", "timings"}`` — the reference's payload (dispatcher.py:120-128).  The
cache directory is ``$TRITONIX_B200_CACHE_DIR`` or ``~/.cache/tritonix_b200`` (the reference
borrowed Triton's cache manager, which this package does not depend on).
"""
from __future__ import annotations

import hashlib
import inspect
import json
import logging
import os
import tempfile
from contextlib import contextmanager
from pathlib import Path
from typing import Callable, Dict, List, Optional

import torch

from tritonix_b200.testing import do_bench

log = logging.getLogger("tritonix.dispatcher")

_CACHE_FILE = "backend_dispatch.json"


def cache_dir() -> Path:
    return Path(os.environ.get("TRITONIX_B200_CACHE_DIR",
                               os.path.join(os.path.expanduser("~"), ".cache", "tritonix_b200")))


def _describe(value):
    if isinstance(value, torch.Tensor):
        return [*value.shape, str(value.dtype)]
    return [value]


def _tuning_key(key_names: List[str], args: tuple, kwargs: dict, arg_names: List[str]) -> tuple:
    """Named key arguments first (tensors contribute their shape and dtype, other values
    themselves), then every remaining tensor argument (dispatcher.py:18-30)."""
    bound = dict(zip(arg_names, args))
    bound.update(kwargs)
    parts: list = []
    for name in key_names:
        if name in bound:
            parts += _describe(bound[name])
    named = set(key_names)
    for name, value in bound.items():
        if name not in named and isinstance(value, torch.Tensor):
            parts += _describe(value)
    return tuple(parts)


def _disk_key(op_name: str, backends: List[str], tuning_key: tuple) -> str:
    text = "-".join([op_name, str(sorted(backends)), str(tuning_key)])
    return hashlib.sha256(text.encode()).hexdigest()


class DynamicDispatcher:
    def __init__(self, fn: Callable, key: List[str], arg_names: List[str], warmup: float = 25,
                 rep: float = 100, use_disk_cache: bool = True):
        self._fn = fn
        self._key_names = list(key)
        self._arg_names = list(arg_names)
        self._warmup = warmup
        self._rep = rep
        self._disk = use_disk_cache
        self._backends: Dict[str, Callable] = {}
        self._forced: Optional[str] = None
        self.cache: Dict[tuple, str] = {}
        self._key_memo: Dict[tuple, tuple] = {}
        self.timings: Dict[tuple, Dict[str, float]] = {}
        self.__name__ = getattr(fn, "__name__", type(fn).__name__)
        self.__doc__ = fn.__doc__

    def register(self, name: str, impl: Callable) -> "DynamicDispatcher":
        self._backends[name] = impl
        return self

    def __call__(self, *args, **kwargs):
        if not self._backends:
            raise RuntimeError(f"[{self.__name__}] No backends registered.")
        if self._forced is not None:
            return self._backends[self._forced](*args, **kwargs)
        key = None
        quick = None
        if not kwargs:
            # the tuning key of a positional call depends only on the tensors' shapes and dtypes
            # and on the other arguments themselves: remember it instead of rebuilding it
            try:
                quick = tuple((a.shape, a.dtype) if isinstance(a, torch.Tensor) else a for a in args)
                key = self._key_memo.get(quick)
            except TypeError:  # an unhashable argument
                quick = None
        if key is None:
            key = _tuning_key(self._key_names, args, kwargs, self._arg_names)
            if quick is not None:
                if len(self._key_memo) >= 4096:
                    self._key_memo.clear()
                self._key_memo[quick] = key
        if key not in self.cache:
            self._bench_and_cache(key, args, kwargs)
        return self._backends[self.cache[key]](*args, **kwargs)

    # ------------------------------------------------------------------ selection
    def _bench_and_cache(self, key: tuple, args: tuple, kwargs: dict) -> None:
        if self._disk and self._load_from_disk(key) is not None:
            return
        results: Dict[str, float] = {}
        for name, impl in self._backends.items():
            try:
                results[name] = do_bench(lambda: impl(*args, **kwargs), warmup=self._warmup,
                                         rep=self._rep)
            except Exception as exc:  # a failing backend is skipped, not fatal
                log.debug("[%s] backend '%s' skipped: %s", self.__name__, name, exc)
        if not results:
            raise RuntimeError(f"[{self.__name__}] All backends failed.")
        winner = min(results, key=results.get)
        log.info("[%s] %s", self.__name__,
                 "  ".join(f"{n}={ms:.3f}ms" for n, ms in results.items()))
        self.cache[key] = winner
        self.timings[key] = results
        if self._disk:
            self._save_to_disk(key, results, winner)

    # ------------------------------------------------------------------ persistence
    def _cache_path(self, key: tuple) -> Path:
        return cache_dir() / _disk_key(self.__name__, list(self._backends), key) / _CACHE_FILE

    def _load_from_disk(self, key: tuple) -> Optional[str]:
        try:
            path = self._cache_path(key)
            if not path.is_file():
                return None
            data = json.loads(path.read_text())
            winner = data["winner"]
            if winner not in self._backends:
                return None
            self.cache[key] = winner
            self.timings[key] = data["timings"]
            return winner
        except Exception as exc:
            log.debug("[%s] disk miss: %s", self.__name__, exc)
            return None

    def _save_to_disk(self, key: tuple, results: Dict[str, float], winner: str) -> None:
        try:
            path = self._cache_path(key)
            path.parent.mkdir(parents=True, exist_ok=True)
            payload = json.dumps({"op": self.__name__, "key": list(key), "winner": winner,
                                  "timings": results})
            fd, tmp = tempfile.mkstemp(dir=path.parent, suffix=".tmp")
            with os.fdopen(fd, "w") as f:
                f.write(payload)
            os.replace(tmp, path)  # atomic: readers never see a partial file
        except Exception as exc:
            log.warning("[%s] disk write failed: %s", self.__name__, exc)

    # ------------------------------------------------------------------ control
    @contextmanager
    def force_backend(self, name: str):
        if name not in self._backends:
            raise KeyError(f"Backend '{name}' not registered in '{self.__name__}'.")
        self._forced = name
        try:
            yield
        finally:
            self._forced = None

    def clear_cache(self) -> None:
        """Forgets the in-memory choices (files on disk are kept)."""
        self.cache.clear()
        self.timings.clear()

    def best_config(self) -> Dict[tuple, str]:
        return dict(self.cache)


def dynamic_dispatch(backends: Optional[Dict[str, Callable]] = None,
                     key: Optional[List[str]] = None, warmup: float = 25, rep: float = 100,
                     use_disk_cache: bool = True):
    """``dynamic_dispatch({"name": impl, ...}, key=[...])`` builds a dispatcher whose signature
    and name come from the first implementation; ``@dynamic_dispatch(key=[...])`` decorates a
    function that then gets backends through ``.register``."""

    def build(fn: Callable) -> DynamicDispatcher:
        return DynamicDispatcher(fn, key=key or [],
                                 arg_names=list(inspect.signature(fn).parameters),
                                 warmup=warmup, rep=rep, use_disk_cache=use_disk_cache)

    if backends is None:
        return build
    dispatcher = build(next(iter(backends.values())))
    for name, impl in backends.items():
        dispatcher.register(name, impl)
    return dispatcher
