"""Shape-keyed backend dispatcher.

Public contract of the reference's tritonix/dispatcher.py:38-175: implementations are registered
under names; the first call for a new tuning key times every implementation; the fastest is
remembered in ``.cache`` (all timings in ``.timings``) and, optionally, in a small JSON file.
``force_backend`` pins one implementation, ``clear_cache`` forgets the in-memory choices.  In
this package the contraction ops register a single implementation, ``"cuda"``; the class itself
stays general.

On disk a choice is ``<cache dir>/<sha256("op-[sorted names]-key")>/backend_dispatch.json`` with
the payload ``{"op", "key", "winner", "timings"}`` — the file name, hash input and payload of
the reference (dispatcher.py:33-35, 100, 120-128), so that caches are interchangeable.  The
cache directory is ``$TRITONIX_B200_CACHE_DIR`` or ``~/.cache/tritonix_b200`` (the reference
borrows Triton's cache manager, which this package does not depend on).
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
from typing import Callable, Dict, Iterable, List, Optional

import torch

from tritonix_b200.testing import do_bench

log = logging.getLogger("tritonix.dispatcher")

_CHOICE_FILE = "backend_dispatch.json"
_MEMO_LIMIT = 4096


def cache_dir() -> Path:
    root = os.environ.get("TRITONIX_B200_CACHE_DIR")
    return Path(root) if root else Path.home() / ".cache" / "tritonix_b200"


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


class _ChoiceFiles:
    """One JSON file per (op, implementation names, tuning key).  Reads never raise: anything
    unreadable is a miss.  Writes go through a temporary file and ``os.replace`` so that a
    concurrent reader never sees half a file; a failed write is reported and otherwise ignored."""

    def __init__(self, op_name: str):
        self.op_name = op_name

    def _path(self, names: Iterable[str], key: tuple) -> Path:
        return cache_dir() / _disk_key(self.op_name, list(names), key) / _CHOICE_FILE

    def read(self, names: Iterable[str], key: tuple) -> Optional[dict]:
        names = list(names)
        try:
            path = self._path(names, key)
            if not path.is_file():
                return None
            record = json.loads(path.read_text())
            if record["winner"] not in names or not isinstance(record["timings"], dict):
                return None
            return record
        except Exception as exc:
            log.debug("%s: stored choice for %s unusable (%s)", self.op_name, key, exc)
            return None

    def write(self, names: Iterable[str], key: tuple, winner: str, timings: Dict[str, float]) -> None:
        try:
            path = self._path(names, key)
            path.parent.mkdir(parents=True, exist_ok=True)
            text = json.dumps({"op": self.op_name, "key": list(key), "winner": winner,
                               "timings": timings})
            handle, scratch = tempfile.mkstemp(dir=path.parent, suffix=".tmp")
            with os.fdopen(handle, "w") as out:
                out.write(text)
            os.replace(scratch, path)
        except Exception as exc:
            log.warning("%s: disk write failed, the choice for %s stays in memory only (%s)",
                        self.op_name, key, exc)


class DynamicDispatcher:
    def __init__(self, fn: Callable, key: List[str], arg_names: List[str], warmup: float = 25,
                 rep: float = 100, use_disk_cache: bool = True):
        self.__name__ = getattr(fn, "__name__", type(fn).__name__)
        self.__doc__ = fn.__doc__
        self.__wrapped__ = fn
        self.cache: Dict[tuple, str] = {}
        self.timings: Dict[tuple, Dict[str, float]] = {}
        self._impls: Dict[str, Callable] = {}
        self._pinned: Optional[str] = None
        self._key_fields = list(key)
        self._params = list(arg_names)
        self._budget = {"warmup": warmup, "rep": rep}
        self._files = _ChoiceFiles(self.__name__) if use_disk_cache else None
        self._memo: Dict[tuple, tuple] = {}

    # ------------------------------------------------------------------ registration
    @property
    def backends(self) -> List[str]:
        """Names of the registered implementations, in registration order."""
        return list(self._impls)

    @property
    def forced(self) -> Optional[str]:
        """The implementation pinned by an active ``force_backend`` block, else None."""
        return self._pinned

    def register(self, name: str, impl: Callable) -> "DynamicDispatcher":
        self._impls[name] = impl
        return self

    # ------------------------------------------------------------------ calls
    def __call__(self, *args, **kwargs):
        if self._pinned is not None:
            return self._impls[self._pinned](*args, **kwargs)
        if not self._impls:
            raise RuntimeError(f"{self.__name__}: no backends registered, nothing to dispatch to")
        key = self._key_of(args, kwargs)
        name = self.cache.get(key)
        if name is None:
            name = self._choose(key, args, kwargs)
        return self._impls[name](*args, **kwargs)

    def _key_of(self, args: tuple, kwargs: dict) -> tuple:
        # A positional call's key depends only on tensor shapes/dtypes and the plain values:
        # remember it under that cheaper signature.
        probe = None
        if not kwargs:
            try:
                probe = tuple((a.shape, a.dtype) if isinstance(a, torch.Tensor) else a for a in args)
                hit = self._memo.get(probe)
                if hit is not None:
                    return hit
            except TypeError:  # an unhashable argument
                probe = None
        key = _tuning_key(self._key_fields, args, kwargs, self._params)
        if probe is not None:
            if len(self._memo) >= _MEMO_LIMIT:
                self._memo.clear()
            self._memo[probe] = key
        return key

    def _choose(self, key: tuple, args: tuple, kwargs: dict) -> str:
        """Stored choice if there is one, else time every implementation and keep the fastest."""
        stored = self._files.read(self._impls, key) if self._files else None
        if stored is not None:
            self.cache[key], self.timings[key] = stored["winner"], stored["timings"]
            return stored["winner"]
        measured: Dict[str, float] = {}
        for name, impl in self._impls.items():
            try:
                measured[name] = do_bench(lambda: impl(*args, **kwargs), **self._budget)
            except Exception as exc:  # one failing implementation does not end the selection
                log.debug("%s: backend %r skipped for %s: %s", self.__name__, name, key, exc)
        if not measured:
            raise RuntimeError(f"{self.__name__}: all backends failed for key {key}")
        best = min(measured, key=measured.get)
        log.info("%s %s -> %s  (%s)", self.__name__, key, best,
                 ", ".join(f"{n} {ms:.3f} ms" for n, ms in measured.items()))
        self.cache[key], self.timings[key] = best, measured
        if self._files:
            self._files.write(self._impls, key, best, measured)
        return best

    # ------------------------------------------------------------------ control
    @contextmanager
    def force_backend(self, name: str):
        """Every call inside the block goes to ``name`` without timing or caching anything.
        Not re-entrant and not thread-safe, like the reference's (dispatcher.py:130-138)."""
        if name not in self._impls:
            raise KeyError(f"{self.__name__} has no backend {name!r}; registered: {self.backends}")
        self._pinned = name
        try:
            yield
        finally:
            self._pinned = None

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
    function that then gets implementations through ``.register``."""

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
