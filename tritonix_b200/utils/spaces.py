"""Value types of a tuning search space.

Same surface as the reference's tritonix/utils/spaces.py:6-86: ``Choice`` (explicit list),
``Range`` (integers lo..hi inclusive with a step), ``PowerOfTwo`` (lo, 2lo, 4lo, ... <= hi) and
``SpaceConfig`` (an ordered dict of those, addressed by index tuples).  The reference's README
and docs call the last one ``ConfigSpace`` (README.md:69-70); both names are exported.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Sequence, Union


class _Axis:
    """Indexing and length for every axis type, in terms of ``values()``."""

    def values(self) -> list:  # pragma: no cover - overridden
        raise NotImplementedError

    def __len__(self) -> int:
        return len(self.values())

    def __getitem__(self, idx: int) -> Any:
        return self.values()[idx]

    def __iter__(self):
        return iter(self.values())


@dataclass
class Choice(_Axis):
    """An explicit list of allowed values, kept in the order given."""

    options: list = field(default_factory=list)

    def __post_init__(self):
        self.options = list(self.options)

    def values(self) -> list:
        return list(self.options)


@dataclass
class Range(_Axis):
    """Integers lo, lo+step, ... up to and including hi (tritonix/utils/spaces.py:26-41)."""

    lo: int
    hi: int
    step: int = 1

    def values(self) -> list[int]:
        return list(range(self.lo, self.hi + 1, self.step))

    def __len__(self) -> int:
        return len(range(self.lo, self.hi + 1, self.step))

    def __getitem__(self, idx: int) -> int:
        # arithmetic, like the reference (no bounds check, negative idx extrapolates)
        return self.lo + idx * self.step


@dataclass
class PowerOfTwo(_Axis):
    """lo, 2*lo, 4*lo, ... not exceeding hi; PowerOfTwo(32, 256) -> [32, 64, 128, 256]."""

    lo: int
    hi: int

    def values(self) -> list[int]:
        out = []
        v = self.lo
        while v <= self.hi:
            out.append(v)
            v <<= 1
        return out


ConfigParam = Union[PowerOfTwo, Range, Choice]


@dataclass
class SpaceConfig:
    """A named, ordered product of axes.  ``shape`` is the tuple of axis lengths; indexing with a
    tuple of per-axis indices returns the list of values at that grid point."""

    params: dict[str, ConfigParam]

    def __post_init__(self):
        empty = [name for name, axis in self.params.items() if len(axis) == 0]
        if empty:
            raise ValueError(f"Param '{empty[0]}' has no values.")

    @property
    def shape(self) -> tuple[int, ...]:
        return tuple(len(axis) for axis in self.params.values())

    @property
    def names(self) -> list[str]:
        return list(self.params)

    def __getitem__(self, idx_tuple: Sequence[int]) -> list:
        if len(idx_tuple) != len(self.params):
            raise AssertionError(
                f"expected {len(self.params)} indices, got {len(idx_tuple)}")
        return [axis[i] for axis, i in zip(self.params.values(), idx_tuple)]

    def __len__(self) -> int:
        return math.prod(self.shape)


ConfigSpace = SpaceConfig
