"""Search-space pruners used by the tuner.

``MonotonicCascadeTrie`` tracks configurations that ran out of resources in a space where
resource use is monotone in every coordinate: once index tuple f fails, every tuple that is
>= f element-wise is known to fail too.  Behaviour follows the reference's
tritonix/utils/pruners.py:15-169 (same constructor, ``shape``, ``_minimal_failures``,
``is_pruned``, ``prune``, ``_is_prefix_doomed`` and the four generators).  With the CUDA
backend "out of resources" means the shared-memory or TMEM budget of an SM is exceeded.

``CoordinateUnimodalFunction`` prunes by assuming the measured time is unimodal along every
axis when the other coordinates are fixed (tritonix/utils/pruners.py:172-225).  The reference's
tuner imports it under the name ``CoordinateMonotonicFunction`` (tritonix/autotune.py:8-11),
so both names are exported.
"""
from __future__ import annotations

import random
from typing import Callable, Dict, Iterator, List, Optional, Sequence, Tuple

from tritonix_b200.utils.spaces import SpaceConfig

Index = Tuple[int, ...]


def _compare_failure_config(failure: Index, candidate: Index) -> bool:
    """True when ``candidate`` needs at least as much as ``failure`` in every coordinate."""
    return all(c >= f for f, c in zip(failure, candidate))


def _compare_failure_dim(failure: int, candidate: int, rank: int = 0) -> bool:
    return candidate >= failure


class _Node:
    """One level of the failure prefix tree: children keyed by the failure's index at this depth."""

    __slots__ = ("children", "terminal")

    def __init__(self):
        self.children: Dict[int, "_Node"] = {}
        self.terminal = False


def _centre_out(n: int) -> Iterator[int]:
    """n//2, then alternately one step down and one step up until 0..n-1 is exhausted."""
    mid = n // 2
    yield mid
    for step in range(1, n + 1):
        lo, hi = mid - step, mid + step
        if lo >= 0:
            yield lo
        if hi < n:
            yield hi


class MonotonicCascadeTrie:
    """Minimal set of failed index tuples, stored as a prefix tree for dominance queries."""

    def __init__(self, space: SpaceConfig,
                 config_comparison_func: Callable[[Index, Index], bool] = _compare_failure_config,
                 dimension_comparison_func: Callable[[int, int, int], bool] = _compare_failure_dim):
        self.shape: Tuple[int, ...] = tuple(space.shape)
        self.dimensions = len(self.shape)
        self._minimal_failures: List[Index] = []
        self._config_compare = config_comparison_func
        self._dim_compare = dimension_comparison_func
        self._root = _Node()

    # ------------------------------------------------------------------ queries
    def is_pruned(self, config_idx: Sequence[int]) -> bool:
        """True iff some recorded failure is dominated element-wise by ``config_idx``."""
        if len(config_idx) != self.dimensions:
            raise ValueError(
                f"is_pruned expects a full-length config of length {self.dimensions}")
        return self._dominated(tuple(config_idx), 0, self._root)

    def _dominated(self, idx: Index, depth: int, node: _Node) -> bool:
        if node.terminal:
            return True
        if depth == self.dimensions:
            return False
        here = idx[depth]
        for fail_idx, child in node.children.items():
            if self._dim_compare(fail_idx, here, depth) and self._dominated(idx, depth + 1, child):
                return True
        return False

    def _is_prefix_doomed(self, prefix: Sequence[int]) -> bool:
        """A prefix is a dead end when even its cheapest completion (zeros) is pruned."""
        prefix = tuple(prefix)
        if not prefix:
            return False
        return self.is_pruned(prefix + (0,) * (self.dimensions - len(prefix)))

    # ------------------------------------------------------------------ updates
    def prune(self, failed_config: Sequence[int]) -> None:
        failed = tuple(failed_config)
        if self.is_pruned(failed):
            return  # already implied by an earlier failure
        # keep the set minimal: drop failures that the new one makes redundant
        self._minimal_failures = [f for f in self._minimal_failures
                                  if not self._config_compare(failed, f)]
        self._minimal_failures.append(failed)
        self._root = _Node()
        for f in self._minimal_failures:
            node = self._root
            for i in f:
                node = node.children.setdefault(i, _Node())
            node.terminal = True

    # ------------------------------------------------------------------ generators
    def _first(self, prefix: Index, order: Callable[[int], Sequence[int]]) -> Optional[Index]:
        if self._is_prefix_doomed(prefix):
            return None
        depth = len(prefix)
        if depth == self.dimensions:
            return prefix
        for i in order(self.shape[depth]):
            found = self._first(prefix + (i,), order)
            if found is not None:
                return found
        return None

    def get_random_unpruned(self) -> Optional[Index]:
        def shuffled(n):
            idx = list(range(n))
            random.shuffle(idx)
            return idx
        return self._first((), shuffled)

    def get_mid_point_unpruned(self) -> Optional[Index]:
        return self._first((), lambda n: list(_centre_out(n)))

    def _walk(self, prefix: Index, order: Callable[[int], Sequence[int]]) -> Iterator[Index]:
        # The doom test runs when a prefix is reached, so prune() calls made while the
        # generator is suspended take effect for everything not yet visited.
        if self._is_prefix_doomed(prefix):
            return
        depth = len(prefix)
        if depth == self.dimensions:
            yield prefix
            return
        for i in order(self.shape[depth]):
            yield from self._walk(prefix + (i,), order)

    def generate_all_unpruned(self) -> Iterator[Index]:
        """Every unpruned index tuple in lexicographic order."""
        yield from self._walk((), range)

    def generate_all_unpruned_midpoint(self) -> Iterator[Index]:
        """Every unpruned tuple, each axis visited from its middle outwards (mid, mid-1, mid+1, ...)."""
        yield from self._walk((), _centre_out)


class CoordinateUnimodalFunction:
    """Per-axis [lo, hi] windows derived from observed values under a unimodality assumption.

    For axis d and a fixed setting of the other axes (a "line"), once two or more points are
    measured the best one is located; the nearest worse point on its right caps the window
    just before it, the nearest worse point on its left raises the floor just after it.  A
    configuration is pruned when it falls outside the window of any line it lies on.
    """

    def __init__(self, space: SpaceConfig):
        self.dim_sizes = list(space.shape)
        self.n_dims = len(self.dim_sizes)
        self._obs: List[Dict[Index, Dict[int, float]]] = [{} for _ in range(self.n_dims)]
        self._ranges: List[Dict[Index, Tuple[int, int]]] = [{} for _ in range(self.n_dims)]

    @staticmethod
    def _line(idx: Index, d: int) -> Index:
        return idx[:d] + idx[d + 1:]

    def record(self, config_idx: Sequence[int], value: float) -> None:
        idx = tuple(config_idx)
        for d in range(self.n_dims):
            line = self._line(idx, d)
            seen = self._obs[d].setdefault(line, {})
            seen[idx[d]] = value
            if len(seen) < 2:
                continue
            best = min(seen, key=seen.get)
            floor, cap = 0, self.dim_sizes[d] - 1
            right = sorted(i for i in seen if i > best)
            left = sorted((i for i in seen if i < best), reverse=True)
            worse_right = next((i for i in right if seen[i] > seen[best]), None)
            worse_left = next((i for i in left if seen[i] > seen[best]), None)
            if worse_right is not None:
                cap = worse_right - 1
            if worse_left is not None:
                floor = worse_left + 1
            if floor > 0 or cap < self.dim_sizes[d] - 1:
                self._ranges[d][line] = (floor, cap)

    def is_pruned(self, config_idx: Sequence[int]) -> bool:
        idx = tuple(config_idx)
        for d in range(self.n_dims):
            window = self._ranges[d].get(self._line(idx, d))
            if window is not None and not (window[0] <= idx[d] <= window[1]):
                return True
        return False


CoordinateMonotonicFunction = CoordinateUnimodalFunction
