"""Oracle case generation — TEST INFRASTRUCTURE.  Restates ``verify/gen_cases.py`` of the
reference: ``TestCase`` (:18-24) and the deterministic edge-size generator
``generate_cases`` (:178-274).

Per symbolic axis (sorted by name) the candidate sizes are {1, 2, 3} ∪ {t−1, t, t+1, 2t+1}
for every tile hint t (caller hints, then ``schedule.tile_m/n/k/vec_width`` that are ints,
default 16) ∪ ``extra_sizes`` ∪ numbers found in ``predicate_clauses`` (±1), ascending,
sizes named by ``counterexample_models`` first.  Cases are the Cartesian product in that
order, cut at ``limit``; with ``needs_mask`` every kept case has a non-divisible axis and
non-divisible sizes come first.  ``seed`` is carried into each case, never consumed.
"""

from __future__ import annotations

import re
from dataclasses import dataclass
from itertools import product
from typing import Any, Dict, List, Optional, Sequence

import numpy as np

__all__ = ["TestCase", "generate_cases", "EDGE_VALUES"]

EDGE_VALUES = [1, 2, 3, 7, 8, 15, 16, 17, 31, 32, 33]


@dataclass
class TestCase:
    shapes: Dict[str, int]
    dtypes: Dict[str, str] = None
    seed: int = 0
    inputs: Optional[Dict[str, np.ndarray]] = None
    __test__ = False  # not a pytest container


def _schedule_tiles(intent) -> List[int]:
    tiles = []
    if intent.schedule:
        for key in ("tile_m", "tile_n", "tile_k", "vec_width"):
            v = getattr(intent.schedule, key)
            if isinstance(v, int):
                tiles.append(v)
    return tiles or [16]


def generate_cases(
    intent,
    constraints: Any = None,
    limit: int = 10,
    seed: int = 0,
    tile_hints: Sequence[int] | None = None,
    axes: Sequence[str] | None = None,
    exclude_axes: Sequence[str] | None = None,
    extra_sizes: Sequence[int] | None = None,
    predicate_clauses: Sequence[str] | None = None,
    counterexample_models: Sequence[Dict[str, int]] | None = None,
) -> List[TestCase]:
    if axes is not None:
        axis_names = list(axes)
    else:
        axis_names = sorted({d.value for t in intent.tensors.values() for d in t.shape if d.kind == "sym"})
    if exclude_axes:
        axis_names = [a for a in axis_names if a not in set(exclude_axes)]
    needs_mask = bool(getattr(constraints, "needs_mask", False)) or bool(predicate_clauses)

    tiles = [int(t) for t in (tile_hints or []) if isinstance(t, (int, float))] + _schedule_tiles(intent)

    first: Dict[str, set] = {}
    for model in counterexample_models or []:
        if not isinstance(model, dict):
            continue
        for ax in axis_names:
            try:
                v = int(model[ax])
            except Exception:
                continue
            if 0 < v <= 2048:
                first.setdefault(ax, set()).update({v, max(1, v - 1), v + 1})

    extra = {int(x) for x in (extra_sizes or []) if isinstance(x, (int, float)) and int(x) > 0}
    for clause in predicate_clauses or []:
        if isinstance(clause, str):
            for tok in re.findall(r"(-?\d+)", clause):
                v = int(tok)
                if 0 < v <= 2048:
                    extra.update({v, max(1, v - 1), v + 1})

    def divisible(v: int) -> bool:
        return all(v % t == 0 for t in tiles if t > 1)

    columns = []
    for ax in axis_names:
        sizes = set(EDGE_VALUES[:3]) | extra
        for t in tiles:
            if t > 0:
                sizes.update((max(1, t - 1), t, t + 1, 2 * t + 1))
        prio = first.get(ax, set())
        order = sorted(sizes, key=lambda v: (0 if v in prio else 1, v))
        if needs_mask:
            order = sorted(order, key=lambda v: (divisible(v), 0 if v in prio else 1, v))
        columns.append(order)

    if not axis_names:
        return [TestCase(shapes={}, dtypes={}, seed=seed)]
    out: List[TestCase] = []
    for combo in product(*columns):
        shapes = dict(zip(axis_names, combo))
        if needs_mask and all(divisible(v) for v in combo):
            continue
        out.append(TestCase(shapes=shapes, dtypes={}, seed=seed))
        if len(out) >= limit:
            break
    return out
