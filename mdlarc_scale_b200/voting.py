"""AAIVR vote aggregation (host side; integer-only, bit-exact with ``src/voting.py``).

Candidates are ``(grid | None, dihedral_idx, colour_perm | None)`` tuples in generation order.
Each valid candidate is mapped back to the task's own orientation and colours, identical
canonical grids are tallied, and the tally is ordered by votes (descending) with ties broken
by one ``rng.random()`` draw per distinct grid, drawn in first-seen order
(``src/voting.py:110-165``).  The draw order is part of the result, so candidates must be
presented in the reference's order (dihedral-major, then permutation, then sample).
"""
from __future__ import annotations

import random

from .data import DIHEDRAL_TRANSFORMS, INVERSE_DIHEDRAL

Grid = list
Prediction = tuple  # (Grid | None, int, tuple[int, ...] | None)


def invert_dihedral(grid: Grid, dihedral_idx: int) -> Grid:
    return DIHEDRAL_TRANSFORMS[INVERSE_DIHEDRAL[dihedral_idx]](grid)


def invert_color_permutation(grid: Grid, perm) -> Grid:
    back = [0] * 10
    for old, new in enumerate(perm):
        back[new] = old
    return [[back[c] for c in row] for row in grid]


def grid_to_tuple(grid: Grid) -> tuple:
    return tuple(tuple(r) for r in grid)


def tuple_to_grid(t: tuple) -> Grid:
    return [list(r) for r in t]


def is_rectangular_grid(grid: Grid) -> bool:
    if not grid or not grid[0]:
        return False
    w = len(grid[0])
    return all(len(r) == w for r in grid)


def _is_valid_grid(grid: Grid, test_input: Grid | None = None, discard_input_copies: bool = True) -> bool:
    if not is_rectangular_grid(grid):
        return False
    return not (discard_input_copies and test_input is not None and grid == test_input)


def _canonicalize_prediction(pred_grid: Grid, dihedral_idx: int, color_perm) -> Grid:
    g = invert_dihedral(pred_grid, dihedral_idx)
    return g if color_perm is None else invert_color_permutation(g, color_perm)


def aggregate_votes(predictions, test_input: Grid | None = None, discard_input_copies: bool = True,
                    rng: random.Random | None = None) -> list[tuple[Grid, int]]:
    tally: dict[tuple, int] = {}  # insertion-ordered: first-seen order of canonical grids
    for grid, dihedral_idx, perm in predictions:
        if grid is None or not _is_valid_grid(grid, test_input, discard_input_copies):
            continue
        key = grid_to_tuple(_canonicalize_prediction(grid, dihedral_idx, perm))
        tally[key] = tally.get(key, 0) + 1
    if not tally:
        return []
    if rng is None:
        rng = random.Random()
    ranked = [(-votes, rng.random(), key) for key, votes in tally.items()]
    ranked.sort(key=lambda r: (r[0], r[1]))
    return [(tuple_to_grid(key), -neg) for neg, _, key in ranked]


def select_top_k(votes, k: int = 2) -> list[Grid]:
    return [g for g, _ in votes[:k]]


def aaivr_predict(predictions, top_k: int = 2, test_input: Grid | None = None,
                  discard_input_copies: bool = True, rng: random.Random | None = None) -> list[Grid]:
    return select_top_k(
        aggregate_votes(predictions, test_input=test_input,
                        discard_input_copies=discard_input_copies, rng=rng), k=top_k)


def compute_voting_stats(predictions, test_input: Grid | None = None,
                         discard_input_copies: bool = True) -> dict:
    votes = aggregate_votes(predictions, test_input=test_input,
                            discard_input_copies=discard_input_copies, rng=random.Random(0))
    n_valid = sum(1 for g, _, _ in predictions
                  if g is not None and _is_valid_grid(g, test_input, discard_input_copies))
    counts = [c for _, c in votes]
    top = counts[0] if counts else 0
    return {
        "total_predictions": len(predictions),
        "valid_predictions": n_valid,
        "invalid_predictions": len(predictions) - n_valid,
        "unique_grids": len(votes),
        "top_vote_count": top,
        "vote_distribution": counts[:10],
        "confidence": (top / n_valid) if (votes and n_valid > 0) else 0.0,
    }
