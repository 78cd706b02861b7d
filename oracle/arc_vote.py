"""Plain-Python restatement of AAIVR voting (src/voting.py:16-213). Test infrastructure."""
import random
from collections import Counter

from .arc_tokens import INVERSE_DIHEDRAL, dihedral


def invert_dihedral(grid, idx):  # src/voting.py:19-31
    return dihedral(grid, INVERSE_DIHEDRAL[idx])


def invert_color_permutation(grid, perm):  # src/voting.py:34-54
    inv = [0] * 10
    for old, new in enumerate(perm):
        inv[new] = old
    return [[inv[c] for c in row] for row in grid]


def is_valid(grid, test_input=None, discard_input_copies=True):  # src/voting.py:67-95
    if not grid or not grid[0]:
        return False
    if any(len(r) != len(grid[0]) for r in grid):
        return False
    if discard_input_copies and test_input is not None and grid == test_input:
        return False
    return True


def aggregate_votes(predictions, test_input=None, discard_input_copies=True, rng=None):  # :110-165
    counter = Counter()
    for grid, d_idx, perm in predictions:
        if grid is None or not is_valid(grid, test_input, discard_input_copies):
            continue
        canon = invert_dihedral(grid, d_idx)
        if perm is not None:
            canon = invert_color_permutation(canon, perm)
        counter[tuple(tuple(r) for r in canon)] += 1
    if not counter:
        return []
    rng = rng or random.Random()
    items = list(counter.items())
    tie = {g: rng.random() for g, _ in items}
    items.sort(key=lambda it: (-it[1], tie[it[0]]))
    return [([list(r) for r in g], c) for g, c in items]


def aaivr_predict(predictions, top_k=2, test_input=None, discard_input_copies=True, rng=None):  # :185-213
    return [g for g, _ in aggregate_votes(predictions, test_input, discard_input_copies, rng)[:top_k]]
