"""Token codec, 3D positions and augmentation primitives (host side of the hot path).

Same vocabulary and rules as the reference's ``src/data.py:26-305``: 14 tokens
(colours 0-9, START 10, NEWLINE 11, IO_SEP 12, END 13), row-major grids with a NEWLINE
after every row, 3D positions (x column, y row, z layer), the 8 dihedral transforms in
the reference's order and its seeded colour permutations.
"""
from __future__ import annotations

import numpy as np

VOCAB_SIZE = 14
START_TOKEN_ID = 10
NEWLINE_TOKEN_ID = 11
IO_SEP_TOKEN_ID = 12
END_TOKEN_ID = 13
PAD_TOKEN_ID = END_TOKEN_ID

MAX_X = 30  # largest x position the grid-state rules produce (src/data.py:126)
MAX_Y = 29  # largest y position (src/data.py:127)

Grid = list  # list[list[int]]


# ---------------------------------------------------------------------------
# token codec (src/data.py:40-117)
# ---------------------------------------------------------------------------
def grid_to_tokens(grid: Grid) -> list[int]:
    out: list[int] = []
    for row in grid:
        out += list(row)
        out.append(NEWLINE_TOKEN_ID)
    return out


def tokens_to_grid(tokens) -> Grid:
    rows: Grid = []
    cur: list[int] = []
    for t in tokens:
        t = int(t)
        if t == NEWLINE_TOKEN_ID:
            if cur:
                rows.append(cur)
                cur = []
        elif t < 10:
            cur.append(t)
        # START / IO_SEP / END inside an output are dropped
    if cur:
        rows.append(cur)
    return rows


def encode_example(input_grid: Grid, output_grid: Grid | None = None) -> list[int]:
    toks = [START_TOKEN_ID] + grid_to_tokens(input_grid) + [IO_SEP_TOKEN_ID]
    if output_grid is not None:
        toks += grid_to_tokens(output_grid) + [END_TOKEN_ID]
    return toks


def decode_output_grid(tokens) -> Grid | None:
    """Grid between the first IO_SEP of ``tokens`` and the next END; None if absent/empty."""
    toks = [int(t) for t in tokens]
    if IO_SEP_TOKEN_ID not in toks:
        return None
    start = toks.index(IO_SEP_TOKEN_ID) + 1
    stop = len(toks)
    for i in range(start, len(toks)):
        if toks[i] == END_TOKEN_ID:
            stop = i
            break
    body = toks[start:stop]
    if not body:
        return None
    return tokens_to_grid(body)


# ---------------------------------------------------------------------------
# 3D positions (src/data.py:124-175)
# ---------------------------------------------------------------------------
def compute_positions_3d(tokens, max_x: int = MAX_X, max_y: int = MAX_Y) -> np.ndarray:
    n = len(tokens)
    pos = np.zeros((n, 3), dtype=np.int64)
    x = y = 0
    in_output = False
    for i in range(n):
        t = int(tokens[i])
        if t == START_TOKEN_ID:
            x = y = 0
            in_output = False  # position stays (0, 0, 0)
        elif t == NEWLINE_TOKEN_ID:
            pos[i, 1] = y
            pos[i, 2] = 3 if in_output else 1
            x = 0
            y = min(y + 1, max_y)
        elif t == IO_SEP_TOKEN_ID:
            pos[i, 2] = 2
            x = y = 0
            in_output = True
        elif t == END_TOKEN_ID:
            pos[i, 2] = 4
        else:
            pos[i, 0] = min(x, max_x)
            pos[i, 1] = min(y, max_y)
            pos[i, 2] = 3 if in_output else 1
            x += 1
    return pos


# ---------------------------------------------------------------------------
# dihedral group (src/data.py:182-233); index order is part of the contract
# ---------------------------------------------------------------------------
def _transposed(grid: Grid) -> Grid:
    """Columns of ``grid`` as rows, truncated to the shortest row (zip semantics)."""
    if not grid:
        return []
    width = min(len(r) for r in grid)
    return [[grid[i][j] for i in range(len(grid))] for j in range(width)]


def identity(grid: Grid) -> Grid:
    return [list(r) for r in grid]


def rot90(grid: Grid) -> Grid:  # clockwise
    return _transposed(grid[::-1])


def rot180(grid: Grid) -> Grid:
    return [list(r)[::-1] for r in grid[::-1]]


def rot270(grid: Grid) -> Grid:
    return _transposed(grid)[::-1]


def flip_h(grid: Grid) -> Grid:
    return [list(r)[::-1] for r in grid]


def flip_v(grid: Grid) -> Grid:
    return [list(r) for r in grid[::-1]]


def flip_diag(grid: Grid) -> Grid:
    return _transposed(grid)


def flip_anti_diag(grid: Grid) -> Grid:
    return [r[::-1] for r in _transposed(grid)[::-1]]


DIHEDRAL_TRANSFORMS = [identity, rot90, rot180, rot270, flip_h, flip_v, flip_diag, flip_anti_diag]
# DIHEDRAL_TRANSFORMS[INVERSE_DIHEDRAL[i]] undoes DIHEDRAL_TRANSFORMS[i] (src/voting.py:16)
INVERSE_DIHEDRAL = [0, 3, 2, 1, 4, 5, 6, 7]
# transforms that swap height and width (src/inference.py:274-282)
TRANSPOSING = frozenset({1, 3, 6, 7})


def apply_dihedral_transform(input_grid: Grid, output_grid: Grid, transform_idx: int):
    f = DIHEDRAL_TRANSFORMS[transform_idx]
    return f(input_grid), f(output_grid)


def inverse_dihedral(grid: Grid, transform_idx: int) -> Grid:
    return DIHEDRAL_TRANSFORMS[INVERSE_DIHEDRAL[transform_idx]](grid)


# ---------------------------------------------------------------------------
# colour permutations (src/data.py:257-305)
# ---------------------------------------------------------------------------
def generate_color_permutations(n_perms: int, seed: int = 42) -> np.ndarray:
    """[n_perms, 10] old->new colour maps; row 0 is the identity, colour 0 is fixed.

    Draws ``default_rng(seed).permutation(arange(1, 10))`` once per further row, which is the
    stream the reference consumes, so the permutations are identical for a given seed.
    """
    rng = np.random.default_rng(seed)
    perms = np.zeros((n_perms, 10), dtype=np.int64)
    if n_perms > 0:
        perms[0] = np.arange(10)
    for i in range(1, n_perms):
        perms[i, 1:] = rng.permutation(np.arange(1, 10))
    return perms


def apply_color_perm_to_tokens(tokens, perm):
    """Token tensor with colours 0-9 mapped through ``perm`` (old -> new) and the special tokens
    left alone (src/data.py:281-298).  Works on torch tensors and numpy arrays."""
    if hasattr(tokens, "clone"):
        out = tokens.clone()
    else:
        out = np.array(tokens, copy=True)
        perm = np.asarray(perm)
    is_colour = tokens < 10
    out[is_colour] = perm[tokens[is_colour]]
    return out


def inverse_color_perm(perm) -> np.ndarray:
    perm = np.asarray(perm)
    inv = np.zeros_like(perm)
    inv[perm] = np.arange(len(perm))
    return inv


def apply_color_perm_grid(grid: Grid, perm) -> Grid:
    lut = [int(v) for v in perm]
    return [[lut[c] for c in row] for row in grid]


# ---------------------------------------------------------------------------
# vectorised serialisation (same tokens and positions as the loops above, for rectangular grids)
# ---------------------------------------------------------------------------
def dihedral_np(grid: np.ndarray, idx: int) -> np.ndarray:
    """DIHEDRAL_TRANSFORMS[idx] on a 2-D array."""
    if idx == 0:
        return grid
    if idx == 1:
        return np.rot90(grid, -1)
    if idx == 2:
        return np.rot90(grid, 2)
    if idx == 3:
        return np.rot90(grid, 1)
    if idx == 4:
        return grid[:, ::-1]
    if idx == 5:
        return grid[::-1]
    if idx == 6:
        return grid.T
    if idx == 7:
        return np.rot90(grid, 2).T
    raise ValueError(idx)


def _grid_tokens_positions(grid: np.ndarray, z: int):
    """Row-major cells with a NEWLINE after every row, and their (x, y, z) positions."""
    h, w = grid.shape
    toks = np.empty((h, w + 1), dtype=np.int64)
    toks[:, :w] = grid
    toks[:, w] = NEWLINE_TOKEN_ID
    pos = np.empty((h, w + 1, 3), dtype=np.int64)
    pos[:, :w, 0] = np.minimum(np.arange(w), MAX_X)[None, :]
    pos[:, w, 0] = 0
    pos[:, :, 1] = np.minimum(np.arange(h), MAX_Y)[:, None]
    pos[:, :, 2] = z
    return toks.reshape(-1), pos.reshape(-1, 3)


def encode_example_np(input_grid: np.ndarray, output_grid: np.ndarray | None = None):
    """encode_example + compute_positions_3d of one pair as arrays (tokens [n], positions [n, 3])."""
    ti, pi = _grid_tokens_positions(input_grid, 1)
    parts_t = [np.array([START_TOKEN_ID]), ti, np.array([IO_SEP_TOKEN_ID])]
    parts_p = [np.zeros((1, 3), np.int64), pi, np.array([[0, 0, 2]])]
    if output_grid is not None:
        to, po = _grid_tokens_positions(output_grid, 3)
        parts_t += [to, np.array([END_TOKEN_ID])]
        parts_p += [po, np.array([[0, 0, 4]])]
    return np.concatenate(parts_t), np.concatenate(parts_p)


def as_rect_array(grid) -> np.ndarray | None:
    """2-D int array of a non-empty rectangular grid, else None."""
    if not grid or not grid[0]:
        return None
    w = len(grid[0])
    if any(len(r) != w for r in grid):
        return None
    return np.asarray(grid, dtype=np.int64)
