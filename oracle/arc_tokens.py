"""Plain-Python restatement of the reference's token / position / augmentation rules.

Test infrastructure (see oracle/__init__.py).  Each function names the reference lines it follows.
"""
import numpy as np

START, NEWLINE, IO_SEP, END = 10, 11, 12, 13


def grid_to_tokens(grid):  # src/data.py:40-51
    out = []
    for row in grid:
        out.extend(row)
        out.append(NEWLINE)
    return out


def tokens_to_grid(tokens):  # src/data.py:54-72
    grid, row = [], []
    for t in tokens:
        if t == NEWLINE:
            if row:
                grid.append(row)
                row = []
        elif t in (START, IO_SEP, END):
            continue
        else:
            row.append(t)
    if row:
        grid.append(row)
    return grid


def encode_example(inp, out=None):  # src/data.py:75-93
    toks = [START] + grid_to_tokens(inp) + [IO_SEP]
    if out is not None:
        toks += grid_to_tokens(out) + [END]
    return toks


def decode_output_grid(tokens):  # src/data.py:96-117
    if IO_SEP not in tokens:
        return None
    body = []
    for t in tokens[tokens.index(IO_SEP) + 1:]:
        if t == END:
            break
        body.append(t)
    return tokens_to_grid(body) if body else None


def positions_3d(tokens, max_x=30, max_y=29):  # src/data.py:124-175
    pos = np.zeros((len(tokens), 3), dtype=np.int64)
    x = y = 0
    in_out = False
    for i, t in enumerate(tokens):
        if t == START:
            pos[i] = (0, 0, 0)
            x = y = 0
            in_out = False
        elif t == NEWLINE:
            pos[i] = (0, y, 3 if in_out else 1)
            x = 0
            y = min(y + 1, max_y)
        elif t == IO_SEP:
            pos[i] = (0, 0, 2)
            x = y = 0
            in_out = True
        elif t == END:
            pos[i] = (0, 0, 4)
        else:
            pos[i] = (min(x, max_x), min(y, max_y), 3 if in_out else 1)
            x += 1
    return pos


def dihedral(grid, idx):  # src/data.py:182-233, same index order
    g = [list(r) for r in grid]
    if idx == 0:
        return g
    if idx == 1:
        return [list(r) for r in zip(*g[::-1])]
    if idx == 2:
        return [r[::-1] for r in g[::-1]]
    if idx == 3:
        return [list(r) for r in zip(*g)][::-1]
    if idx == 4:
        return [r[::-1] for r in g]
    if idx == 5:
        return g[::-1]
    if idx == 6:
        return [list(r) for r in zip(*g)]
    if idx == 7:
        t = [list(r) for r in zip(*g)]
        return [r[::-1] for r in t[::-1]]
    raise ValueError(idx)


INVERSE_DIHEDRAL = [0, 3, 2, 1, 4, 5, 6, 7]  # src/voting.py:16


def color_permutations(n, seed=42):  # src/data.py:257-278
    rng = np.random.default_rng(seed)
    perms = np.zeros((n, 10), dtype=np.int64)
    perms[0, 1:] = np.arange(1, 10)
    for i in range(1, n):
        perms[i, 1:] = rng.permutation(np.arange(1, 10))
    return perms


class GridState:
    """Scalar restatement of GridStateUpdater (src/inference.py:104-168) for one sequence."""

    def __init__(self, x=0, y=0, in_output=True, max_x=30, max_y=29):
        self.x, self.y, self.in_output = x, y, in_output
        self.max_x, self.max_y = max_x, max_y

    def update(self, tok):
        z = 3 if self.in_output else 1
        if tok == START:
            z = 0
        if tok == IO_SEP:
            z = 2
        if tok == END:
            z = 4
        xc = min(max(self.x, 0), self.max_x)
        yc = min(max(self.y, 0), self.max_y)
        px = 0 if tok in (START, IO_SEP, END, NEWLINE) else xc
        py = 0 if tok in (START, IO_SEP, END) else yc
        if tok in (START, IO_SEP):
            self.x = self.y = 0
        if tok == START:
            self.in_output = False
        if tok == IO_SEP:
            self.in_output = True
        if tok == NEWLINE:
            self.x = 0
            self.y = min(self.y + 1, self.max_y)
        if tok < 10:
            self.x = min(self.x + 1, self.max_x)
        self.x = min(max(self.x, 0), self.max_x)
        self.y = min(max(self.y, 0), self.max_y)
        return (px, py, z)


def initial_state(last_tok, last_pos, has_tokens, max_x=30, max_y=29):
    """_derive_initial_state_from_prompt (src/inference.py:171-221) for one sequence."""
    if not has_tokens:
        return 0, 0, True
    x, y, z = (int(v) for v in last_pos)
    in_out = z >= 3
    if last_tok == START:
        in_out = False
    if last_tok == IO_SEP:
        in_out = True
    if last_tok in (START, IO_SEP):
        x = y = 0
    if last_tok == NEWLINE:
        x = 0
        y = min(y + 1, max_y)
    if last_tok < 10:
        x = min(x + 1, max_x)
    return min(max(x, 0), max_x), min(max(y, 0), max_y), in_out
