"""Plain-Python restatement of the augmentation fan-out either side of generation: the prompt of
one (dihedral, colour permutation) variant (src/inference.py:794-827) and the candidate a row of
generated tokens stands for once mapped back (src/inference.py:906-915, src/voting.py:67-108),
laid out as the fixed-width record the CUDA path emits.  Test infrastructure.
"""
from .arc_tokens import END, IO_SEP, decode_output_grid, dihedral, encode_example, positions_3d
from .arc_vote import invert_color_permutation, invert_dihedral

RECORD_BYTES = 944
MAX_CELLS = 936


def variant_prompt(task, test_idx, d_idx, perm, use_train_examples=True):
    """(tokens, positions) of one variant; ``perm`` is an old->new colour map or None."""
    def tr(grid):
        g = dihedral(grid, d_idx)
        return g if perm is None else [[int(perm[c]) for c in row] for row in g]
    toks = []
    for pair in (task["train"] if use_train_examples else []):   # src/inference.py:812-823
        toks += encode_example(tr(pair["input"]), tr(pair["output"]))
    toks += encode_example(tr(task["test"][test_idx]["input"]), None)
    return toks, positions_3d(toks)


def candidate_grid(generated):
    """Grid a row of generated tokens decodes to: cut after the first END, read after the last
    IO_SEP of prompt-IO_SEP + generated (src/inference.py:906-915)."""
    gen = [int(t) for t in generated]
    if END in gen:
        gen = gen[: gen.index(END) + 1]
    seq = [IO_SEP] + gen
    last = max(i for i, t in enumerate(seq) if t == IO_SEP)
    return decode_output_grid(seq[last:]), len(gen)


def candidate_record(generated, d_idx, perm, test_input=None) -> bytes:
    """The 944-byte record: status, input_copy, h, w, n_tokens (little-endian u16), cells.
    n_tokens counts the generated tokens up to and including the first END."""
    grid, n_tokens = candidate_grid(generated)
    status, copy, h, w, cells = 0, 0, 0, 0, []
    if grid is not None:
        rect = bool(grid) and bool(grid[0]) and all(len(r) == len(grid[0]) for r in grid)   # src/voting.py:67-72
        status = 1 if rect else 2
        if rect:
            copy = int(test_input is not None and grid == test_input)                       # src/voting.py:92
            canon = invert_dihedral(grid, d_idx)
            if perm is not None:
                canon = invert_color_permutation(canon, perm)
            h, w = len(canon), len(canon[0])
            cells = [c for row in canon for c in row]
    out = bytearray(RECORD_BYTES)
    out[0], out[1] = status, copy
    out[2:4] = h.to_bytes(2, "little")
    out[4:6] = w.to_bytes(2, "little")
    out[6:8] = n_tokens.to_bytes(2, "little")
    out[8: 8 + len(cells)] = bytes(cells)
    return bytes(out)
