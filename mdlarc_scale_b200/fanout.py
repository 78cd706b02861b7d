"""Augmentation fan-out on the device: prompts for every (dihedral x colour permutation x sample)
variant built by a CUDA kernel from one uploaded table of task grids, and generated tokens turned
into canonical candidate records by another, so that the host touches per-variant metadata only.

Host-side counterparts (bit-identical results, used where a task is malformed):
``inference.build_augmented_prompts`` for prompts (src/inference.py:794-827) and
``sharding.candidates_from_tokens`` + ``voting.aaivr_predict`` for the way back
(src/inference.py:906-915, src/voting.py:110-213).
"""
from __future__ import annotations

import ctypes as C
import random
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib
from .data import TRANSPOSING, as_rect_array, generate_color_permutations
from .engine import PrefillPlan

RECORD_BYTES = 944
MAX_CELLS = 936
MAX_TEMPLATE_GRIDS = 64


@dataclass
class VariantTable:
    """Per-variant metadata in canonical order: task, test index, then the reference's candidate
    order (dihedral-major, permutation, sample; src/inference.py:794-827)."""
    task: np.ndarray       # [n] task index
    test_idx: np.ndarray   # [n]
    template: np.ndarray   # [n] prompt template = index of the (task, test input)
    dihedral: np.ndarray   # [n] 0..7
    perm: np.ndarray       # [n] row of the permutation table (0 = identity)
    length: np.ndarray     # [n] prompt tokens

    def __len__(self) -> int:
        return len(self.task)


class TaskTable:
    """Grids of a task list on the device, plus one prompt template per (task, test input).

    Raises ``ValueError`` for a task the kernels cannot represent (a ragged or empty grid, a
    colour outside 0-9, more than 31 train pairs); callers then use the host path for it.
    """

    def __init__(self, tasks: list[dict], device, num_color_perms: int = 8, use_train_examples: bool = True):
        self.device = torch.device(device)
        self.num_color_perms = int(num_color_perms)
        cells, off, hs, ws = [], [], [], []
        n_cells = 0

        def add(grid) -> int:
            nonlocal n_cells
            a = as_rect_array(grid)
            if a is None or a.min() < 0 or a.max() > 9:
                raise ValueError("grid is ragged, empty or has colours outside 0-9")
            cells.append(a.astype(np.uint8).reshape(-1))
            off.append(n_cells)
            hs.append(a.shape[0])
            ws.append(a.shape[1])
            n_cells += a.size
            return len(off) - 1

        tpl_off, tpl_grid, tpl_task, tpl_test, tpl_test_grid = [0], [], [], [], []
        for ti, task in enumerate(tasks):
            train = []
            for pair in (task["train"] if use_train_examples else []):
                train += [add(pair["input"]), add(pair["output"])]
            for test_idx, test in enumerate(task["test"]):
                g = add(test["input"])
                if len(train) + 1 > MAX_TEMPLATE_GRIDS:
                    raise ValueError("too many train pairs for one prompt template")
                tpl_grid += train + [g]
                tpl_off.append(len(tpl_grid))
                tpl_task.append(ti)
                tpl_test.append(test_idx)
                tpl_test_grid.append(g)
        self.grid_h = np.asarray(hs, np.int32)
        self.grid_w = np.asarray(ws, np.int32)
        self.tpl_off = np.asarray(tpl_off, np.int32)
        self.tpl_grid = np.asarray(tpl_grid, np.int32)
        self.tpl_task = np.asarray(tpl_task, np.int32)
        self.tpl_test = np.asarray(tpl_test, np.int32)
        self.tpl_test_grid = np.asarray(tpl_test_grid, np.int32)
        self.perms = generate_color_permutations(self.num_color_perms, seed=42)   # src/inference.py:790

        def up(a, dtype):
            return torch.from_numpy(np.ascontiguousarray(a, dtype=dtype)).to(self.device)
        self.d_cells = up(np.concatenate(cells) if cells else np.zeros(1, np.uint8), np.uint8)
        self.d_grid_off = up(off, np.int32)
        self.d_grid_h = up(self.grid_h, np.int32)
        self.d_grid_w = up(self.grid_w, np.int32)
        self.d_tpl_off = up(self.tpl_off, np.int32)
        self.d_tpl_grid = up(self.tpl_grid, np.int32)
        self.d_perm_lut = up(self.perms, np.uint8)

    # -- host arithmetic on shapes only -------------------------------------------------
    def template_lengths(self) -> np.ndarray:
        """[n_templates, 2] prompt tokens without / with a transposing dihedral transform."""
        out = np.zeros((len(self.tpl_task), 2), np.int64)
        for t in range(len(self.tpl_task)):
            g = self.tpl_grid[self.tpl_off[t]: self.tpl_off[t + 1]]
            h, w = self.grid_h[g].astype(np.int64), self.grid_w[g].astype(np.int64)
            extra = np.where(np.arange(len(g)) % 2 == 1, 1, 2)      # outputs: END; inputs: START + IO_SEP
            out[t, 0] = int((h * (w + 1) + extra).sum())
            out[t, 1] = int((w * (h + 1) + extra).sum())
        return out

    def variants(self, num_samples: int = 1) -> VariantTable:
        lens = self.template_lengths()
        n_tpl = len(self.tpl_task)
        d = np.repeat(np.arange(8), self.num_color_perms * num_samples)
        p = np.tile(np.repeat(np.arange(self.num_color_perms), num_samples), 8)
        per = len(d)
        tpl = np.repeat(np.arange(n_tpl), per)
        dd, pp = np.tile(d, n_tpl), np.tile(p, n_tpl)
        swaps = np.isin(dd, sorted(TRANSPOSING)).astype(np.int64)
        return VariantTable(task=self.tpl_task[tpl], test_idx=self.tpl_test[tpl], template=tpl.astype(np.int32),
                            dihedral=dd.astype(np.int32), perm=pp.astype(np.int32), length=lens[tpl, swaps])

    def perm_tuple(self, p: int):
        return None if p == 0 else tuple(int(v) for v in self.perms[p])

    # -- device work --------------------------------------------------------------------
    def build_prompts(self, vt: VariantTable, idx: np.ndarray, seq_rows: np.ndarray) -> PrefillPlan:
        """One packed prefill call for variants ``idx`` (cache rows ``seq_rows``): token, position
        and cache-placement arrays are written by the kernel; the host sends per-sequence arrays."""
        lib = _lib.load()
        n = len(idx)
        lens = vt.length[idx].astype(np.int64)
        tok_off = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        total = int(tok_off[-1])
        dev = self.device

        def up(a):
            return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev, non_blocking=True)
        d_tpl, d_dih, d_perm = up(vt.template[idx]), up(vt.dihedral[idx]), up(vt.perm[idx])
        d_off, d_rows = up(tok_off), up(seq_rows)
        out = torch.empty((8, max(total, 1)), dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        args = _lib.PromptBuildArgs(
            n_variants=n, n_perms=self.num_color_perms, d_cells=self.d_cells.data_ptr(),
            d_grid_off=self.d_grid_off.data_ptr(), d_grid_h=self.d_grid_h.data_ptr(),
            d_grid_w=self.d_grid_w.data_ptr(), d_tpl_off=self.d_tpl_off.data_ptr(),
            d_tpl_grid=self.d_tpl_grid.data_ptr(), d_perm_lut=self.d_perm_lut.data_ptr(),
            d_var_template=d_tpl.data_ptr(), d_var_dihedral=d_dih.data_ptr(), d_var_perm=d_perm.data_ptr(),
            d_var_tok_off=d_off.data_ptr(), d_var_seq=d_rows.data_ptr(),
            d_token_ids=out[0].data_ptr(), d_pos_xyz=out[1:4].data_ptr(), d_seq=out[4].data_ptr(),
            d_kv_slot=out[5].data_ptr(), d_kv_count=out[6].data_ptr(), d_kv_row=out[7].data_ptr(),
            d_status=status.data_ptr())
        _lib.check(lib.arcb_build_prompts(C.byref(args), torch.cuda.current_stream(dev).cuda_stream))
        # query blocks of at most 256 consecutive rows of one sequence, from the lengths alone
        nblk = (lens + 255) // 256
        blk_seq = np.repeat(np.arange(n), nblk)
        blk_k = np.arange(int(nblk.sum())) - np.repeat(np.cumsum(nblk) - nblk, nblk)
        qb0 = (tok_off[:-1][blk_seq] + 256 * blk_k).astype(np.int32)
        qbn = np.minimum(256, lens[blk_seq] - 256 * blk_k).astype(np.int32)
        qb_kv0 = tok_off[:-1][blk_seq].astype(np.int32)
        # most expensive blocks first (a block's cost grows with the keys its last row sees), so that
        # the attention kernel's last CTAs are its cheapest ones
        order = np.argsort(-(256 * blk_k + qbn), kind="stable")
        qb0, qbn, qb_kv0 = qb0[order], qbn[order], qb_kv0[order]
        zeros = np.zeros(n, np.int32)
        plan = PrefillPlan(
            n_tokens=total, token_ids=out[0, :total], pos_xyz=out[1:4].reshape(-1)[: 3 * total].view(total, 3),
            seq=out[4, :total], kv_slot=out[5, :total], kv_count=out[6, :total],
            n_qblocks=len(qb0), qblock_row0=up(qb0), qblock_rows=up(qbn), qblock_kv0=up(qb_kv0),
            kv_row=out[7, :total], n_kv_rows=total,
            n_first=n, first_row=up(tok_off[1:] - 1), first_seq=d_rows, prompt_len=up(lens),
            # every prompt ends with IO_SEP: next cell is (0, 0) of the output (src/inference.py:171-221)
            grid_x=up(zeros), grid_y=up(zeros), grid_in_output=up(zeros + 1), kv_row_identity=True)
        plan._status = status          # read by check_status after the stream has run
        plan._keep = (d_tpl, d_dih, d_perm, d_off, out)
        return plan

    def canonicalize(self, tokens: torch.Tensor, vt: VariantTable, idx: np.ndarray, records: torch.Tensor) -> None:
        """Write one candidate record per row of ``tokens`` (int32 [n, max_new], variants ``idx``;
        ``idx < 0`` marks padding rows) into ``records`` (uint8 [n, RECORD_BYTES])."""
        lib = _lib.load()
        n, max_new = tokens.shape
        assert records.shape == (n, RECORD_BYTES) and records.dtype == torch.uint8 and records.is_contiguous()
        assert tokens.dtype == torch.int32 and tokens.is_contiguous()
        dev = self.device
        ok = idx >= 0
        safe = np.where(ok, idx, 0)

        def up(a):
            return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev, non_blocking=True)
        d_dih = up(np.where(ok, vt.dihedral[safe], -1))
        d_perm = up(np.where(ok, vt.perm[safe], 0))
        d_test = up(np.where(ok, self.tpl_test_grid[vt.template[safe]], -1))
        args = _lib.CandidateArgs(
            n_rows=n, max_new=max_new, d_tokens=tokens.data_ptr(), d_row_dihedral=d_dih.data_ptr(),
            d_row_perm=d_perm.data_ptr(), d_perm_lut=self.d_perm_lut.data_ptr(), n_perms=self.num_color_perms,
            d_row_test_grid=d_test.data_ptr(), d_cells=self.d_cells.data_ptr(),
            d_grid_off=self.d_grid_off.data_ptr(), d_grid_h=self.d_grid_h.data_ptr(),
            d_grid_w=self.d_grid_w.data_ptr(), d_records=records.data_ptr())
        _lib.check(lib.arcb_canonicalize_candidates(C.byref(args), torch.cuda.current_stream(dev).cuda_stream))
        torch.cuda.current_stream(dev).synchronize()   # the small index tensors above die with this frame


def check_status(plan: PrefillPlan) -> None:
    """Raise if the prompt-building kernel rejected a variant of ``plan`` (synchronises)."""
    st = getattr(plan, "_status", None)
    if st is not None and int(st.item()) != 0:
        raise RuntimeError(f"prompt construction failed on the device (code {int(st.item())})")


# ---------------------------------------------------------------------------
# voting from records (host; integer only)
# ---------------------------------------------------------------------------
def record_fields(records: np.ndarray):
    """(status, input_copy, h, w, n_tokens, cells) views of a uint8 [n, RECORD_BYTES] array."""
    r = np.ascontiguousarray(records)
    head = r[:, :8].copy().view(np.uint16)   # little-endian: [status | copy << 8, h, w, n_tokens]
    return r[:, 0], r[:, 1], head[:, 1], head[:, 2], head[:, 3], r[:, 8:]


def tally_records(records: np.ndarray, vt: VariantTable, discard_input_copies: bool = True) -> dict:
    """Per (task, test_idx): ``(ranked, n_total, n_valid)`` where ``ranked(rng)`` returns the
    ``[(grid, votes), ...]`` list of ``voting.aggregate_votes`` (src/voting.py:110-165): same tally,
    one ``rng.random()`` tie-break draw per distinct grid in first-seen order, votes descending.
    ``records[i]`` belongs to variant ``i`` (canonical order)."""
    status, copy, hh, ww, _, cells = record_fields(records)
    n = len(vt)
    out: dict = {}
    # variants of one (task, test) are contiguous in canonical order
    bounds = np.flatnonzero(np.diff(vt.template, prepend=-1, append=-1))
    assert n == 0 or bounds[-1] == n
    for b0, b1 in zip(bounds[:-1].tolist(), bounds[1:].tolist()):
        tally: dict = {}
        n_valid = 0
        for i in range(b0, b1):
            if status[i] != 1 or (discard_input_copies and copy[i]):
                continue
            n_valid += 1
            h, w = int(hh[i]), int(ww[i])
            key = (h, w, cells[i, : h * w].tobytes())
            tally[key] = tally.get(key, 0) + 1

        def ranked(rng, tally=tally):
            order = [(-votes, rng.random(), key) for key, votes in tally.items()]
            order.sort(key=lambda r: (r[0], r[1]))
            return [(np.frombuffer(k[2], np.uint8).reshape(k[0], k[1]).tolist(), -neg) for neg, _, k in order]

        out[(int(vt.task[b0]), int(vt.test_idx[b0]))] = (ranked, b1 - b0, n_valid)
    return out


def vote_records(records: np.ndarray, vt: VariantTable, top_k: int = 2, seed: int = 0,
                 discard_input_copies: bool = True) -> dict:
    """AAIVR top-k per (task, test_idx) from canonical records, with the tie-break rng of
    ``sharding.vote_all`` (``random.Random(seed + 1000003 * task + test_idx)``)."""
    out = {}
    for (ti, test_idx), (ranked, _, _) in tally_records(records, vt, discard_input_copies).items():
        out[(ti, test_idx)] = [g for g, _ in ranked(random.Random(seed + 1000003 * ti + test_idx))[:top_k]]
    return out
