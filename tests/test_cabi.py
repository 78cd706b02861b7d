"""The C-ABI library loads and exports exactly what include/arcb200.h declares (no GPU needed)."""
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from mdlarc_scale_b200 import _lib, build
    build.build()
    return _lib.load()


def _declared():
    text = (ROOT / "include" / "arcb200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(arcb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = _declared()
    assert len(names) >= 18
    for n in names:
        assert hasattr(lib, n), f"{n} declared in arcb200.h but not exported"


def test_binding_covers_header():
    from mdlarc_scale_b200 import _lib
    assert sorted(_lib.EXPORTS) == _declared()


def test_struct_sizes_match_c_layout():
    import ctypes as C
    from mdlarc_scale_b200 import _lib
    assert C.sizeof(_lib.Config) == 14 * 4
    assert C.sizeof(_lib.SessionDesc) == 136  # sizeof(arcb_session_desc) printed by a C compile of the header
    assert C.sizeof(_lib.PrefillArgs) == 176
    assert C.sizeof(_lib.PromptBuildArgs) == 160
    assert C.sizeof(_lib.CandidateArgs) == 96
    from mdlarc_scale_b200 import fanout
    assert fanout.RECORD_BYTES == 944 and fanout.MAX_CELLS == 936   # sizeof(arcb_candidate_record)


def test_argument_errors_without_gpu(lib):
    import ctypes as C
    from mdlarc_scale_b200 import _lib
    assert lib.arcb_engine_create(None, None) == _lib.E_ARG
    cfg = _lib.Config(d_model=256, n_heads=4, n_layers=4, d_ff=704, vocab_size=15, num_examples=1280,
                      max_x=32, max_y=32, max_z=8, use_example_embedding=1, norm_eps=1e-5)
    h = C.c_void_p()
    assert lib.arcb_engine_create(C.byref(cfg), C.byref(h)) == _lib.E_UNSUPPORTED
    assert b"vocab" in lib.arcb_last_error()
    assert lib.arcb_attn_scratch_bytes(8, 4, 4) == 8 * 4 * 4 * 68 * 4
    assert lib.arcb_attn_scratch_bytes(8, 4, 1) == 0
