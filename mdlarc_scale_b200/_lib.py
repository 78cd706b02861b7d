"""ctypes binding of libarcb200.so (declarations mirror include/arcb200.h).

The product path has no CPU fallback: if the library is missing, ``load()`` raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libarcb200.so"

ACT_F16, ACT_BF16 = 0, 1
GEMM_AUTO, GEMM_SIMT, GEMM_TC, GEMM_TC_1CTA, GEMM_TC_2CTA = 0, 1, 2, 3, 4
ATTN_AUTO, ATTN_STREAM = 0, 1

E_ARG, E_STATE, E_DEVICE, E_UNSUPPORTED = -1, -2, -3, -4

TENSOR_KINDS = [
    "TOKEN_EMBED", "EXAMPLE_EMBED", "LN1_W", "QKV_W", "OUT_W", "LN2_W", "GATE_W", "GATE_B",
    "UP_W", "UP_B", "DOWN_W", "DOWN_B", "LNF_W", "LM_HEAD", "ROPE_COS_X", "ROPE_SIN_X",
    "ROPE_COS_Y", "ROPE_SIN_Y", "ROPE_COS_Z", "ROPE_SIN_Z",
]
KIND = {name: i for i, name in enumerate(TENSOR_KINDS)}

EXPORTS = [
    "arcb_last_error", "arcb_device_ok", "arcb_engine_create", "arcb_engine_destroy",
    "arcb_engine_load_tensor", "arcb_session_workspace_bytes", "arcb_kv_cache_bytes",
    "arcb_session_create", "arcb_session_destroy", "arcb_prefill", "arcb_decode",
    "arcb_session_poll", "arcb_engine_saturation_count", "arcb_session_attention_probe", "arcb_launch_count", "arcb_op_rmsnorm", "arcb_op_gemm",
    "arcb_op_gemm_residual", "arcb_gemm_splitk_scratch_bytes", "arcb_op_gemm_residual_splitk",
    "arcb_attn_scratch_bytes", "arcb_op_decode_attention", "arcb_op_decode_attention_static",
    "arcb_op_head", "arcb_build_prompts", "arcb_canonicalize_candidates",
]
STATIC_ATTN_MAX_RECORDS = 16384


class Config(C.Structure):
    _fields_ = [
        ("d_model", C.c_int32), ("n_heads", C.c_int32), ("n_layers", C.c_int32), ("d_ff", C.c_int32),
        ("vocab_size", C.c_int32), ("num_examples", C.c_int32),
        ("max_x", C.c_int32), ("max_y", C.c_int32), ("max_z", C.c_int32),
        ("use_example_embedding", C.c_int32), ("act_format", C.c_int32), ("gemm_path", C.c_int32),
        ("attn_path", C.c_int32), ("norm_eps", C.c_float),
    ]


class SessionDesc(C.Structure):
    _fields_ = [
        ("n_seqs", C.c_int32), ("t_max", C.c_int32), ("max_new", C.c_int32),
        ("max_prefill_tokens", C.c_int32), ("attn_splits", C.c_int32), ("stop_on_end", C.c_int32),
        ("d_kv_cache", C.c_void_p), ("kv_cache_bytes", C.c_int64),
        ("d_workspace", C.c_void_p), ("workspace_bytes", C.c_int64),
        ("d_out_tokens", C.c_void_p), ("d_forced", C.c_void_p), ("d_step_logits", C.c_void_p),
        ("d_palette_mask", C.c_void_p), ("d_target_shape", C.c_void_p),
        ("palette_penalty", C.c_float), ("shape_penalty", C.c_float), ("disallow_token_mask", C.c_uint32),
        ("temperature", C.c_float), ("top_k", C.c_int32), ("sample_seed", C.c_uint64),
        ("d_sample_stream", C.c_void_p),
    ]


class PrefillArgs(C.Structure):
    _fields_ = [
        ("n_tokens", C.c_int32),
        ("d_token_ids", C.c_void_p), ("d_pos_xyz", C.c_void_p), ("d_seq", C.c_void_p),
        ("d_kv_slot", C.c_void_p), ("d_kv_count", C.c_void_p), ("d_example_ids", C.c_void_p),
        ("n_qblocks", C.c_int32), ("d_qblock_row0", C.c_void_p), ("d_qblock_rows", C.c_void_p),
        ("d_qblock_kv0", C.c_void_p), ("d_kv_row", C.c_void_p), ("n_kv_rows", C.c_int32),
        ("kv_row_identity", C.c_int32),
        ("d_logits_all", C.c_void_p),
        ("n_first", C.c_int32), ("d_first_row", C.c_void_p), ("d_first_seq", C.c_void_p),
        ("d_prompt_len", C.c_void_p), ("d_grid_x", C.c_void_p), ("d_grid_y", C.c_void_p),
        ("d_grid_in_output", C.c_void_p), ("d_first_logits", C.c_void_p),
    ]


class PromptBuildArgs(C.Structure):
    _fields_ = [
        ("n_variants", C.c_int32), ("n_perms", C.c_int32),
        ("d_cells", C.c_void_p), ("d_grid_off", C.c_void_p), ("d_grid_h", C.c_void_p), ("d_grid_w", C.c_void_p),
        ("d_tpl_off", C.c_void_p), ("d_tpl_grid", C.c_void_p), ("d_perm_lut", C.c_void_p),
        ("d_var_template", C.c_void_p), ("d_var_dihedral", C.c_void_p), ("d_var_perm", C.c_void_p),
        ("d_var_tok_off", C.c_void_p), ("d_var_seq", C.c_void_p),
        ("d_token_ids", C.c_void_p), ("d_pos_xyz", C.c_void_p), ("d_seq", C.c_void_p),
        ("d_kv_slot", C.c_void_p), ("d_kv_count", C.c_void_p), ("d_kv_row", C.c_void_p),
        ("d_status", C.c_void_p),
    ]


class CandidateArgs(C.Structure):
    _fields_ = [
        ("n_rows", C.c_int32), ("max_new", C.c_int32),
        ("d_tokens", C.c_void_p), ("d_row_dihedral", C.c_void_p), ("d_row_perm", C.c_void_p),
        ("d_perm_lut", C.c_void_p), ("n_perms", C.c_int32), ("reserved", C.c_int32),
        ("d_row_test_grid", C.c_void_p), ("d_cells", C.c_void_p), ("d_grid_off", C.c_void_p),
        ("d_grid_h", C.c_void_p), ("d_grid_w", C.c_void_p), ("d_records", C.c_void_p),
    ]


_lib = None


class ArcbError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"arcb200 error {code}: {message}")
        self.code = code


def load() -> C.CDLL:
    """Load the CUDA library; raises if it has not been built (no CPU fallback exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m mdlarc_scale_b200.build` "
            "(the B200 path has no CPU fallback)")
    lib = C.CDLL(str(LIB_PATH))
    vp, i32, i64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float
    lib.arcb_last_error.restype = C.c_char_p
    lib.arcb_last_error.argtypes = []
    lib.arcb_device_ok.restype = C.c_int
    lib.arcb_engine_create.argtypes = [C.POINTER(Config), C.POINTER(vp)]
    lib.arcb_engine_destroy.argtypes = [vp]
    lib.arcb_engine_load_tensor.argtypes = [vp, i32, i32, vp, i64, vp]
    lib.arcb_session_workspace_bytes.restype = i64
    lib.arcb_session_workspace_bytes.argtypes = [vp, i32, i32, i32]
    lib.arcb_kv_cache_bytes.restype = i64
    lib.arcb_kv_cache_bytes.argtypes = [vp, i32, i32]
    lib.arcb_session_create.argtypes = [vp, C.POINTER(SessionDesc), C.POINTER(vp)]
    lib.arcb_session_destroy.argtypes = [vp]
    lib.arcb_prefill.argtypes = [vp, C.POINTER(PrefillArgs), vp]
    lib.arcb_decode.argtypes = [vp, i32, vp]
    lib.arcb_session_poll.argtypes = [vp, C.POINTER(i32), C.POINTER(i32), vp]
    lib.arcb_session_attention_probe.argtypes = [vp, C.POINTER(C.c_float)]
    lib.arcb_engine_saturation_count.argtypes = [vp, C.POINTER(i64), i32, vp]
    lib.arcb_build_prompts.argtypes = [C.POINTER(PromptBuildArgs), vp]
    lib.arcb_canonicalize_candidates.argtypes = [C.POINTER(CandidateArgs), vp]
    lib.arcb_launch_count.restype = i64
    lib.arcb_launch_count.argtypes = [C.c_int]
    lib.arcb_op_rmsnorm.argtypes = [vp, vp, vp, i32, i32, f32, i32, vp]
    lib.arcb_op_gemm.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, vp]
    lib.arcb_op_gemm_residual.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp]
    lib.arcb_gemm_splitk_scratch_bytes.restype = i64
    lib.arcb_gemm_splitk_scratch_bytes.argtypes = [i32, i32, i32]
    lib.arcb_op_gemm_residual_splitk.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, vp, vp]
    lib.arcb_attn_scratch_bytes.restype = i64
    lib.arcb_attn_scratch_bytes.argtypes = [i32, i32, i32]
    lib.arcb_op_decode_attention.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, i32, vp]
    lib.arcb_op_decode_attention_static.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp]
    lib.arcb_op_head.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, f32, vp]
    _lib = lib
    return lib


def check(code: int) -> None:
    if code != 0:
        raise ArcbError(code, load().arcb_last_error().decode("utf-8", "replace"))
