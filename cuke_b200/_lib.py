"""ctypes binding of libkge_b200.so (the C ABI declared in include/kge_b200.h).

This is the thin shim that takes the place of cuke's compile-and-load step
(pycuke1/run/gpu.py:4-19: write the generated .cu, torch.utils.cpp_extension.load, module.run).
There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libkge_b200.so")

MODELS = {"TransE": 0, "TransH": 1, "TransR": 2, "TransF": 3, "DistMult": 4, "RESCAL": 5, "ComplEx": 6}
DTYPES = {"f32": 0, "bf16": 1}
NEG_MODES = {"none": 0, "per_triple": 1, "chunk_shared": 2}
PRECISIONS = {"fp32": 0, "tensor": 1, "tensor_tf32": 2}
FLAG_CHECK_IDS = 1            # kge_problem.reserved
ERR_WAIT_TIMEOUT, ERR_ID_RANGE = 2, 8     # values of the device error word (kge_check)
VECTOR_MODELS = ("TransE", "TransH", "TransR")
MATRIX_MODELS = ("TransR", "RESCAL")


class KgeError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"libkge_b200 error {code}: {message}")
        self.code = code


class KgeProblem(C.Structure):
    _fields_ = [("model", C.c_int32), ("dtype", C.c_int32), ("neg_mode", C.c_int32), ("id_bits", C.c_int32),
                ("dim", C.c_int32), ("n_neg", C.c_int32), ("n_neg_head", C.c_int32), ("chunk", C.c_int32),
                ("batch", C.c_int64), ("n_ent", C.c_int64), ("n_rel", C.c_int64),
                ("precision", C.c_int32), ("reserved", C.c_int32)]


class KgeTensors(C.Structure):
    _fields_ = [("ent", C.c_void_p), ("rel", C.c_void_p), ("rel2", C.c_void_p),
                ("h", C.c_void_p), ("r", C.c_void_p), ("t", C.c_void_p), ("neg", C.c_void_p),
                ("rel_perm", C.c_void_p), ("rel_seg", C.c_void_p), ("rel_uniq", C.c_void_p),
                ("n_rel_groups", C.c_void_p)]


class KgeGrads(C.Structure):
    _fields_ = [("g_head", C.c_void_p), ("g_tail", C.c_void_p), ("g_neg", C.c_void_p),
                ("g_rel", C.c_void_p), ("g_rel2", C.c_void_p)]


class KgeProgram(C.Structure):
    _fields_ = [("n_ops", C.c_int32), ("n_vreg", C.c_int32), ("n_sreg", C.c_int32),
                ("out_kind", C.c_int32), ("out_a", C.c_int32), ("out_b", C.c_int32), ("out_s", C.c_int32),
                ("out_table", C.c_int32), ("out_ids", C.c_int32), ("ops", (C.c_int32 * 5) * 64)]


_lib = None

_vp, _i32, _i64, _sz, _f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t, C.c_float
_PP, _PT, _PG = C.POINTER(KgeProblem), C.POINTER(KgeTensors), C.POINTER(KgeGrads)

# name -> (restype, argtypes); must list every symbol include/kge_b200.h declares
SIGNATURES = {
    "kge_version": (C.c_int, []),
    "kge_last_error": (C.c_char_p, []),
    "kge_launch_count": (C.c_longlong, []),
    "kge_check": (C.c_int, [_vp, C.POINTER(C.c_int32)]),
    "kge_validate_ids": (C.c_int, [_vp, _i32, _i64, _i64, _vp, _vp]),
    "kge_selftest_wait_timeout": (C.c_int, [_i32, _vp]),
    "kge_ref_forward": (C.c_int, [_PP, _PT, _vp, _vp]),
    "kge_inspect_workspace_bytes": (_sz, [_i64]),
    "kge_inspect": (C.c_int, [_vp, _i32, _i64, _i64, _vp, _sz, _vp, _vp, _vp, _vp, _vp, _vp]),
    "kge_legacy_inspect": (C.c_int, [_vp, _i64, _i64, _vp, _vp, _vp, _vp]),
    "kge_gather_rows": (C.c_int, [_vp, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _vp]),
    "kge_scatter_rows": (C.c_int, [_vp, _i32, _vp, _i64, _vp, _i64, _vp, _vp]),
    "kge_profile_gemm": (C.c_int, [_i32]),
    "kge_profile_gemm_read": (C.c_int, [C.POINTER(C.c_double), C.POINTER(C.c_int64), C.POINTER(C.c_double)]),
    "kge_probe_fma": (C.c_int, [_vp, _i32, _i32, C.POINTER(C.c_double), _vp]),
    "kge_segment_reduce_workspace_bytes": (_sz, [_i64, _i32]),
    "kge_segment_reduce": (C.c_int, [_vp, _i32, _i64, _vp, _vp, _vp, _vp, _i64, _vp, _sz, _vp]),
    "kge_pull_reduce": (C.c_int, [_vp, _vp, _vp, _i32, _i32, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _i64, _f32, _vp]),
    "kge_ipc_export": (C.c_int, [_vp, _vp, C.POINTER(C.c_uint64)]),
    "kge_ipc_open": (C.c_int, [_vp, C.c_uint64, C.POINTER(C.c_void_p)]),
    "kge_ipc_close": (C.c_int, [_vp, C.c_uint64]),
    "kge_gather_rows_peers": (C.c_int, [_vp, _i32, _i64, _i64, _i32, _i32, _vp, _i64, _vp, _vp, _vp]),
    "kge_segment_reduce_static": (C.c_int, [_vp, _i32, _i64, _vp, _vp, _vp, _vp, _i64, _vp]),
    "kge_score_workspace_bytes": (_sz, [_PP, _i32]),
    "kge_score_forward": (C.c_int, [_PP, _PT, _vp, _vp, _vp, _sz, _vp]),
    "kge_score_backward": (C.c_int, [_PP, _PT, _vp, _vp, _vp, _vp, _PG, _vp, _sz, _vp]),
    "kge_score_loss_backward_workspace_bytes": (_sz, [_PP]),
    "kge_score_loss_backward": (C.c_int, [_PP, _PT, _f32, _vp, _vp, _PG, _vp, _sz, _vp]),
    "kge_logistic_loss": (C.c_int, [_vp, _i64, _vp, _i64, _f32, _vp, _vp, _vp, _vp, _sz, _vp]),
    "kge_owner_counts": (C.c_int, [_vp, _vp, _i64, _i64, _i32, _vp, _vp]),
    "kge_eval_program": (C.c_int, [C.POINTER(KgeProgram), _i32, _i64, _vp, _i32, _vp, _i32, _i32, _vp, _vp]),
    "kge_sample_uniform": (C.c_int, [_vp, _i32, _i64, _i64, C.c_uint64, C.c_uint32, _vp]),
    "kge_sample_cdf": (C.c_int, [_vp, _i32, _i64, _vp, _vp, _i64, C.c_uint64, C.c_uint32, _vp]),
    "kge_sample_triples": (C.c_int, [_vp, _vp, _vp, _i32, _i64, _vp, _i64, C.c_uint64, C.c_uint32, _vp]),
    "kge_apply_sgd": (C.c_int, [_vp, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _f32, _vp]),
    "kge_apply_adagrad": (C.c_int, [_vp, _i32, _vp, _i32, _vp, _i64, _vp, _i64, _vp, _f32, _f32, _vp]),
}


def lib():
    """The loaded library; raises if it has not been built (python -m cuke_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m cuke_b200.build`; "
                               "there is no CPU or PyTorch fallback for the scoring path")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        if L.kge_version() != 1:
            raise RuntimeError(f"libkge_b200 ABI version {L.kge_version()} != 1")
        _lib = L
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        msg = lib().kge_last_error()
        raise KgeError(rc, msg.decode() if msg else "")
