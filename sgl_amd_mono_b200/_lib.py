"""ctypes binding of ``libmono_b200.so`` (the declarations of ``include/mono_b200.h``).

The reference's runners hand raw pointers to JIT-compiled launchers
(``glm53/gfx950/runner.py:240-321``); this module is the same seam over a C ABI.
There is no fallback: if the library is missing or does not match the header, the
import of a runner raises and the spec refuses to attach.
"""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libmono_b200.so"

MAX_ROWS = 16
GUARD_WORDS = 16
ERR_DEADLINE, ERR_PEER, ERR_ARG, GUARD_FLAGS = 3, 4, 5, 8
ACT_BF16, ACT_A8, ACT_HILO, ACT_MX8, ACT_MX8N, ACT_NVF4 = 0, 1, 2, 3, 4, 5
W_FP8, W_MXFP4, W_BF16, W_NVFP4 = 0, 1, 2, 3
JOB_DENSE, JOB_EXPERT_UP, JOB_EXPERT_DOWN = 0, 1, 2
GEMV_MAX_JOBS = 4

vp, i32, i64, f32, u32, u64 = C.c_void_p, C.c_int, C.c_long, C.c_float, C.c_uint32, C.c_uint64


class Tmap(C.Structure):
    _fields_ = [("opaque", C.c_ubyte * 128)]


class GemvJob(C.Structure):
    _fields_ = [
        ("tmap", Tmap), ("act_tmap", Tmap),
        ("mode", i32), ("n_rows", i32), ("k_tiles", i32), ("split_tiles", i32), ("nsplit", i32),
        ("row_off", i32), ("rb_per_mat", i32), ("n_mats", i32),
        ("wscale_f32", vp), ("wscale_e8", vp), ("wscale_mat_stride", i64), ("wscale_ld", i32),
        ("act", vp), ("planes", i32), ("act_plane_stride", i64), ("act_ld", i32), ("act_seg_stride", i64),
        ("ascale_f32", vp), ("ascale_e8", vp), ("ascale_ld", i32), ("ascale_seg_stride", i64),
        ("coef", vp), ("expert_list", vp), ("n_expert", vp), ("max_expert", i32),
        ("out", vp), ("out_ld", i32), ("out_split_stride", i64),
        ("feeds_job", i32), ("done", vp), ("ready", vp),
        ("_pad4", C.c_ubyte * 40),  # tensor maps are 64-byte aligned in C
        ("tmap4", Tmap), ("act_natural", i32), ("k_tiles4", i32),
        ("stage_planes", vp), ("stage_scale", vp), ("stage_ld", i32), ("stage_scale_ld", i32),
        ("stage_fmt", i32), ("stage_plane_stride", i32),
        ("wglobal", vp), ("wscale_t", vp), ("wscale_t_mat_stride", i64), ("wscale_t_ld", i32),
        ("_tail", C.c_ubyte * 60),
    ]


class GemvArgs(C.Structure):
    _fields_ = [
        ("njobs", i32), ("rows", i32), ("wkind", i32), ("guard", vp), ("max_ctas", i32), ("gen", vp),
        ("wait_ns", u64), ("_pad", C.c_ubyte * 16),  # the job array is 64-byte aligned in C
        ("job", GemvJob * GEMV_MAX_JOBS),
    ]


class ActPrepArgs(C.Structure):
    _fields_ = [
        ("rows", i32), ("k", i32), ("src_bf16", vp), ("src_f32", vp), ("nsum", i32), ("src_ld", i32),
        ("src_sum_stride", i64), ("gamma_bf16", vp), ("eps", f32), ("round_bf16", i32),
        ("fmt", i32), ("planes", vp), ("plane_stride", i64), ("ld", i32), ("scale_f32", vp),
        ("scale_e8", vp), ("scale_ld", i32), ("out_bf16", vp),
        ("segs", i32), ("seg_stride", i64), ("scale_seg_stride", i64),
    ]


class RouteArgs(C.Structure):
    _fields_ = [
        ("rows", i32), ("n_experts", i32), ("top_k", i32), ("route_scale", f32),
        ("logits", vp), ("nsum", i32), ("ld", i32), ("sum_stride", i64), ("bias", vp), ("slots", vp),
        ("ids", vp), ("weights", vp), ("scores", vp), ("expert_list", vp), ("n_expert", vp), ("coef", vp),
    ]


class MidArgs(C.Structure):
    _fields_ = [
        ("rows", i32), ("inter", i32), ("up", vp), ("nsum", i32), ("n_slot", vp), ("max_slot", i32),
        ("fmt", i32), ("round_bf16", i32), ("planes", vp), ("ld", i32), ("scale_f32", vp),
        ("scale_e8", vp), ("scale_ld", i32),
    ]


class SparseMlaArgs(C.Structure):
    _fields_ = [
        ("rows", i32), ("heads", i32), ("topk", i32), ("topk_ld", i32), ("sm_scale", f32),
        ("q", vp), ("kv_pages", vp), ("n_pages", C.c_int64), ("topk_slots", vp), ("out", vp),
        ("scratch", vp), ("guard", vp),
    ]


class ReduceArgs(C.Structure):
    _fields_ = [
        ("rows", i32), ("n", i32), ("partial", vp), ("nsum", i32), ("ld", i32), ("sum_stride", i64),
        ("residual", vp), ("slots", vp), ("out", vp), ("world", i32), ("rank", i32), ("peer_ptrs", vp),
        ("tag", u32), ("parity", i32), ("deadline_ns", u64), ("site", i32), ("guard", vp),
        ("peer_guards", vp), ("mc_ptr", u64), ("rsag", i32),
    ]


PREFETCH_RANGES = 8


class PrefetchArgs(C.Structure):
    _fields_ = [("n", i32), ("ptr", u64 * PREFETCH_RANGES), ("bytes", u64 * PREFETCH_RANGES)]


class RowdotArgs(C.Structure):
    _fields_ = [
        ("rows", i32), ("n", i32), ("k", i32), ("w", vp), ("w_is_f32", i32), ("x_bf16", vp),
        ("out", vp), ("out_ld", i32), ("out_scale", f32),
    ]


class MlaMidArgs(C.Structure):
    _fields_ = [
        ("rows", i32), ("q_lora", i32), ("qkv", vp), ("nsum", i32), ("ld", i32), ("sum_stride", i64),
        ("ik", vp), ("ik_nsum", i32), ("ik_ld", i32), ("ik_sum_stride", i64),
        ("q_a_norm", vp), ("kv_a_norm", vp), ("eps", f32), ("ik_norm_w", vp), ("ik_norm_b", vp),
        ("cos", vp), ("sin", vp), ("positions", vp), ("slots", vp),
        ("qa_planes", vp), ("qa_plane_stride", i64), ("qa_ld", i32), ("qa_scale", vp), ("qa_scale_ld", i32),
        ("kv_pages", vp), ("idx_pages", vp), ("n_pages", C.c_int64), ("kv_out", vp), ("ik_out", vp),
    ]


class QPostArgs(C.Structure):
    _fields_ = [
        ("rows", i32), ("heads", i32), ("qb", vp), ("nsum", i32), ("ld", i32), ("sum_stride", i64),
        ("kv_b", vp), ("kv_b_scale", vp), ("cos", vp), ("sin", vp), ("positions", vp), ("q_full", vp),
        ("index_heads", i32), ("iq", vp), ("iq_nsum", i32), ("iq_ld", i32), ("iq_sum_stride", i64),
        ("idx_q", vp),
    ]


class IndexArgs(C.Structure):
    _fields_ = [
        ("rows", i32), ("index_heads", i32), ("topk", i32), ("idx_q", vp), ("idx_w", vp), ("w_ld", i32),
        ("idx_pages", vp), ("n_pages", C.c_int64), ("page_table", vp), ("pt_ld", i32), ("positions", vp),
        ("slots", vp), ("scores", vp), ("score_ld", i32), ("topk_slots", vp), ("topk_pos", vp),
        ("iq", vp), ("iq_nsum", i32), ("iq_ld", i32), ("iq_sum_stride", i64), ("cos", vp), ("sin", vp),
    ]


class GqaArgs(C.Structure):
    _fields_ = [
        ("rows", i32), ("q_heads", i32), ("kv_heads", i32), ("qkv", vp), ("nsum", i32), ("ld", i32),
        ("sum_stride", i64), ("g_q", vp), ("g_k", vp), ("g_iq", vp), ("g_ik", vp), ("eps", f32),
        ("cos", vp), ("sin", vp), ("positions", vp), ("slots", vp), ("k_scale", f32), ("v_scale", f32),
        ("k_cache", vp), ("v_cache", vp), ("index_cache", vp), ("n_pages", C.c_int64), ("q_out", vp),
        ("iq_out", vp), ("page_table", vp), ("pt_ld", i32), ("scores", vp), ("score_ld", i32),
        ("init_blocks", i32), ("local_blocks", i32), ("sel_pages", vp), ("sel_blocks", vp), ("n_ctx", vp),
        ("sm_scale", f32), ("scratch", vp), ("out", vp),
    ]


class LogitsGatherArgs(C.Structure):
    _fields_ = [
        ("rows", i32), ("n_local", i32), ("partial", vp), ("nsum", i32), ("ld", i32), ("sum_stride", i64),
        ("out", vp), ("out_ld", i32), ("world", i32), ("rank", i32), ("peer_ptrs", vp), ("tag", u32), ("parity", i32),
        ("deadline_ns", u64), ("site", i32), ("guard", vp), ("peer_guards", vp),
    ]


_STRUCTS = [GemvJob, GemvArgs, ActPrepArgs, RouteArgs, MidArgs, SparseMlaArgs, ReduceArgs, RowdotArgs,
            MlaMidArgs, QPostArgs, IndexArgs, GqaArgs, LogitsGatherArgs, PrefetchArgs]

# every symbol include/mono_b200.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "mono_abi_version": (i32, []),
    "mono_set_pdl": (i32, [i32]),
    "mono_last_error": (C.c_char_p, []),
    "mono_sm_count": (i32, []),
    "mono_guard_read": (i32, [vp, C.POINTER(C.c_int32 * 3), vp]),
    "mono_tmap_encode": (i32, [C.POINTER(Tmap), vp, u64, u64, u64, u64, u64]),
    "mono_tmap_encode_box": (i32, [C.POINTER(Tmap), vp, u64, u64, u64, u64, u64, u32]),
    "mono_tmap_encode_fp4": (i32, [C.POINTER(Tmap), vp, u64, u64, u64, u64, u64]),
    "mono_set_gemv_tcgen05": (i32, [i32]),
    "mono_act_prep_launch": (i32, [C.POINTER(ActPrepArgs), vp]),
    "mono_gemv_launch": (i32, [C.POINTER(GemvArgs), vp]),
    "mono_gemv_max_resident_ctas": (i32, [C.POINTER(GemvArgs)]),
    "mono_rowdot_launch": (i32, [C.POINTER(RowdotArgs), vp]),
    "mono_route_launch": (i32, [C.POINTER(RouteArgs), vp]),
    "mono_router_launch": (i32, [C.POINTER(RowdotArgs), C.POINTER(RouteArgs), vp, vp]),
    "mono_mid_launch": (i32, [C.POINTER(MidArgs), vp]),
    "mono_mid_pair_launch": (i32, [C.POINTER(MidArgs), C.POINTER(MidArgs), vp]),
    "mono_sparse_mla_scratch_bytes": (C.c_size_t, [i32, i32, i32]),
    "mono_sparse_mla_launch": (i32, [C.POINTER(SparseMlaArgs), vp]),
    "mono_sparse_mla_quant_launch": (i32, [C.POINTER(SparseMlaArgs), C.POINTER(ActPrepArgs), vp]),
    "mono_sparse_mla_launch_noalloc": (i32, [C.POINTER(SparseMlaArgs), vp]),
    "mono_reduce_peer_bytes": (C.c_size_t, [i32, i32, i32]),
    "mono_reduce_launch": (i32, [C.POINTER(ReduceArgs), vp]),
    "mono_reduce_norm_launch": (i32, [C.POINTER(ReduceArgs), C.POINTER(ActPrepArgs), vp]),
    "mono_epoch_advance_launch": (i32, [vp, vp]),
    "mono_index_prep_launch": (i32, [vp, vp, vp]),
    "mono_l2_prefetch_launch": (i32, [vp, vp]),
    "mono_logits_peer_bytes": (C.c_size_t, [i32, i32]),
    "mono_logits_gather_launch": (i32, [C.POINTER(LogitsGatherArgs), vp]),
    "mono_mla_mid_launch": (i32, [C.POINTER(MlaMidArgs), vp]),
    "mono_q_post_launch": (i32, [C.POINTER(QPostArgs), vp]),
    "mono_index_score_launch": (i32, [C.POINTER(IndexArgs), vp]),
    "mono_index_topk_launch": (i32, [C.POINTER(IndexArgs), vp]),
    "mono_gqa_scratch_bytes": (C.c_size_t, [i32, i32]),
    "mono_gqa_front_launch": (i32, [C.POINTER(GqaArgs), vp]),
    "mono_gqa_score_launch": (i32, [C.POINTER(GqaArgs), vp]),
    "mono_gqa_select_launch": (i32, [C.POINTER(GqaArgs), vp]),
    "mono_gqa_attn_launch": (i32, [C.POINTER(GqaArgs), vp]),
    "mono_struct_size": (C.c_size_t, [i32]),
    "mono_launch_count": (C.c_ulonglong, []),
    "mono_peer_alloc": (i32, [C.c_size_t, C.POINTER(vp)]),
    "mono_peer_export": (i32, [vp, C.POINTER(C.c_ubyte * 64)]),
    "mono_peer_open": (i32, [C.POINTER(C.c_ubyte * 64), C.POINTER(vp)]),
    "mono_peer_close": (i32, [vp]),
    "mono_peer_free": (i32, [vp]),
    "mono_peer_read": (i32, [vp, vp, C.c_size_t]),
}


class MonoLibraryError(RuntimeError):
    pass


_lib = None


def load():
    """The loaded library; raises MonoLibraryError when it is missing or mismatched."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise MonoLibraryError(
            f"{LIB_PATH} is not built: run `python -m sgl_amd_mono_b200.build` "
            "(there is no CPU or eager fallback for the monokernel path)"
        )
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SYMBOLS.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise MonoLibraryError(f"{LIB_PATH} does not export {name}") from e
        fn.restype, fn.argtypes = res, args
    for i, st in enumerate(_STRUCTS):
        want = lib.mono_struct_size(i)
        if want != C.sizeof(st):
            raise MonoLibraryError(f"{st.__name__}: binding has {C.sizeof(st)} bytes, library has {want}")
    # process-wide switches, for A/B measurements: MONO_GEMV_TCGEN05=0|1, MONO_PDL=0|1
    if os.environ.get("MONO_GEMV_TCGEN05", "").isdigit():  # 2..12 also caps the tcgen05 pipeline depth
        lib.mono_set_gemv_tcgen05(int(os.environ["MONO_GEMV_TCGEN05"]))
    if os.environ.get("MONO_PDL") in ("0", "1"):
        lib.mono_set_pdl(int(os.environ["MONO_PDL"]))
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().mono_last_error().decode(errors="replace")
        raise RuntimeError(f"{what} failed with status {rc}: {msg}")
