"""ctypes binding of libjf_hybrid.so (include/jacobi_hybrid.h).  The library is built in-tree on first use when it is
missing or older than its sources (nvcc, sm_100a); there is no CPU fallback."""
from __future__ import annotations

import ctypes as C
import os
import shutil
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(_HERE)
LIB_PATH = os.path.join(_HERE, "libjf_hybrid.so")
SOURCES = [os.path.join(_HERE, "csrc", f) for f in ("hy_engine.cu", "hy_kernels.cuh", "hy_gemm.cuh", "hy_attn.cuh", "hy_mixers.cuh", "hy_experts.cuh", "hy_window.cuh", "hy_biased.cuh",
                                                        "jf_ptx.cuh")] + [
    os.path.join(ROOT, "include", "jacobi_hybrid.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "-shared", "-Xcompiler", "-fPIC"]
EXPORTS = ["hy_create", "hy_destroy", "hy_last_error", "hy_load_tensor", "hy_finalize", "hy_step", "hy_launch_count",
           "hy_last_step_ms", "hy_memory_info", "hy_profile_enable", "hy_profile_read"]
PROFILE_CATEGORIES = ("norm_embed", "gemm_in", "conv_cache", "attention", "small_gemm", "scan", "delta", "gemm_out", "head",
                      "route", "experts")
HY_OK, HY_ERR_INVALID, HY_ERR_CUDA, HY_ERR_CAPACITY, HY_ERR_UNSUPPORTED = 0, -1, -2, -3, -4


class LayerCfg(C.Structure):
    _fields_ = ([("mixer", C.c_int32)] +
                [(n, C.c_int32) for n in ("a_heads", "a_kv_heads", "a_dim", "a_vdim", "a_conv", "a_qt_every")] +
                [("a_scale", C.c_float), ("a_qt_coef", C.c_float)] +
                [(n, C.c_int32) for n in ("s_inner", "s_state", "s_dt_rank", "s_conv")] +
                [("left_scale", C.c_float), ("right_scale", C.c_float)] +
                [(n, C.c_int32) for n in ("d_heads", "d_kv_heads", "d_dim", "d_vdim", "d_conv", "d_low_a", "d_low_g",
                                          "ff_kind", "ff")] +
                [(n, C.c_int32) for n in ("m_heads", "m_vdim", "m_state", "m_groups", "m_conv", "m_norm_groups")] +
                [(n, C.c_int32) for n in ("l_heads", "l_dim", "l_rot_dim", "l_vdim", "l_kv_rank", "l_q_rank", "l_kv_from")] +
                [("l_scale", C.c_float), ("r_dims", C.c_int32)] +
                [(n, C.c_float) for n in ("r_base", "r_factor", "r_original", "r_fast", "r_slow")] +
                [(n, C.c_int32) for n in ("g_heads", "g_dim", "g_vdim", "x_experts", "x_top", "x_groups", "x_keep")] +
                [("x_scale", C.c_float)] +
                [(n, C.c_int32) for n in ("x_route", "x_plain", "x_act", "x_shared_ff", "ff_act")] +
                [(n, C.c_int32) for n in ("w_heads", "w_kv_heads", "w_dim", "w_vdim", "w_window", "w_pool", "w_rot_dims",
                                          "w_rot_values", "w_qk_norm")] +
                [("w_rot_base", C.c_float), ("w_scale", C.c_float)] +
                [(n, C.c_int32) for n in ("t_heads", "t_dim", "t_vdim")] + [("t_gate_cap", C.c_float)] +
                [(n, C.c_int32) for n in ("b_heads", "b_kv_heads", "b_dim", "b_vdim", "b_window", "b_keep_first", "b_v_mix")] +
                [("b_scale", C.c_float), ("b_softcap", C.c_float), ("ff_limit", C.c_float)])


class ModelCfg(C.Structure):
    _fields_ = [("width", C.c_int32), ("vocab", C.c_int32), ("n_layers", C.c_int32), ("dtype", C.c_int32),
                ("emb_scale", C.c_float), ("logit_scale", C.c_float), ("norm_eps", C.c_float),
                ("norm_kind", C.c_int32), ("block_kind", C.c_int32), ("pos_kind", C.c_int32),
                ("embed_norm", C.c_int32), ("tied_head", C.c_int32), ("resid_mult", C.c_float),
                ("canon_taps", C.c_int32), ("side_dim", C.c_int32), ("depth_avg", C.c_int32),
                ("pair_buckets", C.c_int32), ("pair_mul_prev", C.c_int32), ("pair_mul_cur", C.c_int32)]


class RuntimeCfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("device", "max_step_tokens", "max_step_entries", "page_size", "num_pages",
                                         "max_pages_per_seq", "num_slots", "max_want")]


def stale() -> bool:
    srcs = [s for s in SOURCES if os.path.exists(s)]
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(s) > t for s in srcs)


def build(force: bool = False) -> str:
    """Compile csrc/hy_engine.cu into libjf_hybrid.so (only this library: the other model family's is not touched)."""
    if not force and not stale():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        if os.path.exists(LIB_PATH):
            return LIB_PATH
        raise ImportError("nvcc not found and no prebuilt libjf_hybrid.so; there is no CPU fallback")
    tmp = LIB_PATH + f".{os.getpid()}.tmp"
    cmd = [nvcc] + NVCC_FLAGS + ["-I", os.path.join(ROOT, "include"), "-I", os.path.join(_HERE, "csrc"),
                                 os.path.join(_HERE, "csrc", "hy_engine.cu"), "-o", tmp]
    subprocess.check_call(cmd, stdout=subprocess.DEVNULL)
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    build()
    lib = C.CDLL(LIB_PATH)
    vp, i32, i32p, i64p, fp = C.c_void_p, C.c_int32, C.POINTER(C.c_int32), C.POINTER(C.c_int64), C.POINTER(C.c_float)
    lib.hy_create.argtypes = [C.POINTER(ModelCfg), C.POINTER(LayerCfg), C.POINTER(RuntimeCfg), C.POINTER(vp)]
    lib.hy_destroy.argtypes = [vp]
    lib.hy_destroy.restype = None
    lib.hy_last_error.argtypes = [vp]
    lib.hy_last_error.restype = C.c_char_p
    lib.hy_load_tensor.argtypes = [vp, C.c_char_p, vp, i64p, i32, i32]
    lib.hy_finalize.argtypes = [vp]
    lib.hy_step.argtypes = [vp, i32, vp, vp, vp, vp, vp, i32, vp, vp, vp, vp, C.c_uint64, vp]
    lib.hy_launch_count.argtypes = [vp]
    lib.hy_launch_count.restype = C.c_int64
    lib.hy_last_step_ms.argtypes = [vp]
    lib.hy_last_step_ms.restype = C.c_float
    lib.hy_memory_info.argtypes = [vp, i64p, i64p, i64p, i64p]
    lib.hy_profile_enable.argtypes = [vp, i32]
    lib.hy_profile_read.argtypes = [vp, fp]
    for n in ("hy_profile_enable", "hy_profile_read", "hy_create", "hy_load_tensor", "hy_finalize", "hy_step", "hy_memory_info"):
        getattr(lib, n).restype = C.c_int
    _lib = lib
    return lib


_EXC = {HY_ERR_INVALID: ValueError, HY_ERR_CUDA: RuntimeError, HY_ERR_CAPACITY: RuntimeError,
        HY_ERR_UNSUPPORTED: NotImplementedError}


def check(rc: int, handle=None) -> None:
    if rc == HY_OK:
        return
    msg = load().hy_last_error(handle)
    raise _EXC.get(rc, RuntimeError)((msg or b"").decode() or f"libjf_hybrid error {rc}")
