"""ctypes loader for libmsa_b200.so (the C ABI in include/msa_b200.h).

The library is built ahead of time, in-tree, by ``build_library()`` (one nvcc
invocation for sm_100a).  There is no CPU fallback: if the library is missing
or fails to load, every entry point raises.
"""
from __future__ import annotations

import ctypes
import fcntl
import os
import subprocess
import threading
from ctypes import POINTER, Structure, c_char_p, c_float, c_int32, c_int64, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
# MSA_B200_LIB points the loader at another build of the same ABI (e.g. one made with -DMSA_ROLE_TIMING)
LIB_PATH = os.environ.get("MSA_B200_LIB") or os.path.join(_HERE, "libmsa_b200.so")
CSRC = os.path.join(_HERE, "csrc")
SOURCES = ["abi.cu", "topk.cu", "decode.cu", "fmha_host.cu", "kv_quant.cu", "plan_host.cu", "csr.cu", "fp4_indexer.cu"]

MSA_KV_BF16, MSA_KV_FP8_E4M3, MSA_KV_NVFP4 = 0, 1, 2
MSA_ERR_INVALID = -1
MSA_ERR_UNSUPPORTED = -2
MSA_ERR_TIMEOUT = -3
MSA_ERR_BOUNDS = -6
ABI_VERSION = 4


class MsaError(RuntimeError):
    pass


class FmhaArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("out", c_void_p),
        ("lse", c_void_p), ("max_score", c_void_p),
        ("work", c_void_p), ("n_work", c_int32),
        ("kv_indices", c_void_p), ("kv_block_indexes", c_void_p),
        ("k_scale_128x4", c_void_p), ("v_scale_128x4", c_void_p),
        ("total_q", c_int64), ("kv_rows", c_int64),
        ("num_qo_heads", c_int32), ("num_kv_heads", c_int32),
        ("topk", c_int32), ("list_heads", c_int32), ("max_k_tiles", c_int32),
        ("kv_dtype", c_int32), ("paged", c_int32), ("causal", c_int32),
        ("sm_scale", c_float), ("qk_scale", c_float), ("v_scale", c_float),
        ("status", c_void_p), ("max_ctas", c_int32), ("qk_dim", c_int32),
        ("tile_rows", c_int32), ("tile_uniform", c_void_p), ("max_score_tile_stride", c_int64), ("max_score_head_stride", c_int64),
        ("k_scale_format", c_int32), ("score_pack_heads", c_int32), ("score_fill_tail", c_int32), ("fp8_p_f16", c_int32), ("out_rows", c_int64),
    ]


class DecodeArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("out", c_void_p), ("lse", c_void_p),
        ("kv_indices", c_void_p), ("kv_page_indptr", c_void_p), ("kv_block_indexes", c_void_p),
        ("token_request", c_void_p), ("token_pos", c_void_p),
        ("num_tokens", c_int32), ("num_qo_heads", c_int32), ("num_kv_heads", c_int32), ("topk", c_int32),
        ("num_splits", c_int32),
        ("sm_scale", c_float), ("qk_scale", c_float), ("v_scale", c_float),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t),
        ("num_pages", c_int64), ("status", c_void_p),
    ]


class KvAppendArgs(Structure):
    _fields_ = [
        ("struct_size", ctypes.c_uint32), ("format", c_int32),
        ("k_new", c_void_p), ("v_new", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p),
        ("k_block_scales", c_void_p), ("v_block_scales", c_void_p), ("slots", c_void_p),
        ("num_tokens", c_int32), ("num_kv_heads", c_int32), ("head_dim", c_int32), ("num_pages", c_int32),
        ("k_scale", c_float), ("v_scale", c_float),
    ]


class PlanDesc(Structure):
    _fields_ = [
        ("batch", c_int32), ("qo_lens", c_void_p), ("kv_lens", c_void_p), ("qo_offset", c_void_p),
        ("causal", c_int32), ("paged", c_int32), ("num_qo_heads", c_int32), ("num_kv_heads", c_int32),
        ("kv_block_num", c_int32), ("num_kv_splits", c_int32), ("num_sms", c_int32), ("tile_rows", c_int32),
        ("dense_kv_splits", c_int32),
    ]


class ValidateArgs(Structure):
    _fields_ = [
        ("batch", c_int32), ("qo_lens", c_void_p), ("kv_lens", c_void_p),
        ("total_q", c_int64), ("kv_rows", c_int64), ("paged", c_int32),
        ("kv_indices", c_void_p), ("n_kv_indices", c_int64), ("kv_block_indexes", c_void_p),
        ("list_heads", c_int32), ("topk", c_int32), ("num_qo_heads", c_int32), ("num_kv_heads", c_int32),
    ]


class CsrBuildArgs(Structure):
    _fields_ = [
        ("q2k", c_void_p), ("chunk_request", c_void_p), ("chunk_first_query", c_void_p), ("chunk_len", c_void_p),
        ("cu_seqlens_q", c_void_p), ("request_first_chunk", c_void_p), ("request_blocks", c_void_p),
        ("row_of_block", c_void_p), ("workspace", c_void_p), ("workspace_bytes", c_size_t),
        ("row_ptr", c_void_p), ("q_indices", c_void_p), ("total_q", c_int64), ("q_indices_stride", c_int64),
        ("num_kv_heads", c_int32), ("topk", c_int32), ("n_chunks", c_int32), ("batch", c_int32),
        ("max_blocks", c_int32), ("total_rows", c_int32),
    ]


def _sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def build_library(verbose: bool = False, force: bool = True) -> str:
    """Compile every CUDA source for sm_100a into msa_b200/libmsa_b200.so."""
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    # Several processes may get here at once (one rank per GPU importing the package after a source edit):
    # an exclusive file lock serialises them, and the library is written under a temporary name and renamed
    # into place, so a process that is loading the old file never sees a half-written one.
    with open(LIB_PATH + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not _needs_build():
                return LIB_PATH          # another process built it while this one waited
            tmp = f"{LIB_PATH}.{os.getpid()}.tmp"
            cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
                   "--shared", "-Xcompiler", "-fPIC", "-o", tmp] + _sources()
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            r = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
            if r.returncode != 0:
                if os.path.exists(tmp):
                    os.remove(tmp)
                raise MsaError("nvcc failed:\n" + r.stdout + r.stderr)
            if verbose:
                print(r.stderr)
            os.replace(tmp, LIB_PATH)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB_PATH


def _needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(_HERE, "..", "include", "msa_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


_lib = None
_lock = threading.Lock()


def _bind(lib):
    vp = c_void_p
    lib.msa_abi_version.restype = c_int32
    lib.msa_error_string.restype = c_char_p
    lib.msa_error_string.argtypes = [c_int32]
    lib.msa_plan_sizes.restype = c_int32
    lib.msa_plan_sizes.argtypes = [POINTER(PlanDesc), vp, vp, vp]
    lib.msa_plan.restype = c_int32
    lib.msa_plan.argtypes = [POINTER(PlanDesc), vp, vp, vp, vp, vp]
    lib.msa_validate_inputs.restype = c_int32
    lib.msa_validate_inputs.argtypes = [POINTER(ValidateArgs), vp]
    lib.msa_build_k2q_csr_workspace_bytes.restype = c_size_t
    lib.msa_build_k2q_csr_workspace_bytes.argtypes = [c_int32, c_int32, c_int32, c_int32]
    lib.msa_build_k2q_csr.restype = c_int32
    lib.msa_build_k2q_csr.argtypes = [POINTER(CsrBuildArgs), vp]
    lib.msa_k2q_csr_to_lists.restype = c_int32
    lib.msa_k2q_csr_to_lists.argtypes = [vp, vp, vp, vp, vp, c_int32, c_int32, c_int64, c_int64, c_int64, c_int32,
                                         vp, vp, vp]
    lib.msa_topk_select.restype = c_int32
    lib.msa_topk_select.argtypes = [vp, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, vp, vp]
    lib.msa_block_max.restype = c_int32
    lib.msa_block_max.argtypes = [vp, c_int32, c_int32, c_int32, vp, c_int32, vp, vp]
    lib.msa_expand_block_lists.restype = c_int32
    lib.msa_expand_block_lists.argtypes = [vp, vp, c_int32, c_int32, c_int32, vp, vp]
    lib.msa_fmha_combine.restype = c_int32
    lib.msa_fmha_combine.argtypes = [vp, vp, c_int32, c_int64, c_int32, vp, vp, vp]
    lib.msa_fp4_dequant_rows.restype = c_int32
    lib.msa_fp4_dequant_rows.argtypes = [vp, vp, c_int32, c_int32, c_int64, c_int32, vp, vp]
    lib.msa_fp4_reorder_scales.restype = c_int32
    lib.msa_fp4_reorder_scales.argtypes = [vp, c_int32, c_int64, c_int64, c_int32, vp, vp]
    lib.msa_list_uniformity.restype = c_int32
    lib.msa_list_uniformity.argtypes = [vp, c_int32, vp, c_int32, c_int32, vp, vp]
    lib.msa_fmha_fwd.restype = c_int32
    lib.msa_fmha_fwd.argtypes = [POINTER(FmhaArgs), vp]
    lib.msa_decode_workspace_bytes.restype = c_size_t
    lib.msa_decode_workspace_bytes.argtypes = [c_int32, c_int32, c_int32]
    lib.msa_decode_fwd.restype = c_int32
    lib.msa_decode_fwd.argtypes = [POINTER(DecodeArgs), vp]
    lib.msa_decode_fwd_static.restype = c_int32
    lib.msa_decode_fwd_static.argtypes = [POINTER(DecodeArgs), vp]
    lib.msa_kv_append.restype = c_int32
    lib.msa_kv_append.argtypes = [POINTER(KvAppendArgs), vp]
    lib.msa_absmax_bf16.restype = c_int32
    lib.msa_absmax_bf16.argtypes = [vp, c_int64, vp, vp]
    lib.msa_debug_set_timing_buffer.restype = None
    lib.msa_debug_set_timing_buffer.argtypes = [vp]
    lib.msa_umma_selftest.restype = c_int32
    lib.msa_umma_selftest.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp]
    lib.msa_umma_selftest_timeout.restype = c_int32
    lib.msa_umma_selftest_timeout.argtypes = [vp, vp, vp, vp, vp, vp, vp, c_int64, vp]
    return lib


def get_lib():
    """Load (building first if sources are newer and nvcc is present) the C-ABI library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.environ.get("MSA_B200_LIB") and _needs_build():
                nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
                if os.path.exists(nvcc):
                    build_library(force=False)
                elif not os.path.exists(LIB_PATH):
                    raise MsaError(f"{LIB_PATH} is missing and nvcc is not available to build it")
            try:
                _lib = _bind(ctypes.CDLL(LIB_PATH))
            except OSError as e:
                raise MsaError(f"cannot load {LIB_PATH}: {e}") from e
    return _lib


def check(code: int, what: str = "") -> None:
    if code == 0:
        return
    lib = get_lib()
    msg = lib.msa_error_string(code).decode()
    raise MsaError(f"{what or 'libmsa_b200'} failed with {code}: {msg}")
