"""Loader (ctypes) and in-tree build of ``libdst_b200.so``, the C-ABI CUDA library.

The library is compiled with nvcc for sm_100a only and carries no torch types: the Python side
passes raw device pointers, sizes and the current CUDA stream. There is no CPU fallback: when the
library is missing or no GPU is present, the compute entry points raise.
"""

from __future__ import annotations

import ctypes
import os
import subprocess
from functools import lru_cache
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
LIB_PATH = CSRC / "libdst_b200.so"
SOURCES = ["api.cu", "format_kernels.cu", "layout_kernels.cu", "gemm_generic.cu", "gemm_decode.cu", "gemm_decode_tq1.cu", "gemm_prefill.cu", "ep_kernels.cu",
           "moe_kernels.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
              "-Xcompiler", "-fPIC"]

OK, ERR_BAD_ARG, ERR_BAD_SHAPE, ERR_BAD_OFFSETS, ERR_UNSUPPORTED, ERR_ALIGNMENT, ERR_CUDA, ERR_TIMEOUT, ERR_TOO_LARGE = range(9)
NOALLOC_SCRATCH_BYTES = 8 * 1024 * 1024 + 16384
FMT_TQ1, FMT_TQ2 = 1, 2
SCALE_F16, SCALE_F32, SCALE_BF16 = 0, 1, 2
OUT_F32, OUT_BF16, OUT_F16 = 0, 1, 2
ACT_BF16, ACT_F16, ACT_I8, ACT_F16_NORM = 0, 1, 2, 3
ALGO_AUTO, ALGO_GENERIC, ALGO_DECODE, ALGO_PREFILL = 0, 1, 2, 3
MAX_TERMS = 4
MAX_PEERS = 16
LAYOUT_CANONICAL, LAYOUT_TILED = 0, 1
SCORE_FUNCS = {"softmax": 0, "sigmoid": 1, "sqrtsoftplus": 2}


def nvcc_path() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = Path(cuda_home) / "bin" / "nvcc"
    return str(cand) if cand.exists() else "nvcc"


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + list(CSRC.glob("*.cuh")) + [CSRC.parent.parent / "include" / "dst_b200.h"]
    return any(d.exists() and d.stat().st_mtime > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source of the package into ``csrc/libdst_b200.so`` (sm_100a)."""
    if force or needs_build():
        cmd = [nvcc_path(), *NVCC_FLAGS, "-o", str(LIB_PATH), *SOURCES]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        res = subprocess.run(cmd, cwd=str(CSRC), capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed:\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(res.stderr)
    return LIB_PATH


_SIGNATURES = {
    # name: (restype, argtypes)
    "dst_abi_version": (ctypes.c_int, []),
    "dst_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "dst_last_cuda_error": (ctypes.c_char_p, []),
    "dst_packed_cols": (ctypes.c_int64, [ctypes.c_int, ctypes.c_int64]),
    "dst_pack": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]),
    "dst_unpack": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]),
    "dst_quant_act_int8": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p,
                                          ctypes.c_void_p, ctypes.c_void_p]),
    "dst_quant_act_int8_f16": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p,
                                              ctypes.c_void_p, ctypes.c_void_p]),
    "dst_decode_row_limit": (ctypes.c_int64, [ctypes.c_int, ctypes.c_int64, ctypes.c_int64]),
    "dst_ternary_grouped_gemm": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                                                ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                                ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_int64,
                                                ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                                                ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "dst_ternary_grouped_gemm_noalloc": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                                                        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                                        ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int64,
                                                        ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p]),
    "dst_gemm_workspace_bytes": (ctypes.c_size_t, [ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_int64]),
    "dst_tiled_bytes": (ctypes.c_int64, [ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64]),
    "dst_tile_weights": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                        ctypes.c_void_p, ctypes.c_void_p]),
    "dst_untile_weights": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                          ctypes.c_void_p, ctypes.c_void_p]),
    "dst_sort_workspace_bytes": (ctypes.c_size_t, [ctypes.c_int64, ctypes.c_int64]),
    "dst_sort_by_expert": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p,
                                          ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "dst_route_softmax_topk": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_float,
                                              ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "dst_route_softmax_topk_ex": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                                                 ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "dst_route_topk": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                                      ctypes.c_float, ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "dst_combine_add": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int,
                                       ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "dst_ep_combine_pull_add": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                               ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int64, ctypes.c_void_p,
                                               ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]),
    "dst_swiglu_std": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]),
    "dst_swiglu_std_norm": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p,
                                           ctypes.c_void_p]),
    "dst_combine_weighted": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                            ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "dst_gather_rows": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                       ctypes.c_void_p, ctypes.c_void_p]),
    "dst_gather_rows_norm": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "dst_swiglu_norm": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                       ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "dst_swiglu_norm_dev": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64,
                                           ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "dst_swiglu": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                  ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p]),
    "dst_combine": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int,
                                   ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "dst_ep_barrier": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_void_p]),
    "dst_ep_placement": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p,
                                        ctypes.c_void_p, ctypes.c_void_p]),
    "dst_ep_push_rows": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int64,
                                        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                        ctypes.c_void_p, ctypes.c_void_p]),
    "dst_ternary_grouped_gemm_scatter": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                                                        ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                                        ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_int64,
                                                        ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p,
                                                        ctypes.c_size_t, ctypes.c_void_p]),
    "dst_ep_combine_returned": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                               ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                               ctypes.c_void_p]),
    "dst_ep_combine_pull": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                           ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int64, ctypes.c_void_p,
                                           ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]),
    "dst_gather_dequant_rows": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                               ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                               ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "dst_gather_dequant_rows_strided": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                                       ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                                       ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "dst_check_device_status": (ctypes.c_int, [ctypes.c_void_p]),
    "dst_debug_prefill_timeout": (ctypes.c_int, [ctypes.c_longlong, ctypes.c_int, ctypes.c_int]),
}


@lru_cache(1)
def load() -> ctypes.CDLL:
    """dlopen the built library and declare every exported symbol. Raises if it was never built."""
    path = Path(os.environ.get("DST_B200_LIB", str(LIB_PATH)))  # DST_B200_LIB: load a library built elsewhere
    if not path.exists():
        raise RuntimeError(f"{path} is missing: build it with deepseekternarized_b200._lib.build() (there is no CPU fallback)")
    lib = ctypes.CDLL(str(path))
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


def status_string(code: int) -> str:
    return load().dst_status_string(code).decode()


def check(code: int) -> None:
    """Map a status code to the exception type the reference raises for the same mistake."""
    if code == OK:
        return
    msg = status_string(code)
    if code == ERR_BAD_OFFSETS:
        raise ValueError(msg)
    if code == ERR_CUDA:
        raise RuntimeError(f"{msg}: {load().dst_last_cuda_error().decode()}")
    raise RuntimeError(msg)
