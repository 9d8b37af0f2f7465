"""Loader of the C-ABI library `libb200moe.so` (declared in include/b200moe.h) and its build recipe.

The library is the only compute path of this package: if it is missing, importing an operator raises;
there is no CPU or PyTorch fallback.  `build()` compiles it in-tree with nvcc for sm_100a (works without
a GPU); loading it needs only the CUDA runtime it links against.
"""

from __future__ import annotations

import ctypes
import os
import subprocess
import threading

import torch

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libb200moe.so")
SOURCES = ["api.cu", "routing.cu", "rowops.cu", "simt_gemm.cu", "umma_gemm.cu", "umma2_gemm.cu", "ep.cu", "rmsnorm.cu"]
HEADERS = [os.path.join(CSRC, "common.cuh"), os.path.join(PKG_DIR, "..", "include", "b200moe.h")]

F32, BF16, F16 = 0, 1, 2
ENGINE_AUTO, ENGINE_SIMT, ENGINE_UMMA, ENGINE_UMMA_1CTA, ENGINE_UMMA_GATHER4 = 0, 1, 2, 3, 4
OPT_DYNAMIC_TILES, OPT_TILE_VARIANT, OPT_TILE_ORDER, OPT_SM_LIMIT = 1, 2, 3, 4
TILE_PAIR_256x256, TILE_CTA_128x256 = 0, 1
OP_UP_FORWARD, OP_ROW_STORE, OP_DOWN_DGRAD, OP_WGRAD = 0, 1, 2, 3
DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}

_lock = threading.Lock()
_lib = None


NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
OBJ_DIR = os.path.join(PKG_DIR, "build")


def _nvcc() -> str:
    return os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")


def nvcc_command(out: str = LIB_PATH, extra: list[str] | None = None) -> list[str]:
    """The one-command form of the build (every source in one nvcc call); `build()` runs the same flags per source in
    parallel and links the objects."""
    return [_nvcc()] + NVCC_FLAGS + ["-shared"] + (extra or []) + ["-o", out] + [os.path.join(CSRC, s) for s in SOURCES]


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + HEADERS + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]
    return any(os.path.exists(d) and os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library in-tree for sm_100a: one nvcc process per source file, run concurrently, then one link.
    Returns the path of the shared object."""
    if force or needs_build():
        os.makedirs(OBJ_DIR, exist_ok=True)
        tag = f".tmp{os.getpid()}"
        extra = ["-Xptxas", "-v"] if verbose else []
        jobs = []
        for src in SOURCES:
            obj = os.path.join(OBJ_DIR, src + tag + ".o")
            cmd = [_nvcc()] + NVCC_FLAGS + extra + ["-c", "-o", obj, os.path.join(CSRC, src)]
            jobs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        logs, failed = [], []
        for src, obj, proc in jobs:
            out, _ = proc.communicate()
            logs.append(f"== {src}\n{out}")
            if proc.returncode != 0:
                failed.append(src)
        objs = [obj for _, obj, _ in jobs]
        try:
            if failed:
                raise RuntimeError("nvcc failed for " + ", ".join(failed) + ":\n" + "\n".join(logs))
            tmp = LIB_PATH + tag
            proc = subprocess.run([_nvcc(), "-shared", "-o", tmp] + objs, capture_output=True, text=True)
            if proc.returncode != 0:
                raise RuntimeError("link failed:\n" + proc.stdout + proc.stderr)
            os.replace(tmp, LIB_PATH)
        finally:
            for obj in objs:
                if os.path.exists(obj):
                    os.remove(obj)
        if verbose:
            print("\n".join(logs))
    return LIB_PATH


def _declare(lib):
    c = ctypes
    vp, i32, i64, f32 = c.c_void_p, c.c_int, c.c_int64, c.c_float
    sig = {
        "b200moe_version": (i32, []),
        "b200moe_error_string": (c.c_char_p, [i32]),
        "b200moe_last_error_detail": (c.c_char_p, []),
        "b200moe_set_engine": (i32, [i32]),
        "b200moe_set_option": (i32, [i32, i32]),
        "b200moe_get_option": (i32, [i32]),
        "b200moe_tile_table_lookup": (i32, [i32, i32, i32, i64]),
        "b200moe_launch_count": (i64, []),
        "b200moe_check_status": (i32, [vp, vp]),
        "b200moe_selftest_bounded_wait": (i32, [vp, i64, vp, vp]),
        "b200moe_contiguous_count": (i32, [vp, i32, i64, vp, i32, vp]),
        "b200moe_padded_rows_cap": (i64, [i64, i32]),
        "b200moe_route_workspace_bytes": (i64, [i64, i32]),
        "b200moe_route": (i32, [vp, i64, i32, i32, vp, vp, vp, vp, vp, vp, i64, vp, i64, vp, vp]),
        "b200moe_route_static_scratch_bytes": (i64, []),
        "b200moe_route_static": (i32, [vp, i64, i32, i32, vp, vp, vp, vp, vp, vp, i64, vp, vp]),
        "b200moe_scatter2scatter_workspace_bytes": (i64, [i64, i32]),
        "b200moe_scatter2scatter": (i32, [vp, i64, vp, i64, i64, i64, vp, vp, vp, i64, i64, i32, i32, i32, i32, i32, i32, i32, vp, i64, vp, vp]),
        "b200moe_group_bwd_W": (i32, [vp, i64, vp, i64, vp, vp, i64, i64, i64, i64, i32, i32, i32, i32, vp, vp]),
        "b200moe_group": (i32, [vp, i64, vp, vp, i64, vp, i32, i64, i32, i32, vp]),
        "b200moe_gather_rows": (i32, [vp, i64, vp, vp, i64, i64, i32, i32, vp]),
        "b200moe_combine": (i32, [vp, i64, vp, vp, i64, i64, i32, i32, i32, vp]),
        "b200moe_swiglu_unchunked_forward": (i32, [vp, i64, vp, i64, i64, i32, i32, vp]),
        "b200moe_swiglu_unchunked_backward": (i32, [vp, i64, vp, i64, vp, i64, i64, i32, i32, vp]),
        "b200moe_up_forward": (i32, [vp, i64, vp, vp, vp, vp, vp, i64, i32, i32, i32, i64, i32, i32, vp, vp]),
        "b200moe_down_forward": (i32, [vp, vp, vp, vp, vp, vp, i64, i64, i32, i32, i32, i64, i32, vp, vp]),
        "b200moe_gather_grad_rows": (i32, [vp, i64, vp, vp, vp, vp, i64, i32, vp, i64, vp, i64, i32, i32, vp]),
        "b200moe_combine_rows": (i32, [vp, i64, vp, vp, vp, i64, i64, i32, i32, i32, vp]),
        "b200moe_invert_row_map": (i32, [vp, i64, vp, i64, vp]),
        "b200moe_down_dgrad": (i32, [vp, i64, vp, vp, vp, vp, vp, i64, i32, i32, i32, i64, i32, i32, vp, vp]),
        "b200moe_wgrad": (i32, [vp, i64, vp, vp, i64, vp, vp, vp, i32, i32, i32, i64, i32, vp, vp]),
        "b200moe_ep_push_rows": (i32, [vp, i64, vp, i32, vp, vp, vp, vp, i32, i64, i32, i64, i32, vp, vp]),
        "b200moe_ep_pull_combine": (i32, [vp, vp, vp, vp, i32, vp, vp, i64, vp, i64, i32, i32, i32, vp]),
        "b200moe_ep_push_rows_at": (i32, [vp, i64, vp, i32, vp, vp, vp, vp, vp, i32, i64, i32, i64, i32, i32, vp, vp]),
        "b200moe_ep_pull_combine_at": (i32, [vp, vp, vp, vp, vp, i32, i64, i32, vp, vp, i64, vp, i64, i32, i32, i32, vp]),
        "b200moe_zero_filler_rows": (i32, [vp, i64, vp, i32, i32, i64, i32, vp]),
        "b200moe_ep_plan": (i32, [vp, vp, i32, i32, i32, i64, vp, vp, vp, vp, vp, vp, vp]),
        "b200moe_ep_barrier": (i32, [vp, i32, i32, i32, i64, vp, vp]),
        "b200moe_ep_gate_grad": (i32, [vp, i64, vp, i64, vp, i64, i32, i32, i32, vp]),
        "b200moe_up_dgrad": (i32, [vp, vp, vp, vp, vp, i64, i64, i32, i32, i32, i64, i32, vp, vp]),
        "b200moe_router_forward": (i32, [vp, i64, vp, i64, i64, i32, i32, i32, i32, vp, i64, vp, vp, vp, i32, vp, vp]),
        "b200moe_router_forward_scaled": (i32, [vp, i64, vp, i64, vp, i64, i32, i32, i32, i32, vp, i64, vp, vp, vp, i32, vp, vp]),
        "b200moe_rmsnorm_workspace_bytes": (i64, [i64, i32, i32]),
        "b200moe_rmsnorm_forward": (i32, [vp, i64, vp, vp, i64, vp, i64, i32, f32, i32, vp]),
        "b200moe_rmsnorm_backward": (i32, [vp, i64, vp, vp, i64, vp, vp, i64, vp, vp, i64, i64, i32, f32, i32, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)  # AttributeError here means the library does not export a declared symbol
        fn.restype = res
        fn.argtypes = args
    return sig


EXPORTED = None


def lib():
    """The loaded library.  Raises if it has not been built: there is no other compute path."""
    global _lib, EXPORTED
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise RuntimeError(
                        f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                        "(nvcc, sm_100a).  This package has no CPU or PyTorch fallback."
                    )
                handle = ctypes.CDLL(LIB_PATH)
                EXPORTED = _declare(handle)
                _lib = handle
    return _lib


class B200MoEError(RuntimeError):
    pass


def check(code: int, what: str = "") -> None:
    if code != 0:
        L = lib()
        msg = L.b200moe_error_string(code).decode()
        detail = L.b200moe_last_error_detail().decode()
        raise B200MoEError(f"{what}: {msg} ({code}): {detail}")


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def dtype_code(t: torch.Tensor) -> int:
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}: expected float32, bfloat16 or float16") from None


_status = {}


def status_word(device: torch.device) -> torch.Tensor:
    """One int32 per device that kernels write when they give up on a bounded wait or see a bad index."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status[key] = t
    return t


def check_status(device: torch.device) -> None:
    """Synchronises the current stream and raises if a kernel reported a device-side failure."""
    check(lib().b200moe_check_status(ptr(status_word(device)), stream_ptr(device)), "device status")


def set_engine(engine: int) -> int:
    return lib().b200moe_set_engine(engine)


def set_option(option: int, value: int) -> None:
    check(lib().b200moe_set_option(option, value), "set_option")


def get_option(option: int) -> int:
    return lib().b200moe_get_option(option)


def launch_count() -> int:
    return lib().b200moe_launch_count()
