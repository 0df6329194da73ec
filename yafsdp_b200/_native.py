"""Build and load the native sm_100a library (``yafsdp_b200/lib/libyafsdp_b200.so``).

The library is plain CUDA C++ with an ``extern "C"`` interface (``csrc/yafsdp_b200.h``) compiled by
``nvcc`` directly and bound through :mod:`ctypes`: no torch headers, so a full rebuild takes seconds,
and the built ``.so`` sits in the source tree next to the package.

``build()`` compiles every ``csrc/*.cu`` for ``sm_100a``.  ``lib()`` returns the loaded library and
raises if it is missing while a GPU is present: the CUDA path never degrades silently to PyTorch.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import threading
from pathlib import Path

_PKG_DIR = Path(__file__).resolve().parent
_REPO_DIR = _PKG_DIR.parent
_CSRC = _REPO_DIR / "csrc"
_LIB_DIR = _PKG_DIR / "lib"
_LIB_PATH = _LIB_DIR / "libyafsdp_b200.so"
_OBJ_DIR = _LIB_DIR / "obj"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
]

# extra compiler flags, e.g. ``-DYF_DEBUG_BOUNDS`` (the pushing kernels check every peer write against the owners' slots,
# record a violation in the status word and skip the access); part of the rebuild digest
NVCC_FLAGS += [f for f in os.environ.get("YAFSDP_NVCC_FLAGS", "").split() if f]

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None


def _nvcc() -> str | None:
    cand = shutil.which("nvcc")
    if cand:
        return cand
    for root in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if root and (Path(root) / "bin" / "nvcc").exists():
            return str(Path(root) / "bin" / "nvcc")
    return None


def _sources() -> list[Path]:
    return sorted(_CSRC.glob("*.cu"))


def _digest(path: Path) -> str:
    h = hashlib.sha1()
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(path.read_bytes())
    for hdr in sorted(_CSRC.glob("*.h")) + sorted(_CSRC.glob("*.cuh")):
        h.update(hdr.read_bytes())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile ``csrc/*.cu`` to ``libyafsdp_b200.so`` (incremental: an object is rebuilt only when its
    source, a header or the flags changed)."""
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build the native library")
    _OBJ_DIR.mkdir(parents=True, exist_ok=True)
    objs: list[str] = []
    relink = force or not _LIB_PATH.exists()
    procs = []
    for src in _sources():
        obj = _OBJ_DIR / (src.stem + ".o")
        stamp = _OBJ_DIR / (src.stem + ".sha1")
        dig = _digest(src)
        objs.append(str(obj))
        if not force and obj.exists() and stamp.exists() and stamp.read_text() == dig:
            continue
        relink = True
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(_CSRC), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, stamp, dig, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, stamp, dig, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{out}")
        if verbose and out:
            print(out)
        stamp.write_text(dig)
    if relink:
        cmd = [nvcc, "-shared", "-o", str(_LIB_PATH), *objs, "-lcudart"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}")
    return _LIB_PATH


def available() -> bool:
    """True when the built library exists (it may still be unusable without a GPU)."""
    return _LIB_PATH.exists()


def loaded() -> bool:
    """True once :func:`lib` has loaded the library in this process."""
    return _lib is not None


def lib() -> ctypes.CDLL:
    """The loaded native library.  Builds it first when it is missing and ``nvcc`` is present."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not _LIB_PATH.exists():
            if _nvcc() is None:
                raise RuntimeError(
                    f"native library {_LIB_PATH} is missing and nvcc is unavailable; "
                    "run `python -c 'import __graft_entry__ as g; g.build()'` on a machine with CUDA 12.9"
                )
            build()
        _lib = ctypes.CDLL(str(_LIB_PATH))
        _declare(_lib)
        return _lib


_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_longlong
_F = ctypes.c_float


def _declare(l: ctypes.CDLL) -> None:
    sigs = {
        "yf_version": [],
        "yf_sm_count": [],
        "yf_status_read": [_P, _P, _I],
        "yf_gemm_bf16": [_P, _P, _P, _I, _I, _I, _L, _L, _L, _I, _I, _I, _I, _F, _I, _P],
        "yf_rmsnorm_fwd": [_P, _P, _P, _P, _I, _I, _F, _P],
        "yf_rmsnorm_bwd": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
        "yf_rope": [_P, _P, _I, _I, _L, _I, _I, _I, _I, _P],
        "yf_swiglu_fwd": [_P, _P, _L, _I, _P],
        "yf_swiglu_bwd": [_P, _P, _P, _L, _I, _P],
        "yf_cross_entropy": [_P, _P, _P, _I, _I, _L, _F, _P, _I, _P],
        "yf_embedding_fwd": [_P, _P, _P, _L, _I, _I, _P],
        "yf_embedding_bwd": [_P, _P, _P, _L, _I, _I, _P],
        "yf_adamw": [_P, _P, _P, _P, _P, _P, _L, _F, _F, _F, _F, _F, _I, _I, _P],
        "yf_sumsq": [_P, _L, _P, _P],
        "yf_clip_coef": [_P, _F, _P, _P, _P],
        "yf_cast_f32_to_bf16": [_P, _P, _L, _P],
        "yf_accum_bf16_to_f32": [_P, _P, _L, _F, _I, _P],
        "yf_add_bf16": [_P, _P, _P, _L, _P],
        "yf_attn_fwd": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _F, _I, _P],
        "yf_attn_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _L, _L, _L, _F, _I, _P],
        "yf_attn_bwd_noalloc": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _L, _L, _L, _F, _I, _P],
        "yf_gemm_bf16_sumsq": [_P, _P, _P, _I, _I, _I, _L, _L, _L, _I, _I, _I, _I, _F, _I, _P, _P],
        "yf_gemm_bf16_residual": [_P, _P, _P, _P, _I, _I, _I, _L, _L, _L, _L, _I, _I, _F, _I, _P],
        "yf_gemm_bf16_gathered": [_P, _P, _I, _I, _I, _L, _L, _I, _I, _P, _P, _L, _L, _I, _I, _P, _L, _P],
        "yf_gemm_bf16_scatter": [_P, _P, _I, _I, _I, _L, _L, _I, _I, _F, _P, _L, _L, _I, _I, _I, _I, _P],
        "yf_gemm_bf16_scatter_grouped": [_I, _P, _P, _P, _P, _I, _P, _P, _I, _I, _F, _P, _P, _L, _I, _I, _I, _I, _P],
        "yf_allgather_pull": [_P, _P, _L, _I, _I, _I, _P],
        "yf_reduce_scatter_pull": [_P, _P, _L, _I, _I, _F, _I, _I, _I, _P],
        "yf_reduce_scatter_pull_sumsq": [_P, _P, _L, _I, _I, _F, _I, _I, _I, _P, _P],
        "yf_reduce_scatter_mc": [_P, _P, _L, _I, _I, _F, _I, _I, _I, _P, _P],
        "yf_allgather_mc": [_P, _P, _L, _I, _I, _I, _P],
        "yf_signal_barrier": [_P, _I, _I, _I, _L, _L, _P],
        "yf_signal_pad": [_P, _I, _I, _I, _L, _L, _I, _P],
        "yf_push_flat": [_P, _L, _L, _P, _L, _I, _I, _I, _P],
        "yf_flag_wait": [_P, _L, _L, _L, _P],
        "yf_flag_set": [_P, _L, _L, _P],
        "yf_memcpy_async": [_P, _P, _L, _P],
        "yf_ipc_alloc": [_L, _P, _P],
        "yf_ipc_open": [_P, _P],
        "yf_ipc_close": [_P],
        "yf_ipc_free": [_P],
    }
    for name, args in sigs.items():
        fn = getattr(l, name, None)
        if fn is None:
            continue
        fn.argtypes = args
        fn.restype = _I
    # a symbol without a declared signature would be called with C-int arguments and truncate pointers: refuse it loudly
    import re

    header = (_CSRC / "yafsdp_b200.h")
    if header.exists():
        exported = set(re.findall(r"^int (yf_\w+)\(", header.read_text(), flags=re.M))
        missing = sorted(exported - set(sigs))
        if missing:
            raise RuntimeError(f"native functions without a ctypes signature in _native._declare: {missing}")
