"""Builds and loads the package's CUDA library (sm_100a only) and wraps its C entry
points.  There is no other implementation behind these calls: if the library cannot
be built or loaded, or the device is not sm_100, the call fails loudly.

The library is built in-tree (`csrc/_build/`) by nvcc at the first call that needs it
and rebuilt when a source or flag changed; when the tree is not writable it is built
in a per-user folder under the system's temporary directory.

With GGUF_RS_CLI_B200_STAMPS=1 in the environment a second library is built beside it
(`csrc/_build_stamps/`, -DGB_STAMPS) whose kernels write time stamps where they are asked
to (csrc/stamps.cuh, bin/kernel_stamps); the ordinary library has none of that code.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB_NAME = "libgguf_rs_cli_b200.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
STAMPS = os.environ.get("GGUF_RS_CLI_B200_STAMPS") == "1"
if STAMPS:
    NVCC_FLAGS = NVCC_FLAGS + ["-DGB_STAMPS"]
BUILD_DIR = "_build_stamps" if STAMPS else "_build"

_lib = None
_lock = threading.Lock()


class NativeError(RuntimeError):
    """The CUDA library is missing, cannot be built, or an entry point reported an error."""


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise NativeError("nvcc was not found (PATH, $NVCC, /usr/local/cuda/bin): the CUDA library cannot be built, "
                      "and there is no other implementation to fall back to")


def _stamp() -> str:
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()


def _build_dir() -> str:
    d = os.path.join(CSRC, BUILD_DIR)
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        open(probe, "w").close()
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"gguf_rs_cli_b200-{os.getuid()}", BUILD_DIR)
        os.makedirs(d, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[gguf_rs_cli_b200] {msg}", file=sys.stderr, flush=True)


def build(verbose: bool = True, force: bool = False) -> str:
    """Compiles every csrc/*.cu for sm_100a and links the shared library.  Returns its path."""
    bdir = _build_dir()
    lib, stamp_file, stamp = os.path.join(bdir, LIB_NAME), os.path.join(bdir, "stamp"), _stamp()
    if not force and os.path.exists(lib) and os.path.exists(stamp_file) and open(stamp_file).read() == stamp:
        return lib
    nvcc = _nvcc()
    srcs = sources()
    if verbose:
        _say(f"building {LIB_NAME} from {len(srcs)} sources with {nvcc} (first call only)")
    t0 = time.time()

    def compile_one(src):
        obj = os.path.join(bdir, src[:-3] + ".o")
        cmd = [nvcc] + NVCC_FLAGS + ["-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
        p = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        while True:
            try:
                out, _ = p.communicate(timeout=15)
                break
            except subprocess.TimeoutExpired:
                if verbose:
                    _say(f"  still compiling {src} ({time.time() - t0:.0f}s)")
        if p.returncode != 0:
            raise NativeError(f"nvcc failed on {src}:\n{out}")
        if verbose:
            _say(f"  compiled {src} ({time.time() - t0:.0f}s)")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, srcs))
    tmp = lib + f".{os.getpid()}.tmp"
    p = subprocess.run([nvcc, "-shared", "-o", tmp] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise NativeError(f"linking {LIB_NAME} failed:\n{p.stdout}")
    os.replace(tmp, lib)
    with open(stamp_file, "w") as f:
        f.write(stamp)
    if verbose:
        _say(f"built {lib} in {time.time() - t0:.0f}s")
    return lib


_P, _I, _L, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float

_SIGNATURES = {
    "gb_device_arch": [],
    "gb_sm_count": [],
    "gb_set_pdl": [_I],
    "gb_embed": [_P, _I, _P, _I, _I, _I, _P, _P],
    "gb_embed_shadow": [_P, _I, _P, _I, _I, _I, _P, _P, _P, _P],
    "gb_gemm_tc_fused": [_P, _L, _P, _L, _P, _I, _P, _I, _L, _I, _I, _I, _P, _P, _I, _I, _I, _P, _I, _I, _F, _P, _P, _P, _L, _P],
    "gb_add_rmsnorm": [_P, _P, _I, _I, _L, _P, _I, _I, _P, _I, _F, _P, _I, _I, _P],
    "gb_rope_kv_write": [_P, _P, _P, _I, _L, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P, _I, _I, _P, _P, _I, _P],
    "gb_swiglu": [_P, _L, _P, _I, _I, _I, _P],
    "gb_zero_rows": [_P, _P, _I, _I, _P],
    "gb_gemm_generic": [_P, _I, _L, _P, _I, _L, _P, _I, _P, _I, _L, _I, _I, _I, _P],
    "gb_attention_generic": [_P, _I, _L, _P, _I, _L, _I, _I, _I, _I, _P, _P, _P, _I, _I, _P, _P, _I, _I, _F, _P],
    "gb_sample": [_P, _L, _I, _I, _P, _P, _F, _I, _F, _F, _P, _P, _P, _P],
    "gb_gemm_tc": [_P, _L, _P, _L, _P, _I, _P, _I, _L, _I, _I, _I, _P, _P, _I, _I, _I, _P],
    "gb_gemm_tc_tile": [_I],
    "gb_gemm_tc_set_mode": [_I],
    "gb_gemm_tc_set_pair": [_I],
    "gb_gemm_tc_set_tile": [_I],
    "gb_gemm_tc_ctas": [_I, _I, _I, _I],
    "gb_gemm_tc_scratch_floats": [_I, _I, _I, _I],
    "gb_gemm_tc_supported": [_P, _L, _P, _L, _I],
    "gb_attention_decode": [_P, _L, _P, _L, _I, _I, _I, _I, _P, _P, _P, _I, _I, _P, _P, _I, _F, _I, _P, _P, _I, _P],
    "gb_attention_decode_mma": [_P, _L, _P, _L, _I, _I, _I, _I, _P, _P, _P, _I, _I, _P, _P, _I, _F, _I, _P, _P, _I, _P],
    "gb_attention_decode_mma_rope": [_P, _P, _P, _L, _P, _L, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P, _I, _I, _P, _P, _I, _F, _I,
                                     _P, _P, _I, _P],
    "gb_attention_decode_mma_supported": [_I, _I, _I],
    "gb_attention_decode_set_pages_kernel": [_I],
    "gb_attention_decode_set_two_warps": [_I],
    "gb_attention_decode_set_stamps": [_P],
    "gb_gemm_tc_set_stamps": [_P, _I, _I],
    "gb_attention_decode_scratch_floats": [_I, _I, _I, _I],
    "gb_attention_decode_supported": [_I, _I, _I],
    "gb_attention_prefill": [_P, _L, _P, _L, _I, _I, _I, _P, _I, _P, _P, _P, _P, _I, _I, _P, _P, _I, _F, _P],
    "gb_attention_prefill_supported": [_I, _I, _I],
    "gb_attention_prefill_tile": [],
    "gb_attention_prefill_tc": [_P, _L, _P, _L, _I, _I, _I, _I, _P, _I, _P, _P, _P, _P, _I, _I, _P, _P, _L, _I, _F, _P],
    "gb_attention_prefill_tc_supported": [_I, _I, _I],
    "gb_attention_prefill_tc_tile": [],
    "gb_attention_tc_status": [],
    "gb_attention_tc_status_clear": [],
    "gb_tc_status": [],
    "gb_tc_status_clear": [],
}
_RESTYPES = {"gb_gemm_tc_scratch_floats": ctypes.c_longlong, "gb_attention_decode_scratch_floats": ctypes.c_longlong}


def register_signature(name: str, argtypes) -> None:
    """For entry points added by later files of csrc/."""
    _SIGNATURES[name] = list(argtypes)
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.argtypes, fn.restype = list(argtypes), ctypes.c_int


def library():
    """The loaded library; builds it first if needed."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = build()
                try:
                    lib = ctypes.CDLL(path)
                except OSError as e:
                    raise NativeError(f"cannot load {path}: {e}") from None
                lib.gb_last_error.restype = ctypes.c_char_p
                lib.gb_last_error.argtypes = []
                for name, argtypes in _SIGNATURES.items():
                    try:
                        fn = getattr(lib, name)
                    except AttributeError:
                        raise NativeError(f"{path} lacks the entry point {name}; rebuild it") from None
                    fn.argtypes, fn.restype = argtypes, _RESTYPES.get(name, ctypes.c_int)
                _lib = lib
    return _lib


_launches = 0
# kernels launched by one call of an entry point, where that is not one
KERNELS_PER_CALL = {}


def launch_count() -> int:
    """Kernels this process has launched through the library so far."""
    return _launches


def count_launches(n: int) -> None:
    """Adds the kernels of a replayed graph to the count."""
    global _launches
    _launches += n


def call(name: str, *args) -> None:
    """Calls an entry point; a non-zero return becomes a NativeError with its message."""
    global _launches
    lib = library()
    if getattr(lib, name)(*args):
        raise NativeError(lib.gb_last_error().decode("utf-8", "replace"))
    _launches += KERNELS_PER_CALL.get(name, 1)


_checked_device = False


def require_device() -> None:
    """Fails unless a CUDA device of compute capability 10.0 is current."""
    global _checked_device
    if _checked_device:
        return
    import torch
    if not torch.cuda.is_available():
        raise NativeError("no CUDA device: this package runs on an NVIDIA B200 (sm_100) only and has no CPU path")
    arch = library().gb_device_arch()
    if arch != 100:
        raise NativeError(f"the current device has compute capability {arch / 10:.1f}; the kernels are built for "
                          f"sm_100a only")
    _checked_device = True


DTYPE_CODE = {"float32": 0, "bfloat16": 1}


def dtype_code(t) -> int:
    import torch
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise NativeError(f"tensors of {t.dtype} cannot be given to the kernels (float32 or bfloat16)")


def ptr(t) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream
