"""Builds and loads the CUDA kernel library.

The sources under `csrc/` are compiled for sm_100a with nvcc at the first call
and linked into one shared library with a plain C interface, loaded through
ctypes.  The result is kept in `_build/` inside the package (or, when that is
not writable, in a per-user folder under the system's temporary directory) and
reused while the sources are unchanged.  There is no fallback: without the
library, or without nvcc to build it, loading fails with an error.
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

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(_PKG, "csrc")
LIB_NAME = "librdl_b200_kernels.so"
ABI_VERSION = 11

# fast math is never enabled: the 32-bit path relies on exact tanhf/expf/sqrtf and plain FMA
NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC"]


class KernelLibraryError(RuntimeError):
    pass


def _log(msg):
    print(f"[rust_deeplearning_b200] {msg}", file=sys.stderr, flush=True)


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _fingerprint():
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()[:16]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    return None


def _build_dirs():
    yield os.path.join(_PKG, "_build")
    yield os.path.join(tempfile.gettempdir(), f"rust_deeplearning_b200_build_{os.getuid()}")


def _trusted(path):
    """Loading a library runs its code in this process.  The folder inside the package is trusted as the
    package's own Python files are.  The fallback folder lies under the shared temporary directory, where
    another user could have put a folder of that name first: it, and a library in it, must belong to this
    user and be writable by nobody else."""
    if os.path.commonpath([os.path.abspath(path), _PKG]) == _PKG:
        return True
    try:
        st = os.stat(path)
    except OSError:
        return False
    return st.st_uid == os.getuid() and not (st.st_mode & 0o022)


def _writable_dir(path):
    try:
        os.makedirs(path, mode=0o700, exist_ok=True)
        if not _trusted(path):
            return False
        probe = os.path.join(path, f".probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def _compile(build_dir, stamp):
    nvcc = _nvcc()
    if nvcc is None:
        raise KernelLibraryError(
            "the CUDA kernel library is not built and nvcc was not found (looked at $NVCC, PATH and "
            "/usr/local/cuda/bin); there is no fallback path")
    srcs = _sources()
    _log(f"compiling {len(srcs)} CUDA sources for sm_100a into {build_dir} (first call only)")
    t0 = time.time()
    done = []
    lock = threading.Lock()
    # nvcc must not depend on the caller's HOME or working directory
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())

    def one(src):
        obj = os.path.join(build_dir, src[:-3] + f".{stamp}.o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env, cwd=build_dir)
        if r.returncode != 0:
            raise KernelLibraryError(f"nvcc failed on {src}:\n{r.stdout}")
        with lock:
            done.append(src)
            _log(f"  compiled {src} ({len(done)}/{len(srcs)}, {time.time() - t0:.0f} s)")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        objs = list(pool.map(one, srcs))
    out = os.path.join(build_dir, LIB_NAME)
    tmp = out + f".{os.getpid()}.tmp"
    r = subprocess.run([nvcc, "-shared", "-o", tmp, *objs], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                       text=True, env=env, cwd=build_dir)
    if r.returncode != 0:
        raise KernelLibraryError(f"linking {LIB_NAME} failed:\n{r.stdout}")
    os.replace(tmp, out)
    with open(os.path.join(build_dir, "stamp"), "w") as f:
        f.write(stamp)
    for o in objs:
        try:
            os.remove(o)
        except OSError:
            pass
    _log(f"built {LIB_NAME} in {time.time() - t0:.0f} s")
    return out


def build(force: bool = False) -> str:
    """Make sure the library is built for the current sources; return its path."""
    stamp = _fingerprint()
    for d in _build_dirs():
        lib, st = os.path.join(d, LIB_NAME), os.path.join(d, "stamp")
        if not force and os.path.isfile(lib) and os.path.isfile(st) and _trusted(d) and _trusted(lib):
            with open(st) as f:
                if f.read().strip() == stamp:
                    return lib
    for d in _build_dirs():
        if _writable_dir(d):
            return _compile(d, stamp)
    raise KernelLibraryError("no writable folder to build the CUDA kernel library in: tried " + ", ".join(_build_dirs()))


class AttentionArgs(ctypes.Structure):
    _fields_ = [
        ("dtype", ctypes.c_int), ("n_tokens", ctypes.c_int), ("n_seqs", ctypes.c_int),
        ("n_heads", ctypes.c_int), ("n_kv_heads", ctypes.c_int), ("head_dim", ctypes.c_int),
        ("score_scale", ctypes.c_float), ("softcap", ctypes.c_float), ("window", ctypes.c_int),
        ("q", ctypes.c_void_p), ("q_stride", ctypes.c_longlong),
        ("k_new", ctypes.c_void_p), ("v_new", ctypes.c_void_p), ("kv_stride", ctypes.c_longlong),
        ("out", ctypes.c_void_p), ("out_stride", ctypes.c_longlong),
        ("tok_seq", ctypes.c_void_p), ("tok_pos", ctypes.c_void_p),
        ("seq_start", ctypes.c_void_p), ("seq_past", ctypes.c_void_p), ("seq_cached", ctypes.c_void_p),
        ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p),
        ("tables", ctypes.c_void_p), ("table_width", ctypes.c_int), ("page_size", ctypes.c_int),
        ("ring_pages", ctypes.c_int),
        ("tile_seq", ctypes.c_void_p), ("tile_q0", ctypes.c_void_p), ("n_tiles", ctypes.c_int),
        ("keys_per_split", ctypes.c_int), ("max_splits", ctypes.c_int),
        ("scratch", ctypes.c_void_p), ("scratch_bytes", ctypes.c_longlong),
        ("counter_bytes", ctypes.c_longlong), ("status", ctypes.c_void_p),
        ("rope_cos", ctypes.c_void_p), ("rope_sin", ctypes.c_void_p), ("rotary_dim", ctypes.c_int), ("new_rows", ctypes.c_int),
        ("wait_cycles", ctypes.c_longlong), ("test_extra_tx", ctypes.c_int),     # filled in by the launcher
    ]


# What a kernel leaves in a step's status word when it gives up (`csrc/api.h`, RDL_FAULT_*).
FAULTS = {
    1: "embed_rows: a token id outside the vocabulary (its row is NaN)",
    3: "attention_decode: a page copy did not complete",
    4: "gemm_tc: a stage or an accumulator was not handed over",
    5: "attention_prefill_tc: a tile copy or a product did not complete",
    6: "gemm_tc (pairs of blocks): a stage or an accumulator was not handed over",
    7: "gemm_skinny: a weight copy did not complete",
}


class DeferredNormArgs(ctypes.Structure):
    """One side of a deferred norm around a few-row product (`csrc/api.h`)."""
    _fields_ = [
        ("mode", ctypes.c_int), ("sums", ctypes.c_void_p), ("n_sums", ctypes.c_int),
        ("residual", ctypes.c_void_p),
        ("w1", ctypes.c_void_p), ("w1_dtype", ctypes.c_int), ("off1", ctypes.c_float),
        ("w2", ctypes.c_void_p), ("w2_dtype", ctypes.c_int), ("off2", ctypes.c_float),
        ("branch", ctypes.c_void_p), ("scaled", ctypes.c_void_p),
        ("eps1", ctypes.c_float), ("eps2", ctypes.c_float),
        ("branch_in", ctypes.c_void_p), ("residual_in", ctypes.c_void_p), ("residual_out", ctypes.c_void_p),
        ("w_next", ctypes.c_void_p), ("w_next_dtype", ctypes.c_int), ("off_next", ctypes.c_float),
        ("scaled_next", ctypes.c_void_p),
        ("row_index", ctypes.c_void_p), ("n_out", ctypes.c_int),
    ]


NORM_BRANCH, NORM_DEFERRED = 1, 2


class SamplingArgs(ctypes.Structure):
    _fields_ = [("temperature", ctypes.c_float), ("top_k", ctypes.c_int), ("top_p", ctypes.c_float),
                ("repetition_penalty", ctypes.c_float), ("seed", ctypes.c_ulonglong)]


_P, _I, _F, _LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
_SIGNATURES = {
    "rdl_attention_plain": [ctypes.POINTER(AttentionArgs), _P],
    "rdl_attention_prefill": [ctypes.POINTER(AttentionArgs), _P],
    "rdl_attention_decode": [ctypes.POINTER(AttentionArgs), _P],
    "rdl_attention_prefill_tc": [ctypes.POINTER(AttentionArgs), _LL, _P],
    "rdl_embed_rows": [_P, _P, _I, _P, _F, _I, _I, _I, _P, _P],
    "rdl_norm_residual_norm": [_P, _I, _P, _P, _I, _F, _F, _P, _P, _I, _F, _F, _P, _I, _I, _I, _P],
    "rdl_gated_activation": [_P, _P, _I, _I, _I, _I, _P],
    "rdl_softcap_inplace": [_P, _LL, _F, _P],
    "rdl_residual_add": [_P, _P, _I, _LL, _P],
    "rdl_convert_rows": [_P, _I, _P, _I, _P, _I, _I, _P],
    "rdl_rope_cache": [_P, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _P, _P],
    "rdl_gemm_f32": [_P, _P, _P, _I, _I, _I, _P],
    "rdl_gemm_skinny": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _P, _P],
    "rdl_gemm_skinny_norm": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _F, ctypes.POINTER(DeferredNormArgs), _P, _P],
    "rdl_stream_rows": [_P, _I, _F, _P, _P, _P, _P, _I, _F, _P, _I, _I, _P],
    "rdl_gemm_tc": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _P, _P],
    "rdl_random_normal": [_P, _I, _LL, ctypes.c_ulonglong, ctypes.c_double, _P],
    "rdl_sample": [_P, _P, _P, _I, _I, ctypes.POINTER(SamplingArgs), _P, _P, _P, _P, _P, _P],
    "rdl_upload_batch": [_P, _P, _I, _P, _I, _I, _I, _P],
}

_lib = None
_lock = threading.Lock()


def load():
    """The loaded library (built first if needed).  Raises KernelLibraryError if that is impossible."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = build()
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelLibraryError(f"cannot load {path}: {e}") from None
        lib.rdl_abi_version.restype = ctypes.c_int
        if lib.rdl_abi_version() != ABI_VERSION:
            raise KernelLibraryError(f"{path} has interface version {lib.rdl_abi_version()}, expected {ABI_VERSION}")
        lib.rdl_last_error.restype = ctypes.c_char_p
        for name, args in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = ctypes.c_int
        lib.rdl_attention_decode_scratch_bytes.argtypes = [_I, _I, _I, _I, _I]
        lib.rdl_attention_decode_counter_bytes.argtypes = [_I, _I]
        lib.rdl_attention_decode_counter_bytes.restype = _LL
        lib.rdl_attention_decode_scratch_bytes.restype = _LL
        lib.rdl_sampling_uniform.argtypes = [ctypes.c_ulonglong] * 3
        lib.rdl_sampling_uniform.restype = ctypes.c_float
        lib.rdl_set_programmatic_launch.argtypes = [ctypes.c_int]
        lib.rdl_set_programmatic_launch.restype = None
        lib.rdl_set_wait_test.argtypes = [ctypes.c_int, ctypes.c_longlong, ctypes.c_int]
        lib.rdl_set_wait_test.restype = None
        if os.environ.get("RDL_PROGRAMMATIC_LAUNCH") == "0":   # ordinary launches, for comparison
            lib.rdl_set_programmatic_launch(0)
        _lib = lib
        _lib.path = path
    return _lib


class KernelError(RuntimeError):
    """A kernel launcher refused its arguments or the launch failed."""


launch_count = 0   # kernels of this library launched (or captured into a graph) so far


def check(status: int, kernels: int = 1):
    """Raise if a launcher refused or failed; otherwise count its kernels."""
    global launch_count
    if status != 0:
        raise KernelError(load().rdl_last_error().decode(errors="replace"))
    launch_count += kernels
