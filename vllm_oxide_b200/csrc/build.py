"""Compiles the native parts in-tree, at first use or through `build_all()`.

Two libraries:
  * `_host`  (pybind11, g++): block pool, cache manager, scheduler, batch builder;
  * `libvob_kernels.so` (nvcc, sm_100a only, plain C entry points called through ctypes).

Objects go to `csrc/_build/`, the libraries next to the package's Python files.  A stamp
of the sources' hashes decides whether a rebuild is needed, so a fresh checkout compiles
at its first call and a changed source at the next.  Progress lines go to stderr while
the compiler runs.  Nothing is written outside the package folder (the compiler's
temporary files aside), so it works with an empty HOME.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
import threading
import time
from concurrent.futures import ThreadPoolExecutor

_HERE = os.path.dirname(os.path.abspath(__file__))
_PKG = os.path.dirname(_HERE)
_BUILD = os.path.join(_HERE, "_build")
_LOCK = threading.Lock()

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall"]


class BuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[vllm_oxide_b200 build] {msg}", file=sys.stderr, flush=True)


def _hash_files(paths, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _read(path: str) -> str:
    try:
        with open(path) as f:
            return f.read()
    except OSError:
        return ""


def _run(cmd, what: str) -> None:
    """Runs the compiler, printing a line every few seconds until it ends."""
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            _log(f"... still compiling {what} ({time.time() - t0:.0f} s)")
    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        raise BuildError(f"compiling {what} failed:\n$ {' '.join(cmd)}\n{out}")
    if os.environ.get("VOB_BUILD_VERBOSE") and out.strip():
        _log(out.strip())


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc not found: the CUDA kernels of vllm_oxide_b200 cannot be built (set NVCC)")


def host_sources():
    d = os.path.join(_HERE, "host")
    return [os.path.join(d, f) for f in sorted(os.listdir(d)) if f.endswith((".cpp", ".hpp"))]


# Sources compiled once per head size (-DVOB_HD=<n>) into a library of their own.
PER_HEAD_DIM = ("attention_decode.cu", "attention_prefill.cu", "attention_prefill_tc5.cu")
DEFAULT_HEAD_DIMS = (64, 128)


def kernel_sources(per_head_dim: bool = False):
    d = os.path.join(_HERE, "kernels")
    names = [f for f in sorted(os.listdir(d)) if f.endswith((".cu", ".cuh", ".h"))]
    names = [f for f in names if not f.endswith(".cu") or (f in PER_HEAD_DIM) == per_head_dim]
    return [os.path.join(d, f) for f in names]


SANITIZE_FLAGS = ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer", "-g", "-O1"]


def host_sanitized() -> bool:
    """VOB_HOST_SANITIZE=1: the host runtime is built with AddressSanitizer and UndefinedBehaviorSanitizer into a folder
    of its own and loaded from there (the process must have the sanitizer's runtime preloaded: see
    tests/test_host_sanitizers.py)."""
    return os.environ.get("VOB_HOST_SANITIZE", "") not in ("", "0")


def host_library_path() -> str:
    name = "_host" + sysconfig.get_config_var("EXT_SUFFIX")
    return os.path.join(_BUILD, "sanitized", name) if host_sanitized() else os.path.join(_PKG, name)


def kernel_library_path() -> str:
    return os.path.join(_PKG, "libvob_kernels.so")


def attention_library_path(head_dim: int) -> str:
    return os.path.join(_PKG, f"libvob_attn_hd{head_dim}.so")


def build_host(force: bool = False) -> str:
    import pybind11
    with _LOCK:
        os.makedirs(_BUILD, exist_ok=True)
        out = host_library_path()
        os.makedirs(os.path.dirname(out), exist_ok=True)
        flags = CXX_FLAGS + (SANITIZE_FLAGS if host_sanitized() else [])
        stamp_path = os.path.join(_BUILD, "host_sanitized.stamp" if host_sanitized() else "host.stamp")
        stamp = _hash_files(host_sources(), " ".join(flags))
        if not force and os.path.isfile(out) and _read(stamp_path) == stamp:
            return out
        cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
        if not cxx:
            raise BuildError("no C++ compiler found for the host runtime (set CXX)")
        _log("compiling the host runtime (block pool, cache manager, scheduler) ...")
        tmp = out + f".tmp{os.getpid()}"
        cmd = [cxx, *flags, f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}",
               os.path.join(_HERE, "host", "bindings.cpp"), "-o", tmp]
        _run(cmd, "host runtime")
        os.replace(tmp, out)
        with open(stamp_path, "w") as f:
            f.write(stamp)
        _log("host runtime ready")
        return out


def _build_cuda_library(out: str, srcs, tag: str, defines, what: str, force: bool) -> str:
    with _LOCK:
        os.makedirs(_BUILD, exist_ok=True)
        flags = NVCC_FLAGS + list(defines)
        headers = [s for s in srcs if not s.endswith(".cu")]
        cus = [s for s in srcs if s.endswith(".cu")]
        header_hash = _hash_files(headers, " ".join(flags))
        todo, objs, stamps = [], [], []
        for cu in cus:
            obj = os.path.join(_BUILD, os.path.basename(cu)[:-3] + tag + ".o")
            objs.append(obj)
            stamp = _hash_files([cu], header_hash)
            stamps.append(stamp)
            if force or not os.path.isfile(obj) or _read(obj + ".stamp") != stamp:
                todo.append((cu, obj, stamp))
        link_stamp = hashlib.sha256("".join(stamps).encode()).hexdigest()
        link_stamp_path = os.path.join(_BUILD, os.path.basename(out) + ".stamp")
        if not todo and os.path.isfile(out) and _read(link_stamp_path) == link_stamp:
            return out
        nvcc = _nvcc()
        if todo:
            _log(f"compiling {len(todo)} CUDA source file(s) of {what} for sm_100a (first call only) ...")

            def compile_one(item):
                cu, obj, stamp = item
                _run([nvcc, *flags, f"-I{os.path.join(_HERE, 'kernels')}", "-c", cu, "-o", obj], os.path.basename(cu))
                with open(obj + ".stamp", "w") as f:
                    f.write(stamp)
                _log(f"compiled {os.path.basename(cu)}")
            with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
                list(ex.map(compile_one, todo))
        tmp = out + f".tmp{os.getpid()}"
        _run([nvcc, "-shared", "-o", tmp, *objs, "-lcudart"], os.path.basename(out) + " (link)")
        os.replace(tmp, out)
        with open(link_stamp_path, "w") as f:
            f.write(link_stamp)
        _log(f"{what} ready")
        return out


def build_kernels(force: bool = False) -> str:
    return _build_cuda_library(kernel_library_path(), kernel_sources(False), "", [], "the CUDA kernels", force)


def build_attention(head_dim: int, force: bool = False) -> str:
    """The tensor-core attention kernels for one head size (a multiple of 16, at most 256)."""
    if head_dim % 16 or not 16 <= head_dim <= 256:
        raise BuildError(f"the tensor-core attention kernels take head sizes in steps of 16 up to 256, not {head_dim}")
    return _build_cuda_library(attention_library_path(head_dim), kernel_sources(True), f"_hd{head_dim}",
                               [f"-DVOB_HD={head_dim}"], f"the attention kernels for head size {head_dim}", force)


def build_all(force: bool = False, head_dims=None) -> None:
    build_host(force)
    build_kernels(force)
    for hd in head_dims or DEFAULT_HEAD_DIMS:
        build_attention(hd, force)
