"""The host runtime (block pool, cache manager, scheduler, batch builder) under AddressSanitizer and
UndefinedBehaviorSanitizer: the C++ is rebuilt with -fsanitize=address,undefined into a folder of its own and the
cache-manager and scheduler tests run on it in a child process with the sanitizer's runtime preloaded.  A read past a
block table, a page freed twice into freed memory, a signed overflow in the hashes: any of them ends the child with a
report instead of passing by luck."""
import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _compiler_with_runtime(name):
    """(compiler, path of its sanitizer runtime) for the first C++ compiler here that ships one."""
    for cxx in (os.environ.get("CXX"), shutil.which("g++"), "/usr/bin/g++", shutil.which("c++")):
        if not cxx or not os.path.isfile(cxx):
            continue
        path = subprocess.run([cxx, f"-print-file-name={name}"], capture_output=True, text=True).stdout.strip()
        if os.path.isabs(path) and os.path.isfile(path):
            return cxx, path
    return None, None


def test_cache_manager_and_scheduler_under_address_and_undefined_behaviour_sanitizers():
    cxx, asan = _compiler_with_runtime("libasan.so")
    if asan is None:
        pytest.skip("no C++ compiler with an AddressSanitizer runtime here")
    # the interpreter is not linked against the C++ runtime: without it in the preload the sanitizer cannot find the
    # `__cxa_throw` it wraps, and the first exception of the host runtime ends the process
    stdcxx = subprocess.run([cxx, "-print-file-name=libstdc++.so.6"], capture_output=True, text=True).stdout.strip()
    preload = asan + (" " + stdcxx if os.path.isabs(stdcxx) and os.path.isfile(stdcxx) else "")
    env = dict(os.environ, VOB_HOST_SANITIZE="1", CXX=cxx, LD_PRELOAD=preload,
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=0:exitcode=97", UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1:exitcode=98")
    proc = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-p", "no:cacheprovider",
                           os.path.join(ROOT, "tests", "test_cache_manager.py"), os.path.join(ROOT, "tests", "test_scheduler.py")],
                          cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    tail = (proc.stdout + proc.stderr)[-3000:]
    assert proc.returncode == 0, tail
    assert " passed" in proc.stdout and "runtime error" not in tail and "AddressSanitizer" not in tail, tail
