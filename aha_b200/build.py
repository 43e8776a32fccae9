"""Build libaha_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

The library has two translation units -- api.cu (entry points, the Qwen3 family's executors and kernels) and seq_engine.cu (the
layered sequence engine) -- compiled side by side into objects under aha_b200/build/ and linked into one shared object.  An object
is rebuilt only when a source is newer than it."""
import concurrent.futures
import fcntl
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libaha_b200.so")
SOURCES = [os.path.join(CSRC, "api.cu"), os.path.join(CSRC, "seq_engine.cu")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include")]


def _newest_source_mtime():
    newest = 0.0
    for d in (CSRC, os.path.join(ROOT, "include")):
        for f in os.listdir(d):
            newest = max(newest, os.path.getmtime(os.path.join(d, f)))
    return newest


def _obj(src):
    return os.path.join(OBJ, os.path.splitext(os.path.basename(src))[0] + ".o")


def needs_build():
    return not os.path.exists(LIB) or os.path.getmtime(LIB) < _newest_source_mtime()


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), file=sys.stderr)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)


def build_lib(force=False, verbose=False, only=None):
    """only: basenames of the translation units to recompile (the others' objects are reused if present)."""
    if not force and not needs_build():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    os.makedirs(OBJ, exist_ok=True)
    with open(os.path.join(OBJ, ".lock"), "w") as lock:     # two processes of a fresh checkout build once
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and only is None and not needs_build():
            return LIB
        return _build_locked(nvcc, force, verbose, only)


def _build_locked(nvcc, force, verbose, only):
    newest = _newest_source_mtime()
    todo = []
    for s in SOURCES:
        o = _obj(s)
        stale = force or not os.path.exists(o) or os.path.getmtime(o) < newest
        if only is not None:
            stale = os.path.basename(s) in only or not os.path.exists(o)
        if stale:
            todo.append([nvcc] + NVCC_FLAGS + ["-c", "-o", o, s])
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        list(ex.map(lambda c: _run(c, verbose), todo))
    tmp = LIB + ".tmp%d" % os.getpid()
    _run([nvcc, "-shared", "-o", tmp] + [_obj(s) for s in SOURCES] + ["-ldl"], verbose)
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    only = [a.split("=", 1)[1].split(",") for a in sys.argv if a.startswith("--only=")]
    print(build_lib(force="--force" in sys.argv, verbose=True, only=only[0] if only else None))
