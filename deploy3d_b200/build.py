"""Build ``libs/libdeploy3d_b200.so`` from ``csrc/*.cu`` with nvcc for sm_100a.

The reference builds one shared library into ``deploy3d/libs/`` with CMake
(trt/CMakeLists.txt:1-19, -gencode sm_75/sm_86).  This build targets sm_100a only and needs
nothing but nvcc: one translation unit per .cu file, objects cached by content hash under
``csrc/build/``, linked with ``nvcc -shared`` (static cudart, no other dependency).

Run as ``python -m deploy3d_b200.build`` or through ``__graft_entry__.build()``.
"""
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "libs", "libdeploy3d_b200.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]
# nms3d.cu: no fused multiply-add, so the keep-set equals a strict IEEE-754 evaluation of the reference arithmetic
PER_FILE = {"nms3d.cu": ["-fmad=false"]}


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: cannot build libdeploy3d_b200.so")
    return exe


def _digest(path, flags):
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    for name in sorted(os.listdir(CSRC)) + [os.path.join("..", "..", "include", "deploy3d_b200.h")]:
        full = os.path.join(CSRC, name)
        if os.path.isfile(full) and (full == path or full.endswith((".cuh", ".h"))):
            with open(full, "rb") as f:
                h.update(f.read())
    return h.hexdigest()[:16]


def build(verbose=False, ptxas_info=False):
    """Compile and link; returns the library path. Unchanged translation units are reused."""
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    nvcc = _nvcc()
    sources = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    jobs = []
    for src in sources:
        flags = ARCH + COMMON + PER_FILE.get(src, []) + (["-Xptxas", "-v"] if ptxas_info else [])
        path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ, "%s.%s.o" % (src[:-3], _digest(path, flags)))
        jobs.append((src, path, obj, flags))

    def compile_one(job):
        src, path, obj, flags = job
        if os.path.exists(obj) and not ptxas_info:
            return obj, ""
        cmd = [nvcc] + flags + ["-c", path, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, " ".join(cmd), r.stderr))
        return obj, r.stderr

    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
        results = list(ex.map(compile_one, jobs))
    objs = [o for o, _ in results]
    if verbose or ptxas_info:
        for (src, _, _, _), (_, log) in zip(jobs, results):
            if log.strip():
                print("== %s\n%s" % (src, log))
    stamp = os.path.join(OBJ, "link.stamp")
    want = "\n".join(objs)
    if not (os.path.exists(LIB) and os.path.exists(stamp) and open(stamp).read() == want):
        cmd = [nvcc] + ARCH + ["-shared", "-o", LIB] + objs
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s" % r.stderr)
        with open(stamp, "w") as f:
            f.write(want)
    # drop objects of older source revisions
    keep = set(objs) | {stamp}
    for name in os.listdir(OBJ):
        full = os.path.join(OBJ, name)
        if full not in keep:
            os.remove(full)
    return LIB


if __name__ == "__main__":
    print(build(verbose=True, ptxas_info="--ptxas" in sys.argv))
