"""Build ``libs/libdeploy3d_b200.so`` from ``csrc/*.cu`` with nvcc for sm_100a.

The reference builds one shared library into ``deploy3d/libs/`` with CMake
(trt/CMakeLists.txt:1-19, -gencode sm_75/sm_86).  This build targets sm_100a only and needs
nothing but nvcc: one translation unit per .cu file, objects cached by content hash under
``csrc/build/``, linked with ``nvcc -shared`` (static cudart, no other dependency).

Run as ``python -m deploy3d_b200.build`` or through ``__graft_entry__.build()``.

Tuning builds: ``python -m deploy3d_b200.build --tuning NAME -DD3D_TC_PROFILE [-DD3D_TC_NO_MMA] [-DD3D_TC_NO_COPY]``
writes ``libs/libdeploy3d_b200_NAME.so`` with the given macros defined for spconv_mm_tc.cu (per-role cycle
accounting; MMAs / row copies predicated off, which makes the results meaningless and only the timing
informative).  ``microbench.py --lib NAME`` loads such a build; nothing else does.

Checked build: ``python -m deploy3d_b200.build --checked`` writes ``libs/libdeploy3d_b200_checked.so`` with
``-DDEPLOY3D_BOUNDS_CHECK -rdc=true`` on every file: every id a kernel indexes with is range-checked and the first
violation recorded (``d3d_debug_take_bounds_violation``).  ``DEPLOY3D_B200_CHECKED=1`` in the environment makes the
package load it instead of the regular library.
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


def build(verbose=False, ptxas_info=False, tuning=None, defines=(), checked=False):
    """Compile and link; returns the library path. Unchanged translation units are reused.
    `tuning` names a tuning build (see the module docstring): `defines` apply to spconv_mm_tc.cu only."""
    os.makedirs(OBJ, exist_ok=True)
    if checked:
        tuning = "checked"
    lib = LIB if not tuning else LIB[:-3] + "_%s.so" % tuning
    os.makedirs(os.path.dirname(lib), exist_ok=True)
    nvcc = _nvcc()
    sources = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    jobs = []
    for src in sources:
        flags = ARCH + COMMON + PER_FILE.get(src, []) + (["-Xptxas", "-v"] if ptxas_info else [])
        if checked:
            flags = flags + ["-DDEPLOY3D_BOUNDS_CHECK", "-rdc=true"]
        elif tuning and src == "spconv_mm_tc.cu":
            flags = flags + list(defines)
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
    stamp = os.path.join(OBJ, "link.stamp" if not tuning else "link_%s.stamp" % tuning)
    want = "\n".join(objs)
    if not (os.path.exists(lib) and os.path.exists(stamp) and open(stamp).read() == want):
        cmd = [nvcc] + ARCH + ["-shared", "-o", lib] + objs
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s" % r.stderr)
        with open(stamp, "w") as f:
            f.write(want)
    # drop objects of older source revisions (the regular build decides; tuning builds leave the cache alone)
    if not tuning:
        keep = set(objs) | {stamp}
        for name in os.listdir(OBJ):
            full = os.path.join(OBJ, name)
            if full not in keep and not name.startswith("link_"):
                os.remove(full)
    return lib


if __name__ == "__main__":
    _tuning = sys.argv[sys.argv.index("--tuning") + 1] if "--tuning" in sys.argv else None
    print(build(verbose=True, ptxas_info="--ptxas" in sys.argv, tuning=_tuning,
                defines=[a for a in sys.argv[1:] if a.startswith("-D")], checked="--checked" in sys.argv))
