"""The command lines quoted in the profiler summaries and the documents must still parse: every `--flag` written after
`python bench.py` / `python microbench.py` is an option the script knows, and every file a summary's command names
exists in the repository.  (CPU only: the scripts are asked for their --help, nothing runs.)"""
import glob
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DOCS = sorted(glob.glob(os.path.join(ROOT, "profiles", "*.md"))) + [
    os.path.join(ROOT, name) for name in ("README.md", "DESIGN.md", "INTEGRATION.md")]


def _options(script):
    out = subprocess.run([sys.executable, os.path.join(ROOT, script), "--help"], capture_output=True, text=True,
                         timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    return set(re.findall(r"(--[a-z][a-z0-9-]*)", out.stdout))


def test_quoted_flags_exist():
    known = {"bench.py": _options("bench.py"), "microbench.py": _options("microbench.py")}
    seen = 0
    for path in DOCS:
        text = open(path).read().replace("\\\n", " ")
        for script, rest in re.findall(r"python (bench\.py|microbench\.py)([^\n`|>#]*)", text):
            for flag in re.findall(r"(--[a-z][a-z0-9-]*)", rest):
                assert flag in known[script], "%s quotes `%s %s`, which the script does not know" % (
                    os.path.basename(path), script, flag)
                seen += 1
    assert seen > 20


def test_quoted_source_files_exist():
    for path in DOCS:
        for name in re.findall(r"`((?:deploy3d_b200|tests|oracle|profiles|include)/[A-Za-z0-9_./-]+\.[a-z]+)`",
                               open(path).read()):
            if "*" in name or "<" in name:
                continue
            assert os.path.exists(os.path.join(ROOT, name)) or name.endswith(".so"), "%s names %s" % (
                os.path.basename(path), name)
