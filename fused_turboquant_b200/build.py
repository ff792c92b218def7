"""Builds libftq_b200.so (the CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

    python -m fused_turboquant_b200.build [--force] [--verbose]

The per-head_dim translation units compile in parallel.  No fast-math flag is
ever passed: the encode kernel's bit-exactness depends on IEEE arithmetic.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import re
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
OBJ_DIR = os.path.join(PKG_DIR, "build")
LIB_PATH = os.path.join(PKG_DIR, "libftq_b200.so")
# A second library for ONE test (tests/test_gpu_wait_expiry.py): the same objects, except that the
# head_dim-128 decode unit is compiled with FTQ_TEST_WAIT_EXPIRY (one page copy of one warp is
# never issued and the poll limit is small), so that a bounded wait runs out and the give-up path
# (NaN rows, status word, the context stays usable) executes.  Never loaded by the package.
TEST_LIB_PATH = os.path.join(PKG_DIR, "libftq_b200_waittest.so")
TEST_UNIT = ("ftq_attn_inst.cu", "attn_d128_waittest",
             ["-DFTQ_D=128", "-DFTQ_ONLY_BITS=4", "-DFTQ_TEST_WAIT_EXPIRY"])

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]

# (source, object suffix, extra defines)
# (the slowest units first: the pool then finishes them while the short ones fill the gaps)
UNITS = []
for _d in (256, 128, 64):
    UNITS.append(("ftq_tq_v1_inst.cu", f"tq_v1_store_d{_d}", [f"-DFTQ_D={_d}", "-DFTQ_TQ_PART=0"]))
    UNITS.append(("ftq_tq_v1_inst.cu", f"tq_v1_decode_d{_d}", [f"-DFTQ_D={_d}", "-DFTQ_TQ_PART=1"]))
for _d in (256, 128, 64):
    UNITS.append(("ftq_attn_inst.cu", f"attn_d{_d}", [f"-DFTQ_D={_d}"]))
    UNITS.append(("ftq_encode_inst.cu", f"encode_d{_d}", [f"-DFTQ_D={_d}"]))
UNITS.append(("ftq_api.cu", "api", []))


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: cannot build libftq_b200.so")


def _sources_mtime() -> float:
    m = os.path.getmtime(os.path.join(PKG_DIR, "..", "include", "ftq_b200.h"))
    for f in os.listdir(CSRC):
        m = max(m, os.path.getmtime(os.path.join(CSRC, f)))
    return m


_INCLUDE = re.compile(r'^\s*#\s*include\s+"([^"]+)"', re.M)


def _deps(path: str, seen=None) -> set:
    """The file and every project header it includes, transitively."""
    seen = set() if seen is None else seen
    path = os.path.normpath(path)
    if path in seen or not os.path.exists(path):
        return seen
    seen.add(path)
    with open(path) as f:
        text = f.read()
    for inc in _INCLUDE.findall(text):
        _deps(os.path.join(os.path.dirname(path), inc), seen)
    return seen


def _unit_stale(src: str, obj: str) -> bool:
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    return any(os.path.getmtime(d) > t for d in _deps(os.path.join(CSRC, src)))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile and link the library (and the wait-expiry test library) if missing or older than
    the sources."""
    if not force and all(os.path.exists(l) and os.path.getmtime(l) >= _sources_mtime()
                         for l in (LIB_PATH, TEST_LIB_PATH)):
        return LIB_PATH
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(unit):
        src, tag, defs = unit
        obj = os.path.join(OBJ_DIR, f"{tag}.o")
        if not force and not verbose and not _unit_stale(src, obj):
            return obj      # up to date: only units whose sources changed are recompiled
        cmd = [nvcc, *NVCC_FLAGS, *extra, *defs, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src} {defs}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, UNITS + [TEST_UNIT]))
    test_obj = objs.pop()
    for lib, members in ((LIB_PATH, objs),
                         (TEST_LIB_PATH, [test_obj if o.endswith("attn_d128.o") else o for o in objs])):
        cmd = [nvcc, "-shared", "-o", lib, *members, "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register/spill report")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
