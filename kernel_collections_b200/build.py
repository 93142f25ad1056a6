"""Builds libxkv.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m kernel_collections_b200.build [--force] [--verbose]

Every kernel_collections_b200/csrc/*.cu is compiled to an object file under csrc/build/ (in
parallel, only when the source or a header is newer than the object) and the objects are linked
into libxkv.so next to this file.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
OBJ_DIR = os.path.join(CSRC, "build")
LIB_PATH = os.path.join(PKG_DIR, "libxkv.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC)
                  if f.endswith(".cu") and os.path.isfile(os.path.join(CSRC, f)))


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    hs.append(os.path.join(ROOT, "include", "xkv.h"))
    return hs


def _obj(src: str) -> str:
    return os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def needs_build() -> bool:
    return _stale(LIB_PATH, sources() + _headers())


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; libxkv.so cannot be built")
    return nvcc


def build(force: bool = False, verbose: bool = False, defines=(), lib_path: str = LIB_PATH, overrides=None) -> str:
    """Compile what is stale and link.  `defines` (e.g. ["XKV_TC_PROFILE"]) and another `lib_path`
    give an instrumented copy of the library next to the regular one (its objects live in their own
    directory); `overrides` maps a source's file name to another path to compile in its place."""
    overrides = dict(overrides or {})
    if not force and not defines and not overrides and not needs_build():
        return lib_path
    nvcc = find_nvcc()
    tag = "_".join(list(defines) + sorted(overrides)).replace(".", "_").replace("=", "_")
    obj_dir = OBJ_DIR if not (defines or overrides) else OBJ_DIR + "_" + tag
    os.makedirs(obj_dir, exist_ok=True)
    base = [nvcc, *NVCC_FLAGS, "-I", os.path.join(ROOT, "include"), "-I", CSRC] + [f"-D{d}" for d in defines]
    if verbose:
        base += ["-Xptxas", "-v"]
    hdrs = _headers()
    jobs = []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        src = overrides.get(os.path.basename(src), src)
        if force or _stale(obj, [src] + hdrs):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        return src, subprocess.run(base + ["-c", src, "-o", obj], capture_output=True, text=True)

    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as pool:
        results = list(pool.map(compile_one, jobs))
    failed = False
    for src, proc in results:
        if verbose or proc.returncode != 0:
            sys.stderr.write(f"--- {os.path.basename(src)}\n{proc.stdout}{proc.stderr}")
        failed = failed or proc.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed building libxkv.so")
    objs = [os.path.join(obj_dir, os.path.basename(s)[:-3] + ".o") for s in sources()]
    proc = subprocess.run([nvcc, "--shared", "-gencode", "arch=compute_100a,code=sm_100a", *objs, "-o", lib_path,
                           "-lcudart"], capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("linking libxkv.so failed")
    return lib_path


FAULT_TEST_LIB = os.path.join(PKG_DIR, "libxkv_faulttest.so")


def build_fault_test(force: bool = False) -> str:
    """The test-only copy of the library (-DXKV_FAULT_TEST): device-side waits give up after 20 ms and a
    flag bit makes one kernel's producer skip a load it announced.  tests/test_gpu_timeout.py uses it to
    run the time-out path on purpose; the regular library is not affected."""
    if not force and not _stale(FAULT_TEST_LIB, sources() + _headers()):
        return FAULT_TEST_LIB
    return build(defines=["XKV_FAULT_TEST"], lib_path=FAULT_TEST_LIB)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
