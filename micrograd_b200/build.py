"""In-tree build of the two product libraries.

    python -m micrograd_b200.build            # incremental
    python -m micrograd_b200.build --force

``lib/libmg_cuda.so``   CUDA kernels + device C ABI (include/mg_cuda.h), compiled
                        by nvcc for sm_100a only.
``lib/libmicrograd.so`` the C++ Tensor/Linear/SGD layer (include/micrograd/*.h)
                        and its flat C binding (include/mg_tensor_c.h), linked
                        against libmg_cuda.so through an $ORIGIN rpath.

nvcc cross-compiles without a GPU, so this runs on any machine with the CUDA
toolkit.  Objects are rebuilt when their source or any header is newer.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
SRC = os.path.join(HERE, "src")
LIB = os.path.join(HERE, "lib")
OBJ = os.path.join(HERE, "build")
INCLUDE = os.path.join(ROOT, "include")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CXX = "/usr/bin/g++"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-ccbin", CXX,
              f"-I{INCLUDE}", f"-I{CSRC}", "-I/usr/include"]
# Files whose arithmetic must round every multiply and add separately, like the
# reference (built without FMA contraction).
NO_FMA = {"elementwise.cu"}
CXX_FLAGS = ["-O2", "-std=c++20", "-fPIC", "-Wall", "-Wextra", "-DMG_B200_EXTENSIONS",
             f"-I{INCLUDE}"]


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _glob(root: str, exts) -> list[str]:
    out = []
    for d, _, files in os.walk(root):
        for f in sorted(files):
            if f.endswith(tuple(exts)):
                out.append(os.path.join(d, f))
    return sorted(out)


def _run(cmd, verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError(f"build step failed: {' '.join(cmd)}")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr, flush=True)


def build_cuda(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    headers = _glob(CSRC, (".cuh", ".h")) + _glob(INCLUDE, (".h",))
    sources = _glob(CSRC, (".cu",))
    objs, jobs = [], []
    for src in sources:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or _newer(obj, [src] + headers):
            cmd = [NVCC] + ARCH + NVCC_FLAGS
            if os.path.basename(src) in NO_FMA:
                cmd += ["-fmad=false"]
            if ptxas_info:
                cmd += ["-Xptxas", "-v"]
            cmd += ["-c", src, "-o", obj]
            jobs.append(cmd)
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        list(pool.map(lambda c: _run(c, verbose or ptxas_info), jobs))
    out = os.path.join(LIB, "libmg_cuda.so")
    if force or jobs or _newer(out, objs):
        _run([NVCC] + ARCH + ["-shared", "-ccbin", CXX, "-o", out] + objs + ["-ldl"], verbose)
    return out


def build_tensor(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    headers = _glob(INCLUDE, (".h",)) + _glob(SRC, (".h",))
    sources = _glob(SRC, (".cpp",))
    objs, jobs = [], []
    for src in sources:
        rel = os.path.relpath(src, SRC).replace(os.sep, "_")
        obj = os.path.join(OBJ, "host_" + rel[:-4] + ".o")
        objs.append(obj)
        if force or _newer(obj, [src] + headers):
            jobs.append([CXX] + CXX_FLAGS + [f"-I{SRC}", "-c", src, "-o", obj])
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        list(pool.map(lambda c: _run(c, verbose), jobs))
    out = os.path.join(LIB, "libmicrograd.so")
    cuda_lib = os.path.join(LIB, "libmg_cuda.so")
    if force or jobs or _newer(out, objs + [cuda_lib]):
        _run([CXX, "-shared", "-o", out] + objs +
             [f"-L{LIB}", "-lmg_cuda", "-Wl,-rpath,$ORIGIN", "-Wl,-Bsymbolic"], verbose)
    return out


def reference_dir() -> str:
    """The reference checkout: $MICROGRAD_REFERENCE, else a sibling of this repository."""
    return os.environ.get("MICROGRAD_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")


def build_cpp_tests(force: bool = False, verbose: bool = False, reference: str | None = None):
    """C++ test binaries, all under tests/cpp/bin/:

    buckets_test       CPU-only unit tests of the data-parallel bookkeeping
                       (header-only logic, no CUDA link; run by the CPU test suite)
    api_test           this repository's own C++ API tests (GPU)
    trainer_loop       the reference trainer's per-sample loop on synthetic images (GPU)
    tensor_test_b200   the reference's test/tensor_test.cpp, compiled unchanged
                       against this backend's headers and library — only where
                       the reference tree is mounted; elsewhere the prebuilt
                       binary is used.
    main_b200          the reference's src/main.cpp, compiled unchanged.
    """
    tests = os.path.join(ROOT, "tests", "cpp")
    bindir = os.path.join(tests, "bin")
    os.makedirs(bindir, exist_ok=True)
    common = [CXX, "-O2", "-std=c++20", f"-I{INCLUDE}", f"-I{tests}"]
    link = [f"-L{LIB}", "-lmicrograd", "-lmg_cuda"]
    rpath = ["-Wl,-rpath,$ORIGIN/../../../micrograd_b200/lib"]
    lib = os.path.join(LIB, "libmicrograd.so")
    gtest = os.path.join(tests, "gtest", "gtest.h")
    built = []
    out = os.path.join(bindir, "buckets_test")
    src = os.path.join(tests, "buckets_test.cpp")
    if force or _newer(out, [src, gtest, os.path.join(INCLUDE, "micrograd", "detail", "GradBuckets.h")]):
        _run(common + [src, "-o", out], verbose)
    built.append(out)
    out = os.path.join(bindir, "api_test")
    src = os.path.join(tests, "api_test.cpp")
    if force or _newer(out, [src, lib, gtest]):
        _run(common + [src, "-o", out] + link + rpath, verbose)
    built.append(out)
    out = os.path.join(bindir, "trainer_loop")
    src = os.path.join(tests, "trainer_loop.cpp")
    if force or _newer(out, [src, lib]):
        _run(common + ["-DMG_TRAINER_RECORDED", src, "-o", out] + link + rpath, verbose)
    built.append(out)
    reference = reference or reference_dir()
    ref_test = os.path.join(reference, "test", "tensor_test.cpp")
    if os.path.exists(ref_test):
        out = os.path.join(bindir, "tensor_test_b200")
        if force or _newer(out, [ref_test, lib]):
            _run(common + [ref_test, "-o", out] + link + rpath, verbose)
        built.append(out)
        # the reference's trainer application, compiled unchanged (it needs MNIST
        # files under ./data to do anything; building it proves the API surface)
        ref_main = os.path.join(reference, "src", "main.cpp")
        out = os.path.join(bindir, "main_b200")
        if os.path.exists(ref_main) and (force or _newer(out, [ref_main, lib])):
            _run([CXX, "-O2", "-std=c++20", f"-I{INCLUDE}", ref_main, "-o", out] + link + rpath, verbose)
        built.append(out)
    return built


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cuda(force, verbose)
    build_tensor(force, verbose)
    build_cpp_tests(force, verbose)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers/spills per kernel")
    ap.add_argument("--cuda-only", action="store_true")
    a = ap.parse_args()
    build_cuda(a.force, a.verbose, a.ptxas_info)
    if not a.cuda_only:
        build_tensor(a.force, a.verbose)
        build_cpp_tests(a.force, a.verbose)
    print("built:", os.listdir(LIB))
