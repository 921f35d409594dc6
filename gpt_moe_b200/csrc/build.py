"""In-tree build of the CUDA extension.

`.cu` files are compiled by nvcc for sm_100a only (`-gencode arch=compute_100a,code=sm_100a
-lineinfo`); they include no torch headers, so each compiles in seconds.  The two binding files
are compiled by g++ against torch's headers.  Everything is linked into
`gpt_moe_b200/_C.so`, which is imported as a regular Python extension module.  Object files are
cached by a hash of source + flags, so rebuilding after an edit recompiles only what changed.
nvcc cross-compiles, so this runs on a machine without a GPU.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sysconfig
from concurrent.futures import ThreadPoolExecutor

CSRC = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(CSRC)
BUILD = os.path.join(CSRC, "build_checked" if os.environ.get("GM_CHECK_BOUNDS", "0") == "1" else "build")
TARGET = os.path.join(PKG, "_C_checked.so" if os.environ.get("GM_CHECK_BOUNDS", "0") == "1" else "_C.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
# --use_fast_math only where the arithmetic is an exponential / reciprocal inside a softmax or a GEMM epilogue; the
# optimizer, normalisation, loss and quantisation kernels keep IEEE division and square root (they name the fast
# intrinsics they want explicitly)
FAST_MATH_DIRS = ("gemm", "attention")
# GM_CHECK_BOUNDS=1 in the environment builds the checked variant (`_C_checked.so`): every guarded index is tested, an
# out-of-range access is skipped and recorded in the status word (code 9xx) instead of touching memory
CHECKED = os.environ.get("GM_CHECK_BOUNDS", "0") == "1"


def _sources():
    cu, cpp = [], []
    for folder, _, files in os.walk(CSRC):
        if os.path.relpath(folder, CSRC).startswith("build"):
            continue
        for name in sorted(files):
            path = os.path.join(folder, name)
            if name.endswith(".cu"):
                cu.append(path)
            elif name.endswith(".cpp"):
                cpp.append(path)
    return cu, cpp


def _headers_digest() -> str:
    h = hashlib.sha256()
    for folder, _, files in os.walk(CSRC):
        if os.path.relpath(folder, CSRC).startswith("build"):
            continue
        for name in sorted(files):
            if name.endswith((".h", ".cuh")):
                with open(os.path.join(folder, name), "rb") as f:
                    h.update(f.read())
    return h.hexdigest()


def source_digest() -> str:
    """Digest of every source and header: the loader compares it with the stamp written at build time."""
    h = hashlib.sha256(_headers_digest().encode())
    for group in _sources():
        for path in group:
            with open(path, "rb") as f:
                h.update(f.read())
    return h.hexdigest()


def _compile(cmd, src, obj, digest_key):
    stamp = obj + ".hash"
    if os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == digest_key:
        return
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"compilation failed: {' '.join(cmd)}\n{result.stdout}\n{result.stderr}")
    with open(stamp, "w") as f:
        f.write(digest_key)


def build(verbose: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension
    os.makedirs(BUILD, exist_ok=True)
    cu, cpp = _sources()
    headers = _headers_digest()
    cuda_home = cpp_extension.CUDA_HOME or "/usr/local/cuda"
    nvcc = os.path.join(cuda_home, "bin", "nvcc")
    includes = [f"-I{p}" for p in cpp_extension.include_paths(device_type="cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    ext_name = "_C_checked" if CHECKED else "_C"
    cxx_flags = ["-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", f"-DTORCH_EXTENSION_NAME={ext_name}",
                 "-DTORCH_API_INCLUDE_EXTENSION_H", "-Wno-deprecated-declarations"] + (["-DGM_CHECK_BOUNDS=1"] if CHECKED else [])
    jobs, objects = [], []
    for src in cu:
        obj = os.path.join(BUILD, os.path.relpath(src, CSRC).replace(os.sep, "_") + ".o")
        objects.append(obj)
        extra = ["--use_fast_math"] if os.path.relpath(src, CSRC).split(os.sep)[0] in FAST_MATH_DIRS else []
        if CHECKED:
            extra.append("-DGM_CHECK_BOUNDS=1")
        cmd = [nvcc] + NVCC_FLAGS + extra + [f"-I{CSRC}", "-c", src, "-o", obj]
        key = hashlib.sha256((open(src).read() + headers + " ".join(cmd)).encode()).hexdigest()
        jobs.append((cmd, src, obj, key))
    for src in cpp:
        obj = os.path.join(BUILD, os.path.relpath(src, CSRC).replace(os.sep, "_") + ".o")
        objects.append(obj)
        cmd = ["g++"] + cxx_flags + includes + [f"-I{CSRC}", "-c", src, "-o", obj]
        key = hashlib.sha256((open(src).read() + headers + " ".join(cmd)).encode()).hexdigest()
        jobs.append((cmd, src, obj, key))
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        for future in [pool.submit(_compile, *job) for job in jobs]:
            future.result()
    lib_dirs = cpp_extension.library_paths(device_type="cuda")
    link = ["g++", "-shared", "-o", TARGET] + objects + [f"-L{d}" for d in lib_dirs] + \
           [f"-Wl,-rpath,{d}" for d in lib_dirs] + ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    result = subprocess.run(link, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"link failed:\n{result.stderr}")
    with open(os.path.join(BUILD, "stamp.txt"), "w") as f:
        f.write(source_digest())
    if verbose:
        print(f"built {TARGET}")
    return TARGET


if __name__ == "__main__":
    build(verbose=True)
