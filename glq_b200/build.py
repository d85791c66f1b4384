"""Build libglq_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libglq_b200.so")
SOURCES = ["glqb_api.cu", "glqb_gemm_inst.cu", "glqb_fused.cu", "glqb_noalloc.cu", "glqb_moe.cu", "glqb_comm.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared", "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: libglq_b200.so cannot be built")
    return exe


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    for root, _, files in os.walk(CSRC):
        for f in files:
            if os.path.getmtime(os.path.join(root, f)) > t:
                return True
    hdr = os.path.join(os.path.dirname(HERE), "include", "glq_b200.h")
    return os.path.exists(hdr) and os.path.getmtime(hdr) > t


def build(force: bool = False, verbose: bool = False, out: str = LIB, defines=()) -> str:
    """``out`` / ``defines`` build a tuning variant beside the default library (see GLQB_LIB_PATH).
    The translation units are compiled side by side, then linked."""
    if not force and out == LIB and not needs_build():
        return LIB
    import tempfile
    from concurrent.futures import ThreadPoolExecutor
    flags = [f for f in NVCC_FLAGS if f != "-shared"] + [f"-D{d}" for d in defines]
    if verbose:
        flags += ["-Xptxas", "-v"]
    with tempfile.TemporaryDirectory(prefix="glqb_build_") as tmp:
        def compile_one(src):
            obj = os.path.join(tmp, src.replace(".cu", ".o"))
            res = subprocess.run([_nvcc(), *flags, "-c", os.path.join(CSRC, src), "-o", obj],
                                 capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}:\n" + res.stdout + res.stderr)
            return obj, res.stderr
        with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
            results = list(pool.map(compile_one, SOURCES))
        if verbose:
            for _, log in results:
                print(log)
        res = subprocess.run([_nvcc(), "-shared", "-Xcompiler", "-fPIC", *[o for o, _ in results], "-o", out],
                             capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("link failed:\n" + res.stdout + res.stderr)
    return out


if __name__ == "__main__":
    _defs = [a[2:] for a in sys.argv[1:] if a.startswith("-D")]
    _out = next((a.split("=", 1)[1] for a in sys.argv[1:] if a.startswith("--out=")), LIB)
    print(build(force="--force" in sys.argv or bool(_defs), verbose="-v" in sys.argv, out=_out, defines=_defs))
