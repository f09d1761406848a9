"""Builds libbrasa_cuda.so for sm_100a with nvcc, in-tree (brasa_b200/libbrasa_cuda.so)."""

from __future__ import annotations

import concurrent.futures
import os
import pathlib
import subprocess
import sys

HERE = pathlib.Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "_build"
LIB = HERE / "libbrasa_cuda.so"
SOURCES = ["ctx.cu", "quant.cu", "gemv.cu", "ops.cu", "attn.cu", "flash_tc.cu", "gemm.cu", "gemm_tc.cu", "sample.cu", "host_util.cu", "decode_token.cu", "model.cu", "batch.cu", "tp.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
              "-Xcompiler", "-fPIC", "-diag-suppress", "550"]
# extra compiler flags for a developer's build, e.g. BRASA_NVCC_FLAGS="-DBRASA_TRACE_BUILD" (phase time stamps in the
# GEMV and whole-token kernels)
NVCC_FLAGS += os.environ.get("BRASA_NVCC_FLAGS", "").split()


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (cand == "nvcc" or pathlib.Path(cand).exists()):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target: pathlib.Path, deps: list[pathlib.Path]) -> bool:
    return not target.exists() or any(d.stat().st_mtime > target.stat().st_mtime for d in deps)


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    OBJ.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "brasa_cuda.h"]
    nvcc = _nvcc()
    jobs = []
    for name in SOURCES:
        src, obj = CSRC / name, OBJ / (name + ".o")
        if force or _stale(obj, [src] + headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        return r.stderr

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        for out in ex.map(compile_one, jobs):
            if verbose and out:
                print(out, file=sys.stderr)
    objs = [OBJ / (n + ".o") for n in SOURCES]
    if force or jobs or _stale(LIB, objs):
        tmp = LIB.with_suffix(f".{os.getpid()}.tmp")
        subprocess.check_call([nvcc, "-shared", "-o", str(tmp), *map(str, objs)])
        os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
