"""Builds libpm_b200.so (sm_100a) in-tree with nvcc.  Usage: python build.py [--force] [--verbose]"""
import hashlib
import pathlib
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = pathlib.Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "pm_b200" / "libpm_b200.so"
OBJ = HERE / "build"
SOURCES = ["abi.cu", "elementwise.cu", "ssd.cu", "gemm_simt.cu", "gemm_tc.cu", "block.cu", "lm.cu", "decode.cu", "ssd_tc.cu", "ssd_fused.cu", "ssd_pairs.cu", "gemm_bf16.cu", "gemm_tc_small.cu", "optim.cu", "dp.cu", "primitives.cu", "checkpoint.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]


def _digest():
    h = hashlib.sha256()
    for f in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) +
                    [HERE.parent / "include" / "pm_b200.h"]):
        h.update(f.name.encode()); h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force=False, verbose=False):
    OBJ.mkdir(exist_ok=True)
    stamp = OBJ / "stamp.txt"
    dig = _digest()
    if not force and OUT.exists() and stamp.exists() and stamp.read_text() == dig:
        return OUT
    srcs = [s for s in SOURCES if (CSRC / s).exists()]

    def compile_one(src):
        obj = OBJ / (src + ".o")
        cmd = ["nvcc", *NVCC_FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas"); cmd.insert(2, "-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, srcs))
    cmd = ["nvcc", "-shared", "-o", str(OUT), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    stamp.write_text(dig)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
