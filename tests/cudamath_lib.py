"""A second, TEST-ONLY build of the library's kernels: CUDA's own math library and nvcc's default contraction.

The shipped library defines its elementary functions itself (include/srf_canon_math.h) and is compiled with
-fmad=false so that host and device agree bit for bit.  The reference calls atan2f/asinf/cosf/__expf/__logf from the
CUDA math library and is compiled with nvcc's defaults.  This module compiles the same sources with
-DSRF_CANON_CUDA_MATH and -fmad=true into tests/_cudamath/libsrf_b200_cudamath.so, so that a GPU test can measure
how far the shipped results are from what a CUDA build of the reference's expressions computes.  Never loaded by the
package.
"""
import os
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "sphericalrf_b200" / "csrc"
OUT = Path(__file__).resolve().parent / "_cudamath"
# "fast": __expf/__logf as the reference writes them.  "accurate": the same build with expf/logf, to show how much of
# the difference is the fast intrinsics' error in 1 - exp(-sigma*dt) for small sigma*dt.
LIBS = {"fast": OUT / "libsrf_b200_cudamath.so", "accurate": OUT / "libsrf_b200_cudamath_accurate_exp.so"}

FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-DSRF_CANON_CUDA_MATH",
         "-fmad=true", "-Xcompiler", "-fPIC,-O2"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    return None


def build(variant="fast"):
    """Returns the library's path; builds it where nvcc exists, otherwise it must already be there (None if not)."""
    LIB = LIBS[variant]
    extra = ["-DSRF_CANON_CUDA_MATH_ACCURATE_EXP"] if variant == "accurate" else []
    nvcc = _nvcc()
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + sorted((ROOT / "include").glob("*.h"))
    if nvcc is None:
        return LIB if LIB.exists() else None
    newest = max(p.stat().st_mtime for p in sources + headers + [Path(__file__)])
    if LIB.exists() and LIB.stat().st_mtime >= newest:
        return LIB
    OUT.mkdir(exist_ok=True)
    ccbin = ["-ccbin", "/usr/bin/g++"] if Path("/usr/bin/g++").exists() else []
    procs, objs = [], []
    for src in sources:
        obj = OUT / (f"{variant}_{src.stem}.o")
        objs.append(str(obj))
        procs.append((src, subprocess.Popen([nvcc] + ccbin + FLAGS + extra + ["-c", str(src), "-o", str(obj)],
                                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{out}")
    r = subprocess.run([nvcc] + ccbin + ["-shared", "-o", str(LIB)] + objs + ["-lcudart"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    return LIB


def load(variant="fast"):
    from sphericalrf_b200 import abi
    path = build(variant)
    if path is None:
        return None
    return abi.load_from(path)


if __name__ == "__main__":
    for v in LIBS:
        print(build(v))
