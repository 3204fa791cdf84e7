"""Builds baseline/_ref/libsrf_refgpu.so: the reference's own CUDA kernels for sm_100a, as a same-GPU comparator.

NOT part of the library.  The kernels are cut, by line range, out of the reference's sources where they lie
(oracle/build_ref.py holds the ranges and the reference's location), written to a temporary directory and compiled
by nvcc with its default flags together with baseline/refgpu_harness.cu and the stand-in headers under
oracle/ref_stub/.  Only the shared object (git-ignored) remains; it travels to the GPU box with the repository.
Where the reference is not mounted, build() returns the earlier build if there is one, else None.
"""
from __future__ import annotations

import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
sys.path.insert(0, str(ROOT))
from oracle import build_ref  # noqa: E402

OUT = HERE / "_ref" / "libsrf_refgpu.so"


def build(force: bool = False):
    nvcc = "/usr/local/cuda/bin/nvcc"
    if not build_ref.available() or not Path(nvcc).exists():
        return OUT if OUT.exists() else None
    deps = [HERE / "refgpu_harness.cu", HERE / "build_refgpu.py", ROOT / "oracle" / "build_ref.py", ROOT / "include" / "srf_abi.h"]
    deps += [d for d in sorted((ROOT / "oracle" / "ref_stub").rglob("*")) if d.is_file()]
    if OUT.exists() and not force and all(d.stat().st_mtime <= OUT.stat().st_mtime for d in deps):
        return OUT
    OUT.parent.mkdir(parents=True, exist_ok=True)
    with tempfile.TemporaryDirectory(prefix="srf_refgpu_") as tmp:
        build_ref.extract(Path(tmp))
        ccbin = ["-ccbin", "/usr/bin/g++"] if Path("/usr/bin/g++").exists() else []
        cmd = [nvcc] + ccbin + ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
                                "--extended-lambda", "-w", "-Xcompiler", "-fPIC", "-shared",
                                "-I", str(ROOT / "oracle" / "ref_stub"), "-I", str(build_ref.REFERENCE_ROOT), "-I", tmp,
                                str(HERE / "refgpu_harness.cu"), "-o", str(OUT), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("GPU build of the reference kernels failed:\n" + r.stdout + r.stderr)
    return OUT


if __name__ == "__main__":
    p = build(force=True)
    print(p if p else "reference not mounted: nothing built")
