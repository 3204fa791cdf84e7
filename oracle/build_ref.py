"""Builds oracle/_ref/libsrf_ref.so: the reference's own kernels compiled for the host.  TEST INFRASTRUCTURE.

The kernels and device functions are cut, by line range, out of the reference's source files where they lie
(the directory SRF_REFERENCE_ROOT names, or the default checkout location below), written to a temporary directory and compiled together with
oracle/ref_harness.cpp and the stand-in headers under oracle/ref_stub/.  Nothing of the reference is copied into
this repository: only the shared object under oracle/_ref/ (git-ignored) remains.  Where the reference is not
mounted, build() returns None and callers skip.

Usage: python oracle/build_ref.py [--fma]     (--fma: let gcc contract a*b+c into fused multiply-adds, the way
                                               nvcc's default -fmad=true may; written to libsrf_ref_fma.so)
"""
from __future__ import annotations

import os
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
REFERENCE_ROOT = Path(os.environ.get("SRF_REFERENCE_ROOT", "/root/reference"))

# file under internal/, first line, last line (1-based, inclusive), name of the extract
RANGES = [
    ("utils/loss.cu", 3, 98, "loss.inc"),                                  # the seven losses + loss_and_gradient
    ("sampler/occupancy_sampler.cu", 6, 863, "sampler_kernels.inc"),       # every kernel / device function of the sampler
    ("render/ray_marcher.cu", 5, 282, "marcher_kernels.inc"),              # both compositing kernels
    ("testbed.cu", 423, 477, "testbed_kernels.inc"),                       # compact_rays_kernel, shade_kernel
    ("utils/render_buffer.cu", 46, 181, "render_buffer_kernels.inc"),      # accumulate_kernel, tonemap, tonemap_kernel
]
# first and last extracted lines must look like this: a guard against a reference tree with other line numbers
EXPECT = {
    "loss.inc": ("#ifdef copysign", "}"),
    "sampler_kernels.inc": ("using namespace Eigen;", "}"),
    "marcher_kernels.inc": ("using namespace Eigen;", "}"),
    "testbed_kernels.inc": ("__global__ void compact_rays_kernel(", "}"),
    "render_buffer_kernels.inc": ("__global__ void accumulate_kernel(", "}"),
}


def available() -> bool:
    return (REFERENCE_ROOT / "internal" / "sampler" / "occupancy_sampler.cu").exists()


def lib_path(fma: bool = False) -> Path:
    return OUT_DIR / ("libsrf_ref_fma.so" if fma else "libsrf_ref.so")


def extract(tmp: Path) -> None:
    """Writes the kernel extracts (*.inc) of the mounted reference into the temporary directory `tmp`."""
    for rel, first, last, name in RANGES:
        lines = (REFERENCE_ROOT / "internal" / rel).read_text().splitlines()
        cut = lines[first - 1:last]
        head, tail = EXPECT[name]
        if not cut or not cut[0].strip().startswith(head) or cut[-1].strip() != tail:
            raise RuntimeError(f"{rel}:{first}-{last} does not hold the expected text; the reference tree differs")
        (tmp / name).write_text("\n".join(cut) + "\n")


def build(fma: bool = False, force: bool = False):
    """Returns the path of the shared object, or None when the reference is not mounted and no earlier build exists."""
    out = lib_path(fma)
    if not available():
        return out if out.exists() else None
    deps = [HERE / "ref_harness.cpp", HERE / "build_ref.py"] + sorted((HERE / "ref_stub").rglob("*"))
    deps = [d for d in deps if d.is_file()]
    if out.exists() and not force and all(d.stat().st_mtime <= out.stat().st_mtime for d in deps):
        return out
    OUT_DIR.mkdir(exist_ok=True)
    with tempfile.TemporaryDirectory(prefix="srf_ref_") as tmp:
        extract(Path(tmp))
        cxx = "/usr/bin/g++" if Path("/usr/bin/g++").exists() else "g++"
        cmd = [cxx, "-std=c++17", "-O2", "-fPIC", "-shared", "-fno-fast-math", "-fopenmp", "-w",
               "-ffp-contract=fast" if fma else "-ffp-contract=off"] + (["-mfma"] if fma else []) + [
               "-I", str(HERE / "ref_stub"), "-I", "/usr/local/cuda/include", "-I", str(REFERENCE_ROOT), "-I", tmp,
               str(HERE / "ref_harness.cpp"), "-o", str(out)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("host build of the reference kernels failed:\n" + r.stdout + r.stderr)
    return out


if __name__ == "__main__":
    p = build(fma="--fma" in sys.argv, force=True)
    print(p if p else "reference not mounted: nothing built")
