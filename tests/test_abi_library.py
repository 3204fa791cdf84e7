"""The C-ABI library: it loads, exports every symbol include/srf_abi.h declares (and nothing is
declared that the Python binding does not know), and the ctypes structures have the C layout.
No compute call is made here (there is no GPU on this side)."""
import ctypes as C
import re
import shutil
import subprocess
from pathlib import Path

import pytest

from sphericalrf_b200 import abi

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "srf_abi.h"


def _declared_functions():
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(srf_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert _declared_functions() == sorted(abi.SYMBOLS)


def test_library_exports_every_declared_symbol(built_lib):
    for name in _declared_functions():
        assert hasattr(built_lib, name), name


def test_struct_layouts_match_the_header(tmp_path):
    cc = "/usr/bin/gcc" if Path("/usr/bin/gcc").exists() else shutil.which("gcc")
    if not cc:
        pytest.skip("no C compiler")
    src = tmp_path / "sz.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "srf_abi.h"\nint main(void){printf("%zu %zu %zu %zu %zu %zu %zu\\n",'
                   'sizeof(srf_config_t),sizeof(srf_view_t),sizeof(srf_post_t),sizeof(srf_frame_stats_t),'
                   'offsetof(srf_config_t,n_levels),offsetof(srf_view_t,shard_rows),offsetof(srf_frame_stats_t,ms_sampler));return 0;}\n')
    exe = tmp_path / "sz"
    subprocess.run([cc, "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    want = [C.sizeof(abi.Config), C.sizeof(abi.View), C.sizeof(abi.Post), C.sizeof(abi.FrameStats),
            abi.Config.n_levels.offset, abi.View.shard_rows.offset, abi.FrameStats.ms_sampler.offset]
    assert got == want


def test_defaults_match_the_library(built_lib):
    c = abi.Config()
    built_lib.srf_config_default(C.byref(c))
    d = abi.default_config()
    for name, _ in abi.Config._fields_:
        if name == "reserved":
            continue
        assert getattr(c, name) == getattr(d, name), name


def test_layout_query_needs_no_gpu(built_lib):
    import numpy as np
    from sphericalrf_b200 import synth
    cfg = abi.default_config()
    cfg.per_level_scale = 1.447
    off = np.zeros(17, np.uint32); res = np.zeros(16, np.uint32); sc = np.zeros(16, np.float32)
    assert built_lib.srf_hashgrid_layout(C.byref(cfg), off.ctypes.data, res.ctypes.data, sc.ctypes.data) == abi.OK
    o2, r2, s2 = synth.hashgrid_layout(cfg)
    assert np.array_equal(off, o2) and np.array_equal(res, r2) and np.array_equal(sc.view(np.uint32), s2.view(np.uint32))


def test_no_gpu_is_an_error_not_a_fallback(built_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    ctx = C.c_void_p()
    cfg = abi.default_config()
    st = built_lib.srf_create(C.byref(cfg), 0, C.byref(ctx))
    assert st == abi.ERR_CUDA and not ctx.value
    assert b"no CUDA device" in built_lib.srf_last_error(None)


def test_product_never_touches_the_oracle():
    """The library, the package and their build inputs do not reference oracle/ ."""
    for p in list((ROOT / "sphericalrf_b200").rglob("*.py")) + list((ROOT / "sphericalrf_b200" / "csrc").glob("*")) + \
            list((ROOT / "include").glob("*.h")):
        if p.is_file() and p.suffix in (".py", ".cu", ".cuh", ".h"):
            assert "oracle" not in p.read_text().replace("test oracle", "").lower() or p.name == "synth.py", p


def test_cpp_shim_compiles():
    cxx = "/usr/bin/g++" if Path("/usr/bin/g++").exists() else shutil.which("g++")
    if not cxx:
        pytest.skip("no C++ compiler")
    r = subprocess.run([cxx, "-std=c++17", "-fsyntax-only", "-Wall", "-Werror", "-I", str(ROOT / "include"), "-x", "c++", "-"],
                       input='#include "srf_shim.hpp"\nint main() { return 0; }\n', capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
