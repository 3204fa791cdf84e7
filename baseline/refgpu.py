"""ctypes binding of baseline/_ref/libsrf_refgpu.so: the reference's own CUDA kernels on the GPU (a comparator, not part
of the library).  The network is this library's stage entry srf_network_inference, passed as a function pointer."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import build_refgpu

_lib = None


def available() -> bool:
    try:
        return build_refgpu.build() is not None
    except Exception:
        return False


def lib():
    global _lib
    if _lib is None:
        path = build_refgpu.build()
        if path is None:
            raise RuntimeError("the reference is not mounted and baseline/_ref holds no earlier build")
        _lib = C.CDLL(str(path))
        _lib.refgpu_last_ms.restype = C.c_float
        _lib.refgpu_last_rounds.restype = C.c_uint32
        _lib.refgpu_last_network_samples.restype = C.c_uint64
    return _lib


class RefGpu:
    """One reference-kernel pipeline on the device of `renderer` (a sphericalrf_b200.testbed.Renderer, which supplies the
    network and the occupancy bitfield)."""

    def __init__(self, renderer):
        self.r = renderer
        bits = np.ascontiguousarray(renderer.download_bitfield(), np.uint8)
        self.ctx = C.c_void_p()
        rc = lib().refgpu_create(C.byref(renderer.cfg), renderer.device, bits.ctypes.data_as(C.c_void_p), C.c_size_t(bits.size), C.byref(self.ctx))
        if rc != 0:
            raise RuntimeError(f"refgpu_create failed ({rc})")
        self.network = C.cast(renderer.lib.srf_network_inference, C.c_void_p)

    def close(self):
        if getattr(self, "ctx", None):
            lib().refgpu_destroy(self.ctx)
            self.ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def render_frame_device(self, view, post, out, accum, rgba_raw=None, n_samples=None):
        """torch CUDA tensors (H*W, 4) float32 / (H*W,) int32; synchronises (the reference's loop does)."""
        p = lambda t: None if t is None else C.c_void_p(t.data_ptr())
        rc = lib().refgpu_render_frame(self.ctx, C.byref(view), C.byref(post), self.network, self.r.ctx, p(out), p(accum), p(rgba_raw), p(n_samples))
        if rc != 0:
            raise RuntimeError(f"refgpu_render_frame failed ({rc})")

    def render_frame(self, view, post, taps=True):
        import torch
        dev = torch.device("cuda", self.r.device)
        n = view.width * view.height
        out = torch.zeros((n, 4), device=dev); acc = torch.zeros((n, 4), device=dev)
        raw = torch.zeros((n, 4), device=dev) if taps else None
        ns = torch.zeros(n, dtype=torch.int32, device=dev) if taps else None
        self.render_frame_device(view, post, out, acc, raw, ns)
        res = dict(out=out.cpu().numpy(), accum=acc.cpu().numpy(), ms=self.last_ms(), rounds=int(lib().refgpu_last_rounds(self.ctx)),
                   network_samples=int(lib().refgpu_last_network_samples(self.ctx)))
        if taps:
            res["rgba_raw"] = raw.cpu().numpy(); res["n_samples"] = ns.cpu().numpy().astype(np.uint32)
        return res

    def last_ms(self):
        return float(lib().refgpu_last_ms(self.ctx))
