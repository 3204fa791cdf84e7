"""Stand-in for the reference's Python module, so that a driver written as `import pyngp as ngp`
(experiment/*/python/run.py) runs its inference half on this library with
`from sphericalrf_b200 import pyngp as ngp`.

Mirrors the names of internal/python_api.cu:43-134: the enums (with their values exported at module
level, as `export_values()` does) and `Testbed`.  Members that belong to training (`train`,
`load_training_data`, `save_snapshot`, `training_buffer`) exist and raise: the optimizer loop is not part
of this library.
"""
from __future__ import annotations

import enum

from . import abi
from .testbed import Testbed as _Testbed

Activation = enum.IntEnum("Activation", {"None": abi.ACT_NONE, "ReLU": abi.ACT_RELU, "Logistic": abi.ACT_LOGISTIC,
                                         "Exponential": abi.ACT_EXPONENTIAL})
RenderMode = enum.IntEnum("RenderMode", {"AO": abi.MODE_AO, "Shade": abi.MODE_SHADE, "Normals": abi.MODE_NORMALS,
                                         "Depth": abi.MODE_DEPTH, "Distance": abi.MODE_DISTANCE, "Cost": abi.MODE_COST})
ColorSpace = enum.IntEnum("ColorSpace", {"Linear": abi.COLOR_LINEAR, "SRGB": abi.COLOR_SRGB})
TonemapCurve = enum.IntEnum("TonemapCurve", {"Identity": abi.TONEMAP_IDENTITY, "ACES": abi.TONEMAP_ACES,
                                             "Hable": abi.TONEMAP_HABLE, "Reinhard": abi.TONEMAP_REINHARD})
LossType = enum.IntEnum("LossType", {"L2": 0, "L1": 1, "Mape": 2, "Smape": 3, "SmoothL1": 4, "LogL1": 5, "RelativeL2": 6})

for _e in (Activation, RenderMode, ColorSpace, TonemapCurve, LossType):
    for _m in _e:
        if _m.name != "None":
            globals()[_m.name] = _m


class Testbed(_Testbed):
    """`pyngp.Testbed`: configuration, camera and `render` are served by the CUDA library; the training
    members raise."""

    def __init__(self):
        super().__init__(0)
        self.loss_type = LossType.L2

    @property
    def training_buffer(self):
        raise RuntimeError("training is not part of this library: no training buffer")

    def train(self, *args, **kwargs):
        raise RuntimeError("training is not part of this library")

    def load_training_data(self, *args, **kwargs):
        raise RuntimeError("training is not part of this library")

    def save_snapshot(self, *args, **kwargs):
        raise RuntimeError("training is not part of this library: nothing to snapshot")
