"""Test helpers for the reference's snapshot files (the reader that ships is C++: include/srf_testbed.hpp).

A snapshot is the model configuration (the JSON of `load_model_config`) serialised as msgpack with one extra
section, written by Testbed::save_snapshot and read by Testbed::load_snapshot (internal/testbed.cu:135-171):

    snapshot.scene_scale    number
    snapshot.scene_offset   [x, y, z]                       (internal/utils/json_binding.h:13-26)
    snapshot.density_grid   binary: cells * cascades fp32, Morton order
    snapshot.n_params, snapshot.params_type ("__half" | "float"), snapshot.params_binary
                            the trainer's parameter vector, in the network's order
                            (internal/network/ngp_network.h:491-536): density MLP, colour MLP, hash grid
                            (the spherical-harmonics encoding has no parameters)
    snapshot.optimizer      optional, ignored here

The trainer is the reference's tiny-cuda-nn dependency, which is not part of its tree; the three field names
and the parameter layout restated here (row-major `[out][in]` weight matrices layer after layer, the last
layer padded to 16 outputs; hash-grid levels one after the other, each `hashgrid_layout` entries of
n_features halves) are that library's published format.  No snapshot written by the reference was available
to check against: the writer below produces the same structure and the tests are round trips.
"""
from __future__ import annotations

import numpy as np

from . import abi

DENSITY_MLP_PARAMS = 64 * 32 + 16 * 64
RGB_MLP_PARAMS = 64 * 32 + 64 * 64 + 16 * 64


def table_entries(cfg: abi.Config) -> int:
    """Number of hash-grid parameters (halves) of a configuration."""
    from .synth import hashgrid_layout
    offsets, _, _ = hashgrid_layout(cfg)
    return int(offsets[-1]) * cfg.n_features_per_level


def read_snapshot(path: str) -> dict:
    """Parses a snapshot file with the C++ host's msgpack reader into dict(model_config, scene_scale, scene_offset,
    density_grid, density_mlp, rgb_mlp, hash_table) with fp32 grid and fp16 parameters: a test helper that mirrors
    srf_host::parse_snapshot (include/srf_testbed.hpp), which is what `pyngp.Testbed.load_snapshot` runs."""
    from . import pyngp
    with open(path, "rb") as f:
        model_config = pyngp.parse_msgpack(f.read())
    if not isinstance(model_config, dict) or "snapshot" not in model_config:
        raise RuntimeError("ERROR in loading snapshot.")
    snap = model_config["snapshot"]
    grid = np.frombuffer(snap["density_grid"], dtype=np.float32).copy()
    ptype = snap.get("params_type", "__half")
    raw = snap["params_binary"]
    if ptype == "float":
        params = np.frombuffer(raw, dtype=np.float32).astype(np.float16)
    elif ptype == "__half":
        params = np.frombuffer(raw, dtype=np.float16).copy()
    else:
        raise RuntimeError(f"snapshot parameters of type {ptype!r} are not supported")
    n_params = int(snap.get("n_params", params.size))
    if params.size < n_params or n_params < DENSITY_MLP_PARAMS + RGB_MLP_PARAMS:
        raise RuntimeError("snapshot parameter vector is shorter than n_params")
    params = params[:n_params]
    a, b = DENSITY_MLP_PARAMS, DENSITY_MLP_PARAMS + RGB_MLP_PARAMS
    return dict(model_config={k: v for k, v in model_config.items() if k != "snapshot"},
                scene_scale=float(snap["scene_scale"]),
                scene_offset=np.asarray(snap["scene_offset"], np.float32).reshape(3),
                density_grid=grid, density_mlp=params[:a].copy(), rgb_mlp=params[a:b].copy(),
                hash_table=params[b:].copy())


def write_snapshot(path: str, model_config: dict, density_grid, density_mlp, rgb_mlp, hash_table,
                   scene_scale=1.0, scene_offset=(0.5, 0.5, 0.5), full_precision=False):
    """Writes the structure Testbed::save_snapshot writes (no optimizer state)."""
    from . import pyngp
    params = np.concatenate([np.asarray(density_mlp, np.float16).reshape(-1), np.asarray(rgb_mlp, np.float16).reshape(-1),
                             np.asarray(hash_table, np.float16).reshape(-1)])
    doc = dict(model_config)
    doc["snapshot"] = {
        "n_params": int(params.size),
        "params_type": "float" if full_precision else "__half",
        "params_binary": (params.astype(np.float32) if full_precision else params).tobytes(),
        "density_grid": np.ascontiguousarray(density_grid, np.float32).tobytes(),
        "scene_scale": float(scene_scale),
        "scene_offset": [float(x) for x in scene_offset],
    }
    with open(path, "wb") as f:
        f.write(pyngp.write_msgpack(doc))
