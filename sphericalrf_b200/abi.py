"""ctypes view of include/srf_abi.h: structures, enumerators and the loader of libsrf_b200.so.

The library is the product; there is no Python or CPU fallback.  `load()` raises when the
shared object is missing or lacks a declared symbol.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

ABI_VERSION = 1

# status codes
OK, ERR_ARG, ERR_CUDA, ERR_CAPACITY, ERR_TIMEOUT, ERR_STATE = range(6)

# enumerators (order of internal/utils/common.h:61-115 in the reference)
ACT_NONE, ACT_RELU, ACT_LOGISTIC, ACT_EXPONENTIAL = range(4)
MODE_AO, MODE_SHADE, MODE_NORMALS, MODE_DEPTH, MODE_DISTANCE, MODE_COST = range(6)
COLOR_LINEAR, COLOR_SRGB, COLOR_VISPOSNEG = range(3)
TONEMAP_IDENTITY, TONEMAP_ACES, TONEMAP_HABLE, TONEMAP_REINHARD = range(4)
LOSS_L2, LOSS_L1, LOSS_MAPE, LOSS_SMAPE, LOSS_SMOOTH_L1, LOSS_LOG_L1, LOSS_RELATIVE_L2 = range(7)
REG_NONE, REG_DISTORTION = range(2)
WARP_NGP, WARP_MIPNERF360, WARP_DONERF, WARP_SIGMOID, WARP_ERP, WARP_SINUSOIDAL = range(6)
SAMPLING_ORIGINAL, SAMPLING_DISPARITY, SAMPLING_LOG = range(3)
GRID_WARPED_EXP, GRID_WARPED_RECIPROCAL, GRID_METRIC_EXP, GRID_METRIC_RECIPROCAL = range(4)
FIELD_NETWORK, FIELD_BLOBS = range(2)


class Config(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("version", C.c_uint32),
        ("warping_type", C.c_int32), ("aabb_scale", C.c_uint32), ("use_grid", C.c_int32),
        ("grid_size", C.c_uint32), ("num_cascades", C.c_uint32), ("ema_decay", C.c_float),
        ("grid_distribution_type", C.c_int32), ("maximum_marching_steps", C.c_uint32),
        ("cone_angle_constant", C.c_float), ("min_cone_stepsize", C.c_float),
        ("max_cone_stepsize", C.c_float), ("near_distance", C.c_float), ("far_distance", C.c_float),
        ("sampling_type", C.c_int32), ("snap_to_pixel_centers_in_rendering", C.c_int32),
        ("min_optical_thickness", C.c_float),
        ("transmittance_threshold", C.c_float), ("train_in_linear_color", C.c_int32),
        ("n_levels", C.c_uint32), ("n_features_per_level", C.c_uint32),
        ("log2_hashmap_size", C.c_uint32), ("base_resolution", C.c_uint32),
        ("per_level_scale", C.c_float), ("desired_resolution", C.c_float),
        ("density_activation", C.c_int32), ("rgb_activation", C.c_int32), ("field_type", C.c_int32),
        ("march_iter", C.c_uint32), ("max_samples_per_ray", C.c_uint32),
        ("reserved", C.c_uint32 * 8),
    ]


class View(C.Structure):
    _fields_ = [
        ("camera", C.c_float * 12), ("width", C.c_uint32), ("height", C.c_uint32),
        ("relative_focal_length", C.c_float * 2), ("principal_point", C.c_float * 2),
        ("spp_index", C.c_uint32), ("render_mode", C.c_int32), ("depth_scale", C.c_float),
        ("shard_rows", C.c_uint32), ("shard_count", C.c_uint32), ("shard_rank", C.c_uint32),
    ]


class Post(C.Structure):
    _fields_ = [
        ("exposure", C.c_float), ("background_color", C.c_float * 4), ("color_space", C.c_int32),
        ("tonemap_curve", C.c_int32), ("to_srgb", C.c_int32),
    ]


class TrainViews(C.Structure):
    _fields_ = [
        ("n_images", C.c_uint32), ("width", C.c_int32), ("height", C.c_int32),
        ("focal_length", C.c_float * 2), ("principal_point", C.c_float * 2),
        ("d_xforms", C.c_void_p), ("d_images", C.c_void_p), ("d_sampling_probability", C.c_void_p),
    ]


class LossParams(C.Structure):
    _fields_ = [
        ("n_rays", C.c_uint32), ("n_max_compacted_coords", C.c_uint32), ("loss_type", C.c_int32), ("loss_scale", C.c_float),
        ("regularization_type", C.c_int32), ("background_color", C.c_float * 3), ("color_space", C.c_int32),
        ("train_with_random_bg_color", C.c_int32), ("rng_state", C.c_uint64), ("rng_inc", C.c_uint64),
        ("padded_output_width", C.c_uint32),
    ]


class FrameStats(C.Structure):
    _fields_ = [
        ("n_rays", C.c_uint64), ("n_rays_alive", C.c_uint64), ("n_march_steps", C.c_uint64),
        ("n_samples", C.c_uint64), ("n_samples_composited", C.c_uint64), ("n_rays_hit", C.c_uint64),
        ("n_batches", C.c_uint32), ("error_flags", C.c_uint32),
        ("ms_sampler", C.c_float), ("ms_field", C.c_float), ("ms_composite", C.c_float), ("ms_post", C.c_float),
        ("n_waves", C.c_uint32),
    ]

    def as_dict(self):
        return {name: getattr(self, name) for name, _ in self._fields_}


def default_config() -> Config:
    """The reference's defaults (internal/sampler/occupancy_sampler.cu:909-944,
    internal/render/ray_marcher.cu:294-301, internal/testbed.h:114-117) and the network shape
    every shipped config uses.  Pure Python so that it works without the library."""
    c = Config()
    c.struct_size = C.sizeof(Config)
    c.version = ABI_VERSION
    c.warping_type = WARP_NGP
    c.aabb_scale = 1
    c.use_grid = 1
    c.grid_size = 128
    c.num_cascades = 1
    c.ema_decay = 0.95
    c.grid_distribution_type = GRID_WARPED_EXP   # the reference's default string "Exp" throws
    c.maximum_marching_steps = 1024
    c.cone_angle_constant = 0.0
    c.min_cone_stepsize = 0.0
    c.max_cone_stepsize = 0.0
    c.near_distance = 0.2
    c.far_distance = 100.0
    c.sampling_type = SAMPLING_ORIGINAL
    c.snap_to_pixel_centers_in_rendering = 1
    c.min_optical_thickness = 0.01
    c.transmittance_threshold = 1e-4
    c.train_in_linear_color = 0
    c.n_levels = 16
    c.n_features_per_level = 2
    c.log2_hashmap_size = 19
    c.base_resolution = 16
    c.per_level_scale = 0.0
    c.desired_resolution = 2048.0
    c.density_activation = ACT_EXPONENTIAL
    c.rgb_activation = ACT_LOGISTIC
    c.field_type = FIELD_NETWORK
    c.march_iter = 10000
    c.max_samples_per_ray = 0
    return c


def default_post() -> Post:
    p = Post()
    p.exposure = 0.0
    p.background_color[:] = [0.0, 0.0, 0.0, 1.0]
    p.color_space = COLOR_LINEAR
    p.tonemap_curve = TONEMAP_IDENTITY
    p.to_srgb = 0
    return p


def make_view(camera, width, height, relative_focal_length, principal_point=(0.5, 0.5), spp_index=0,
              render_mode=MODE_SHADE, depth_scale=1.0, shard_rows=8, shard_count=1, shard_rank=0) -> View:
    v = View()
    flat = [float(x) for row in camera for x in row] if hasattr(camera[0], "__len__") else [float(x) for x in camera]
    assert len(flat) == 12
    v.camera[:] = flat
    v.width, v.height = int(width), int(height)
    v.relative_focal_length[:] = [float(relative_focal_length[0]), float(relative_focal_length[1])]
    v.principal_point[:] = [float(principal_point[0]), float(principal_point[1])]
    v.spp_index = spp_index
    v.render_mode = render_mode
    v.depth_scale = depth_scale
    v.shard_rows, v.shard_count, v.shard_rank = shard_rows, shard_count, shard_rank
    return v


_P = C.POINTER
_vp = C.c_void_p
_ctx = C.c_void_p

# name -> (restype, argtypes): every symbol include/srf_abi.h declares
SYMBOLS = {
    "srf_config_default": (None, [_P(Config)]),
    "srf_create": (C.c_int, [_P(Config), C.c_int, _P(_ctx)]),
    "srf_destroy": (None, [_ctx]),
    "srf_last_error": (C.c_char_p, [_ctx]),
    "srf_set_timing": (C.c_int, [_ctx, C.c_int]),
    "srf_hashgrid_layout": (C.c_int, [_P(Config), _vp, _vp, _vp]),
    "srf_upload_network": (C.c_int, [_ctx, _vp, C.c_size_t, _vp, C.c_size_t, _vp, C.c_size_t]),
    "srf_upload_blobs": (C.c_int, [_ctx, _vp, C.c_uint32, _vp]),
    "srf_upload_density_grid": (C.c_int, [_ctx, _vp, C.c_size_t, _vp]),
    "srf_download_density_grid": (C.c_int, [_ctx, _vp, C.c_size_t, _vp]),
    "srf_upload_bitfield": (C.c_int, [_ctx, _vp, C.c_size_t, _vp]),
    "srf_download_bitfield": (C.c_int, [_ctx, _vp, C.c_size_t, _vp]),
    "srf_download_grid_mean": (C.c_int, [_ctx, _vp, _vp]),
    "srf_update_grid_bitfield": (C.c_int, [_ctx, _vp]),
    "srf_refresh_reset": (C.c_int, [_ctx, C.c_uint64]),
    "srf_refresh_grid": (C.c_int, [_ctx, C.c_uint32, _vp]),
    "srf_shard_ray_count": (C.c_int, [_P(View), _P(C.c_uint64)]),
    "srf_generate_rays": (C.c_int, [_ctx, _P(View), _vp, _vp, _vp, _vp, _vp]),
    "srf_sample_count": (C.c_int, [_ctx, _P(View), _vp, _vp]),
    "srf_sample_offsets": (C.c_int, [_ctx, _vp, C.c_uint64, _vp, _vp]),
    "srf_sample_emit": (C.c_int, [_ctx, _P(View), _vp, C.c_uint64, _vp, _vp, _vp, _vp]),
    "srf_network_inference": (C.c_int, [_ctx, _vp, C.c_uint64, _vp, _vp]),
    "srf_network_density": (C.c_int, [_ctx, _vp, C.c_uint64, _vp, _vp]),
    "srf_volume_rendering": (C.c_int, [_ctx, _P(View), _vp, C.c_uint64, _vp, _vp, _vp, _vp, _vp]),
    "srf_render_frame": (C.c_int, [_ctx, _P(View), _P(Post), _vp, _vp, _vp, _vp, _P(FrameStats), _vp]),
    "srf_render_frame_scatter": (C.c_int, [_ctx, _P(View), _P(Post), _vp, _vp, _P(FrameStats), _vp]),
    "srf_render": (C.c_int, [_ctx, _P(View), _P(Post), C.c_uint32, _vp, _P(FrameStats)]),
    "srf_dump_samples": (C.c_int, [_ctx, _P(View), C.c_uint64, C.c_uint64, C.c_uint64, _vp, _vp, _vp, _vp,
                                   _P(C.c_uint64)]),
    "srf_check_errors": (C.c_int, [_ctx, _vp, _P(C.c_uint32)]),
    "srf_comm_init": (C.c_int, [_P(_ctx), C.c_uint32, _P(C.c_void_p)]),
    "srf_comm_destroy": (None, [C.c_void_p]),
    "srf_comm_last_error": (C.c_char_p, [C.c_void_p]),
    "srf_render_frames_sharded": (C.c_int, [C.c_void_p, _P(View), C.c_uint32, _P(Post), C.c_uint32, _vp, _vp, _P(FrameStats)]),
    "srf_get_timings": (C.c_int, [C.c_void_p, _P(C.c_float), C.c_uint32]),
    "srf_reserve": (C.c_int, [_ctx, C.c_uint64]),
    "srf_set_wave_schedule": (C.c_int, [_ctx, _vp, C.c_uint32]),
    "srf_set_cell_table_budget": (C.c_int, [_ctx, C.c_uint64]),
    "srf_sampler_init": (C.c_int, [_ctx, _P(TrainViews), C.c_int, C.c_uint64, _vp]),
    "srf_sample_training_rays": (C.c_int, [_ctx, _P(TrainViews), C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64, C.c_uint64,
                                           C.c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "srf_volume_rendering_loss": (C.c_int, [_ctx, _P(LossParams), _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "srf_sample_offsets_static": (C.c_int, [C.c_int, _vp, C.c_uint64, _vp, _vp, C.c_char_p, C.c_size_t]),
    "srf_eval_math": (C.c_int, [C.c_int, C.c_int, _vp, _vp, _vp, C.c_size_t]),
}

LIB_NAME = "libsrf_b200.so"
_lib = None


def lib_path() -> Path:
    override = os.environ.get("SRF_B200_LIB")
    return Path(override) if override else Path(__file__).resolve().parent / LIB_NAME


def load_from(path):
    """Loads a build of the C-ABI library from `path` and types every declared symbol."""
    lib = C.CDLL(str(path))
    for name, (restype, argtypes) in SYMBOLS.items():
        fn = getattr(lib, name)   # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


def load():
    """Loads libsrf_b200.so and types every declared symbol.  Raises if anything is missing."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not path.exists():
        raise RuntimeError(f"{path} is missing: build it with `python __graft_entry__.py build` "
                           "(nvcc, sm_100a). There is no fallback path.")
    _lib = load_from(path)
    return _lib


class SrfError(RuntimeError):
    def __init__(self, status, text):
        super().__init__(f"srf status {status}: {text}")
        self.status = status


def check(status, ctx=None):
    if status != OK:
        lib = load()
        msg = lib.srf_last_error(ctx)
        raise SrfError(status, msg.decode() if msg else "")
