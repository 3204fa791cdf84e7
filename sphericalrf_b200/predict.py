"""Prediction driver: the inference half of the reference's run script on the compiled `pyngp` module.

Mirrors the `--predict_transforms` and `--test_transforms` branches of experiment/*/python/run.py:128-250: load a
snapshot, set background and field of view (or the transforms file's intrinsics), and for every frame of a transforms
file set the camera, render the colour image with `spp` samples per pixel and then the depth image, timing the colour
render.  Images are returned (and written as .npy when `output_dir` is given); image metrics against ground-truth
photographs (PSNR / SSIM / LPIPS) and video encoding are outside this library.

    python -m sphericalrf_b200.predict --load_snapshot scene.msgpack --predict_transforms transforms_spherical.json \
           --predict_width 1245 --predict_height 825 --predict_angle_x 60 --output_dir out/
"""
from __future__ import annotations

import argparse
import json
import math
import os
import time

import numpy as np


def predict(testbed, transforms: dict, width: int, height: int, angle_x_deg: float | None = None, spp: int = 8,
            background=(1.0, 1.0, 1.0, 1.0), with_depth: bool = True, output_dir: str | None = None):
    """Renders every frame of `transforms` (the reference's transforms JSON: `frames[i].transform_matrix`, 4x4).

    With `angle_x_deg` the field of view is set as the predict branch does (run.py:226-235: fov_y from the aspect ratio);
    without it the file's intrinsics are used as the test branch does (run.py:143-147).  Returns
    dict(images, depths, seconds, fps)."""
    from . import pyngp as ngp
    testbed.background_color = [float(x) for x in background]
    if angle_x_deg is not None:
        fov_rad_x = math.radians(angle_x_deg)
        aspect_ratio = float(width) / float(height)
        fov_rad_y = math.radians(math.degrees(math.radians(angle_x_deg * 0.5) / aspect_ratio) * 2.0)
        testbed.fov_xy = [fov_rad_x, fov_rad_y]
    else:
        testbed.rendering_buffer.relative_focal_length = [transforms["fx"] / transforms["w"], transforms["fy"] / transforms["h"]]
        testbed.rendering_buffer.principal_point = [transforms["cx"], transforms["cy"]]
    if output_dir:
        os.makedirs(os.path.join(output_dir, "image_predict"), exist_ok=True)
        os.makedirs(os.path.join(output_dir, "depth_predict"), exist_ok=True)
    images, depths, seconds = [], [], []
    for i, frame in enumerate(transforms["frames"]):
        testbed.set_nerf_camera_matrix(np.asarray(frame["transform_matrix"], np.float32)[:-1, :])
        t0 = time.perf_counter()
        image = testbed.render(width, height, spp, False)
        seconds.append(time.perf_counter() - t0)
        depth = None
        if with_depth:
            testbed.rendering_buffer.render_mode = ngp.RenderMode.Depth
            depth = testbed.render(width, height, spp, False)
            testbed.rendering_buffer.render_mode = ngp.RenderMode.Shade
        images.append(image)
        depths.append(depth)
        if output_dir:
            name = os.path.splitext(os.path.basename(frame.get("file_path", f"{i:04d}")))[0]
            np.save(os.path.join(output_dir, "image_predict", name + ".npy"), image[..., :3])
            if depth is not None:
                np.save(os.path.join(output_dir, "depth_predict", name + ".npy"), depth[..., 0])
    mean = float(np.mean(seconds)) if seconds else 0.0
    return dict(images=images, depths=depths, seconds=seconds, fps=(1.0 / mean if mean > 0 else 0.0))


def main():
    ap = argparse.ArgumentParser(description="Render the frames of a transforms file from a snapshot (the reference's predict branch).")
    ap.add_argument("--load_snapshot", required=True)
    ap.add_argument("--predict_transforms", required=True)
    ap.add_argument("--predict_width", type=int, default=1245)
    ap.add_argument("--predict_height", type=int, default=825)
    ap.add_argument("--predict_angle_x", type=float, default=60.0)
    ap.add_argument("--spp", type=int, default=8)
    ap.add_argument("--output_dir", default=None)
    args = ap.parse_args()
    from . import pyngp as ngp
    testbed = ngp.Testbed()
    testbed.load_snapshot(args.load_snapshot)
    with open(args.predict_transforms) as f:
        transforms = json.load(f)
    res = predict(testbed, transforms, args.predict_width, args.predict_height, args.predict_angle_x, args.spp, output_dir=args.output_dir)
    print(f"{len(res['images'])} frames, {np.mean(res['seconds']):.4f} s per colour image, FPS={res['fps']:.2f}")


if __name__ == "__main__":
    main()
