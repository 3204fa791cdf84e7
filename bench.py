#!/usr/bin/env python
"""Benchmark of the render hot path (rays/s), one JSON line on stdout.

Workloads (seed-generated stand-ins for the datasets the reference is evaluated on):
  1 (default, the headline): full inference frames of configuration 1 (1245x825, camera inside the unit sphere, 128^3
     spherical occupancy bitfield, 16x2 hash grid with 2^19 entries per level, 64-wide fp16 MLPs, random-init
     parameters).  A step renders N such frames on N GPUs, every frame's rays cut into blocks of 8 image rows dealt
     round-robin to the ranks: the work per GPU is one frame's worth of rays whatever N is (weak scaling).
  2: the 32-view 360-degree orbit of configuration 2 (32.9 M rays per step), the same batch whatever N is (strong
     scaling): every view's row blocks are dealt to the N ranks.
  4: the four 3840x2160 views of the dense scene of configuration 4 (33.2 M rays per step, 2048-sample cap), strong.
  0O / 0D / 0X: sampler + compositing on the analytic field (configuration 0), one 800x800 frame per GPU.
Weights, grid and bitfield are replicated; the ranks' pixels meet in rank 0's image (peer stores from the output
stage, or an NCCL gather of tiles with --gather nccl).

  value : Mrays/s with the cameras already on the device side of the call and the images left in HBM
  e2e   : Mrays/s through srf_render(), the call a user of the reference's Testbed.render makes:
          camera in host memory, image copied back to (pinned) host memory inside the timed region
  --impl reference : the reference's own sampler / compositing kernels compiled for the host cores (oracle/_ref, built
          from the reference's sources where they are mounted; the network comes from the CPU oracle because
          tiny-cuda-nn is not available), or the CPU oracle alone where that build does not exist; on a bounded sample.
  --single-process : N GPUs driven by one host process through srf_comm_init / srf_render_frames_sharded (no torch
          distributed, no torchrun) instead of one process per GPU.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WIDTH, HEIGHT = 1245, 825
ALG_BYTES_PER_SAMPLE = 588.0      # hash encoding: 12 B position + 16 levels x 8 corners x 4 B + 64 B encoded
ALG_FLOP_PER_SAMPLE = 18816.0     # the two MLPs
# DRAM bytes per sample of the two dominant kernels, from the ncu captures named in `roofline.scaled_from`
# (dram__bytes_read.sum + dram__bytes_write.sum of one launch / its samples)
FIELD_DRAM_BYTES_PER_SAMPLE = 36.3
SAMPLER_DRAM_BYTES_PER_SAMPLE = 16.1


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


WORKLOAD = "1"          # "1" is the headline; the others are BASELINE's other configurations, for the record
WORKLOAD_NAMES = {
    "1": "config1 full inference frame {w}x{h}, fp16 network, 128^3 bitfield",
    "2": "config2 32-view orbit of config1 frames {w}x{h}, fp16 network, 128^3 bitfield",
    "0O": "config0-O sampler+compositing, analytic blob field fp32, Original sampling, {w}x{h}",
    "0D": "config0-D sampler+compositing, analytic blob field fp32, Disparity sampling, {w}x{h}",
    "0X": "config0-O with opaque blobs (rays saturate early), analytic blob field fp32, Original sampling, {w}x{h}",
    "4": "config4 dense inward-facing scene, 4 views {w}x{h}, fp16 network, Original sampling, 2048-sample cap",
}
FIXED_VIEWS = {"2": 32, "4": 4}     # workloads whose batch of views does not grow with N (strong scaling)


def build_scene():
    from sphericalrf_b200 import abi, synth
    if WORKLOAD == "1":
        return synth.scene_config1(grid_size=128, width=WIDTH, height=HEIGHT)
    if WORKLOAD == "2":
        return synth.scene_config1(grid_size=128, width=WIDTH, height=HEIGHT, n_views=32)
    if WORKLOAD in ("0O", "0D", "0X"):
        return synth.scene_config0(WORKLOAD[1], 128, WIDTH, HEIGHT)
    if WORKLOAD == "4":
        return synth.scene_config4(128, WIDTH, HEIGHT)
    raise SystemExit(f"unknown workload {WORKLOAD}")


def workload_name():
    return WORKLOAD_NAMES[WORKLOAD].format(w=WIDTH, h=HEIGHT)


def upload_scene(r, sc):
    from sphericalrf_b200 import abi
    if sc["cfg"].field_type == abi.FIELD_NETWORK:
        r.upload_network(sc["hash_table"], sc["density_mlp"], sc["rgb_mlp"])
    else:
        r.upload_blobs(sc["blobs"], sc["color_map"])
    r.upload_density_grid(sc["grid"])
    r.update_grid_bitfield()


def _host_threads():
    """One OpenMP thread per core this process may run on (launchers such as torchrun export OMP_NUM_THREADS=1)."""
    return max(1, len(os.sched_getaffinity(0)))


def cpu_reference_sample(sc, target_seconds=15.0):
    """Times the reference's CPU-side logic on a bounded sample of the workload's first view.

    kind "reference": the reference's own kernels compiled for the host (oracle/_ref/libsrf_ref.so: ray generation,
    occupancy-guided marching, compaction, compositing, shading, accumulation and tonemapping of
    Testbed::render_frame; the network is the CPU oracle's because tiny-cuda-nn is not available), rendering the
    view at a lower resolution sized for the time budget.  kind "port": the CPU oracle on a stripe of consecutive
    rays, where that build does not exist or the field is the analytic stand-in.
    Returns (Mrays/s, threads, kind, description, seconds)."""
    from oracle import srf_oracle
    from sphericalrf_b200 import abi, synth
    cfg = sc["cfg"]
    threads = srf_oracle.set_num_threads(_host_threads())
    bits = synth.bitfield_from_grid(cfg, sc["grid"])
    orc = srf_oracle.Oracle(cfg, bits, sc.get("hash_table"), sc.get("density_mlp"), sc.get("rgb_mlp"), sc.get("blobs"), sc.get("color_map"))
    b2, _ = orc.update_grid_bitfield(sc["grid"])
    orc.bitfield = b2
    post = abi.default_post()
    use_ref = False
    if cfg.field_type == abi.FIELD_NETWORK:
        try:
            from oracle import srf_ref
            use_ref = srf_ref.available()
        except Exception:
            use_ref = False
    if use_ref:
        threads = min(threads, srf_ref.set_num_threads(_host_threads()))

        def render(w):
            h = max(1, round(w * HEIGHT / WIDTH))
            view = abi.make_view(sc["cameras"][0], w, h, sc["rfl"])
            t0 = time.perf_counter()
            res = srf_ref.render_frame(cfg, view, post, b2, orc)
            return w * h, int(res["n_samples"].astype(np.int64).sum()), time.perf_counter() - t0

        n0, _, dt0 = render(48)
        rate = n0 / max(dt0, 1e-3)
        w = int(min(WIDTH, max(48, (rate * target_seconds * WIDTH / HEIGHT) ** 0.5)))
        n, n_samples, dt = render(w)
        desc = (f"the first view at {w}x{max(1, round(w * HEIGHT / WIDTH))} ({n} rays, {n_samples} samples) through the reference's "
                f"kernels compiled for the host, OpenMP over rays; network from the CPU oracle")
        return n / dt / 1e6, threads, "reference", desc, dt
    view = abi.make_view(sc["cameras"][0], WIDTH, HEIGHT, sc["rfl"])
    n = orc.n_rays(view)
    first = (HEIGHT // 2) * WIDTH
    probe = 256
    t0 = time.perf_counter()
    orc.render_frame(view, post, first, probe)
    dt = time.perf_counter() - t0
    count = int(max(probe, min(n - first - probe, probe * target_seconds / max(dt, 1e-3))))
    t0 = time.perf_counter()
    res = orc.render_frame(view, post, first + probe, count)
    dt = time.perf_counter() - t0
    desc = (f"{count} consecutive rays from the middle rows of the first view ({res['stats']['n_samples']} samples) through the CPU "
            f"oracle, OpenMP over rays")
    return count / dt / 1e6, threads, "port", desc, dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sc = build_scene()
    vals, cores, kind, desc = [], 1, "port", ""
    for _ in range(max(0, args.warmup)):
        cpu_reference_sample(sc, target_seconds=2.0)
    t_tot = 0.0
    for _ in range(max(1, args.steps)):
        v, cores, kind, desc, dt = cpu_reference_sample(sc, target_seconds=12.0)
        vals.append(v); t_tot += dt
    value = float(np.mean(vals))
    n_views = FIXED_VIEWS.get(WORKLOAD, args.gpus)
    line = {
        "impl": "reference", "metric": "render throughput", "value": value, "unit": "Mrays/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_tot / max(1, args.steps), "higher_is_better": True,
        "scaling": "strong" if WORKLOAD in FIXED_VIEWS else "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": workload_name(), "frames_per_step": n_views, "rays_per_frame": WIDTH * HEIGHT},
        "cpu_baseline": {"value": value, "unit": "Mrays/s", "cores": cores, "kind": kind, "sample": desc},
        "e2e": {"value": value, "unit": "Mrays/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist
    from sphericalrf_b200 import abi
    from sphericalrf_b200.testbed import Renderer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    n_views = FIXED_VIEWS.get(WORKLOAD, world)       # frames per step: one per GPU (weak) or the workload's fixed batch (strong)

    sc = build_scene()
    if world > 1:
        # replication at load: rank 0's parameters, grid and scene arrays go to every rank (NCCL broadcast)
        from sphericalrf_b200.sharding import broadcast_arrays
        import numpy as np
        names = [k for k, v in sc.items() if isinstance(v, np.ndarray)]
        sc.update(broadcast_arrays({k: sc[k] for k in names} if rank == 0 else None, src=0, device=dev))
    cfg = sc["cfg"]
    r = Renderer(cfg, local_rank)
    upload_scene(r, sc)
    post = abi.default_post()
    cams = sc["cameras"]
    views = [abi.make_view(cams[k % len(cams)], WIDTH, HEIGHT, sc["rfl"], shard_rows=8, shard_count=world, shard_rank=rank)
             for k in range(n_views)]
    view = views[0]
    n_local = r.n_rays(view)
    rays_per_step = WIDTH * HEIGHT * n_views

    from sphericalrf_b200.sharding import PeerImage, TileGather
    tg = TileGather(WIDTH, HEIGHT, n_views, 4, 8, dev)
    assert tg.n_local == n_local
    out = tg.tiles
    accum = torch.zeros((tg.n_pad, 4), dtype=torch.float32, device=dev)
    # N > 1: the output stage stores pixels straight into rank 0's image over NVLink (peer stores); NCCL gather of
    # tiles is the fallback when symmetric memory cannot be set up
    peer, gather_kind = None, "none"
    if world > 1:
        gather_kind = "nccl gather of tiles"
        if args.gather == "peer":
            try:
                peer = PeerImage(WIDTH, HEIGHT, n_views, dev)
                gather_kind = "peer stores into rank 0's image (fused into the output stage) + barrier"
            except Exception as e:          # noqa: BLE001
                if rank == 0:
                    print(f"symmetric memory unavailable ({type(e).__name__}: {e}); using the NCCL gather", file=sys.stderr)
    host_img = torch.zeros((n_views, HEIGHT, WIDTH, 4), dtype=torch.float32).pin_memory() if rank == 0 else None
    stats = abi.FrameStats()

    def step_device():
        if peer is not None:
            for k in range(n_views):
                r.render_frame_scatter_device(views[k], post, peer.root[k], accum)
            peer.barrier()
            return
        for k in range(n_views):
            r.render_frame_device(views[k], post, out[k], accum, None, None, None, None)
        if world > 1:
            tg.gather()

    def step_e2e():
        if world == 1:
            # the reference-facing call: host camera in, host image out
            for k in range(n_views):
                st = r.lib.srf_render(r.ctx, C.byref(views[k]), C.byref(post), 1, C.c_void_p(host_img[k].data_ptr()), None)
                assert st == 0, r.lib.srf_last_error(r.ctx)
        else:
            step_device()
            if rank == 0:
                host_img.view(n_views, HEIGHT * WIDTH, 4).copy_(peer.local if peer is not None else tg.image, non_blocking=True)
                torch.cuda.current_stream().synchronize()

    def timed(fn, steps, warmup, sample_clocks=False):
        for _ in range(warmup):
            fn()
        sampler = ClockSampler(local_rank) if (sample_clocks and rank == 0) else None
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        if sampler:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        clocks = sampler.stop() if sampler else None
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), clocks

    ms_total, clocks = timed(step_device, args.steps, args.warmup, sample_clocks=True)
    r.check_errors()                                 # a frame cut short on the device must not pass for a timed one
    ms_step = ms_total / args.steps
    value = rays_per_step / (ms_step * 1e-3) / 1e6
    ms_e2e, _ = timed(step_e2e, args.steps, 1)
    r.check_errors()
    e2e_value = rays_per_step / (ms_e2e / args.steps * 1e-3) / 1e6

    # What reached rank 0 over NVLink, against the same view rendered whole on rank 0's GPU: the driver's box has one
    # GPU for its tests, so this is where the assembled image is checked on real links.
    gather_check = "single GPU: nothing gathered"
    if world > 1:
        step_device()
        torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            k = n_views - 1
            whole = abi.View.from_buffer_copy(views[k])
            whole.shard_count, whole.shard_rank = 1, 0
            ref_img = torch.zeros((HEIGHT * WIDTH, 4), dtype=torch.float32, device=dev)
            ref_acc = torch.zeros((HEIGHT * WIDTH, 4), dtype=torch.float32, device=dev)
            r.render_frame_device(whole, post, ref_img, ref_acc, None, None, None, None)
            torch.cuda.synchronize()
            got = (peer.local if peer is not None else tg.image)[k]
            gather_check = "equal" if torch.equal(got.view(torch.int32), ref_img.view(torch.int32)) else "DIFFERS"
        dist.barrier()

    # per-kernel durations of the dominant kernel (field: hash encoding + MLPs), CUDA events inside the library
    r.set_timing(True)
    t_field = t_sampler = t_comp = 0.0
    n_samples = n_batches = 0
    for _ in range(args.steps):
        r.render_frame_device(views[0], post, out[0], accum, None, None, stats, None)
        t_field += stats.ms_field; t_sampler += stats.ms_sampler; t_comp += stats.ms_composite
        n_samples = stats.n_samples; n_batches = stats.n_batches * max(stats.n_waves, 1)   # launches of each stage per frame
    r.set_timing(False)
    t_field /= args.steps; t_sampler /= args.steps; t_comp /= args.steps
    imbalance = None
    if world > 1:
        # samples each rank marches for one step's views: how evenly the row blocks split the work
        mine = 0
        for k in range(n_views):
            r.render_frame_device(views[k], post, out[0], accum, None, None, stats, None)
            mine += int(stats.n_samples)
        t = torch.zeros(world, dtype=torch.int64, device=dev)
        t[rank] = mine
        dist.all_reduce(t)
        per_rank = [int(x) for x in t.tolist()]
        imbalance = {"samples_per_rank": per_rank, "max_over_mean": max(per_rank) / (sum(per_rank) / world)}
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peak, peak_kind = _peaks()
    launches_per_frame = 3 * n_batches               # march, field, composite per batch of rays and wave
    achieved = ALG_BYTES_PER_SAMPLE * n_samples / max(n_batches, 1) / (t_field / max(n_batches, 1) * 1e-3) / 1e9 if t_field > 0 else 0.0
    roof_kernel = "k_field_network_tc (hash-grid gather + tcgen05 MLPs + shading)"
    roof_ms = t_field / max(n_batches, 1)
    roof_traffic = FIELD_DRAM_BYTES_PER_SAMPLE * n_samples / max(n_batches, 1)
    roof_capture = "profiles/field_network_tcgen05_config1_320x208.md"
    roof_limiter = "instruction issue and the group barriers around the five tcgen05.mma issues (ncu: issue-active 72 %, top stall barrier, L1 68 %, DRAM 5 %, tensor pipe 12 %)"
    if cfg.field_type != abi.FIELD_NETWORK:
        # sampler + compositing configurations: the sampler is the kernel of interest (28 B/sample + 80 B/ray)
        roof_kernel = "k_march_paged (single-pass sampler)"
        roof_ms = t_sampler / max(n_batches, 1)
        achieved = (28.0 * n_samples + 80.0 * n_local) / (t_sampler * 1e-3) / 1e9 if t_sampler > 0 else 0.0
        roof_traffic = SAMPLER_DRAM_BYTES_PER_SAMPLE * n_samples / max(n_batches, 1)
        roof_capture = "profiles/march_paged_config1_320x208.md"
        roof_limiter = "dependent arithmetic per march step (ncu: issue-active 58 %, top stall wait, DRAM 12 %)"
    line = {
        "metric": "render throughput", "value": value, "unit": "Mrays/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong" if WORKLOAD in FIXED_VIEWS else "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": workload_name(),
                   "frames_per_step": n_views, "rays_per_frame": WIDTH * HEIGHT, "samples_per_frame_shard": int(n_samples),
                   "partition": f"rows in blocks of 8 round-robin over {world} rank(s)", "gather": gather_kind,
                   "gather_check": gather_check,
                   "l2": "per-frame working set (sample buffers) far larger than L2; no flush needed",
                   "schedule": f"{stats.n_batches} ray batch(es) x {stats.n_waves} wave(s) per frame (trailing waves empty when every ray has ended)",
                   "device_memory": "library defaults: 16 GB sample pool; cell-major copies of the leading hash-grid levels within 4 GiB (network workloads)"},
        "frames_per_s": n_views / (ms_step * 1e-3),
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "Mrays/s", "h2d_bytes_per_step": int(C.sizeof(abi.View) + C.sizeof(abi.Post)) * n_views,
                "d2h_bytes_per_step": int(HEIGHT * WIDTH * 16 * n_views)},
        "gpu_launches": int(launches_per_frame * n_views * args.steps),
        # achieved / frac follow the benchmark contract: algorithmic bytes (the gathers and records the stage is defined
        # by) over the kernel's CUDA-event time, against the measured HBM copy peak.  For the field kernel those bytes are
        # table gathers served by L1/L2, so the number is not DRAM bandwidth: `traffic` and `frac_dram` give the DRAM
        # side (bytes per sample from an ncu capture of this kernel on a smaller frame, scaled by the samples of a
        # launch; not re-measured by this run) and `limiter` names what the counters say the kernel waits for.
        "roofline": {"kernel": roof_kernel, "bound": "hbm", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak,
                     "traffic": roof_traffic, "frac_dram": (roof_traffic / (roof_ms * 1e-3) / 1e9 / peak) if roof_ms > 0 else 0.0,
                     "scaled_from": roof_capture, "limiter": roof_limiter, "peak_kind": peak_kind,
                     "ms_per_launch": roof_ms, "launches_per_frame": int(n_batches),
                     "mlp_tflops": ALG_FLOP_PER_SAMPLE * n_samples / (t_field * 1e-3) / 1e12 if t_field > 0 else 0.0},
        "stage_ms": {"sampler": t_sampler, "field": t_field, "composite_output": t_comp},
        "rank_balance": imbalance,
    }
    if world == 1 and WORKLOAD == "1" and cfg.field_type == abi.FIELD_NETWORK:
        # training-side kernels on the same scene: one batch of Testbed::train_nerf_step's data path
        # (testbed.cu:317-380) -- sample 4096 training rays (<= 1024 samples each, 4 Mi sample slots), evaluate
        # the network on them, composite with loss and gradient into a 2^18-sample compacted batch
        from sphericalrf_b200 import synth
        tviews = synth.training_views(5000, n_images=8, width=400, height=400, radius=0.5, fov_deg=60.0, zero_probability=0.05)
        tv, keep = r._device_views(tviews)
        n_tr, n_coords, n_comp = 4096, 1 << 22, 1 << 18
        ctr = torch.zeros(4, dtype=torch.int32, device=dev)
        t_rays = torch.zeros((n_tr, 6), device=dev); t_rgba = torch.zeros((n_tr, 4), device=dev)
        t_idx = torch.zeros((n_tr, 2), dtype=torch.int32, device=dev); t_idx0 = torch.zeros_like(t_idx)
        t_coords = torch.zeros((n_coords, 7), device=dev); t_out = torch.zeros((n_coords, 4), dtype=torch.float16, device=dev)
        t_cc = torch.zeros((n_comp, 7), device=dev); t_dl = torch.zeros((n_comp, 4), dtype=torch.float16, device=dev)
        t_loss = torch.zeros(n_tr, device=dev)
        lp = abi.LossParams()
        lp.n_rays, lp.n_max_compacted_coords, lp.loss_type, lp.loss_scale = n_tr, n_comp, abi.LOSS_SMOOTH_L1, 128.0
        lp.background_color[:] = [1.0, 1.0, 1.0]
        lp.color_space, lp.train_with_random_bg_color, lp.padded_output_width = abi.COLOR_SRGB, 1, 4
        lp.rng_state, lp.rng_inc = 0x853c49e6748fea9b, 0xda3e39cb94b95bdb
        P = lambda t, off=0: C.c_void_p(t.data_ptr() + off)
        n_used = [0]

        def train_sample():
            st = r.lib.srf_sample_training_rays(r.ctx, C.byref(tv), n_tr, 0, n_coords, lp.rng_state, lp.rng_inc, 1, P(ctr), P(ctr, 4),
                                                P(t_rays), P(t_rgba), P(t_idx0), P(t_coords), None)
            assert st == 0, r.lib.srf_last_error(r.ctx)

        def train_infer():
            st = r.lib.srf_network_inference(r.ctx, P(t_coords), n_used[0], P(t_out), None)
            assert st == 0, r.lib.srf_last_error(r.ctx)

        def train_loss():
            t_idx.copy_(t_idx0)                      # the compositor rewrites the (count, base) pairs
            st = r.lib.srf_volume_rendering_loss(r.ctx, C.byref(lp), P(ctr), P(t_idx), P(t_rgba), P(t_coords), P(t_out), P(t_cc),
                                                 P(ctr, 8), P(t_dl), P(t_loss), None, None)
            assert st == 0, r.lib.srf_last_error(r.ctx)

        def ms_of(fn, reps=5):
            fn(); fn()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(); a.record()
            for _ in range(reps):
                fn()
            b.record(); torch.cuda.synchronize()
            return a.elapsed_time(b) / reps

        ms_s = ms_of(train_sample)
        kept, total = int(ctr[0].item()), int(ctr[1].item())
        n_used[0] = min(total, n_coords)
        ms_i = ms_of(train_infer)
        ms_l = ms_of(train_loss)
        line["training_side"] = {
            "rays": n_tr, "rays_kept": kept, "samples": total, "samples_consumed": int(ctr[2].item()),
            "samples_with_gradient": min(int(ctr[2].item()), n_comp),
            "ms_sample_rays": ms_s, "ms_network_inference": ms_i, "ms_loss_and_gradient": ms_l,
            "sampler_msamples_per_s": total / (ms_s * 1e-3) / 1e6, "inference_msamples_per_s": n_used[0] / (ms_i * 1e-3) / 1e6,
            # sampler: 28 B/sample + 80 B/ray; compositor forward+backward: 2 x (8 + 4) B read per sample + 28 B copied and
            # 8 B gradient written per compacted sample
            "sampler_algorithmic_gbs": (28.0 * total + 80.0 * n_tr) / (ms_s * 1e-3) / 1e9,
            "loss_algorithmic_gbs": (24.0 * total + 64.0 * min(int(ctr[2].item()), n_comp)) / (ms_l * 1e-3) / 1e9,
        }
    if world == 1 and WORKLOAD == "1" and cfg.field_type == abi.FIELD_NETWORK:
        # density-grid refresh (Testbed::train_prep_nerf): 16 consecutive refreshes of the 128^3 grid, all-cells mode
        r.refresh_reset(3001)
        for _ in range(2):
            r.refresh_grid(0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(16):
            r.refresh_grid(0)
        e1.record()
        torch.cuda.synchronize()
        ms_refresh = e0.elapsed_time(e1) / 16
        cells = cfg.grid_size ** 3
        line["refresh"] = {"ms_per_refresh": ms_refresh, "cells": cells, "refreshes_per_s": 1e3 / ms_refresh,
                           "algorithmic_gbs": cells * 532.125 / (ms_refresh * 1e-3) / 1e9,
                           "algorithmic_tflops": cells * 4224.0 / (ms_refresh * 1e-3) / 1e12}
    if world == 1 and not args.no_cpu_baseline:
        v, cores, kind, desc, _ = cpu_reference_sample(sc, target_seconds=15.0)
        line["cpu_baseline"] = {"value": v, "unit": "Mrays/s", "cores": cores, "kind": kind, "sample": desc}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_refgpu(args):
    """The reference's own CUDA kernels (ray generation, marching, compaction, compositing, shading, accumulation,
    tonemapping; compiled for sm_100a from its sources by baseline/build_refgpu.py) in the reference's host loop on one
    GPU, with this library's srf_network_inference where the reference calls tiny-cuda-nn.  A same-GPU baseline for the
    frame time; not the library, and not the reference's network."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from baseline import refgpu
    from sphericalrf_b200 import abi
    from sphericalrf_b200.testbed import Renderer
    if not refgpu.available():
        print(json.dumps({"impl": "refgpu", "unavailable": "baseline/_ref/libsrf_refgpu.so is missing and the reference is not mounted to build it"}), flush=True)
        return
    sc = build_scene()
    if sc["cfg"].field_type != abi.FIELD_NETWORK:
        print(json.dumps({"impl": "refgpu", "unavailable": "the analytic stand-in field has no counterpart in the reference's pipeline"}), flush=True)
        return
    r = Renderer(sc["cfg"], 0)
    upload_scene(r, sc)
    ref = refgpu.RefGpu(r)
    dev = torch.device("cuda", 0)
    n_views = FIXED_VIEWS.get(WORKLOAD, 1)
    cams = sc["cameras"]
    views = [abi.make_view(cams[k % len(cams)], WIDTH, HEIGHT, sc["rfl"]) for k in range(n_views)]
    post = abi.default_post()
    out = torch.zeros((HEIGHT * WIDTH, 4), device=dev); acc = torch.zeros((HEIGHT * WIDTH, 4), device=dev)
    host = torch.zeros((HEIGHT * WIDTH, 4)).pin_memory()

    def step(copy):
        ms = 0.0
        for v in views:
            ref.render_frame_device(v, post, out, acc)
            ms += ref.last_ms()
            if copy:
                host.copy_(out, non_blocking=True); torch.cuda.synchronize()
        return ms

    for _ in range(args.warmup):
        step(False)
    sampler = ClockSampler(0); sampler.start()
    ms = sum(step(False) for _ in range(args.steps))
    clocks = sampler.stop()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step(True)
    wall = time.perf_counter() - t0
    rays = WIDTH * HEIGHT * n_views * args.steps
    import ctypes as Cc
    rounds = int(refgpu.lib().refgpu_last_rounds(ref.ctx)); slots = int(refgpu.lib().refgpu_last_network_samples(ref.ctx))
    line = {
        "impl": "refgpu", "metric": "render throughput", "value": rays / (ms * 1e-3) / 1e6, "unit": "Mrays/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong" if WORKLOAD in FIXED_VIEWS else "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": workload_name(), "frames_per_step": n_views, "rays_per_frame": WIDTH * HEIGHT,
                   "pipeline": "the reference's CUDA kernels and host loop (one alive-counter read-back per round, <= 8 samples per ray "
                               "per round) + this library's network stage entry in place of tiny-cuda-nn",
                   "rounds_per_frame": rounds, "network_slots_per_frame": slots},
        "frames_per_s": n_views * args.steps / (ms * 1e-3), "clocks": clocks,
        "e2e": {"value": rays / wall / 1e6, "unit": "Mrays/s", "h2d_bytes_per_step": int(C.sizeof(abi.View) + C.sizeof(abi.Post)) * n_views,
                "d2h_bytes_per_step": int(HEIGHT * WIDTH * 16 * n_views)},
        "gpu_launches": None,
    }
    print(json.dumps(line), flush=True)


def run_single_process(args):
    """N GPUs of the box driven by this one process through the C-ABI's srf_comm_init / srf_render_frames_sharded:
    no torch.distributed, no NCCL.  Device time of a step = the slowest GPU's stream (CUDA events inside the library)."""
    import torch
    from sphericalrf_b200 import abi
    from sphericalrf_b200.testbed import Comm, Renderer
    n = args.gpus
    if torch.cuda.device_count() < n:
        raise SystemExit(f"--single-process --gpus {n}: only {torch.cuda.device_count()} GPU(s) visible")
    sc = build_scene()
    rs = []
    for d in range(n):
        r = Renderer(sc["cfg"], d)
        upload_scene(r, sc)
        rs.append(r)
    comm = Comm(rs)
    n_views = FIXED_VIEWS.get(WORKLOAD, n)
    cams = sc["cameras"]
    views = [abi.make_view(cams[k % len(cams)], WIDTH, HEIGHT, sc["rfl"]) for k in range(n_views)]
    post = abi.default_post()
    host = torch.zeros((n_views, HEIGHT, WIDTH, 4), dtype=torch.float32).pin_memory()
    rays_per_step = WIDTH * HEIGHT * n_views
    for _ in range(args.warmup):
        comm.render(views, post, 1, host_images=False)
    sampler = ClockSampler(0)
    sampler.start()
    ms = 0.0
    t0 = time.perf_counter()
    for _ in range(args.steps):
        comm.render(views, post, 1, host_images=False)
        ms += max(comm.timings())
    wall_resident = time.perf_counter() - t0
    clocks = sampler.stop()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        comm.render(views, post, 1, host_images=host)
    wall = time.perf_counter() - t0
    whole = rs[0].render(views[-1], post, 1)
    check = "equal" if whole.tobytes() == host[-1].numpy().tobytes() else "DIFFERS"
    line = {
        "metric": "render throughput", "value": rays_per_step * args.steps / (ms * 1e-3) / 1e6, "unit": "Mrays/s", "n_gpus": n,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong" if WORKLOAD in FIXED_VIEWS else "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": workload_name(), "frames_per_step": n_views, "rays_per_frame": WIDTH * HEIGHT,
                   "partition": f"rows in blocks of 8 round-robin over {n} GPU(s) of one process",
                   "gather": "peer stores into the first GPU's image (srf_render_frames_sharded), ordered by stream events",
                   "gather_check": check if n > 1 else "single GPU: nothing gathered",
                   "l2": "per-frame working set (sample buffers) far larger than L2; no flush needed"},
        "frames_per_s": n_views * args.steps / (ms * 1e-3), "clocks": clocks,
        "e2e": {"value": rays_per_step * args.steps / wall / 1e6, "unit": "Mrays/s",
                "h2d_bytes_per_step": int(C.sizeof(abi.View) + C.sizeof(abi.Post)) * n_views, "d2h_bytes_per_step": int(HEIGHT * WIDTH * 16 * n_views)},
        "gpu_launches": None, "mode": "single process, srf_comm",
        "wall_ms_per_step": wall_resident * 1e3 / args.steps,     # host clock around the same calls: must agree with ms_per_step
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "refgpu"],
                    help="ours: the library; reference: the reference's CPU-side logic on the host cores; refgpu: the reference's CUDA kernels on one GPU")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"], help="N > 1: how tiles reach rank 0")
    ap.add_argument("--single-process", action="store_true", help="drive --gpus N devices from this one process (srf_comm), no torchrun")
    ap.add_argument("--workload", default="1", choices=sorted(WORKLOAD_NAMES), help="configuration to time; the benchmark is 1")
    ap.add_argument("--res", default=None, help="WxH: a smaller image of the same scene, for profiler captures only "
                                                "(the benchmark number is the default 1245x825)")
    args = ap.parse_args()
    global WIDTH, HEIGHT, WORKLOAD
    WORKLOAD = args.workload
    if WORKLOAD in ("0O", "0D", "0X"):
        WIDTH, HEIGHT = 800, 800
    elif WORKLOAD == "4":
        WIDTH, HEIGHT = 3840, 2160
    if args.res:
        WIDTH, HEIGHT = (int(x) for x in args.res.lower().split("x"))
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "refgpu":
        run_refgpu(args)
    elif args.single_process:
        run_single_process(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
