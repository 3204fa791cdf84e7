"""Two GPUs: every rank's output stage stores its pixels straight into rank 0's image (peer stores through
torch symmetric memory); the assembled image must equal the single-GPU frame byte for byte, and the NCCL
tile gather must give the same.  Skipped on a box with one GPU."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def _worker(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT)); sys.path.insert(0, str(ROOT / "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from sphericalrf_b200 import abi
    from sphericalrf_b200.sharding import PeerImage, TileGather
    from sphericalrf_b200.testbed import Renderer
    from helpers import small_scene
    W, H = 40, 37
    sc = small_scene(kind="net", width=W, height=H)
    r = Renderer(sc["cfg"], rank)
    r.upload_network(sc["hash_table"], sc["density_mlp"], sc["rgb_mlp"])
    r.upload_density_grid(sc["grid"]); r.update_grid_bitfield()
    post = abi.default_post()
    v = abi.View.from_buffer_copy(sc["view"])
    v.shard_rows, v.shard_count, v.shard_rank = 8, world, rank
    n_local = r.n_rays(v)
    accum = torch.zeros((n_local, 4), device=dev)
    peer = PeerImage(W, H, 1, dev)
    r.render_frame_scatter_device(v, post, peer.root[0], accum)
    peer.barrier()
    tg = TileGather(W, H, 1, 4, 8, dev)
    r.render_frame_device(v, post, tg.tiles[0], accum)
    img = tg.gather()
    torch.cuda.synchronize()
    if rank == 0:
        whole_view = abi.View.from_buffer_copy(sc["view"])
        out = torch.zeros((W * H, 4), device=dev); acc = torch.zeros((W * H, 4), device=dev)
        r.render_frame_device(whole_view, post, out, acc)
        torch.cuda.synchronize()
        np.savez(os.path.join(tmp, "res.npz"), peer=peer.local[0].cpu().numpy(), nccl=img[0].cpu().numpy(), whole=out.cpu().numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_store_gather_two_gpus(tmp_path, built_lib):
    import torch.multiprocessing as mp
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    d = np.load(tmp_path / "res.npz")
    assert d["peer"].tobytes() == d["whole"].tobytes()
    assert d["nccl"].tobytes() == d["whole"].tobytes()


def _comm_scene(n_dev):
    from helpers import small_scene
    from sphericalrf_b200.testbed import Renderer
    W, H = 40, 37
    sc = small_scene(kind="net", width=W, height=H)
    rs = []
    for d in range(n_dev):
        r = Renderer(sc["cfg"], d)
        r.upload_network(sc["hash_table"], sc["density_mlp"], sc["rgb_mlp"])
        r.upload_density_grid(sc["grid"]); r.update_grid_bitfield()
        rs.append(r)
    return sc, rs, W, H


@pytest.mark.parametrize("n_dev", [1, 2, 4])
def test_single_process_sharded_frames_equal_the_single_gpu_frames(built_lib, n_dev):
    """srf_comm_init + srf_render_frames_sharded: one host process, one context per GPU, pixels stored into the first
    GPU's image over peer mappings.  Three views, two passes per pixel: bytes equal to srf_render on one GPU."""
    import ctypes as C
    from sphericalrf_b200 import abi, synth
    from sphericalrf_b200.testbed import Comm
    if torch.cuda.device_count() < n_dev:
        pytest.skip(f"needs {n_dev} GPUs")
    sc, rs, W, H = _comm_scene(n_dev)
    sc["cfg"].snap_to_pixel_centers_in_rendering = 1
    post = abi.default_post()
    post.background_color[:] = [0.2, 0.4, 0.6, 1.0]
    views = [abi.make_view(synth.orbit_camera(0.5, 10.0 * k, 25.0 + 70.0 * k), W, H, synth.relative_focal_length(60.0, W, H)) for k in range(3)]
    comm = Comm(rs)
    imgs, stats = comm.render(views, post, spp=2, want_stats=True)
    assert imgs.shape == (3, H, W, 4)
    assert len(comm.timings()) == n_dev and all(t > 0 for t in comm.timings())
    assert sum(s["n_samples"] for s in stats) > 0 and all(s["error_flags"] == 0 for s in stats)
    for k, v in enumerate(views):
        whole = rs[0].render(v, post, spp=2)
        assert whole.tobytes() == imgs[k].tobytes(), f"view {k}"
    comm.close()


def test_comm_rejects_bad_arguments(built_lib):
    import ctypes as C
    from sphericalrf_b200 import abi
    sc, rs, W, H = _comm_scene(1)
    lib = rs[0].lib
    comm = C.c_void_p()
    arr = (C.c_void_p * 2)(rs[0].ctx, rs[0].ctx)
    assert lib.srf_comm_init(arr, 2, C.byref(comm)) == abi.ERR_ARG           # two contexts on one device
    assert b"one context per GPU" in lib.srf_comm_last_error(None)
    assert lib.srf_comm_init(arr, 0, C.byref(comm)) == abi.ERR_ARG
