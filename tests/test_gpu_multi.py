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
