"""Two gloo ranks on the CPU: each renders its row-block shard of a frame (with the oracle standing
in for the GPU library) and the tiles are gathered and assembled on rank 0 by the same TileGather
the benchmark uses.  The assembled image must equal the single-rank frame byte for byte."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT)); sys.path.insert(0, str(ROOT / "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import srf_oracle
    from sphericalrf_b200 import abi
    from sphericalrf_b200.sharding import TileGather
    from helpers import make_oracle, small_scene
    sc = small_scene(kind="blobs", width=16, height=21, sampling="Original", radius=4.0)
    orc = make_oracle(srf_oracle, sc, None)
    bits, _ = orc.update_grid_bitfield(sc["grid"])
    orc.bitfield = bits
    tg = TileGather(16, 21, n_views=2, channels=4, shard_rows=4, device="cpu")
    for k in range(2):
        v = abi.View.from_buffer_copy(sc["view"])
        v.shard_rows, v.shard_count, v.shard_rank = 4, world, rank
        v.spp_index = k
        res = orc.render_frame(v, abi.default_post())
        assert res["out"].shape[0] == tg.n_local
        tg.tiles[k, : tg.n_local] = torch.from_numpy(res["out"])
    img = tg.gather()
    if rank == 0:
        np.save(os.path.join(tmp, "gathered.npy"), img.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gather_equals_whole_frame(tmp_path, oracle_mod):
    sys.path.insert(0, str(ROOT / "tests"))
    from sphericalrf_b200 import abi
    from helpers import make_oracle, small_scene
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    got = np.load(tmp_path / "gathered.npy")
    sc = small_scene(kind="blobs", width=16, height=21, sampling="Original", radius=4.0)
    orc = make_oracle(oracle_mod, sc, None)
    bits, _ = orc.update_grid_bitfield(sc["grid"])
    orc.bitfield = bits
    for k in range(2):
        v = abi.View.from_buffer_copy(sc["view"])
        v.spp_index = k
        whole = orc.render_frame(v, abi.default_post())["out"]
        assert got[k].tobytes() == whole.tobytes()


def _replicate_worker(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from sphericalrf_b200.sharding import broadcast_arrays, reduce_counters
    arrays = None
    if rank == 0:
        rng = np.random.Generator(np.random.PCG64(5))
        arrays = {"hash_table": rng.standard_normal(1000).astype(np.float16), "density_grid": rng.random((8, 8, 8)).astype(np.float32),
                  "bitfield": rng.integers(0, 256, 64, dtype=np.uint8)}
    got = broadcast_arrays(arrays, src=0)
    np.savez(os.path.join(tmp, f"rank{rank}.npz"), **got)
    total = reduce_counters({"n_rays": 10 + rank, "n_samples": 1000 * (rank + 1), "ms": 1.5}, dst=0)
    if rank == 0:
        assert total == {"n_rays": 21, "n_samples": 3000}
    else:
        assert total is None
    dist.barrier()
    dist.destroy_process_group()


def test_load_time_replication_and_counter_reduction(tmp_path):
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    mp.spawn(_replicate_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    a, b = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    assert sorted(a.files) == sorted(b.files) == ["bitfield", "density_grid", "hash_table"]
    for k in a.files:
        assert a[k].dtype == b[k].dtype and a[k].shape == b[k].shape and a[k].tobytes() == b[k].tobytes()
    assert a["density_grid"].shape == (8, 8, 8) and a["hash_table"].dtype == np.float16
