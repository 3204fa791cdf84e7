"""Ray sharding across ranks and the gather of rendered tiles.

A frame's rays are cut into blocks of `shard_rows` image rows; block b belongs to rank
b % world.  Every rank renders its blocks into a compact tile buffer (blocks concatenated, the
layout srf_render_frame writes) and rank 0 gathers the tiles and scatters them back into image
order.  The per-ray arithmetic does not depend on the partition, so the assembled image is
byte-identical to the single-rank image.  The only exchange step is this gather; weights, grid
and bitfield are replicated.

Two ways to move the tiles:
  PeerImage  -- the output stage of the render kernel stores every pixel directly at its position in
                rank 0's image over NVLink (srf_render_frame_scatter on a peer-mapped buffer from torch's
                symmetric memory), followed by one barrier: no staging tile, no collective, no un-interleave;
  TileGather -- NCCL/gloo `gather` of padded tiles + scatter into image order on rank 0 (works everywhere,
                used by the CPU tests).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_row_indices(height: int, shard_rows: int, world: int, rank: int):
    """Image rows owned by `rank`, in the order they appear in its tile buffer."""
    return [y for y in range(height) if (y // shard_rows) % world == rank]


def shard_ray_count(width: int, height: int, shard_rows: int, world: int, rank: int) -> int:
    return len(shard_row_indices(height, shard_rows, world, rank)) * width


class TileGather:
    """Gathers per-rank tile buffers (n_views, n_local_rays, C) on rank 0 and assembles images.

    Tiles are padded to the largest shard so that every rank contributes an equal-sized buffer
    (a plain `gather`); the padding rows are never read."""

    def __init__(self, width: int, height: int, n_views: int, channels: int = 4, shard_rows: int = 8,
                 device="cpu", dtype=torch.float32, group=None):
        self.width, self.height, self.n_views, self.channels = width, height, n_views, channels
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.counts = [shard_ray_count(width, height, shard_rows, self.world, r) for r in range(self.world)]
        self.n_local = self.counts[self.rank]
        self.n_pad = max(self.counts)
        self.device = torch.device(device)
        # the tile buffer the renderer writes into
        self.tiles = torch.zeros((n_views, self.n_pad, channels), dtype=dtype, device=self.device)
        self.image = None
        self._recv = None
        self._pix = None
        if self.rank == 0:
            self.image = torch.zeros((n_views, height * width, channels), dtype=dtype, device=self.device)
            if self.world > 1:
                self._recv = [torch.zeros_like(self.tiles) for _ in range(self.world)]
            cols = torch.arange(width, device=self.device)[None, :]
            self._pix = []
            for r in range(self.world):
                rows = torch.tensor(shard_row_indices(height, shard_rows, self.world, r), dtype=torch.int64, device=self.device)
                self._pix.append((rows[:, None] * width + cols).reshape(-1))

    def gather(self):
        """Collective: after it, rank 0's `image` holds the n_views assembled images."""
        if self.world == 1:
            self.image[:, self._pix[0]] = self.tiles[:, : self.counts[0]]
            return self.image
        dist.gather(self.tiles, self._recv if self.rank == 0 else None, dst=0, group=self.group)
        if self.rank == 0:
            for r in range(self.world):
                self.image[:, self._pix[r]] = self._recv[r][:, : self.counts[r]]
        return self.image


class PeerImage:
    """n_views whole images on rank 0 that every rank's output stage writes into with plain peer stores.

    Every rank allocates the same symmetric buffer (the rendezvous is symmetric); only rank 0's copy
    receives pixels.  `root` is this rank's view of rank 0's buffer; `barrier()` orders all ranks' stores
    before rank 0 reads `local`.  NVLink multicast objects are not used (plain stores only)."""

    def __init__(self, width: int, height: int, n_views: int, device, group=None):
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        shape = (n_views, height * width, 4)
        self.local = symm_mem.empty(shape, dtype=torch.float32, device=torch.device(device))
        self.local.zero_()
        self.handle = symm_mem.rendezvous(self.local, self.group)
        self.root = self.handle.get_buffer(0, shape, torch.float32)

    def barrier(self):
        self.handle.barrier()


def broadcast_arrays(arrays, src: int = 0, device="cpu", group=None):
    """Replication at load time: rank `src` holds a dict name -> numpy array (hash table, MLP weights, density
    grid, ...); every rank returns the same dict.  One broadcast of the directory (names, dtypes, shapes)
    and one per array; other ranks pass None."""
    import numpy as np
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return arrays
    rank = dist.get_rank(group)
    directory = [None]
    if rank == src:
        directory = [[(k, str(np.asarray(v).dtype), tuple(np.asarray(v).shape)) for k, v in arrays.items()]]
    dist.broadcast_object_list(directory, src=src, group=group)
    out = {}
    for name, dtype, shape in directory[0]:
        nbytes = int(np.prod(shape, dtype=np.int64)) * np.dtype(dtype).itemsize
        if rank == src:
            t = torch.from_numpy(np.ascontiguousarray(arrays[name]).reshape(-1).view(np.uint8).copy()).to(device)
        else:
            t = torch.empty(nbytes, dtype=torch.uint8, device=device)
        dist.broadcast(t, src=src, group=group)
        out[name] = t.cpu().numpy().view(np.dtype(dtype)).reshape(shape)
    return out


def reduce_counters(stats: dict, dst: int = 0, device="cpu", group=None):
    """Sum of per-rank frame counters (rays, march steps, samples, ...) on rank `dst`; other ranks get None."""
    keys = sorted(k for k, v in stats.items() if isinstance(v, int))
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return {k: stats[k] for k in keys}
    t = torch.tensor([stats[k] for k in keys], dtype=torch.int64, device=device)
    dist.reduce(t, dst=dst, op=dist.ReduceOp.SUM, group=group)
    return dict(zip(keys, t.tolist())) if dist.get_rank(group) == dst else None
