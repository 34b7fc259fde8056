"""Host-side sharding logic on CPU: index arithmetic, and the blur halo exchange as two gloo
ranks (the per-band compute is the CPU oracle here; on GPUs it is the C ABI)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gern_b200 import sharding


def test_row_blocks_cover_without_overlap():
    for total in (0, 1, 7, 8, 65536, 8191):
        for world in (1, 2, 3, 4, 8):
            blocks = [sharding.row_block(total, world, r) for r in range(world)]
            assert blocks[0][0] == 0 and blocks[-1][1] == total
            for a, b in zip(blocks, blocks[1:]):
                assert a[1] == b[0]
            sizes = [e - b for b, e in blocks]
            assert max(sizes) - min(sizes) <= 1


def test_blur_bands_partition_the_output():
    for in_rows in (8192, 8190, 1001, 16):
        for world in (1, 2, 4, 8):
            bands = [sharding.blur_band(in_rows, world, r) for r in range(world)]
            assert bands[0].out_begin == 0 and bands[-1].out_end == in_rows - 2
            for a, b in zip(bands, bands[1:]):
                assert a.out_end == b.out_begin and a.halo_rows == 2
                assert a.out_end + 2 <= b.in_begin + 2 <= in_rows   # halo rows exist in the next band
            assert bands[-1].halo_rows == 0
            assert not bands[0].sends_halo and all(b.sends_halo for b in bands[1:])
    with pytest.raises(ValueError):
        sharding.blur_band(6, 4, 0)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _blur_worker(rank, world, port, in_rows, cols, out_path):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle import pyoracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    oracle = pyoracle.Oracle()
    full = np.random.default_rng(42).random((in_rows, cols), dtype=np.float32)   # same on all ranks
    band = sharding.blur_band(in_rows, world, rank)
    own = torch.from_numpy(full[band.in_begin:band.in_end].copy())
    halo = torch.empty((2, cols), dtype=torch.float32)
    for w in sharding.exchange_blur_halo(dist, band, own[0:2].contiguous(), halo):
        w.wait()
    stacked = torch.cat([own, halo]) if band.recvs_halo else own
    out = oracle.blur_xy(np.ascontiguousarray(stacked.numpy()))
    assert out.shape[0] == band.out_rows
    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    if rank == 0:
        np.save(out_path, np.concatenate(gathered))
    dist.destroy_process_group()


@pytest.mark.parametrize("world,in_rows", [(2, 67), (2, 64), (3, 100)])
def test_blur_halo_exchange_two_ranks_gloo(tmp_path, oracle, world, in_rows):
    cols = 131
    out_path = str(tmp_path / "out.npy")
    mp.spawn(_blur_worker, args=(world, _free_port(), in_rows, cols, out_path), nprocs=world, join=True)
    full = np.random.default_rng(42).random((in_rows, cols), dtype=np.float32)
    assert np.array_equal(np.load(out_path), oracle.blur_xy(full))


def _rows_worker(rank, world, port, out_path):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle import pyoracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    oracle = pyoracle.Oracle()
    x = (np.random.default_rng(1).standard_normal((37, 300)) * 3).astype(np.float32)
    b, e = sharding.row_block(x.shape[0], world, rank)
    part = oracle.softmax_rows(np.ascontiguousarray(x[b:e]))
    gathered = [None] * world
    dist.all_gather_object(gathered, part)
    if rank == 0:
        np.save(out_path, np.concatenate(gathered))
    dist.destroy_process_group()


def test_row_sharded_softmax_two_ranks_gloo(tmp_path, oracle):
    out_path = str(tmp_path / "sm.npy")
    mp.spawn(_rows_worker, args=(2, _free_port(), out_path), nprocs=2, join=True)
    x = (np.random.default_rng(1).standard_normal((37, 300)) * 3).astype(np.float32)
    assert np.array_equal(np.load(out_path), oracle.softmax_rows(x))
