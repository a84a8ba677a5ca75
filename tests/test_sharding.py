"""Multi-GPU host logic on CPU: partitioning, and the one exchange step of the decode path over a world_size-2 gloo
group (the oracle stands in for the per-rank kernels)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def test_tile_row_ranges(pkg):
    sh = pkg.sharding
    for rows, world in ((768, 8), (768, 1), (10, 4), (3, 8), (1792, 3)):
        spans = [sh.tile_row_range(rows, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == rows
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [e - b for b, e in spans]
        assert max(sizes) - min(sizes) <= 1
    assert sh.block_row_range(57344, 3, 8) == (3 * 7168, 7168)
    with pytest.raises(ValueError):
        sh.block_row_range(96, 0, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import __graft_entry__ as g
    pkg = g.load_package()
    from oracle.oracle import Oracle
    O = Oracle()
    s = pkg.synth
    tl = s.seeded_tlut(1).view(np.uint16)
    # decode: each rank multiplies its contiguous block-rows, z slices are all-gathered (rank-major = row order)
    n_in, n_out = 384, 128
    tr = s.random_trellis(n_out, n_in, 9)
    u = s.bf16_bits_to_f32(s.f32_to_bf16_bits(np.random.default_rng(3).standard_normal(n_in).astype(np.float32)))
    row0, rows = pkg.sharding.block_row_range(n_out, rank, world)
    per = (n_in // 32) * 128
    shard = tr[(row0 // 32) * per:((row0 + rows) // 32) * per]
    z_local = O.decode_rows(shard, n_in, rows, tl, 0, rows, True).astype(np.float64) @ u
    parts = [torch.zeros(rows, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(z_local))
    z = torch.cat(parts).numpy()
    z_full = O.decode_rows(tr, n_in, n_out, tl, 0, n_out, True).astype(np.float64) @ u
    assert np.array_equal(z, z_full)
    # encode: tile rows split over ranks, no exchange; the concatenation equals the single-rank result
    W = s.gaussian_matrix(64, 32, 2)
    lut, _ = O.build_lut(tl)
    b, e = pkg.sharding.tile_row_range(64 // 16, rank, world)
    st_local, _ = O.quantize_tiles(s.tile_sequences(W[16 * b:16 * e]), lut)
    np.save(os.path.join(out_dir, "st_%d.npy" % rank), st_local)
    dist.barrier()
    if rank == 0:
        st = np.concatenate([np.load(os.path.join(out_dir, "st_%d.npy" % r)) for r in range(world)])
        st_full, _ = O.quantize_tiles(s.tile_sequences(W), lut)
        assert np.array_equal(st, st_full)
    dist.destroy_process_group()


def test_two_rank_gloo(tmp_path):
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
