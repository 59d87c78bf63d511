"""Column-shard arithmetic (CPU) and a world_size-2 gloo run of the sharded operator with the
oracle standing in for the GPU kernel: shards + all-gather must equal the unsharded result."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from amd_developer_challenge_2025_b200.inputs import make_inputs
from amd_developer_challenge_2025_b200.sharding import (choose_grid, gather_c, grid_inputs, grid_spec, shard_inputs,
                                                      shard_spec)
from oracle import fp8_mm_oracle as oracle


def test_spec_4608_over_8_ranks():
    for r in range(8):
        s = shard_spec(4608, 8, r)
        assert s.n_local == 576
        assert s.n_phase == (64 if r % 2 else 0)
        assert s.scale_row_end - s.scale_row_begin == 5
        assert s.scale_row_begin == (576 * r) // 128
    assert [shard_spec(4608, 4, r).n_phase for r in range(4)] == [0, 0, 0, 0]
    assert shard_spec(4608, 1, 0).scale_row_end == 36


def test_spec_rejects_bad_splits():
    with pytest.raises(ValueError):
        shard_spec(100, 8, 0)      # not a multiple of 32
    with pytest.raises(ValueError):
        shard_spec(4608, 8, 8)     # rank out of range
    with pytest.raises(ValueError):
        shard_spec(128, 4, 0)      # two 64-column units cannot feed four ranks


def test_uneven_units_576_over_8():
    specs = [shard_spec(576, 8, r) for r in range(8)]
    assert [s.n_local for s in specs] == [128] + [64] * 7
    assert specs[0].col_begin == 0 and specs[-1].col_end == 576
    for a, b in zip(specs, specs[1:]):
        assert a.col_end == b.col_begin
    assert all(s.n_phase in (0, 64) for s in specs)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_shards_tile_the_columns_and_reproduce_the_full_result(world):
    m, n, k = 16, 576, 256
    a, b, a_s, b_s, _ = make_inputs(m, n, k, seed=21)
    full = oracle.dequant_matmul(a, b, a_s, b_s)
    cols = []
    for r in range(world):
        s = shard_spec(n, world, r)
        bb, bs = shard_inputs(b, b_s, s)
        assert bs.shape[0] == (s.n_local + s.n_phase + 127) // 128
        cols.append(oracle.dequant_matmul(a, bb, a_s, bs, s.n_phase))
    assert torch.equal(torch.cat(cols, dim=1).view(torch.int16), full.view(torch.int16))


@pytest.mark.parametrize("gm,gn", [(1, 4), (2, 2), (4, 1), (3, 2), (2, 4)])
def test_grid_blocks_tile_c_and_reproduce_the_full_result(gm, gn):
    m, n, k = 520, 576, 256   # 5 row blocks (the last one short), 9 column units
    a, b, a_s, b_s, _ = make_inputs(m, n, k, seed=33)
    full = oracle.dequant_matmul(a, b, a_s, b_s)
    got = torch.full((m, n), float("nan"), dtype=torch.bfloat16)
    covered = torch.zeros(m, n, dtype=torch.int32)
    for r in range(gm * gn):
        s = grid_spec(m, n, gm * gn, r, gm, gn)
        aa, bb, aas, bs = grid_inputs(a, b, a_s, b_s, s)
        assert aa.shape[0] == s.m_local and bb.shape[0] == s.n_local and s.row_begin % 128 == 0
        got[s.row_begin:s.row_end, s.cols.col_begin:s.cols.col_end] = oracle.dequant_matmul(aa, bb, aas, bs, s.n_phase)
        covered[s.row_begin:s.row_end, s.cols.col_begin:s.cols.col_end] += 1
    assert bool((covered == 1).all())
    assert torch.equal(got.view(torch.int16), full.view(torch.int16))


def test_choose_grid_minimises_the_slowest_rank():
    # a cost that only counts whole waves of 128 x 128 tiles on 4 "SMs"
    waves = lambda m, n, k: -(-(-(-m // 128) * -(-n // 128)) // 4) * k
    assert choose_grid(1024, 256, 128, 4, estimate=waves) in ((2, 2), (4, 1))   # 4 tiles per rank either way
    assert choose_grid(128, 4096, 128, 4, estimate=waves) == (1, 4)            # one row block: columns only
    assert choose_grid(4096, 64, 128, 4, estimate=waves) == (4, 1)             # one column unit: rows only
    with pytest.raises(ValueError):
        choose_grid(128, 64, 128, 4, estimate=waves)                           # nothing to cut four ways
    with pytest.raises(ValueError):
        grid_spec(1024, 1024, 4, 0, 3, 2)


def test_choose_grid_with_the_library_model(built_library):
    # the headline GEMM over 8 GPUs: 4 x 2 gives every GPU one wave of 256 x 256 pair tiles
    assert choose_grid(8192, 4608, 7168, 8) == (4, 2)
    assert choose_grid(8192, 4608, 7168, 1) == (1, 1)
    import amd_developer_challenge_2025_b200 as pkg
    assert pkg.estimate_clocks(8192, 4608, 7168) > pkg.estimate_clocks(2048, 2304, 7168) * 7
    with pytest.raises(Exception):
        pkg.estimate_clocks(128, 128, 100)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, m, n, k, grid, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        a, b, a_s, b_s, _ = make_inputs(m, n, k, seed=77)
        if grid is None:
            spec = shard_spec(n, world, rank)   # the one-dimensional column scheme
            bb, bs = shard_inputs(b, b_s, spec)
            mine = oracle.dequant_matmul(a, bb.contiguous(), a_s, bs.contiguous(), spec.n_phase)
        else:
            spec = grid_spec(m, n, world, rank, *grid)
            aa, bb, aas, bs = grid_inputs(a, b, a_s, b_s, spec)
            mine = oracle.dequant_matmul(aa, bb, aas, bs, spec.n_phase)
        c = gather_c(mine, spec, m, n)
        full = oracle.dequant_matmul(a, b, a_s, b_s)
        out.put((rank, bool(torch.equal(c.view(torch.int16), full.view(torch.int16)))))
        dist.barrier()
    finally:
        dist.destroy_process_group()


# (world, m, n, k, grid): column shards of equal width; a 2 x 1 row cut; a 2 x 2 grid whose row blocks are
# uneven (5 row units over 2) and whose column blocks are uneven too (9 column units over 2)
@pytest.mark.parametrize("world,m,n,k,grid", [(2, 8, 1152, 256, None), (2, 256, 256, 128, (2, 1)),
                                              (4, 520, 576, 128, (2, 2))])
def test_gloo_ranks_gather_equals_unsharded(world, m, n, k, grid):
    """The oracle stands in for the kernel on each rank; what is tested is the shard arithmetic and
    gather_c's collective + re-interleave, on every rank."""
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, m, n, k, grid, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    got = sorted(out.get(timeout=5) for _ in range(world))
    assert got == [(r, True) for r in range(world)]
