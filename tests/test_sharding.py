"""Column-shard arithmetic (CPU) and a world_size-2 gloo run of the sharded operator with the
oracle standing in for the GPU kernel: shards + all-gather must equal the unsharded result."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from amd_developer_challenge_2025_b200.inputs import make_inputs
from amd_developer_challenge_2025_b200.sharding import shard_inputs, shard_spec
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


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, m, n, k, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        a, b, a_s, b_s, _ = make_inputs(m, n, k, seed=77)
        spec = shard_spec(n, world, rank)
        bb, bs = shard_inputs(b, b_s, spec)
        mine = oracle.dequant_matmul(a, bb.contiguous(), a_s, bs.contiguous(), spec.n_phase)
        # all_gather concatenates along dim 0: gather [world][M][N/world] and re-interleave
        gathered = torch.empty(world * m, spec.n_local, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(gathered, mine.contiguous())
        c = gathered.view(world, m, spec.n_local).permute(1, 0, 2).reshape(m, n)
        full = oracle.dequant_matmul(a, b, a_s, b_s)
        if rank == 0:
            out.put(bool(torch.equal(c.view(torch.int16), full.view(torch.int16))))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_gather_equals_unsharded():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, 8, 1152, 256, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert out.get(timeout=5) is True
