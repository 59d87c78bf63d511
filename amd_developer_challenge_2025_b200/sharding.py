"""Column (N) sharding of b and b_scale across the GPUs of one box.

The reference has no multi-GPU code. Output columns are independent, so rank r of g
owns columns [r*N/g, (r+1)*N/g) of c: the matching rows of b and the rows of b_scale
that cover them. When N/g is not a multiple of 128 a shard can start inside a scale
block (N=4608, g=8: 576 columns per rank, odd ranks start 64 columns in); the kernel
then needs `n_phase` = first column mod 128 and indexes b_scale with
(local column + n_phase) // 128, where the reference kernels index a whole matrix with
column // 128 (1-amd-fp8-mm/amd-fp8-mm-submission.py:75, 316)."""
from __future__ import annotations

from dataclasses import dataclass

SCALE_BLOCK = 128


@dataclass(frozen=True)
class ShardSpec:
    rank: int
    world: int
    col_begin: int      # first global column owned
    col_end: int        # one past the last
    n_phase: int        # col_begin % 128
    scale_row_begin: int
    scale_row_end: int  # one past the last b_scale row that covers the shard

    @property
    def n_local(self) -> int:
        return self.col_end - self.col_begin


def shard_spec(n: int, world: int, rank: int) -> ShardSpec:
    """Columns of rank `rank` of `world`. Columns are dealt in units of 64 (32 when N is not a
    multiple of 64) so that every shard starts on a boundary the kernel's n_phase can express;
    when the units do not divide evenly the first ranks get one unit more (N=576 over 8 ranks:
    128 columns on rank 0, 64 on the others)."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad rank/world")
    unit = 64 if n % 64 == 0 else 32
    if n % unit != 0:
        raise ValueError(f"N={n} is not a multiple of 32: shards could not start on an n_phase boundary")
    units = n // unit
    if units < world:
        raise ValueError(f"N={n} has only {units} shardable units for {world} ranks")
    base, extra = divmod(units, world)
    u0 = rank * base + min(rank, extra)
    u1 = u0 + base + (1 if rank < extra else 0)
    c0, c1 = u0 * unit, u1 * unit
    return ShardSpec(rank, world, c0, c1, c0 % SCALE_BLOCK, c0 // SCALE_BLOCK, (c1 - 1) // SCALE_BLOCK + 1)


def shard_inputs(b, b_scale, spec: ShardSpec):
    """The (b, b_scale) rows rank `spec.rank` holds. Views; call .contiguous() to own them."""
    return b[spec.col_begin : spec.col_end], b_scale[spec.scale_row_begin : spec.scale_row_end]
