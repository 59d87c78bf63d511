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


# ---------------------------------------------------------------------------------------------
# Two-dimensional sharding: a grid of row blocks x column blocks
# ---------------------------------------------------------------------------------------------
# Every output tile is independent, so the ranks may also cut c along M: rank (i, j) of a
# grid_m x grid_n grid owns row block i (its rows of a and a_scale) and column block j (as above).
# Still no data-path collective. Which grid is best depends on how the per-rank problem fills the
# SMs: 8192 x 4608 x 7168 over 8 GPUs as 1 x 8 leaves each GPU 2.2 waves of work, as 4 x 2 each
# GPU gets 2048 x 2304 = 72 pair tiles of 256 x 256 on 74 SM pairs, one wave.


@dataclass(frozen=True)
class GridSpec:
    rank: int
    world: int
    grid_m: int
    grid_n: int
    row_begin: int
    row_end: int
    cols: ShardSpec  # the column block, as for one-dimensional sharding over grid_n ranks

    @property
    def m_local(self) -> int:
        return self.row_end - self.row_begin

    @property
    def n_local(self) -> int:
        return self.cols.n_local

    @property
    def n_phase(self) -> int:
        return self.cols.n_phase


def _row_range(m: int, parts: int, index: int):
    """Rows dealt in units of 128 (one tile row); the first blocks get one unit more when uneven."""
    units = -(-m // 128)
    if units < parts:
        raise ValueError(f"M={m} has only {units} row blocks for {parts} row shards")
    base, extra = divmod(units, parts)
    u0 = index * base + min(index, extra)
    u1 = u0 + base + (1 if index < extra else 0)
    return u0 * 128, min(u1 * 128, m)


def grid_spec(m: int, n: int, world: int, rank: int, grid_m: int, grid_n: int) -> GridSpec:
    """The block of rank `rank` in a grid_m x grid_n grid (rank = i * grid_n + j)."""
    if grid_m * grid_n != world or not (0 <= rank < world):
        raise ValueError("grid does not match world, or bad rank")
    i, j = divmod(rank, grid_n)
    r0, r1 = _row_range(m, grid_m, i)
    return GridSpec(rank, world, grid_m, grid_n, r0, r1, shard_spec(n, grid_n, j))


def choose_grid(m: int, n: int, k: int, world: int, estimate=None):
    """(grid_m, grid_n) with grid_m * grid_n = world that minimises the slowest rank's estimated time.
    `estimate(m, n, k) -> cost` defaults to the library's own model (b200_fp8_mm_estimate_clocks);
    ties go to the grid with fewer row shards (a is then replicated rather than cut, as in the
    one-dimensional scheme)."""
    if estimate is None:
        from .fp8_mm import estimate_clocks as estimate
    best = None
    for gm in range(1, world + 1):
        if world % gm:
            continue
        gn = world // gm
        try:
            worst = max(estimate(s.m_local, s.n_local, k)
                        for s in (grid_spec(m, n, world, r, gm, gn) for r in range(world)))
        except ValueError:
            continue
        if best is None or worst < best[0] * (1 - 1e-9):
            best = (worst, gm, gn)
    if best is None:
        raise ValueError(f"no grid of {world} ranks fits M={m}, N={n}")
    return best[1], best[2]


def grid_inputs(a, b, a_scale, b_scale, spec: GridSpec):
    """The (a, b, a_scale, b_scale) blocks rank `spec.rank` holds. Views."""
    bb, bs = shard_inputs(b, b_scale, spec.cols)
    return a[spec.row_begin : spec.row_end], bb, a_scale[spec.row_begin : spec.row_end], bs


# ---------------------------------------------------------------------------------------------
# Optional all-gather of c
# ---------------------------------------------------------------------------------------------


def gather_c(c_local, spec, m: int, n: int, group=None):
    """All-gathers the ranks' blocks of c into the whole [m, n] matrix on every rank.

    `spec` is this rank's GridSpec (or a ShardSpec for the one-dimensional column scheme). One
    collective: `all_gather_into_tensor` of the blocks (padded to the largest block when the cut is
    uneven), then a local re-interleave, since rank r's block is a rectangle of c, not a run of its
    rows. Column shards of equal width need no padding and the re-interleave is one permute. Works
    with any torch.distributed backend (NCCL over NVLink on the GPUs; gloo in the CPU tests)."""
    import torch
    import torch.distributed as dist

    if isinstance(spec, ShardSpec):
        spec = GridSpec(spec.rank, spec.world, 1, spec.world, 0, m, spec)
    world = spec.world
    if world == 1:
        return c_local
    if tuple(c_local.shape) != (spec.m_local, spec.n_local):
        raise ValueError("c_local does not have the shape of this rank's block")
    blocks = [grid_spec(m, n, world, r, spec.grid_m, spec.grid_n) for r in range(world)]
    m_max = max(b.m_local for b in blocks)
    n_max = max(b.n_local for b in blocks)
    uniform = all(b.m_local == m_max and b.n_local == n_max for b in blocks)
    if uniform:
        send = c_local.contiguous()
    else:
        send = c_local.new_zeros(m_max, n_max)
        send[: spec.m_local, : spec.n_local] = c_local
    flat = c_local.new_empty(world * m_max, n_max)  # the blocks end to end along dim 0
    dist.all_gather_into_tensor(flat, send, group=group)
    recv = flat.view(world, m_max, n_max)
    if uniform:
        # [grid_m, grid_n, m_loc, n_loc] -> [grid_m, m_loc, grid_n, n_loc] -> [m, n]
        return recv.view(spec.grid_m, spec.grid_n, m_max, n_max).permute(0, 2, 1, 3).reshape(m, n)
    out = c_local.new_empty(m, n)
    for r, b in enumerate(blocks):
        out[b.row_begin : b.row_end, b.cols.col_begin : b.cols.col_end] = recv[r, : b.m_local, : b.n_local]
    return out
