"""Host-side sharding plans for one 8xB200 box: one process per GPU.

GEMMs shard by output-column blocks (every output element is independent in the reference's
`materializec`, catena-lang/src/codegen/ops/materializec.rs:36-82) and decode attention by
(batch, kv-head) units.  The plans are pure functions of the problem and the world size; tile
shape, k order and KV split count never depend on them, which is what keeps results bitwise
identical across 1/2/4/8 GPUs.  The only collective is the final gather of the output.
"""
from dataclasses import dataclass


@dataclass(frozen=True)
class ColumnBlock:
    rank: int
    n0: int      # first output column (= first row of column-major B)
    n1: int      # one past the last


def column_blocks(n, world, align=256):
    """Splits N output columns into `world` contiguous blocks whose boundaries are multiples of the
    GEMM tile width (so a rank's tiles are exactly tiles of the unsharded problem)."""
    if world <= 0:
        raise ValueError("world must be positive")
    tiles = (n + align - 1) // align
    out = []
    for r in range(world):
        t0 = tiles * r // world
        t1 = tiles * (r + 1) // world
        out.append(ColumnBlock(r, min(n, t0 * align), min(n, t1 * align)))
    return out


@dataclass(frozen=True)
class RowBlock:
    rank: int
    m0: int      # first output row (= first row of A)
    m1: int      # one past the last


def row_blocks(m, world, align=256):
    """Splits M output rows into `world` contiguous blocks on tile boundaries.  Row blocks of a row-major C are
    contiguous in memory, so the final gather needs no repacking (column blocks do)."""
    if world <= 0:
        raise ValueError("world must be positive")
    tiles = (m + align - 1) // align
    return [RowBlock(r, min(m, tiles * r // world * align), min(m, tiles * (r + 1) // world * align)) for r in range(world)]


def _as_wire(t):
    """NCCL has no 16-bit integer type; bf16 bit patterns held as int16 travel as bfloat16 (a gather only copies bits)."""
    import torch
    return (t.view(torch.bfloat16), True) if t.dtype == torch.int16 and t.is_cuda else (t, False)


def _from_wire(t, was_int16):
    import torch
    return t.view(torch.int16) if was_int16 else t


def gather_rows(local_block, blocks, dist=None, group=None, out=None):
    """All-gathers contiguous row blocks [m1-m0, N] into the full [M, N] matrix on every rank (one collective when
    the blocks are equal, padded otherwise).  `out`: a preallocated [M, N] tensor to gather into when the blocks are
    equal (a serving loop reuses its output buffer instead of allocating one per step)."""
    import torch
    if dist is None or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return local_block
    local_block, was_int16 = _as_wire(local_block)
    heights = [b.m1 - b.m0 for b in blocks]
    if len(set(heights)) == 1:
        if out is not None:
            full = _as_wire(out)[0]
        else:
            full = torch.empty((sum(heights),) + tuple(local_block.shape[1:]), dtype=local_block.dtype, device=local_block.device)
        dist.all_gather_into_tensor(full, local_block.contiguous(), group=group)
        return _from_wire(full, was_int16)
    hmax = max(heights)
    pad = torch.zeros((hmax,) + tuple(local_block.shape[1:]), dtype=local_block.dtype, device=local_block.device)
    pad[: local_block.shape[0]] = local_block
    parts = [torch.empty_like(pad) for _ in blocks]
    dist.all_gather(parts, pad, group=group)
    return _from_wire(torch.cat([p[:h] for p, h in zip(parts, heights)], dim=0), was_int16)


@dataclass(frozen=True)
class UnitRange:
    rank: int
    u0: int
    u1: int


def unit_ranges(units, world):
    """Contiguous ranges of (batch, kv-head) units per rank."""
    if world <= 0:
        raise ValueError("world must be positive")
    return [UnitRange(r, units * r // world, units * (r + 1) // world) for r in range(world)]


@dataclass(frozen=True)
class IndexRange:
    rank: int
    i0: int
    i1: int


def index_ranges(n, world, align=1):
    """Contiguous ranges of the n independent elements of a map (`materializec`: out[i] = f(env, i)) per rank, boundaries on
    multiples of `align` elements.  Every rank runs the same kernel — or the same register program with its range's first
    index (`MapProgram.launch(i1 - i0, env, index0=i0)`) — so the bits do not depend on the world size; `gather_units` with a
    row width of 1 assembles the ranges."""
    if world <= 0:
        raise ValueError("world must be positive")
    chunks = (n + align - 1) // align
    return [IndexRange(r, min(n, chunks * r // world * align), min(n, chunks * (r + 1) // world * align)) for r in range(world)]


def gather_columns(local_block, blocks, rows, dist=None, group=None):
    """All-gathers row-major column blocks [rows, n1-n0] into the full [rows, N] matrix.
    `local_block` is a torch tensor on this rank's device; returns the assembled tensor on every rank."""
    import torch
    if dist is None or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return local_block
    local_block, was_int16 = _as_wire(local_block)
    widths = [b.n1 - b.n0 for b in blocks]
    wmax = max(widths)
    pad = torch.zeros((rows, wmax), dtype=local_block.dtype, device=local_block.device)
    pad[:, : local_block.shape[1]] = local_block
    parts = [torch.empty_like(pad) for _ in blocks]
    dist.all_gather(parts, pad, group=group)
    return _from_wire(torch.cat([p[:, :w] for p, w in zip(parts, widths)], dim=1), was_int16)


def gather_units(local_rows, ranges, row_width, dist=None, group=None, out=None):
    """All-gathers per-unit output rows (attention O) in unit order — or the elements of a map sharded by `index_ranges`, as
    rows of width 1; `out` as in gather_rows."""
    import torch
    if dist is None or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return local_rows
    local_rows, was_int16 = _as_wire(local_rows)
    counts = [(r.u1 - r.u0) if isinstance(r, UnitRange) else (r.i1 - r.i0) for r in ranges]
    if len(set(counts)) == 1:                                  # equal ranges: one collective straight into place
        full = _as_wire(out)[0] if out is not None else torch.empty((sum(counts), row_width), dtype=local_rows.dtype, device=local_rows.device)
        dist.all_gather_into_tensor(full, local_rows.contiguous(), group=group)
        return _from_wire(full, was_int16)
    cmax = max(counts)
    pad = torch.zeros((cmax, row_width), dtype=local_rows.dtype, device=local_rows.device)
    pad[: local_rows.shape[0]] = local_rows
    parts = [torch.empty_like(pad) for _ in ranges]
    dist.all_gather(parts, pad, group=group)
    return _from_wire(torch.cat([p[:c] for p, c in zip(parts, counts)], dim=0), was_int16)


def max_over_ranks(ms, dist=None, device="cpu"):
    """Device-timed milliseconds -> max over ranks (the number every multi-GPU figure is quoted on)."""
    import torch
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(ms)
    t = torch.tensor([float(ms)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
