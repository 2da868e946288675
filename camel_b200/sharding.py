"""Host-side partitioning of the hot path over the GPUs of one node (one process per GPU).

Samples of a batched forward pass and row blocks of the left GEMM operand are independent, so
most of the path shards without any exchange.  The one exchange is the reassembly of a
row-sharded product C = A.B on every rank: an all-gather of C's row blocks, issued per row panel
so that a finished panel travels while the next one is computed.  The functions here hold only
the index arithmetic and the collective calls; they work on any `torch.distributed` backend (NCCL
on the GPUs, gloo in the CPU tests) and on tensors of any device.
"""
from __future__ import annotations

from typing import List, Tuple


def batch_shard(batch: int, world: int, rank: int) -> Tuple[int, int]:
    """(first sample, count) of rank's part of a batch: contiguous, sizes differ by at most one."""
    if world <= 0 or not 0 <= rank < world or batch < 0:
        raise ValueError("bad shard request")
    base, extra = divmod(batch, world)
    first = rank * base + min(rank, extra)
    return first, base + (1 if rank < extra else 0)


def row_shard(rows: int, world: int, rank: int) -> Tuple[int, int]:
    """(first row, count) of rank's row block of A and C.  The blocks must be equal because the
    all-gather moves equal pieces."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad shard request")
    if rows % world != 0:
        raise ValueError(f"{rows} rows do not split evenly over {world} ranks")
    per = rows // world
    return rank * per, per


def panel_plan(rows: int, panels: int) -> List[Tuple[int, int]]:
    """Splits a rank's row block into at most `panels` consecutive panels (offset, count) of
    near-equal size, none empty."""
    if rows < 0 or panels <= 0:
        raise ValueError("bad panel request")
    panels = min(panels, rows) or 1
    base, extra = divmod(rows, panels)
    plan, at = [], 0
    for p in range(panels):
        cnt = base + (1 if p < extra else 0)
        if cnt:
            plan.append((at, cnt))
        at += cnt
    return plan


def tapered_panel_plan(rows: int, smallest: int = 256, unit: int = 128) -> List[Tuple[int, int]]:
    """Consecutive panels (offset, count) whose sizes halve: rows/2, rows/4, ... down to `smallest`
    (the last two about equal), sizes multiples of `unit` where the row count allows.  Panel j's
    all-gather runs while panel j+1 is computed, so only the last panel's gather is exposed:
    tapering makes that one small while the early panels stay large enough to fill the GPU."""
    if rows < 0 or smallest <= 0 or unit <= 0:
        raise ValueError("bad panel request")
    if rows <= 2 * smallest:
        return [(0, rows)] if rows else []
    sizes, left = [], rows
    while left > 2 * smallest:
        take = max(smallest, (left // 2) // unit * unit)
        sizes.append(take)
        left -= take
    half = max(unit, (left // 2) // unit * unit) if left > smallest else left
    sizes += [left - half, half] if 0 < half < left else [left]
    plan, at = [], 0
    for cnt in sizes:
        if cnt:
            plan.append((at, cnt))
            at += cnt
    assert at == rows
    return plan


def banded_rows(plan: List[Tuple[int, int]], world: int, rank: int) -> List[Tuple[int, int, int, int]]:
    """Row ownership that makes every gathered panel one contiguous band of C.

    With one contiguous row block per rank, panel j of all ranks lies in `world` separate places of
    C, and an all-gather into a list of such views goes through a temporary buffer and one copy per
    rank.  Here the rows are dealt out band by band instead: band j holds panel j of every rank,
    rank r's piece at position r inside it.  A rank still owns rows_per_rank rows of A and C (its
    pieces of all bands); each band is contiguous, so its all-gather runs in place.

    `plan` is the panel plan of one rank, [(local offset, count)].  Returns, per panel,
    (local offset, count, first global row of this rank's piece, first global row of the band)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad shard request")
    out, band0 = [], 0
    for off, cnt in plan:
        out.append((off, cnt, band0 + rank * cnt, band0))
        band0 += world * cnt
    return out


def gather_band(dist, c_full, band0: int, cnt: int, rank: int, world: int) -> None:
    """In-place all-gather of one band of C (see banded_rows): rows [band0, band0 + world*cnt), of
    which rank r's piece [band0 + r*cnt, +cnt) must already be in place on rank r."""
    band = c_full[band0: band0 + world * cnt]
    dist.all_gather_into_tensor(band, band[rank * cnt: (rank + 1) * cnt])


def gather_panel(dist, c_full, rows_per_rank: int, panel_off: int, panel_rows: int, rank: int, world: int) -> None:
    """All-gather of one row panel of the sharded product: rank r's rows
    [r*rows_per_rank + panel_off, +panel_rows) of `c_full` are filled on every rank from rank r.
    `c_full` is the full [rows_per_rank*world, n] result; this rank's own panel must already be
    in place.  The views are contiguous row ranges, so the collective moves them in place."""
    outs = [c_full[r * rows_per_rank + panel_off: r * rows_per_rank + panel_off + panel_rows] for r in range(world)]
    dist.all_gather(outs, outs[rank])


def reduce_max(dist, torch, value: float, device) -> float:
    """Largest `value` over the ranks (the time of a step is the slowest rank's)."""
    if dist is None or not dist.is_initialized():
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
