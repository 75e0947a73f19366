"""Row sharding of a matrix product across the GPUs of one box.

The product shards along M: rank r owns a contiguous block of rows of A and of C, B is replicated, and no
rank needs another rank's data to compute its block.  The only exchange the path ever has is the optional
all-gather of the C blocks afterwards, for which blocks are laid out in rank order (block r starts at row
`row_shard(m, world, r)[0]` of the gathered matrix)."""
from __future__ import annotations

TILE_ROWS = 128  # rows of one CTA tile: shard boundaries sit on tile boundaries so that no tile is split


def row_shard(m: int, world: int, rank: int, align: int = TILE_ROWS) -> tuple[int, int]:
    """(first row, row count) of `rank`'s block when `m` rows are split over `world` ranks.

    Rows are dealt out in units of `align`: every rank gets floor(units / world) units, the first
    (units mod world) ranks one more; the last rank's block ends at m (it may hold a ragged unit).
    A rank can end up with no rows when there are fewer units than ranks."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank out of range")
    if m < 0 or align <= 0:
        raise ValueError("negative size")
    units = -(-m // align)
    base, extra = divmod(units, world)
    first_unit = rank * base + min(rank, extra)
    unit_count = base + (1 if rank < extra else 0)
    first = min(first_unit * align, m)
    last = min((first_unit + unit_count) * align, m)
    return first, last - first


def shard_table(m: int, world: int, align: int = TILE_ROWS) -> list[tuple[int, int]]:
    """All ranks' blocks; they are disjoint, in rank order, and cover [0, m)."""
    return [row_shard(m, world, r, align) for r in range(world)]


def equal_shards(m: int, world: int, align: int = TILE_ROWS) -> bool:
    """True when every rank holds the same number of rows (what an in-place all-gather needs)."""
    return len({rows for _, rows in shard_table(m, world, align)}) == 1


def broadcast_from_rank0(dist):
    """An `exchange` for `Communicator` and friends built on a torch.distributed process group of any backend: returns
    a function that hands rank 0's bytes to every rank."""

    def exchange(payload):
        box = [payload if dist.get_rank() == 0 else None]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    return exchange


def allgather_objects(dist):
    """An `exchange` for `GatheredMatrix`: every rank's bytes, in rank order, on every rank."""

    def exchange(payload):
        everyone = [None] * dist.get_world_size()
        dist.all_gather_object(everyone, payload)
        return everyone

    return exchange
