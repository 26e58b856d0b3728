"""How the benchmark workloads are split over ranks (one process per GPU).

Config 3 (one large mul): the destination columns are cut into equal contiguous blocks; with a
column-major destination a rank's block is one contiguous byte range of the full destination, so the
gather is an in-place all-gather with no repacking.  Config 2 (many independent muls): contiguous ranges
of the mul index; no exchange at all."""


def column_shard(cols, rank, world):
    """(first column, column count) of `rank`; cols must divide evenly so that shards are equal-sized."""
    if cols % world:
        raise ValueError(f"{cols} columns do not split evenly over {world} ranks")
    per = cols // world
    return rank * per, per


def mul_range(n, rank, world):
    """(first mul, count) of `rank` for n independent muls; the last ranks may get fewer."""
    per = (n + world - 1) // world
    first = min(n, rank * per)
    return first, max(0, min(per, n - first))
