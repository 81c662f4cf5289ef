"""Work partition of the KDA op over the GPUs of one node.

KDA is independent per (sequence, head), and the reference's own parallelism is plain data
parallel (k3mini/training.py:192-197), so every rank gets whole sequences and the kernel path
needs no collective.  Batches are split batch-major; packed documents (``cu_seqlens``) are
dealt to ranks so that token counts balance, because the state kernels cost time in
proportion to a rank's longest chain of chunks."""

from __future__ import annotations


def shard_batch(batch: int, world: int, rank: int) -> range:
    """Contiguous slice of the batch for this rank; the first ``batch % world`` ranks get one more."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    base, extra = divmod(batch, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def shard_documents(lengths, world: int, rank: int) -> list[int]:
    """Indices of the documents this rank processes: longest-first greedy assignment to the
    least loaded rank (ties to the lower rank), returned in ascending order.  Deterministic,
    so every rank computes the same table without talking to the others."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    load = [0] * world
    owner = {}
    for idx in sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i)):
        r = min(range(world), key=lambda x: (load[x], x))
        owner[idx] = r
        load[r] += int(lengths[idx])
    return sorted(i for i, r in owner.items() if r == rank)


def aggregate_throughput(local_ms: float, tokens_per_rank: int, steps: int, world: int, reduce_max=None) -> float:
    """Whole-job tokens per second: every rank's tokens over the slowest rank's time.
    ``reduce_max`` maps the local time to the maximum over ranks (identity on one rank)."""
    ms = reduce_max(local_ms) if reduce_max is not None else local_ms
    return world * tokens_per_rank * steps / (ms / 1e3)
