"""Request sharding for more than one GPU.

Every (request, KV head) pair of the block-sparse path is independent: no stage needs another request's K/V,
scores or page lists.  A batch therefore spreads over N processes (one per GPU) by giving each a subset of the
requests, with no collective on the data path; each rank runs the unchanged single-GPU pipeline on its subset.
The reference has no multi-GPU layer of its own (its callers shard by request or by head in the serving engine),
so this module only provides the deterministic host-side split: every rank computes the same assignment from
the same lengths, without communicating.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

PAGE = 128


def request_cost(qo_len: int, kv_len: int, topk: int = 0, causal: bool = True) -> int:
    """Attended (query, key) pairs of one request for one head: the work the attention stage does.

    Row i of the request (0-based, bottom-right aligned causal mask) sees ``kv_len - qo_len + i + 1`` keys;
    with ``topk`` > 0 a row reads at most ``topk`` pages of 128 keys.
    """
    qo_len, kv_len = int(qo_len), int(kv_len)
    if qo_len <= 0 or kv_len <= 0:
        return 0
    cap = topk * PAGE if topk > 0 else kv_len
    if not causal:
        return qo_len * min(cap, kv_len)
    first = kv_len - qo_len + 1                       # keys visible to row 0 (may be <= 0 when qo_len > kv_len)
    total = 0
    # rows with visible <= cap form an arithmetic series; the rest read cap keys
    lo = max(0, 1 - first)                            # first row that sees at least one key
    hi = min(qo_len, cap - first + 1)                 # rows [lo, hi) see first + i <= cap keys
    if hi > lo:
        n = hi - lo
        total += n * (first + lo) + n * (n - 1) // 2
    total += max(0, qo_len - max(hi, lo)) * cap
    return total


def shard_requests(qo_lens: Sequence[int], kv_lens: Sequence[int], world_size: int, topk: int = 0,
                   causal: bool = True) -> List[List[int]]:
    """Assign requests to ``world_size`` ranks, heaviest first onto the least loaded rank.

    Deterministic (ties go to the lower request id, then the lower rank), so every rank can call it on its own.
    Returns one ascending list of request ids per rank; a rank may get none.
    """
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    if len(qo_lens) != len(kv_lens):
        raise ValueError("qo_lens and kv_lens differ in length")
    costs = [request_cost(q, k, topk, causal) for q, k in zip(qo_lens, kv_lens)]
    order = sorted(range(len(costs)), key=lambda r: (-costs[r], r))
    load = [0] * world_size
    out: List[List[int]] = [[] for _ in range(world_size)]
    for r in order:
        dst = min(range(world_size), key=lambda w: (load[w], w))
        out[dst].append(r)
        load[dst] += costs[r]
    return [sorted(x) for x in out]


def shard_batch(rank: int, world_size: int, qo_lens: Sequence[int], kv_lens: Sequence[int], topk: int = 0,
                causal: bool = True, page_size: int = PAGE) -> Dict[str, object]:
    """What rank ``rank`` needs to cut its part out of a packed batch.

    ``requests``: its request ids; ``qo_lens`` / ``kv_lens``: their lengths; ``q_ranges``: (start, end) token
    ranges in the packed Q/O tensors; ``page_ranges``: (start, end) slot ranges in the flat page table
    (``kv_indices``), whose per-request extents are ``ceil(kv_len / page_size)``.
    """
    if not 0 <= rank < world_size:
        raise ValueError("rank out of range")
    mine = shard_requests(qo_lens, kv_lens, world_size, topk, causal)[rank]
    q_start, p_start = [0], [0]
    for q, k in zip(qo_lens, kv_lens):
        q_start.append(q_start[-1] + int(q))
        p_start.append(p_start[-1] + (int(k) + page_size - 1) // page_size)
    return dict(
        requests=mine,
        qo_lens=[int(qo_lens[r]) for r in mine],
        kv_lens=[int(kv_lens[r]) for r in mine],
        q_ranges=[(q_start[r], q_start[r + 1]) for r in mine],
        page_ranges=[(p_start[r], p_start[r + 1]) for r in mine],
        cost=sum(request_cost(qo_lens[r], kv_lens[r], topk, causal) for r in mine),
    )


def scatter_rows(dst, shard: Dict[str, object], src) -> None:
    """Copy a rank's packed output rows ``src`` (its requests back to back) into the full packed tensor ``dst``."""
    at = 0
    for s, e in shard["q_ranges"]:
        dst[s:e] = src[at:at + (e - s)]
        at += e - s
    if at != src.shape[0]:
        raise ValueError("shard output has %d rows, its requests hold %d" % (src.shape[0], at))


def shard_kv_heads(num_kv_heads: int, world_size: int, rank: int) -> List[int]:
    """KV heads of rank ``rank`` when a batch is split by KV-head group: heads ``rank, rank + world_size, ...``.

    With ``world_size == num_kv_heads`` every GPU holds exactly one KV head and the query heads that attend to it
    (how the NVFP4 prefill case of the benchmark is spread over 8 GPUs).  Like the request split this needs no
    collective on the data path: attention never mixes KV heads.
    """
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError("rank out of range")
    return list(range(rank, int(num_kv_heads), world_size))


def head_shard(kv_head: int, num_qo_heads: int, num_kv_heads: int) -> Dict[str, object]:
    """Index ranges of one KV-head group: ``q_heads`` (slice of the query-head axis of Q and O), ``kv_head``
    (index into the head axis of paged K/V and, for page lists given per KV head, of ``kv_block_indexes``)."""
    if num_qo_heads % num_kv_heads:
        raise ValueError("num_qo_heads must be a multiple of num_kv_heads")
    hr = num_qo_heads // num_kv_heads
    if not 0 <= kv_head < num_kv_heads:
        raise ValueError("kv_head out of range")
    return dict(kv_head=int(kv_head), q_heads=slice(kv_head * hr, (kv_head + 1) * hr), heads_per_kv=hr)


def gather_heads(dst, kv_head: int, num_qo_heads: int, num_kv_heads: int, src) -> None:
    """Copy one head group's output ``src[total_q, hr, D]`` into its query-head columns of ``dst[total_q, Hq, D]``."""
    dst[:, head_shard(kv_head, num_qo_heads, num_kv_heads)["q_heads"]] = src
