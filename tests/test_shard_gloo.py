"""Request sharding across ranks (world_size 2, gloo, CPU).

The oracle stands in for the kernels: what is under test is the host logic of the N > 1 path -- every rank derives
the same split on its own, cuts its requests out of the packed batch, and the per-rank results put back together
equal the single-process result bit for bit (requests are independent, so no data-path collective exists).
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from msa_b200.shard import (gather_heads, head_shard, request_cost, scatter_rows, shard_batch, shard_kv_heads,
                            shard_requests)
from oracle import msa_oracle as O
from util import make_paged

QO = [256, 128, 384, 40, 1]
KV = [1024, 128, 640, 1500, 900]
HQ, HKV, TOPK = 4, 2, 4


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_request_cost_matches_brute_force():
    for q, k, topk, causal in [(5, 300, 0, True), (300, 300, 1, True), (700, 1000, 2, True), (64, 32, 0, True),
                               (10, 1000, 3, False), (0, 5, 0, True), (257, 257, 0, True)]:
        cap = topk * 128 if topk else k
        want = sum(min(cap, max(0, (k - q + i + 1) if causal else k)) for i in range(q))
        assert request_cost(q, k, topk, causal) == want, (q, k, topk, causal)


def test_split_is_a_partition_and_balanced():
    lens = [16384, 32768, 65536, 131072, 8192, 8192, 4096, 100]
    for world in (1, 2, 3, 4, 8):
        parts = shard_requests(lens, lens, world, topk=16)
        assert sorted(r for p in parts for r in p) == list(range(len(lens)))
        loads = [sum(request_cost(lens[r], lens[r], 16) for r in p) for p in parts]
        heaviest = max(request_cost(n, n, 16) for n in lens)
        assert max(loads) <= max(heaviest, sum(loads) / world * 4 / 3 + 1)      # the LPT bound
    with pytest.raises(ValueError):
        shard_requests([1], [1, 2], 2)


def _problem():
    kp, vp, table = make_paged(KV, HKV, 21, dtype=torch.float32)
    g = torch.Generator().manual_seed(22)
    q = torch.randn(sum(QO), HQ, 128, generator=g).to(torch.bfloat16)
    ms = O.tile_max_score_paged(q, kp.to(torch.bfloat16), table, QO, KV, 12)
    kvh = ms.view(HKV, HQ // HKV, *ms.shape[1:]).amax(dim=1)
    idx = O.topk_select(kvh, 16, ms.shape[1])[:, :, :TOPK].contiguous()
    return q, kp.to(torch.bfloat16), vp.to(torch.bfloat16), table, idx


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v, table, idx = _problem()                     # same seeds: every rank holds the same batch
        sh = shard_batch(rank, world, QO, KV, topk=TOPK)
        rows = [torch.arange(s, e) for s, e in sh["q_ranges"]]
        slots = [torch.arange(s, e) for s, e in sh["page_ranges"]]
        if rows:
            rows, slots = torch.cat(rows), torch.cat(slots)
            out, lse = O.sparse_attention_paged(q[rows], k, v, table[slots], sh["qo_lens"], sh["kv_lens"], idx[rows])
        else:
            out, lse = torch.zeros(0, HQ, 128), torch.zeros(0, HQ)
        # what bench.py does around the timed loop: max of the per-rank times, gather of per-rank checksums
        t = torch.tensor([10.0 + rank])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        gathered = [None] * world
        dist.all_gather_object(gathered, (sh, out, lse))
        if rank == 0:
            full = torch.zeros(sum(QO), HQ, 128)
            for s, o, _ in gathered:
                scatter_rows(full, s, o)
            ret["t_max"] = float(t)
            ret["out"] = full
            ret["requests"] = [s["requests"] for s, _, _ in gathered]
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_the_single_process_result():
    world = 2
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        out, reqs, t_max = ret["out"], ret["requests"], ret["t_max"]
    assert sorted(r for p in reqs for r in p) == list(range(len(QO)))
    assert all(len(p) > 0 for p in reqs)
    assert t_max == 11.0
    q, k, v, table, idx = _problem()
    ref, _ = O.sparse_attention_paged(q, k, v, table, QO, KV, idx)
    assert torch.equal(out, ref.float())


def _head_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v, table, idx = _problem()
        outs = []
        for g in shard_kv_heads(HKV, world, rank):
            hs = head_shard(g, HQ, HKV)
            # this rank's slice of the problem: its KV head, the query heads on it, its page lists
            o, _ = O.sparse_attention_paged(q[:, hs["q_heads"]], k[:, g:g + 1], v[:, g:g + 1], table, QO, KV,
                                            idx[:, g:g + 1])
            outs.append((g, o))
        gathered = [None] * world
        dist.all_gather_object(gathered, outs)              # what the benchmark does with NCCL all_gather
        if rank == 0:
            full = torch.zeros(sum(QO), HQ, 128)
            for part in gathered:
                for g, o in part:
                    gather_heads(full, g, HQ, HKV, o)
            ret["out"] = full
            ret["heads"] = [[g for g, _ in part] for part in gathered]
    finally:
        dist.destroy_process_group()


def test_kv_head_split_two_ranks_reproduce_the_single_process_result():
    """Split by KV-head group (the 8-GPU NVFP4 case, here 2 KV heads on 2 gloo ranks): each rank attends with its
    KV head only, the gathered outputs equal the unsplit result bit for bit."""
    assert shard_kv_heads(8, 8, 3) == [3] and shard_kv_heads(8, 2, 1) == [1, 3, 5, 7] and shard_kv_heads(8, 16, 9) == []
    assert head_shard(3, 64, 8)["q_heads"] == slice(24, 32)
    world = 2
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_head_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        out, heads = ret["out"], ret["heads"]
    assert heads == [[0], [1]]
    q, k, v, table, idx = _problem()
    ref, _ = O.sparse_attention_paged(q, k, v, table, QO, KV, idx)
    assert torch.equal(out, ref.float())
