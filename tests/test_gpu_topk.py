"""Top-k page selector: bit-exact index parity with the oracle through the C ABI."""
import os

import numpy as np
import pytest
import torch

import msa_b200
from oracle import msa_oracle as O

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")


def _scores(H, K, T, nvp, seed, ties=True):
    g = torch.Generator().manual_seed(seed)
    ms = torch.randn(H, K, T, generator=g)
    for t in range(T):
        ms[:, 1 + (t * nvp) // max(T, 1):, t] = float("-inf")     # causal frontier, rows with < k finite
    if ties and K >= 4:
        ms[0, 3, T // 2:] = ms[0, 2, T // 2:]
    return ms


@pytest.mark.parametrize("H,K,T,topk,nvp,fb,fe", [
    (3, 128, 96, 16, 40, 0, 0),
    (2, 1024, 200, 16, 1000, 1, 2),
    (2, 2304, 37, 32, 2300, 0, 1),
    (8, 1024, 32, 64, 1024, 0, 0),       # the decode configuration of the benchmark set
    (1, 128, 5, 16, 9, 0, 0),            # fewer valid pages than k
    (1, 128, 33, 16, 16, 3, 4),
    (2, 4096, 19, 64, 4096, 2, 2),
    (1, 17, 3, 16, 17, 0, 0),
])
def test_topk_bit_exact(H, K, T, topk, nvp, fb, fe):
    ms = _scores(H, K, T, nvp, K * 7 + T)
    ref = O.topk_select(ms, topk, nvp, fb, fe)
    got = msa_b200.sparse_topk_select(ms.cuda(), topk, nvp, force_begin_blocks=fb, force_end_blocks=fe).cpu()
    assert torch.equal(ref, got)


def test_topk_reference_fixture():
    z = np.load(os.path.join(G, "topk.npz"))
    got = msa_b200.sparse_topk_select(torch.from_numpy(z["ms"]).cuda(), 16, 40).cpu()
    assert torch.equal(got, torch.from_numpy(z["sel"]))


def test_topk_all_equal_and_all_masked_rows():
    ms = torch.zeros(1, 300, 20)
    ms[:, :, 10:] = float("-inf")
    got = msa_b200.sparse_topk_select(ms.cuda(), 16, 300).cpu()
    assert torch.equal(got[:10, 0], torch.arange(16, dtype=torch.int32).expand(10, 16))   # lowest indices win ties
    assert (got[10:] == -1).all()


@pytest.mark.parametrize("H,K,T,topk", [(2, 1024, 40, 64), (1, 2304, 700, 32), (4, 1024, 640, 16), (1, 3000, 50, 16),
                                         (148, 512, 64, 16)])
def test_topk_heavy_ties(H, K, T, topk):
    # scores drawn from a handful of values (signed zeros among them): the cut falls inside a run of ties, in
    # the first slab or across slabs, and the lowest page ids of the run must win; narrow and wide CTA shapes
    g = torch.Generator().manual_seed(K + T)
    vals = torch.tensor([-2.5, -0.0, 0.0, 1.0, 1.0, 3.25, float("-inf")])
    ms = vals[torch.randint(0, len(vals), (H, K, T), generator=g)]
    ms[:, :, 0] = 1.0                                   # one row of all-equal scores
    ms[:, K // 2:, 1] = float("-inf")
    ref = O.topk_select(ms, topk, K)
    got = msa_b200.sparse_topk_select(ms.cuda(), topk, K).cpu()
    assert torch.equal(ref, got)


@pytest.mark.parametrize("H,K,T,topk,nvp,fb,fe,mode", [
    (2, 1024, 20000, 16, 1024, 0, 0, "causal"),      # the prefill shape
    (3, 300, 13000, 32, 290, 2, 1, "random"),        # num_valid_pages < K, forced pages, k = 32
    (2, 1024, 20000, 16, 1024, 1, 1, "ties"),        # few distinct values: the cut falls inside long runs of ties
    (1, 2500, 40000, 16, 2500, 0, 0, "causal"),      # more than 1024 pages
    (2, 64, 19999, 32, 40, 0, 0, "ties"),            # few pages, ragged last CTA
    (1, 1024, 8192, 64, 1000, 1, 0, "random"),       # k = 64 on the slab-resident kernel (128 groups per row)
    (1, 1000, 6004, 64, 1000, 0, 2, "ties"),         # k = 64, ties, last CTA holds 4 of its 16 tokens
    (1, 1024, 20004, 16, 1024, 0, 0, "causal"),      # ragged last CTA of the slab-resident kernel
])
def test_topk_many_rows(H, K, T, topk, nvp, fb, fe, mode):
    g = torch.Generator().manual_seed(K + T + topk)
    if mode == "ties":
        vals = torch.tensor([-2.5, -0.0, 0.0, 1.0, 1.0, 3.25, float("-inf")])
        ms = vals[torch.randint(0, len(vals), (H, K, T), generator=g)]
    else:
        ms = torch.randn(H, K, T, generator=g)
    if mode == "random":
        ms[:, 5, ::17] = float("inf")                                    # +inf ranks with FLT_MAX
        ms[:, 9, ::17] = 3.402823466e38
        ms[:, 11, 3::29] = float("nan")
    if mode == "causal":
        frontier = 1 + (torch.arange(T) * nvp) // T                      # tokens see a growing prefix of pages
        ms.masked_fill_(torch.arange(K)[None, :, None] >= frontier[None, None, :], float("-inf"))
        ms[:, :, 7] = float("nan")                                       # NaN never wins
    ref = O.topk_select(ms, topk, nvp, fb, fe)
    got = msa_b200.sparse_topk_select(ms.cuda(), topk, nvp, force_begin_blocks=fb, force_end_blocks=fe).cpu()
    assert torch.equal(ref, got)


def test_topk_block_granularity():
    torch.manual_seed(1)
    qo = [250, 128, 7]
    starts = [0, 128, 250, 378, 385]
    ms = torch.randn(2, 256, sum(qo))
    got = msa_b200.sparse_topk_select(ms.cuda(), 16, 200, q_block_starts=torch.tensor(starts, dtype=torch.int32)).cpu()
    ref = O.topk_select(O.block_max_score(ms, starts), 16, 200)
    for i in range(4):
        assert torch.equal(got[starts[i]:starts[i + 1]], ref[i:i + 1].expand(starts[i + 1] - starts[i], 2, 16))


def test_topk_block_granularity_into_a_given_buffer():
    """Same through `output=`: msa_expand_block_lists writes the caller's [T, H, topk] tensor, every row of it."""
    torch.manual_seed(2)
    starts = [0, 1, 129, 257, 300]
    ms = torch.randn(3, 128, 300)
    out = torch.full((300, 3, 32), -7, dtype=torch.int32, device="cuda")
    got = msa_b200.sparse_topk_select(ms.cuda(), 32, 100, output=out,
                                      q_block_starts=torch.tensor(starts, dtype=torch.int32))
    assert got.data_ptr() == out.data_ptr()
    ref = O.topk_select(O.block_max_score(ms, starts), 32, 100)
    for i in range(4):
        assert torch.equal(out[starts[i]:starts[i + 1]].cpu(), ref[i:i + 1].expand(starts[i + 1] - starts[i], 3, 32))


def test_topk_large_multiset_property():
    """Full prefill-sized head slice: the selected scores equal torch.topk's as a multiset
    (the check of tests/integration/test_proxy_kv_e2e.py:77-116 of the reference) and rows ascend."""
    H, K, T = 1, 1024, 65536
    g = torch.Generator(device="cuda").manual_seed(0)
    ms = torch.randn(H, K, T, device="cuda", generator=g)
    sel = msa_b200.sparse_topk_select(ms, 16, K)
    s = ms.permute(2, 0, 1)
    ref = torch.topk(s, 16, dim=-1).values.sort(dim=-1).values
    got = torch.gather(s, -1, sel.long()).sort(dim=-1).values
    assert torch.equal(ref, got)
    assert (sel[..., 1:] > sel[..., :-1]).all()
