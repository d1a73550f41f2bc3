"""FP4 indexer (fp4_indexer_block_scores and its scale helpers) against the oracle and the reference fixture.
Scores are float32 sums of exact products, so the only difference to the oracle is summation order: rtol 2e-5."""
import os

import numpy as np
import pytest
import torch

import msa_b200
from oracle import msa_oracle as O

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")
SCALE_DTYPE = {"nvfp4": torch.float8_e4m3fn, "mxfp4": torch.float8_e8m0fnu}
RAW_RANGE = {"nvfp4": (16, 89), "mxfp4": (122, 133)}     # the scale bytes the reference's tests draw from


def _case(fmt, q_lens, k_lens, Hq, Hk, seed, extra_pages=2):
    g = torch.Generator().manual_seed(seed)
    pages = [(x + 127) // 128 for x in k_lens]
    P = sum(pages) + extra_pages
    G_ = O.FP4_GROUPS[fmt]
    q = torch.randint(0, 256, (sum(q_lens), Hq, 64), dtype=torch.uint8, generator=g)
    k = torch.randint(0, 256, (P, Hk, 128, 64), dtype=torch.uint8, generator=g)
    lo, hi = RAW_RANGE[fmt]
    qs = torch.randint(lo, hi, (sum(q_lens), Hq, G_), dtype=torch.uint8, generator=g)
    ks = torch.randint(lo, hi, (P, Hk, 128, G_), dtype=torch.uint8, generator=g)
    cu = lambda v: torch.tensor([0] + list(np.cumsum(v)), dtype=torch.int32)
    kvi = torch.randperm(P, generator=g)[:sum(pages)].to(torch.int32)
    return dict(q=q, k=k, qs=qs, ks=ks, cu_q=cu(q_lens), cu_k=cu(k_lens), cu_p=cu(pages), kvi=kvi,
                max_q=max(q_lens), max_k=max(k_lens))


def _run(fmt, c, causal, off, layout):
    dt = SCALE_DTYPE[fmt]
    qs, ks = c["qs"].cuda().view(dt), c["ks"].cuda().view(dt)
    if layout == "preordered_mma":
        qs, ks = msa_b200.fp4_indexer_reorder_scales_for_mma_cute(qs, ks, fp4_format=fmt)
    return msa_b200.fp4_indexer_block_scores(
        c["q"].cuda(), c["k"].cuda(), qs, ks, c["cu_q"].cuda(), c["cu_k"].cuda(), c["cu_p"].cuda(),
        max_seqlen_q=c["max_q"], max_seqlen_k=c["max_k"], kv_indices=c["kvi"].cuda(), fp4_format=fmt, causal=causal,
        qo_offset=None if off is None else off.cuda(), scale_layout=layout).cpu()


def _check(got, ref):
    assert got.shape == ref.shape
    fin = torch.isfinite(ref)
    assert torch.equal(fin, torch.isfinite(got))
    assert torch.allclose(got[fin], ref[fin], rtol=2e-5, atol=1e-2)


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
@pytest.mark.parametrize("layout", ["public", "preordered_mma"])
def test_reference_fixture_through_the_kernel(fmt, layout):
    z = np.load(os.path.join(G, "fp4_indexer.npz"))
    c = dict(q=torch.from_numpy(z[f"{fmt}_q"]), k=torch.from_numpy(z[f"{fmt}_k"]), qs=torch.from_numpy(z[f"{fmt}_qs"]),
             ks=torch.from_numpy(z[f"{fmt}_ks"]), cu_q=torch.from_numpy(z["cu_q"]), cu_k=torch.from_numpy(z["cu_k"]),
             cu_p=torch.from_numpy(z["cu_p"]), kvi=torch.from_numpy(z[f"{fmt}_kvi"]), max_q=130, max_k=300)
    off = torch.from_numpy(z["off"])
    for name, causal, o in (("dense", False, None), ("causal", True, None), ("offset", True, off)):
        _check(_run(fmt, c, causal, o, layout), torch.from_numpy(z[f"{fmt}_{name}"]))


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
def test_scale_reorder_and_q_dequant_kernels(fmt):
    z = np.load(os.path.join(G, "fp4_indexer.npz"))
    dt = SCALE_DTYPE[fmt]
    qs, ks = torch.from_numpy(z[f"{fmt}_qs"]).cuda().view(dt), torch.from_numpy(z[f"{fmt}_ks"]).cuda().view(dt)
    q_mma, k_mma = msa_b200.fp4_indexer_reorder_scales_for_mma_cute(qs, ks, fp4_format=fmt)
    T, Hq = qs.shape[0], qs.shape[1]
    assert tuple(q_mma.shape) == msa_b200.fp4_indexer_mma_scale_shape(T, Hq, fp4_format=fmt)
    assert tuple(q_mma.stride()) == msa_b200.fp4_indexer_mma_scale_stride(T, Hq, fp4_format=fmt)
    # back to the contiguous storage order (L, restM, restG, 32, 4, 4)
    assert torch.equal(q_mma.permute(5, 2, 4, 0, 1, 3).contiguous().view(torch.uint8).reshape(-1).cpu(),
                       torch.from_numpy(z[f"{fmt}_qs_mma"]))
    assert torch.equal(k_mma.permute(5, 2, 4, 0, 1, 3).contiguous().view(torch.uint8).reshape(-1).cpu(),
                       torch.from_numpy(z[f"{fmt}_ks_mma"]))
    # Q dequantisation from either scale layout, bit for bit (the products are exact in bf16)
    lib = msa_b200.get_lib()
    from msa_b200.api import _ptr, _stream
    q = torch.from_numpy(z[f"{fmt}_q"]).cuda()
    want = torch.from_numpy(z[f"{fmt}_deq_q"])
    for layout, sc in ((0, qs), (1, q_mma)):
        out = torch.empty(T, Hq, 128, dtype=torch.bfloat16, device="cuda")
        assert lib.msa_fp4_dequant_rows(_ptr(q), _ptr(sc), 0 if fmt == "nvfp4" else 1, layout, T, Hq, _ptr(out),
                                        _stream()) == 0
        assert torch.equal(out.float().cpu(), want)


@pytest.mark.parametrize("fmt,q_lens,k_lens,Hq,Hk,causal", [
    ("nvfp4", [300, 17, 129], [700, 900, 129], 8, 2, True),        # ragged, GQA 4, odd page counts
    ("mxfp4", [300, 17, 129], [700, 900, 129], 8, 2, True),
    ("nvfp4", [256, 512], [2048, 512], 2, 1, False),
    ("mxfp4", [3, 3, 3], [1000, 130, 4097], 16, 1, True),          # decode-like: a few new tokens per request
    ("nvfp4", [400], [200], 1, 1, True),                           # more queries than keys: early rows see nothing
])
def test_block_scores_against_the_oracle(fmt, q_lens, k_lens, Hq, Hk, causal):
    c = _case(fmt, q_lens, k_lens, Hq, Hk, seed=len(q_lens) * 7 + Hq)
    ref = O.fp4_indexer_block_scores(c["q"], c["k"], c["qs"], c["ks"], c["cu_q"], c["cu_k"], c["cu_p"], c["kvi"], fmt,
                                     causal=causal)
    for layout in ("public", "preordered_mma"):
        _check(_run(fmt, c, causal, None, layout), ref)


def test_argument_checks():
    c = _case("nvfp4", [10], [200], 2, 1, seed=1)
    e4 = torch.float8_e4m3fn
    args = (c["q"].cuda(), c["k"].cuda(), c["qs"].cuda().view(e4), c["ks"].cuda().view(e4), c["cu_q"].cuda(),
            c["cu_k"].cuda(), c["cu_p"].cuda())
    kw = dict(max_seqlen_q=10, max_seqlen_k=200, kv_indices=c["kvi"].cuda())
    with pytest.raises(ValueError):
        msa_b200.fp4_indexer_block_scores(*args, fp4_format="fp4", scale_layout="public", **kw)
    with pytest.raises(ValueError):                                  # qo_offset needs causal
        _run("nvfp4", c, False, torch.zeros(1, dtype=torch.int32), "public")
    with pytest.raises(ValueError):                                  # public-shaped scales passed as preordered
        msa_b200.fp4_indexer_block_scores(*args, fp4_format="nvfp4", **kw)
