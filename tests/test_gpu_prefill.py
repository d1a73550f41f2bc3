"""Dense / score-only / block-sparse paged prefill against the oracle, through the
C ABI.  Tolerances (max-abs vs the fp32 oracle): 2e-2 bf16, 6e-2 fp8, 1.5e-1 nvfp4."""
import os

import numpy as np
import pytest
import torch

import msa_b200
from msa_b200 import quant
from oracle import msa_oracle as O
from util import block_starts, causal_scores, make_paged

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")
TOL = {"bf16": 2e-2, "fp8": 6e-2, "nvfp4": 1.5e-1}


def test_umma_selftest():
    lib = msa_b200.get_lib()
    from msa_b200.api import _ptr, _stream
    torch.manual_seed(0)
    q, k, v = (torch.randn(128, 128, device="cuda").to(torch.bfloat16) for _ in range(3))
    p = torch.rand(128, 128, device="cuda").to(torch.bfloat16)
    s = torch.zeros(128, 128, device="cuda")
    o = torch.zeros(128, 128, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.msa_umma_selftest(_ptr(q), _ptr(k), _ptr(v), _ptr(p), _ptr(s), _ptr(o), _ptr(st), _stream()) == 0
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert (s - q.float() @ k.float().T).abs().max() < 1e-3
    assert (o - p.float() @ v.float()).abs().max() < 1e-3


def test_bounded_wait_runs_out_and_the_context_stays_usable():
    """The timeout path shared by every kernel (bounded mbarrier wait -> abort flag -> teardown with TMEM freed ->
    status word): the self-test kernel is launched with its operand loads withheld and a wait limit of about a
    millisecond; it must return normally with MSA_ERR_TIMEOUT in the status word, and an ordinary launch right
    after it (same process, same context) must compute correctly.  Nothing faults or hangs."""
    lib = msa_b200.get_lib()
    from msa_b200.api import _ptr, _stream
    torch.manual_seed(1)
    q, k, v = (torch.randn(128, 128, device="cuda").to(torch.bfloat16) for _ in range(3))
    p = torch.rand(128, 128, device="cuda").to(torch.bfloat16)
    s = torch.full((128, 128), 7.0, device="cuda")
    o = torch.full((128, 128), 7.0, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.msa_umma_selftest_timeout(_ptr(q), _ptr(k), _ptr(v), _ptr(p), _ptr(s), _ptr(o), _ptr(st), 1 << 21,
                                       _stream())
    assert rc == 0
    torch.cuda.synchronize()                                   # returns: the kernel ended by itself
    assert int(st.item()) == msa_b200._lib.MSA_ERR_TIMEOUT
    assert bool((s == 7.0).all()) and bool((o == 7.0).all())  # nothing was computed
    st.zero_()
    assert lib.msa_umma_selftest(_ptr(q), _ptr(k), _ptr(v), _ptr(p), _ptr(s), _ptr(o), _ptr(st), _stream()) == 0
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert (s - q.float() @ k.float().T).abs().max() < 1e-3
    assert (o - p.float() @ v.float()).abs().max() < 1e-3


def _quantise(kp, vp, kind):
    """-> (device k, device v, oracle k, oracle v, kwargs for fmha_sm100)"""
    if kind == "bf16":
        return kp.cuda(), vp.cuda(), kp, vp, {}
    k8, ks = O.quantize_fp8_per_tensor(kp.float())
    v8, vs = O.quantize_fp8_per_tensor(vp.float())
    return k8.cuda(), v8.cuda(), k8.float() * ks, v8.float() * vs, dict(k_scale=ks, v_scale=vs)


@pytest.mark.parametrize("qo_lens,kv_lens,Hq,Hkv,kind", [
    ([128], [128], 2, 1, "bf16"),
    ([70, 128, 200], [300, 128, 457], 4, 2, "bf16"),      # ragged, GQA 2, partial pages, q < kv
    ([200], [333], 1, 1, "bf16"),                          # MHA -> one query head per CTA
    ([1, 127, 129], [1, 127, 129], 8, 2, "bf16"),          # the reference's corner lengths
    ([384], [1024], 8, 1, "fp8"),
    ([70, 128, 200], [300, 128, 457], 4, 2, "fp8"),
])
def test_dense_full_mode(qo_lens, kv_lens, Hq, Hkv, kind):
    """Mode Full: O and the per-page max score in one pass."""
    kp, vp, table = make_paged(kv_lens, Hkv, 8)
    q = torch.randn(sum(qo_lens), Hq, 128, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
    kd, vd, kr, vr, kw = _quantise(kp, vp, kind)
    plan = msa_b200.fmha_sm100_plan(torch.tensor(qo_lens), torch.tensor(kv_lens), Hq, num_kv_heads=Hkv, page_size=128,
                                    output_maxscore=True)
    out, ms, lse = msa_b200.fmha_sm100(q.cuda(), kd, vd, plan, kv_indices=table.cuda(), output_maxscore=True,
                                       check_input_valid=True, return_lse=True, **kw)
    assert msa_b200.plan_status(plan) == 0
    ref, lse_ref = O.dense_attention_paged(q, kr, vr, table, qo_lens, kv_lens)
    assert (out.float().cpu() - ref).abs().max() <= TOL[kind]
    assert torch.allclose(lse.cpu(), lse_ref, atol=2e-2, rtol=1e-3)
    # max score: raw stored values (no scales), -inf pattern exact
    kraw = kd.float().cpu() if kind == "fp8" else kp
    msref = O.tile_max_score_paged(q, kraw, table, qo_lens, kv_lens, ms.shape[1])
    got = ms.cpu()
    assert ms.shape == (Hq, 128, sum(qo_lens))
    assert torch.equal(torch.isfinite(got), torch.isfinite(msref))
    fin = torch.isfinite(msref)
    assert torch.allclose(got[fin], msref[fin], atol=2e-3 if kind == "bf16" else 1e-1, rtol=1e-3)


@pytest.mark.parametrize("kind", ["bf16", "fp8"])
def test_row_maximum_grows_on_every_page(kind):
    """The walk runs from the last page down; here the scores of logical page j are about 4 * (7 - j) nats, so
    every row's maximum grows by ~5.8 in log2 on each step, past the lazy-rescale threshold of either P format:
    O is rescaled on every page and P must stay inside its number range (e4m3 tops out at 448)."""
    kv_len, n_pages, Hq, Hkv = 1024, 8, 2, 1
    g = torch.Generator().manual_seed(77)
    w = torch.randn(128, generator=g)
    q = (w[None, None, :] + 0.1 * torch.randn(128, Hq, 128, generator=g)).to(torch.bfloat16)
    kp = 0.3 * torch.randn(n_pages, Hkv, 128, 128, generator=g)
    vp = torch.randn(n_pages, Hkv, 128, 128, generator=g).to(torch.bfloat16)
    table = torch.randperm(n_pages, generator=g).int()
    for j in range(n_pages):
        kp[table[j]] += 4.0 * (n_pages - 1 - j) * (128 ** 0.5) * w / w.pow(2).sum()
    kp = kp.to(torch.bfloat16)
    kd, vd, kr, vr, kw = _quantise(kp, vp, kind)
    plan = msa_b200.fmha_sm100_plan(torch.tensor([128]), torch.tensor([kv_len]), Hq, num_kv_heads=Hkv, page_size=128)
    out, _, lse = msa_b200.fmha_sm100(q.cuda(), kd, vd, plan, kv_indices=table.cuda(), return_lse=True, **kw)
    assert msa_b200.plan_status(plan) == 0
    ref, lse_ref = O.dense_attention_paged(q, kr, vr, table, [128], [kv_len])
    assert bool(torch.isfinite(out.float()).all())
    assert (out.float().cpu() - ref).abs().max() <= TOL[kind]
    assert torch.allclose(lse.cpu(), lse_ref, atol=2e-2, rtol=1e-3)


@pytest.mark.parametrize("qo_lens,kv_lens,Hq,Hkv,kind,splits,causal", [
    ([40, 3], [5000, 9000], 8, 2, "bf16", -1, True),       # planner's own choice (few tiles, long contexts)
    ([40, 3], [5000, 9000], 8, 2, "fp8", 3, True),
    ([130], [2100], 2, 1, "bf16", 5, True),                # two tiles; upper splits see nothing of the first rows
    ([5], [300], 4, 4, "bf16", 7, True),                   # more splits than pages: empty splits
    ([17], [4000], 6, 2, "fp8", 4, False),
])
def test_dense_short_query_kv_splits(qo_lens, kv_lens, Hq, Hkv, kind, splits, causal):
    """A dense call with few query tiles is split over page ranges and merged (msa_fmha_combine): same output,
    LSE and max score as the unsplit oracle."""
    kp, vp, table = make_paged(kv_lens, Hkv, 18)
    q = torch.randn(sum(qo_lens), Hq, 128, generator=torch.Generator().manual_seed(19)).to(torch.bfloat16)
    kd, vd, kr, vr, kw = _quantise(kp, vp, kind)
    plan = msa_b200.fmha_sm100_plan(torch.tensor(qo_lens), torch.tensor(kv_lens), Hq, num_kv_heads=Hkv, page_size=128,
                                    output_maxscore=True, num_kv_splits=splits, causal=causal)
    assert plan[3]["dense_kv_splits"] > 1 and not plan[3]["use_decode_kernel"]
    out, ms, lse = msa_b200.fmha_sm100(q.cuda(), kd, vd, plan, kv_indices=table.cuda(), output_maxscore=True,
                                       return_lse=True, **kw)
    assert msa_b200.plan_status(plan) == 0
    ref, lse_ref = O.dense_attention_paged(q, kr, vr, table, qo_lens, kv_lens, causal=causal)
    assert (out.float().cpu() - ref).abs().max() <= TOL[kind]
    assert torch.allclose(lse.cpu(), lse_ref, atol=2e-2, rtol=1e-3)
    if causal:
        kraw = kd.float().cpu() if kind == "fp8" else kp
        msref = O.tile_max_score_paged(q, kraw, table, qo_lens, kv_lens, ms.shape[1])
        got = ms.cpu()
        assert torch.equal(torch.isfinite(got), torch.isfinite(msref))
        fin = torch.isfinite(msref)
        assert torch.allclose(got[fin], msref[fin], atol=2e-3 if kind == "bf16" else 1e-1, rtol=1e-3)
    # the same call again reuses the plan's partial buffers
    out2, _ = msa_b200.fmha_sm100(q.cuda(), kd, vd, plan, kv_indices=table.cuda(), output_maxscore=False, **kw)
    assert torch.equal(out2, out)


def test_score_only_mode_and_reference_fixture():
    z = np.load(os.path.join(G, "maxscore.npz"))
    q = torch.from_numpy(z["q"]).to(torch.bfloat16)
    k = torch.from_numpy(z["k"]).to(torch.bfloat16)
    qo, kv = z["qo_lens"].tolist(), z["kv_lens"].tolist()
    plan = msa_b200.fmha_sm100_plan(torch.tensor(qo), torch.tensor(kv), 4, num_kv_heads=2, output_maxscore=True)
    # ragged (non-paged) K, no O requested
    out, ms = msa_b200.fmha_sm100(q.cuda(), k.cuda(), k.cuda(), plan, output_maxscore=True, output_o=False)
    assert out is None
    ref = torch.from_numpy(z["ms_default"])
    got = ms.cpu()
    assert (got[:, 4:] == float("-inf")).all()
    assert torch.equal(torch.isfinite(got[:, :4]), torch.isfinite(ref))
    fin = torch.isfinite(ref)
    assert torch.allclose(got[:, :4][fin], ref[fin], atol=2e-3, rtol=1e-3)
    # runtime causal-offset override
    offs = torch.from_numpy(z["offs"])
    _, ms2 = msa_b200.fmha_sm100(q.cuda(), k.cuda(), k.cuda(), plan, output_maxscore=True, output_o=False,
                                 q_offset_override=offs.cuda())
    ref2 = torch.from_numpy(z["ms_off"])
    got2 = ms2.cpu()[:, :4]
    assert torch.equal(torch.isfinite(got2), torch.isfinite(ref2))
    assert torch.allclose(got2[torch.isfinite(ref2)], ref2[torch.isfinite(ref2)], atol=2e-3, rtol=1e-3)


@pytest.mark.parametrize("kind,Hq,Hkv", [("bf16", 1, 1), ("fp8", 1, 1), ("fp8", 4, 2), ("bf16", 6, 2)])
def test_score_only_proxy_slice(kind, Hq, Hkv):
    """The proxy pass: long requests (many pages per tile, so the two S buffers and their barriers wrap many
    times), one or several heads, and score_dim=64 on a 64-wide slice zero-padded to 128."""
    qo = kv = [2048, 700, 1300]
    g = torch.Generator().manual_seed(12)
    q = torch.randn(sum(qo), Hq, 128, generator=g).to(torch.bfloat16)
    kp, _, table = make_paged(kv, Hkv, 13, dtype=torch.float32)
    q[..., 64:] = 0
    kp[..., 64:] = 0
    if kind == "fp8":
        k_dev, ks = O.quantize_fp8_per_tensor(kp)
        k_ref = k_dev.float()
    else:
        k_dev = kp.to(torch.bfloat16)
        k_ref = k_dev.float()
    plan = msa_b200.fmha_sm100_plan(torch.tensor(qo), torch.tensor(kv), Hq, num_kv_heads=Hkv, page_size=128,
                                    output_maxscore=True)
    full = msa_b200.fmha_sm100(q.cuda(), k_dev.cuda(), None, plan, kv_indices=table.cuda(), output_maxscore=True,
                               output_o=False)[1].cpu()
    half = msa_b200.fmha_sm100(q.cuda(), k_dev.cuda(), None, plan, kv_indices=table.cuda(), output_maxscore=True,
                               output_o=False, score_dim=64)[1].cpu()
    assert torch.equal(full, half)                      # the skipped half of the contraction is exactly zero
    ref = O.tile_max_score_paged(q, k_ref, table, qo, kv, half.shape[1])
    assert torch.equal(torch.isfinite(half), torch.isfinite(ref))
    fin = torch.isfinite(ref)
    assert torch.allclose(half[fin], ref[fin], atol=2e-3 if kind == "bf16" else 1e-1, rtol=1e-3)
    with pytest.raises(msa_b200.MsaError):
        msa_b200.fmha_sm100(q.cuda(), k_dev.cuda(), k_dev.cuda(), plan, kv_indices=table.cuda(), score_dim=64)


def test_dense_ragged_kv_off_mode():
    qo, kv = [100, 260], [100, 700]
    g = torch.Generator().manual_seed(4)
    q = torch.randn(sum(qo), 4, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(sum(kv), 2, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(sum(kv), 2, 128, generator=g).to(torch.bfloat16)
    plan = msa_b200.fmha_sm100_plan(torch.tensor(qo), torch.tensor(kv), 4, num_kv_heads=2)
    out, ms = msa_b200.fmha_sm100(q.cuda(), k.cuda(), v.cuda(), plan, output_maxscore=False)
    assert ms is None
    # oracle wants pages: pad each request to whole pages
    ind = O.page_indptr(kv)
    kp = torch.zeros(ind[-1], 2, 128, 128, dtype=torch.bfloat16)
    vp = torch.zeros_like(kp)
    off = 0
    for b, kl in enumerate(kv):
        for pg in range(ind[b + 1] - ind[b]):
            t0, t1 = pg * 128, min(kl, (pg + 1) * 128)
            kp[ind[b] + pg, :, :t1 - t0] = k[off + t0:off + t1].permute(1, 0, 2)
            vp[ind[b] + pg, :, :t1 - t0] = v[off + t0:off + t1].permute(1, 0, 2)
        off += kl
    ref, _ = O.dense_attention_paged(q, kp, vp, torch.arange(ind[-1]).int(), qo, kv)
    assert (out.float().cpu() - ref).abs().max() <= TOL["bf16"]


def _sparse_case(qo_lens, kv_lens, Hq, Hkv, topk, kind, lists, seed=21, per_q_head=False):
    kp, vp, table = make_paged(kv_lens, Hkv, seed, extra_pages=2)
    q = torch.randn(sum(qo_lens), Hq, 128, generator=torch.Generator().manual_seed(seed + 1)).to(torch.bfloat16)
    LH = Hq if per_q_head else Hkv
    ms = causal_scores(LH, qo_lens, kv_lens, seed + 2)
    maxp = max((k + 127) // 128 for k in kv_lens)
    if lists == "block":
        st = block_starts(qo_lens)
        sel = O.topk_select(O.block_max_score(ms, st), 64, maxp)[:, :, :topk]
        idx = torch.cat([sel[i:i + 1].expand(st[i + 1] - st[i], LH, topk) for i in range(len(st) - 1)]).contiguous()
    else:
        idx = O.topk_select(ms, 64, maxp)[:, :, :topk].contiguous()
        if lists == "padded":
            idx[::3, :, topk // 2:] = -1
            idx[5::7] = -1                                  # rows that selected nothing
    return q, kp, vp, table, idx


@pytest.mark.parametrize("qo_lens,kv_lens,Hq,Hkv,topk,kind,lists", [
    ([512], [512], 4, 2, 2, "bf16", "block"),
    ([300, 100], [900, 1000], 4, 2, 4, "bf16", "token"),
    ([300, 100], [900, 1000], 8, 2, 4, "fp8", "token"),
    ([256, 33], [2048, 4000], 16, 2, 16, "fp8", "block"),
    ([130], [1300], 8, 8, 8, "bf16", "padded"),             # MHA + short / empty lists
    ([640], [640], 8, 1, 16, "fp8", "block"),               # more slots than visible pages
])
def test_sparse_prefill(qo_lens, kv_lens, Hq, Hkv, topk, kind, lists):
    q, kp, vp, table, idx = _sparse_case(qo_lens, kv_lens, Hq, Hkv, topk, kind, lists)
    kd, vd, kr, vr, kw = _quantise(kp, vp, kind)
    plan = msa_b200.fmha_sm100_plan(torch.tensor(qo_lens), torch.tensor(kv_lens), Hq, num_kv_heads=Hkv, page_size=128,
                                    kv_block_num=topk, sparse_kernel_mode="prefill")
    out, ms, lse = msa_b200.fmha_sm100(q.cuda(), kd, vd, plan, kv_indices=table.cuda(), kv_block_indexes=idx.cuda(),
                                       check_input_valid=True, return_lse=True, **kw)
    assert ms is None and msa_b200.plan_status(plan) == 0
    ref, lse_ref = O.sparse_attention_paged(q, kr, vr, table, qo_lens, kv_lens, idx)
    o = out.float().cpu()
    assert not o.isnan().any()
    assert (o - ref).abs().max() <= TOL[kind]
    assert torch.equal(torch.isfinite(lse.cpu()), torch.isfinite(lse_ref))
    fin = torch.isfinite(lse_ref)
    assert torch.allclose(lse.cpu()[fin], lse_ref[fin], atol=2e-2, rtol=1e-3)


@pytest.mark.parametrize("lists,qo_lens,kv_lens,Hq,Hkv,topk", [
    (None, [70, 128, 200], [300, 128, 457], 4, 2, 0),        # dense, ragged
    ("block", [256, 33], [2048, 4000], 16, 2, 16),
    ("token", [300, 100], [900, 1000], 6, 6, 4),             # one query head per CTA
])
def test_fp8_with_p_in_f16(lists, qo_lens, kv_lens, Hq, Hkv, topk):
    """msa_fmha_args.fp8_p_f16 (msa_b200.fp8_pv_precision("f16")): V dequantised to f16, P kept in f16.  The error
    against the fp32 oracle on the same dequantised K/V is that of the 16-bit paths, and the default (P rounded to
    e4m3) stays within the FP8 tolerance on the same inputs."""
    if lists is None:
        kp, vp, table = make_paged(kv_lens, Hkv, 8)
        q = torch.randn(sum(qo_lens), Hq, 128, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
        idx, plan_kw = None, {}
    else:
        q, kp, vp, table, idx = _sparse_case(qo_lens, kv_lens, Hq, Hkv, topk, "fp8", lists, seed=61)
        plan_kw = dict(kv_block_num=topk, sparse_kernel_mode="prefill")
    kd, vd, kr, vr, kw = _quantise(kp, vp, "fp8")
    plan = msa_b200.fmha_sm100_plan(torch.tensor(qo_lens), torch.tensor(kv_lens), Hq, num_kv_heads=Hkv, page_size=128,
                                    **plan_kw)
    call_kw = dict(kv_indices=table.cuda(), **kw)
    if idx is not None:
        call_kw["kv_block_indexes"] = idx.cuda()
        ref, _ = O.sparse_attention_paged(q, kr, vr, table, qo_lens, kv_lens, idx)
    else:
        ref, _ = O.dense_attention_paged(q, kr, vr, table, qo_lens, kv_lens)
    assert msa_b200.get_fp8_pv_precision() == "e4m3"
    out8, _ = msa_b200.fmha_sm100(q.cuda(), kd, vd, plan, **call_kw)
    with msa_b200.fp8_pv_precision("f16"):
        out16, _ = msa_b200.fmha_sm100(q.cuda(), kd, vd, plan, **call_kw)
    assert msa_b200.get_fp8_pv_precision() == "e4m3" and msa_b200.plan_status(plan) == 0
    e8 = (out8.float().cpu() - ref).abs().max()
    e16 = (out16.float().cpu() - ref).abs().max()
    assert e16 <= TOL["bf16"] and e8 <= TOL["fp8"]
    assert e16 <= e8 + 4e-3          # bf16 output rounding is common to both


def test_sparse_per_query_head_lists():
    qo, kv = [200], [1500]
    q, kp, vp, table, idx = _sparse_case(qo, kv, 4, 2, 4, "bf16", "token", per_q_head=True)
    plan = msa_b200.fmha_sm100_plan(torch.tensor(qo), torch.tensor(kv), 4, num_kv_heads=2, page_size=128,
                                    kv_block_num=4, sparse_kernel_mode="prefill")
    out, _ = msa_b200.fmha_sm100(q.cuda(), kp.cuda(), vp.cuda(), plan, kv_indices=table.cuda(),
                                 kv_block_indexes=idx.cuda())
    # oracle: treat every query head as its own KV head
    kx = kp.repeat_interleave(2, dim=1)
    vx = vp.repeat_interleave(2, dim=1)
    ref, _ = O.sparse_attention_paged(q, kx, vx, table, qo, kv, idx)
    assert (out.float().cpu() - ref).abs().max() <= TOL["bf16"]


def test_sparse_nvfp4():
    qo, kv, Hq, Hkv, topk = [256, 60], [1024, 700], 8, 2, 4
    q, kp, vp, table, idx = _sparse_case(qo, kv, Hq, Hkv, topk, "bf16", "block", seed=33)
    kq, vq = quant.quantize_kv_bf16_to_nvfp4_128x4(kp, vp)
    kr, vr = quant.dequantize_nvfp4_128x4(kq), quant.dequantize_nvfp4_128x4(vq)
    plan = msa_b200.fmha_sm100_plan(torch.tensor(qo), torch.tensor(kv), Hq, num_kv_heads=Hkv, page_size=128,
                                    kv_block_num=topk, sparse_kernel_mode="prefill")
    dev = lambda t: quant.Nvfp4QuantizedTensor(t.data.cuda(), t.scale_128x4.cuda(), t.global_scale.cuda(),  # noqa: E731
                                               t.logical_scale_shape, t.original_shape)
    out = msa_b200.sparse_prefill_nvfp4(q.cuda(), dev(kq), dev(vq), plan, table.cuda(), idx.cuda())
    assert msa_b200.plan_status(plan) == 0
    ref, _ = O.sparse_attention_paged(q, kr, vr, table, qo, kv, idx)
    # same dequantised values on both sides: the bf16 bound applies; 1.5e-1 is the bound vs unquantised K/V
    assert (out.float().cpu() - ref).abs().max() <= TOL["bf16"]
    ref_fp, _ = O.sparse_attention_paged(q, kp, vp, table, qo, kv, idx)
    assert (out.float().cpu() - ref_fp).abs().max() <= TOL["nvfp4"] * 4


def test_reference_fixtures_through_the_kernel():
    # sparse_ref (tests/regression/test_sparse_attn.py:46-75 of the reference)
    z = np.load(os.path.join(G, "sparse_ref.npz"), allow_pickle=True)
    q = torch.from_numpy(z["q"]).to(torch.bfloat16)
    kp = torch.from_numpy(z["k_pages"]).to(torch.bfloat16)
    vp = torch.from_numpy(z["v_pages"]).to(torch.bfloat16)
    qo, kv = z["qo_lens"].tolist(), z["kv_lens"].tolist()
    blocks = [z["blocks0"].tolist(), z["blocks1"].tolist()]
    rows = []
    for b, ql in enumerate(qo):
        per = torch.full((2, 4), -1, dtype=torch.int32)
        for h in range(2):
            per[h, :len(blocks[b][h])] = torch.tensor(blocks[b][h], dtype=torch.int32)
        rows.append(per.unsqueeze(0).expand(ql, 2, 4))
    idx = torch.cat(rows, 0).contiguous()
    table = torch.arange(kp.shape[0], dtype=torch.int32)
    for mode in ("prefill", "auto"):       # "auto" with q_len <= 32 and bf16 K/V still takes the prefill kernel
        plan = msa_b200.fmha_sm100_plan(torch.tensor(qo), torch.tensor(kv), 4, num_kv_heads=2, page_size=128,
                                        kv_block_num=4, sparse_kernel_mode=mode)
        out, _ = msa_b200.fmha_sm100(q.cuda(), kp.cuda(), vp.cuda(), plan, kv_indices=table.cuda(),
                                     kv_block_indexes=idx.cuda())
        ref = torch.from_numpy(z["out"])
        assert (out.float().cpu() - ref).abs().max() <= TOL["bf16"]
        assert torch.nn.functional.cosine_similarity(out.float().cpu().flatten(), ref.flatten(), dim=0) > 0.9999

    # sparse_attention_ref through the CSR entry point
    z = np.load(os.path.join(G, "sparse_attention_ref.npz"))
    q = torch.from_numpy(z["q"]).to(torch.bfloat16)
    k = torch.from_numpy(z["k"]).to(torch.bfloat16)
    v = torch.from_numpy(z["v"]).to(torch.bfloat16)
    q2k = torch.from_numpy(z["q2k"])
    seqused = torch.from_numpy(z["seqused"])
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    kp = k.reshape(B * Sk // 128, 128, Hkv, D).permute(0, 2, 1, 3).contiguous()
    vp = v.reshape(B * Sk // 128, 128, Hkv, D).permute(0, 2, 1, 3).contiguous()
    page_table = torch.arange(B * Sk // 128, dtype=torch.int32).view(B, Sk // 128)
    cu_q = torch.arange(0, (B + 1) * Sq, Sq, dtype=torch.int32)
    cu_k = torch.arange(0, (B + 1) * Sk, Sk, dtype=torch.int32)
    q2k_flat = q2k.permute(1, 0, 2, 3).reshape(Hkv, B * Sq, -1).contiguous()
    rp, qi = msa_b200.build_k2q_csr(q2k_flat.cuda(), cu_q, cu_k, 128)
    # topK = 4 (>= the 3 entries per row of the fixture)
    q2k4 = torch.cat([q2k_flat, torch.full_like(q2k_flat[..., :1], -1)], dim=-1)
    rp, qi = msa_b200.build_k2q_csr(q2k4.cuda(), cu_q, cu_k, 128)
    out, lse = msa_b200.sparse_atten_func(q.reshape(B * Sq, Hq, D).cuda(), kp.cuda(), vp.cuda(), rp, qi, 4,
                                          cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, max_seqlen_q=Sq, max_seqlen_k=Sk,
                                          causal=True, return_softmax_lse=True, page_table=page_table.cuda(),
                                          seqused_k=seqused)
    ref_o = torch.from_numpy(z["out"]).reshape(B * Sq, Hq, D)
    ref_l = torch.from_numpy(z["lse"]).reshape(B * Sq, Hq)
    assert (out.float().cpu() - ref_o).abs().max() <= TOL["bf16"]
    assert torch.allclose(lse.cpu(), ref_l, atol=2e-2, rtol=1e-3)


def test_mixed_decode_prefill_split_equals_separate_runs():
    qo, kv = [1, 2, 300], [500, 900, 1000]
    kp, vp, table = make_paged(kv, 2, 5, dtype=torch.float32)
    k8, ks = O.quantize_fp8_per_tensor(kp)
    v8, vs = O.quantize_fp8_per_tensor(vp)
    q = torch.randn(sum(qo), 8, 128, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16)
    idx = O.topk_select(causal_scores(2, qo, kv, 7), 16, 8)[:, :, :4].contiguous()
    plan = msa_b200.fmha_sm100_plan(torch.tensor(qo), torch.tensor(kv), 8, num_kv_heads=2, page_size=128,
                                    kv_block_num=4)
    assert plan[0] and plan[1] == 2
    out, _ = msa_b200.fmha_sm100(q.cuda(), k8.cuda(), v8.cuda(), plan, kv_indices=table.cuda(),
                                 kv_block_indexes=idx.cuda(), k_scale=ks, v_scale=vs)
    ref, _ = O.sparse_attention_paged(q, k8, v8, table, qo, kv, idx, k_scale=ks, v_scale=vs)
    assert (out.float().cpu() - ref).abs().max() <= TOL["fp8"]


def test_properties_at_benchmark_scale():
    """Prefill-sized slice (one 32K request, 16/2 heads): results must not depend on how the
    pages are laid out physically (bit-exact under a page permutation), and a page list that
    names every visible page must reproduce the dense pass bit for bit."""
    L, Hq, Hkv = 32768, 16, 2
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(L, Hq, 128, device="cuda", generator=g).to(torch.bfloat16)
    kp = torch.randn(L // 128, Hkv, 128, 128, device="cuda", generator=g).to(torch.bfloat16)
    vp = torch.randn(L // 128, Hkv, 128, 128, device="cuda", generator=g).to(torch.bfloat16)
    n = L // 128
    ms = torch.rand(Hkv, n, n, device="cuda", generator=g)
    ms = ms.masked_fill(torch.arange(n, device="cuda").view(1, n, 1) > torch.arange(n, device="cuda").view(1, 1, n),
                        float("-inf"))
    sel = msa_b200.sparse_topk_select(ms.contiguous(), 16, n, force_end_blocks=1)          # [n blocks, Hkv, 16]
    idx = sel.repeat_interleave(128, dim=0).contiguous()
    plan = msa_b200.fmha_sm100_plan(torch.tensor([L]), torch.tensor([L]), Hq, num_kv_heads=Hkv, page_size=128,
                                    kv_block_num=16, sparse_kernel_mode="prefill")
    t1 = torch.arange(n, dtype=torch.int32, device="cuda")
    out1, _ = msa_b200.fmha_sm100(q, kp, vp, plan, kv_indices=t1, kv_block_indexes=idx)
    perm = torch.randperm(n, device="cuda", generator=g)
    kp2, vp2 = torch.empty_like(kp), torch.empty_like(vp)
    kp2[perm] = kp
    vp2[perm] = vp
    out2, _ = msa_b200.fmha_sm100(q, kp2, vp2, plan, kv_indices=perm.int(), kv_block_indexes=idx)
    assert msa_b200.plan_status(plan) == 0
    assert torch.equal(out1, out2)
    # sampled oracle check on the last query block (all 16 heads)
    ref, _ = O.sparse_attention_paged(q[-128:].cpu(), kp.cpu(), vp.cpu(), t1.cpu(), [128], [L], idx[-128:].cpu())
    assert (out1[-128:].float().cpu() - ref).abs().max() <= TOL["bf16"]
    # dense == sparse with full lists, on a 2K prefix
    Ls = 2048
    full = O.dense_block_indexes([Ls], [Ls]).unsqueeze(1).expand(-1, Hkv, -1).contiguous().cuda()
    p_d = msa_b200.fmha_sm100_plan(torch.tensor([Ls]), torch.tensor([Ls]), Hq, num_kv_heads=Hkv, page_size=128)
    p_s = msa_b200.fmha_sm100_plan(torch.tensor([Ls]), torch.tensor([Ls]), Hq, num_kv_heads=Hkv, page_size=128,
                                   kv_block_num=16, sparse_kernel_mode="prefill")
    od, _ = msa_b200.fmha_sm100(q[:Ls], kp, vp, p_d, kv_indices=t1[:16], output_maxscore=False)
    os_, _ = msa_b200.fmha_sm100(q[:Ls], kp, vp, p_s, kv_indices=t1[:16], kv_block_indexes=full)
    assert torch.equal(od, os_)


def _csr_inputs(qo, kv, idx):
    """(cu_q, cu_k, page_table, seqused_k, row_ptr, q_indices) for per-token lists ``idx[total_q, Hkv, topk]``."""
    cu_q = torch.tensor([0] + list(np.cumsum(qo)), dtype=torch.int32)
    cu_k = torch.tensor([0] + list(np.cumsum(kv)), dtype=torch.int32)
    rp, qi = msa_b200.build_k2q_csr(idx.permute(1, 0, 2).contiguous(), cu_q, cu_k, 128)
    return cu_q, cu_k, rp, qi


def test_sparse_atten_nvfp4_kv_func_entry_point():
    """The reference-named NVFP4 entry point (python/fmha_sm100/cute/interface.py:768): CSR in, paged NVFP4
    K/V; bit-identical to the page-list entry point and within the bf16 bound of the oracle on the dequantised
    values."""
    qo, kv, Hq, Hkv, topk = [256, 60], [1024, 700], 8, 2, 4
    q, kp, vp, table, idx = _sparse_case(qo, kv, Hq, Hkv, topk, "bf16", "token", seed=35)
    kq, vq = quant.quantize_kv_bf16_to_nvfp4_128x4(kp, vp)
    cu_q, cu_k, rp, qi = _csr_inputs(qo, kv, idx)
    ind = O.page_indptr(kv)
    pt = torch.zeros(2, 8, dtype=torch.int32)
    for b in range(2):
        pt[b, :ind[b + 1] - ind[b]] = table[ind[b]:ind[b + 1]]
    # the CSR rows are laid out over the page-table capacity (8 pages per request)
    cu_k_cap = torch.tensor([0, 1024, 2048], dtype=torch.int32)
    rp, qi = msa_b200.build_k2q_csr(idx.permute(1, 0, 2).contiguous(), cu_q, cu_k_cap, 128)
    out, lse = msa_b200.sparse_atten_nvfp4_kv_func(
        q.cuda(), kq.data.cuda(), vq.data.cuda(), kq.scale_128x4.cuda(), vq.scale_128x4.cuda(),
        kq.global_scale.cuda(), vq.global_scale.cuda(), rp.cuda(), qi.cuda(), topk, cu_seqlens_q=cu_q.cuda(),
        cu_seqlens_k=cu_k_cap.cuda(), max_seqlen_q=max(qo), max_seqlen_k=max(kv), blk_kv=128, causal=True,
        return_softmax_lse=True, page_table=pt.cuda(), seqused_k=torch.tensor(kv, dtype=torch.int32).cuda())
    plan = msa_b200.fmha_sm100_plan(torch.tensor(qo), torch.tensor(kv), Hq, num_kv_heads=Hkv, page_size=128,
                                    kv_block_num=topk, sparse_kernel_mode="prefill")
    dev = lambda t: quant.Nvfp4QuantizedTensor(t.data.cuda(), t.scale_128x4.cuda(), t.global_scale.cuda(),  # noqa: E731
                                               t.logical_scale_shape, t.original_shape)
    out2 = msa_b200.sparse_prefill_nvfp4(q.cuda(), dev(kq), dev(vq), plan, table.cuda(), idx.cuda())
    assert torch.equal(out, out2)
    kr, vr = quant.dequantize_nvfp4_128x4(kq), quant.dequantize_nvfp4_128x4(vq)
    ref, lse_ref = O.sparse_attention_paged(q, kr, vr, table, qo, kv, idx)
    assert (out.float().cpu() - ref).abs().max() <= TOL["bf16"]
    fin = torch.isfinite(lse_ref)
    assert torch.allclose(lse.cpu()[fin], lse_ref[fin], atol=2e-2, rtol=1e-3)


def test_csr_to_lists_kernel_inverts_build_k2q_csr():
    """msa_k2q_csr_to_lists on the device == the host inverse, for ragged requests with short and empty lists."""
    g = torch.Generator().manual_seed(8)
    qo, kv, Hkv, topk = [37, 0, 300], [1000, 128, 5000], 3, 8
    T = sum(qo)
    idx = torch.full((T, Hkv, topk), -1, dtype=torch.int32)
    t = 0
    for ql, kl in zip(qo, kv):
        npg = (kl + 127) // 128
        for i in range(ql):
            for h in range(Hkv):
                n = int(torch.randint(0, min(topk, npg) + 1, (1,), generator=g))
                idx[t, h, :n] = torch.randperm(npg, generator=g)[:n].sort().values.int()
            t += 1
    cu_q, cu_k, rp, qi = _csr_inputs(qo, kv, idx)
    from msa_b200.sparse import _row_map_np
    rr, rb = _row_map_np(kv, 128)
    got = msa_b200.k2q_csr_to_lists(rp.cuda(), qi.cuda(), topk, cu_q.cuda(), torch.from_numpy(rr).cuda(),
                                    torch.from_numpy(rb).cuda(), T)
    assert torch.equal(got.cpu(), idx)
    assert torch.equal(msa_b200.k2q_csr_to_q2k(rp, qi, topk, cu_q, kv, 128), idx)


def test_usable_sm_count_caps_the_grid_without_changing_results():
    qo, kv, Hq, Hkv, topk = [700, 300], [2000, 1500], 8, 2, 8
    q, kp, vp, table, idx = _sparse_case(qo, kv, Hq, Hkv, topk, "fp8", "token", seed=51)
    kd, vd, _, _, kw = _quantise(kp, vp, "fp8")
    outs = []
    for sm in (-1, 16, 1):
        plan = msa_b200.fmha_sm100_plan(torch.tensor(qo), torch.tensor(kv), Hq, num_kv_heads=Hkv, page_size=128,
                                        kv_block_num=topk, sparse_kernel_mode="prefill", usable_SM_count=sm)
        outs.append(msa_b200.fmha_sm100(q.cuda(), kd, vd, plan, kv_indices=table.cuda(), kv_block_indexes=idx.cuda(),
                                        **kw)[0])
        assert msa_b200.plan_status(plan) == 0
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_mixed_batch_writes_straight_into_caller_buffers():
    """Dense mixed batch (two short requests, one long): O and the max scores land in the caller's tensors,
    decode and prefill halves side by side, and equal the two halves run separately."""
    qo, kv = [1, 2, 300], [500, 900, 1000]
    kp, vp, table = make_paged(kv, 2, 5)
    q = torch.randn(sum(qo), 8, 128, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16)
    plan = msa_b200.fmha_sm100_plan(torch.tensor(qo), torch.tensor(kv), 8, num_kv_heads=2, page_size=128,
                                    output_maxscore=True)
    assert plan[0] and plan[1] == 2         # split at the first request longer than 128 query tokens
    out_buf = torch.zeros(sum(qo), 8, 128, dtype=torch.bfloat16, device="cuda")
    ms_buf = torch.full((8, 128, sum(qo)), -float("inf"), device="cuda")
    out, ms = msa_b200.fmha_sm100(q.cuda(), kp.cuda(), vp.cuda(), plan, kv_indices=table.cuda(), out=out_buf,
                                  max_score=ms_buf, output_maxscore=True)
    assert out.data_ptr() == out_buf.data_ptr() and ms.data_ptr() == ms_buf.data_ptr()
    ref, _ = O.dense_attention_paged(q, kp, vp, table, qo, kv)
    assert (out.float().cpu() - ref).abs().max() <= TOL["bf16"]
    msref = O.tile_max_score_paged(q, kp, table, qo, kv, 128)
    assert torch.equal(torch.isfinite(ms.cpu()), torch.isfinite(msref))


def test_build_k2q_csr_kernels_match_the_host_builder_and_the_reference_fixture():
    """msa_build_k2q_csr (count / chunk offsets / row_ptr scan / ordered scatter) == the tensor-op builder on
    ragged requests with short, empty and full lists; and == the reference's own output on its fixture."""
    from msa_b200.sparse import _build_k2q_csr_host
    z = np.load(os.path.join(G, "k2q_csr.npz"))
    q2k = torch.from_numpy(z["q2k"])
    cu_q, cu_k = torch.from_numpy(z["cu_q"]), torch.from_numpy(z["cu_k"])
    rp, qi = msa_b200.build_k2q_csr(q2k.cuda(), cu_q.cuda(), cu_k.cuda(), 128)
    assert torch.equal(rp.cpu(), torch.from_numpy(z["row_ptr"])) and torch.equal(qi.cpu(), torch.from_numpy(z["q_indices"]))
    g = torch.Generator().manual_seed(9)
    qo, kv, Hkv, topk = [700, 0, 33, 1500], [5000, 128, 300, 20000], 3, 8
    T = sum(qo)
    q2k = torch.full((Hkv, T, topk), -1, dtype=torch.int32)
    t = 0
    for ql, kl in zip(qo, kv):
        npg = (kl + 127) // 128
        for i in range(ql):
            for h in range(Hkv):
                n = int(torch.randint(0, min(topk, npg) + 1, (1,), generator=g))
                # popular first block + random others: long rows and short rows
                pick = torch.randperm(npg, generator=g)[:n]
                if n > 0 and i % 3:
                    pick[0] = 0
                u = torch.unique(pick).int()            # ascending, distinct (the forced block may repeat one)
                q2k[h, t, :u.numel()] = u
            t += 1
    cu_q = torch.tensor([0] + list(np.cumsum(qo)), dtype=torch.int32)
    cu_k = torch.tensor([0] + list(np.cumsum(kv)), dtype=torch.int32)
    rp_h, qi_h = _build_k2q_csr_host(q2k, cu_q, cu_k, 128)
    rp_d, qi_d = msa_b200.build_k2q_csr(q2k.cuda(), cu_q.cuda(), cu_k.cuda(), 128)
    assert torch.equal(rp_d.cpu(), rp_h) and torch.equal(qi_d.cpu(), qi_h)


def test_sparse_atten_func_temperature_lse():
    """return_temperature_lse: the LSE of the logits at softmax_scale / lse_temperature_scale
    (python/fmha_sm100/cute/interface.py:665-699), next to the ordinary output and LSE."""
    qo, kv, Hq, Hkv, topk = [200, 90], [1000, 640], 4, 2, 4
    q, kp, vp, table, idx = _sparse_case(qo, kv, Hq, Hkv, topk, "bf16", "token", seed=61)
    cu_q, cu_k, rp, qi = _csr_inputs(qo, kv, idx)
    ind = O.page_indptr(kv)
    pt = torch.zeros(2, 8, dtype=torch.int32)
    for b in range(2):
        pt[b, :ind[b + 1] - ind[b]] = table[ind[b]:ind[b + 1]]
    cu_k_cap = torch.tensor([0, 1024, 2048], dtype=torch.int32)
    rp, qi = msa_b200.build_k2q_csr(idx.permute(1, 0, 2).contiguous().cuda(), cu_q.cuda(), cu_k_cap.cuda(), 128)
    out, lse, lse_t = msa_b200.sparse_atten_func(
        q.cuda(), kp.cuda(), vp.cuda(), rp, qi, topk, cu_seqlens_q=cu_q.cuda(), cu_seqlens_k=cu_k_cap.cuda(),
        max_seqlen_q=max(qo), max_seqlen_k=max(kv), causal=True, return_softmax_lse=True, return_temperature_lse=True,
        lse_temperature_scale=2.5, page_table=pt.cuda(), seqused_k=torch.tensor(kv, dtype=torch.int32).cuda())
    ref, lse_ref = O.sparse_attention_paged(q, kp, vp, table, qo, kv, idx)
    _, lse_t_ref = O.sparse_attention_paged(q, kp, vp, table, qo, kv, idx, sm_scale=128 ** -0.5 / 2.5)
    assert (out.float().cpu() - ref).abs().max() <= TOL["bf16"]
    fin = torch.isfinite(lse_ref)
    assert torch.allclose(lse.cpu()[fin], lse_ref[fin], atol=2e-2, rtol=1e-3)
    assert torch.allclose(lse_t.cpu()[fin], lse_t_ref[fin], atol=2e-2, rtol=1e-3)
    with pytest.raises(ValueError):
        msa_b200.sparse_atten_func(q.cuda(), kp.cuda(), vp.cuda(), rp, qi, topk, cu_seqlens_q=cu_q.cuda(),
                                   cu_seqlens_k=cu_k_cap.cuda(), max_seqlen_q=max(qo), max_seqlen_k=max(kv),
                                   causal=True, return_temperature_lse=True, page_table=pt.cuda())


def test_corrupt_page_table_is_reported_not_followed():
    """A page-table entry beyond the page pool: the kernel reads page 0 instead, finishes normally and the status
    word reads MSA_ERR_BOUNDS (what the reference's FMHA_GMEM_CHECK build reports, csrc/gmem_bounds_check.h:27-95).
    Nothing is read out of bounds, so nothing faults; a clean call on the same plan then reads status 0 again."""
    kv_lens = [700]
    kp, vp, table = make_paged(kv_lens, 2, 51)
    q = torch.randn(64, 4, 128, generator=torch.Generator().manual_seed(52)).to(torch.bfloat16)
    plan = msa_b200.fmha_sm100_plan(torch.tensor([64]), torch.tensor(kv_lens), 4, num_kv_heads=2, page_size=128,
                                    output_maxscore=True)
    bad = table.clone()
    bad[2] = kp.shape[0] + 5
    for kwargs in (dict(output_o=True, output_maxscore=False), dict(output_o=False, output_maxscore=True)):
        msa_b200.fmha_sm100(q.cuda(), kp.cuda(), vp.cuda(), plan, kv_indices=bad.cuda(), **kwargs)
        assert msa_b200.plan_status(plan) == msa_b200._lib.MSA_ERR_BOUNDS
        plan[3]["status"].zero_()
        msa_b200.fmha_sm100(q.cuda(), kp.cuda(), vp.cuda(), plan, kv_indices=table.cuda(), **kwargs)
        assert msa_b200.plan_status(plan) == 0
