"""Parity at the shapes the benchmark times, sub-sampled: a few (request, 128-query block) slices of a
full-size launch against the oracle (max-abs <= 6e-2 for FP8 K/V, 1.5e-1 for NVFP4 K/V vs unquantised values
and 2e-2 on the dequantised values).  Full-size inputs live on the GPU only; the slices and the pages they
touch are copied to the host for the oracle."""
import pytest
import torch

import msa_b200
from msa_b200 import quant
from oracle import msa_oracle as O

pytestmark = pytest.mark.gpu
PAGE, D = 128, 128


def _pages_of(pool, table_dev, lo, hi):
    """The request's pages, gathered on the device and copied to the host in logical order."""
    return pool[table_dev[lo:hi].long()].cpu()


def test_c3_sparse_prefill_fp8_sampled_against_oracle():
    """Ragged 16384/32768/65536/131072 batch, 64/8 heads, FP8 K/V, top-16 per 128-query block from this
    library's proxy pass + selector: the last and one middle query block of EVERY request, all 64 heads.
    The 131072-token request has 1024 logical pages (multi-word page bitmaps)."""
    lens, hq, hkv, topk = (16384, 32768, 65536, 131072), 64, 8, 16
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(2)
    T, n_pages = sum(lens), sum(lens) // PAGE
    q = torch.randn(T, hq, D, device=dev, dtype=torch.bfloat16, generator=g)
    k8, ks = quant.quantize_fp8_per_tensor(torch.randn(n_pages, hkv, PAGE, D, device=dev, dtype=torch.bfloat16,
                                                       generator=g))
    v8, vs = quant.quantize_fp8_per_tensor(torch.randn(n_pages, hkv, PAGE, D, device=dev, dtype=torch.bfloat16,
                                                       generator=g))
    table = torch.randperm(n_pages, device=dev, generator=g).int()
    qo = torch.tensor(lens)
    qp = torch.zeros(T, 1, D, device=dev, dtype=torch.bfloat16)
    qp[:, 0, :64] = q[:, 0, :64]
    kp = torch.zeros(n_pages, 1, PAGE, D, device=dev, dtype=torch.float8_e4m3fn)
    kp.view(torch.uint8)[:, 0, :, :64] = k8.view(torch.uint8)[:, 0, :, :64]
    plan_p = msa_b200.fmha_sm100_plan(qo, qo, 1, num_kv_heads=1, page_size=PAGE, output_maxscore=True)
    ms = msa_b200.fmha_sm100(qp, kp, None, plan_p, kv_indices=table, output_maxscore=True, output_o=False,
                             score_dim=64)[1]
    starts = torch.arange(0, T + 1, PAGE, dtype=torch.int32, device=dev)
    idx = msa_b200.sparse_topk_select(ms, topk, num_valid_pages=max(lens) // PAGE, q_block_starts=starts)
    idx = idx.expand(-1, hkv, -1).contiguous()
    plan = msa_b200.fmha_sm100_plan(qo, qo, hq, num_kv_heads=hkv, page_size=PAGE, kv_block_num=topk,
                                    sparse_kernel_mode="prefill")
    out = msa_b200.fmha_sm100(q, k8, v8, plan, kv_indices=table, kv_block_indexes=idx, k_scale=ks, v_scale=vs)[0]
    torch.cuda.synchronize()
    assert msa_b200.plan_status(plan) == 0
    assert not bool(out.isnan().any())
    tok0 = pg0 = 0
    worst = 0.0
    for L in lens:
        npg = L // PAGE
        kreq, vreq = _pages_of(k8, table, pg0, pg0 + npg), _pages_of(v8, table, pg0, pg0 + npg)
        local = torch.arange(npg, dtype=torch.int32)
        for blk in (npg - 1, npg // 2 + 3):
            s = tok0 + blk * PAGE
            # the proxy scores of the sampled block: exact -inf pattern and values of the visible pages
            ms_ref = O.tile_max_score_paged(qp[s:s + PAGE].cpu(), kp.view(torch.uint8)[table[pg0:pg0 + npg].long()]
                                            .view(torch.float8_e4m3fn).cpu(), local, [PAGE], [L], ms.shape[1],
                                            qo_offset=[blk * PAGE])
            got = ms[:, :, s:s + PAGE].cpu()
            assert torch.equal(torch.isfinite(got), torch.isfinite(ms_ref))
            fin = torch.isfinite(ms_ref)
            assert torch.allclose(got[fin], ms_ref[fin], atol=1e-1, rtol=1e-3)
            # the page list of the block is the oracle's selection on the kernel's own scores
            bm = O.block_max_score(got, [0, PAGE])
            assert torch.equal(idx[s, 0].cpu(), O.topk_select(bm, topk, max(lens) // PAGE)[0, 0])
            err = O.sampled_sparse_error(out[s:s + PAGE].cpu(), q[s:s + PAGE].cpu(), kreq, vreq, local, L,
                                         blk * PAGE, idx[s:s + PAGE].cpu(), k_scale=ks, v_scale=vs)
            worst = max(worst, err)
            assert err <= 6e-2, (L, blk, err)
        tok0 += L
        pg0 += npg
    print(f"C3 sampled max-abs vs oracle: {worst:.4f}")


def test_c4_decode_131072_contexts_sampled_against_oracle():
    """32 requests x 1 token over 131072-token contexts (1024 logical pages each, 32768 physical), 64/8 heads,
    top-64 from sparse_topk_select over uniform scores: two of the requests, all heads."""
    batch, ctx, hq, hkv, topk = 32, 131072, 64, 8, 64
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(3)
    ppr = ctx // PAGE
    n_pages = batch * ppr
    scale = 5.5 / 448.0
    k8 = torch.empty(n_pages, hkv, PAGE, D, device=dev, dtype=torch.float8_e4m3fn)
    v8 = torch.empty_like(k8)
    for s in range(0, n_pages, 2048):
        e = min(n_pages, s + 2048)
        k8[s:e] = (torch.randn(e - s, hkv, PAGE, D, device=dev, generator=g) / scale).clamp(-448, 448).to(k8.dtype)
        v8[s:e] = (torch.randn(e - s, hkv, PAGE, D, device=dev, generator=g) / scale).clamp(-448, 448).to(k8.dtype)
    q = torch.randn(batch, hq, D, device=dev, dtype=torch.bfloat16, generator=g)
    table = torch.randperm(n_pages, device=dev, generator=g).int()
    scores = torch.rand(hkv, ppr, batch, device=dev, generator=g)
    idx = msa_b200.sparse_topk_select(scores, topk, num_valid_pages=ppr)
    assert torch.equal(idx.cpu(), O.topk_select(scores.cpu(), topk, ppr))
    plan = msa_b200.fmha_sm100_plan(torch.tensor([1] * batch), torch.tensor([ctx] * batch), hq, num_kv_heads=hkv,
                                    page_size=PAGE, kv_block_num=topk)
    assert plan[3]["use_decode_kernel"]
    out = msa_b200.fmha_sm100(q, k8, v8, plan, kv_indices=table, kv_block_indexes=idx, k_scale=scale,
                              v_scale=scale)[0]
    torch.cuda.synchronize()
    assert msa_b200.plan_status(plan) == 0
    local = torch.arange(ppr, dtype=torch.int32)
    for b in (0, 21):
        kreq, vreq = _pages_of(k8, table, b * ppr, (b + 1) * ppr), _pages_of(v8, table, b * ppr, (b + 1) * ppr)
        err = O.sampled_sparse_error(out[b:b + 1].cpu(), q[b:b + 1].cpu(), kreq, vreq, local, ctx, ctx - 1,
                                     idx[b:b + 1].cpu(), k_scale=scale, v_scale=scale)
        assert err <= 6e-2, (b, err)


def test_c5_nvfp4_share_sampled_against_oracle():
    """One GPU's share of the NVFP4 case: 8 x 32768 tokens, 8 query heads on 1 KV head, top-32 per
    128-query block: the last block and a middle block of two requests."""
    n_req, L, hq, hkv, topk = 8, 32768, 8, 1, 32
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(4)
    T, n_pages, ppr = n_req * L, n_req * L // PAGE, L // PAGE
    q = torch.randn(T, hq, D, device=dev, dtype=torch.bfloat16, generator=g)
    kf = torch.randn(n_pages, hkv, PAGE, D, device=dev, dtype=torch.bfloat16, generator=g)
    vf = torch.randn(n_pages, hkv, PAGE, D, device=dev, dtype=torch.bfloat16, generator=g)
    kq, vq = msa_b200.quantize_kv_bf16_to_nvfp4_128x4(kf, vf)
    kd, vd = quant.dequantize_nvfp4_128x4(kq), quant.dequantize_nvfp4_128x4(vq)
    table = torch.randperm(n_pages, device=dev, generator=g).int()
    nblk = T // PAGE
    sc = torch.rand(hkv, ppr, nblk, device=dev, generator=g)
    blk_in_req = torch.arange(nblk, device=dev) % ppr
    sc.masked_fill_(torch.arange(ppr, device=dev)[None, :, None] > blk_in_req[None, None, :], -float("inf"))
    idx = msa_b200.sparse_topk_select(sc, topk, num_valid_pages=ppr).repeat_interleave(PAGE, dim=0).contiguous()
    qo = torch.tensor([L] * n_req)
    plan = msa_b200.fmha_sm100_plan(qo, qo, hq, num_kv_heads=hkv, page_size=PAGE, kv_block_num=topk,
                                    sparse_kernel_mode="prefill")
    out = msa_b200.sparse_prefill_nvfp4(q, kq, vq, plan, table, idx)
    torch.cuda.synchronize()
    assert msa_b200.plan_status(plan) == 0
    local = torch.arange(ppr, dtype=torch.int32)
    for b, blk in ((0, ppr - 1), (5, ppr // 2), (7, ppr - 1)):
        s = b * L + blk * PAGE
        args = (q[s:s + PAGE].cpu(),)
        kreq, vreq = _pages_of(kd, table, b * ppr, (b + 1) * ppr), _pages_of(vd, table, b * ppr, (b + 1) * ppr)
        err = O.sampled_sparse_error(out[s:s + PAGE].cpu(), args[0], kreq, vreq, local, L, blk * PAGE,
                                     idx[s:s + PAGE].cpu())
        assert err <= 2e-2, (b, blk, err)          # same dequantised values on both sides
        kraw, vraw = _pages_of(kf, table, b * ppr, (b + 1) * ppr), _pages_of(vf, table, b * ppr, (b + 1) * ppr)
        err_raw = O.sampled_sparse_error(out[s:s + PAGE].cpu(), args[0], kraw, vraw, local, L, blk * PAGE,
                                         idx[s:s + PAGE].cpu())
        assert err_raw <= 1.5e-1 * 4, (b, blk, err_raw)
