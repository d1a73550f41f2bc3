"""Paged FP8 sparse decode against the oracle (tolerance: max-abs <= 6e-2 vs fp32)."""
import pytest
import torch

import msa_b200
from oracle import msa_oracle as O
from util import make_paged

pytestmark = pytest.mark.gpu
TOL_FP8 = 6e-2


def _run(qo_lens, kv_lens, Hq, Hkv, topk, splits, seed, drop_tail=0, sm_scale=None):
    B = len(qo_lens)
    kp, vp, table = make_paged(kv_lens, Hkv, seed, dtype=torch.float32, extra_pages=3)
    k8, ks = O.quantize_fp8_per_tensor(kp)
    v8, vs = O.quantize_fp8_per_tensor(vp)
    g = torch.Generator().manual_seed(seed + 1)
    T = sum(qo_lens)
    q = torch.randn(T, Hq, 128, generator=g).to(torch.bfloat16)
    ms = torch.rand(Hkv, 128, T, generator=g)
    off = 0
    for ql, kl in zip(qo_lens, kv_lens):
        for i in range(ql):
            ms[:, (min(kl, kl - ql + i + 1) + 127) // 128:, off + i] = float("-inf")
        off += ql
    idx = O.topk_select(ms, 64, 128)[:, :, :topk].contiguous()
    if drop_tail:
        idx[:, :, topk - drop_tail:] = -1
    ref, lse_ref = O.sparse_attention_paged(q, k8, v8, table, qo_lens, kv_lens, idx, sm_scale=sm_scale, k_scale=ks,
                                            v_scale=vs)
    plan = msa_b200.fmha_sm100_plan(torch.tensor(qo_lens), torch.tensor(kv_lens), Hq, num_kv_heads=Hkv, page_size=128,
                                    kv_block_num=topk, num_kv_splits=splits)
    assert plan[3]["use_decode_kernel"]
    out, _, lse = msa_b200.fmha_sm100(q.cuda(), k8.cuda(), v8.cuda(), plan, kv_indices=table.cuda(),
                                      kv_block_indexes=idx.cuda(), k_scale=ks, v_scale=vs, sm_scale=sm_scale,
                                      return_lse=True)
    return out.float().cpu(), ref, lse.cpu(), lse_ref


@pytest.mark.parametrize("Hq,Hkv,topk,splits", [(64, 8, 64, -1), (16, 2, 8, 1), (16, 2, 8, 4), (16, 1, 16, 2),
                                                (4, 4, 4, 1), (6, 2, 5, 5)])
def test_decode_parity(Hq, Hkv, topk, splits):
    out, ref, lse, lse_ref = _run([1, 1, 1, 1], [1500, 8192, 300, 1024], Hq, Hkv, topk, splits, seed=Hq + topk)
    assert (out - ref).abs().max() <= TOL_FP8
    assert torch.allclose(lse, lse_ref, atol=2e-2)
    assert torch.nn.functional.cosine_similarity(out.flatten(), ref.flatten(), dim=0) > 0.999


def test_decode_multi_token_and_padding():
    # several new tokens per request (each masks by its own position), short lists padded with -1
    out, ref, _, _ = _run([3, 1, 17], [700, 129, 2000], 16, 2, 8, 2, seed=3, drop_tail=3)
    assert (out - ref).abs().max() <= TOL_FP8


def test_decode_wrapper_dense():
    kv_lens = [900, 2048, 130]
    kp, vp, table = make_paged(kv_lens, 2, 11, dtype=torch.float32)
    k8, ks = O.quantize_fp8_per_tensor(kp)
    v8, vs = O.quantize_fp8_per_tensor(vp)
    q = torch.randn(3, 16, 128).to(torch.bfloat16)
    ref, _ = O.dense_attention_paged(q, k8, v8, table, [1, 1, 1], kv_lens, k_scale=ks, v_scale=vs)
    pt = torch.zeros(3, 16, dtype=torch.int32)
    ind = O.page_indptr(kv_lens)
    for b in range(3):
        pt[b, :ind[b + 1] - ind[b]] = table[ind[b]:ind[b + 1]]
    w = msa_b200.SparseDecodePagedAttentionWrapper().plan(pt.cuda(), torch.tensor(kv_lens, dtype=torch.int32),
                                                          num_qo_heads=16, num_kv_heads=2)
    out = w.run(q.cuda(), k8.cuda(), v8.cuda(), k_scale=ks, v_scale=vs).float().cpu()
    assert (out - ref).abs().max() <= TOL_FP8


def _page_table(table, kv_lens, width):
    pt = torch.zeros(len(kv_lens), width, dtype=torch.int32)
    ind = O.page_indptr(kv_lens)
    for b in range(len(kv_lens)):
        pt[b, :ind[b + 1] - ind[b]] = table[ind[b]:ind[b + 1]]
    return pt


@pytest.mark.parametrize("kv_lens", [[20000, 17000], [40000, 128 * 65]])
def test_decode_wrapper_dense_long_lists(kv_lens):
    """Dense decode over 157 / 313 pages: one split holds more than 64 list entries, which the ring kernel
    walks in chunks of 64.  Reference-style keyword call (python/fmha_sm100/cute/interface.py:1175-1195,
    1336-1346)."""
    kp, vp, table = make_paged(kv_lens, 2, 21, dtype=torch.float32)
    k8, ks = O.quantize_fp8_per_tensor(kp)
    v8, vs = O.quantize_fp8_per_tensor(vp)
    q = torch.randn(2, 16, 128, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    ref, lse_ref = O.dense_attention_paged(q, k8, v8, table, [1, 1], kv_lens, k_scale=ks, v_scale=vs)
    pt = _page_table(table, kv_lens, 320).cuda()
    lens = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    for kwargs in (dict(), dict(disable_split_kv=True), dict(fixed_split_size=100)):
        w = msa_b200.SparseDecodePagedAttentionWrapper(blk_kv=128, causal=True)
        w.plan(page_table=pt, seqused_k=lens, seqlen_q=1, max_seqlen_k=max(kv_lens), q2k_indices=None,
               num_qo_heads=16, num_kv_heads=2, head_dim=128, enable_cuda_graph=False, **kwargs)
        if "disable_split_kv" in kwargs:
            assert not w.split_kv
        out_buf = torch.empty(2, 16, 128, dtype=torch.bfloat16, device="cuda")
        out, lse = w.run(q.cuda(), k8.cuda(), v8.cuda(), k_scale=ks, v_scale=vs, return_softmax_lse=True, out=out_buf)
        assert out.data_ptr() == out_buf.data_ptr()
        assert (out.float().cpu() - ref).abs().max() <= TOL_FP8, kwargs
        assert torch.allclose(lse.cpu(), lse_ref, atol=2e-2), kwargs


@pytest.mark.parametrize("splits", [1, 2])
def test_decode_lists_longer_than_64_per_split(splits):
    """fmha_sm100 decode with 128-entry page lists and 1 or 2 splits (128 / 64 entries per split)."""
    kv_lens = [128 * 200, 128 * 150 + 17]
    Hq, Hkv, topk = 16, 2, 128
    kp, vp, table = make_paged(kv_lens, Hkv, 31, dtype=torch.float32)
    k8, ks = O.quantize_fp8_per_tensor(kp)
    v8, vs = O.quantize_fp8_per_tensor(vp)
    g = torch.Generator().manual_seed(32)
    q = torch.randn(2, Hq, 128, generator=g).to(torch.bfloat16)
    idx = torch.full((2, Hkv, topk), -1, dtype=torch.int32)
    for t, kl in enumerate(kv_lens):
        npg = (kl + 127) // 128
        for h in range(Hkv):
            idx[t, h] = torch.randperm(npg, generator=g)[:topk].sort().values.int()
    ref, lse_ref = O.sparse_attention_paged(q, k8, v8, table, [1, 1], kv_lens, idx, k_scale=ks, v_scale=vs)
    plan = msa_b200.fmha_sm100_plan(torch.tensor([1, 1]), torch.tensor(kv_lens), Hq, num_kv_heads=Hkv, page_size=128,
                                    kv_block_num=topk, num_kv_splits=splits)
    assert plan[3]["use_decode_kernel"] and plan[3]["num_kv_splits"] == splits
    out, _, lse = msa_b200.fmha_sm100(q.cuda(), k8.cuda(), v8.cuda(), plan, kv_indices=table.cuda(),
                                      kv_block_indexes=idx.cuda(), k_scale=ks, v_scale=vs, return_lse=True)
    assert (out.float().cpu() - ref).abs().max() <= TOL_FP8
    assert torch.allclose(lse.cpu(), lse_ref, atol=2e-2)


def test_sparse_decode_atten_func_reference_signature():
    """sparse_decode_atten_func(q, k, v, q2k_indices[Hkv, total_q, topK], page_table=..., ...) with two new
    tokens per request and e4m3 queries, as the reference's decode entry takes them."""
    kv_lens = [3000, 1111]
    Hq, Hkv, topk, sq = 16, 2, 8, 2
    kp, vp, table = make_paged(kv_lens, Hkv, 41, dtype=torch.float32)
    k8, ks = O.quantize_fp8_per_tensor(kp)
    v8, vs = O.quantize_fp8_per_tensor(vp)
    g = torch.Generator().manual_seed(42)
    q = torch.randn(2 * sq, Hq, 128, generator=g).to(torch.float8_e4m3fn)
    idx = torch.full((2 * sq, Hkv, topk), -1, dtype=torch.int32)
    for b, kl in enumerate(kv_lens):
        for j in range(sq):
            vis = (kl - sq + j + 1 + 127) // 128
            for h in range(Hkv):
                idx[b * sq + j, h] = torch.randperm(vis, generator=g)[:topk].sort().values.int()
    ref, lse_ref = O.sparse_attention_paged(q.float(), k8, v8, table, [sq, sq], kv_lens, idx, k_scale=ks, v_scale=vs)
    pt = _page_table(table, kv_lens, 24).cuda()
    # the reference entry has no scale arguments: the K scale rides on softmax_scale, the V scale on the output
    out, lse = msa_b200.sparse_decode_atten_func(
        q.cuda(), k8.cuda(), v8.cuda(), idx.permute(1, 0, 2).contiguous().cuda(), page_table=pt,
        seqused_k=torch.tensor(kv_lens, dtype=torch.int32, device="cuda"), seqlen_q=sq, max_seqlen_k=max(kv_lens),
        blk_kv=128, causal=True, softmax_scale=ks / 128 ** 0.5, return_softmax_lse=True)
    assert (out.float().cpu() * vs - ref).abs().max() <= TOL_FP8
    assert torch.allclose(lse.cpu(), lse_ref, atol=2e-2)
