"""Pins oracle/msa_oracle.py to outputs of the reference's own PyTorch code
(fixtures made by tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest
import torch

from oracle import msa_oracle as O

G = os.path.join(os.path.dirname(__file__), "golden")


def _ragged_to_pages(k, kv_lens, Hkv, shuffle_seed=None):
    """ragged [sum kv, H, D] -> pages [n, H, 128, D] + flat page table."""
    indptr = O.page_indptr(kv_lens)
    n = indptr[-1]
    D = k.shape[-1]
    pages = torch.zeros(n, Hkv, 128, D, dtype=k.dtype)
    perm = torch.arange(n)
    if shuffle_seed is not None:
        perm = torch.randperm(n, generator=torch.Generator().manual_seed(shuffle_seed))
    off = 0
    for b, kl in enumerate(kv_lens):
        for p in range(indptr[b + 1] - indptr[b]):
            t0, t1 = p * 128, min((p + 1) * 128, kl)
            pages[perm[indptr[b] + p], :, :t1 - t0] = k[off + t0:off + t1].permute(1, 0, 2)
        off += kl
    return pages, perm.to(torch.int32)


def test_max_score_matches_reference():
    z = np.load(os.path.join(G, "maxscore.npz"))
    q = torch.from_numpy(z["q"]).to(torch.bfloat16)
    k = torch.from_numpy(z["k"]).to(torch.bfloat16)
    qo, kv = z["qo_lens"].tolist(), z["kv_lens"].tolist()
    pages, table = _ragged_to_pages(k, kv, int(z["Hkv"]), shuffle_seed=3)
    assert bool(z["tail_all_neg_inf"])
    for key, off in (("ms_default", None), ("ms_off", z["offs"].tolist())):
        got = O.tile_max_score_paged(q, pages, table, qo, kv, 4, causal=True, qo_offset=off)
        ref = torch.from_numpy(z[key])
        assert torch.equal(torch.isinf(got), torch.isinf(ref))
        fin = torch.isfinite(ref)
        assert torch.allclose(got[fin], ref[fin], atol=1e-4, rtol=1e-5)


def test_topk_passes_reference_verifier():
    z = np.load(os.path.join(G, "topk.npz"))
    assert bool(z["verifier_ok"]) and int(z["n_mismatch"]) == 0
    ms = torch.from_numpy(z["ms"])
    sel = O.topk_select(ms, 16, num_valid_pages=40)
    assert torch.equal(sel, torch.from_numpy(z["sel"]))
    # re-derive the multiset check (tests/integration/test_proxy_kv_e2e.py:77-116)
    s = ms.permute(2, 0, 1)
    valid = sel >= 0
    got = torch.gather(s, -1, torch.where(valid, sel, torch.zeros_like(sel)).long())
    got = torch.where(valid, got, torch.full_like(got, float("-inf"))).sort(dim=-1).values
    ref = torch.from_numpy(z["ref_sorted_scores"])
    assert torch.equal(torch.isfinite(got), torch.isfinite(ref))
    assert torch.equal(got[torch.isfinite(ref)], ref[torch.isfinite(ref)])
    # ascending, -1 only at the tail, lower index wins the tie injected at head 1
    v = sel.clone().long()
    v[v < 0] = 1 << 30
    assert (v[..., 1:] >= v[..., :-1]).all()


def test_topk_forced_blocks_and_k():
    torch.manual_seed(0)
    ms = torch.randn(2, 256, 10)
    for topk in (16, 32, 64):
        sel = O.topk_select(ms, topk, num_valid_pages=200, force_begin=2, force_end=3)
        for t in range(10):
            for h in range(2):
                row = set(sel[t, h].tolist())
                assert {0, 1, 197, 198, 199} <= row
                assert len(row) == topk and max(row) < 200


def test_sparse_ref_fixture():
    z = np.load(os.path.join(G, "sparse_ref.npz"), allow_pickle=True)
    q = torch.from_numpy(z["q"]).to(torch.bfloat16)
    kp = torch.from_numpy(z["k_pages"]).to(torch.bfloat16)
    vp = torch.from_numpy(z["v_pages"]).to(torch.bfloat16)
    qo, kv = z["qo_lens"].tolist(), z["kv_lens"].tolist()
    blocks = [z["blocks0"].tolist(), z["blocks1"].tolist()]
    Hkv, topk = 2, 4
    rows = []
    for b, ql in enumerate(qo):
        per = torch.full((Hkv, topk), -1, dtype=torch.int32)
        for h in range(Hkv):
            per[h, :len(blocks[b][h])] = torch.tensor(blocks[b][h], dtype=torch.int32)
        rows.append(per.unsqueeze(0).expand(ql, Hkv, topk))
    idx = torch.cat(rows, 0).contiguous()
    table = torch.arange(kp.shape[0], dtype=torch.int32)
    out, _ = O.sparse_attention_paged(q, kp, vp, table, qo, kv, idx)
    ref = torch.from_numpy(z["out"])
    assert (out - ref).abs().max() < 1.6e-2          # ref output is rounded to bf16
    assert torch.nn.functional.cosine_similarity(out.flatten(), ref.flatten(), dim=0) > 0.99999


def test_sparse_attention_ref_fixture():
    z = np.load(os.path.join(G, "sparse_attention_ref.npz"))
    q = torch.from_numpy(z["q"]).to(torch.bfloat16)     # [B,Sq,Hq,D]
    k = torch.from_numpy(z["k"]).to(torch.bfloat16)
    v = torch.from_numpy(z["v"]).to(torch.bfloat16)
    q2k = torch.from_numpy(z["q2k"])                    # [B,Hkv,Sq,topk]
    seqused = z["seqused"].tolist()
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    kp = k.reshape(B * Sk // 128, 128, Hkv, D).permute(0, 2, 1, 3).contiguous()
    vp = v.reshape(B * Sk // 128, 128, Hkv, D).permute(0, 2, 1, 3).contiguous()
    # page table: request b owns pages [b*Sk/128, ...) but only ceil(seqused/128) are listed
    table = torch.cat([torch.arange(b * Sk // 128, b * Sk // 128 + (seqused[b] + 127) // 128) for b in range(B)]).int()
    idx = q2k.permute(0, 2, 1, 3).reshape(B * Sq, Hkv, -1).contiguous()
    out, lse = O.sparse_attention_paged(q.reshape(B * Sq, Hq, D), kp, vp, table, [Sq] * B, seqused, idx)
    ref_o = torch.from_numpy(z["out"]).reshape(B * Sq, Hq, D)
    ref_l = torch.from_numpy(z["lse"]).reshape(B * Sq, Hq)
    assert torch.allclose(out, ref_o, atol=2e-5, rtol=1e-4)
    assert torch.allclose(lse, ref_l, atol=1e-4, rtol=1e-5)


def test_k2q_csr_fixture():
    z = np.load(os.path.join(G, "k2q_csr.npz"))
    rp, qi = O.build_k2q_csr(torch.from_numpy(z["q2k"]), z["cu_q"].tolist(), z["cu_k"].tolist(), 128)
    assert torch.equal(rp, torch.from_numpy(z["row_ptr"]))
    assert torch.equal(qi, torch.from_numpy(z["q_indices"]))


def test_nvfp4_layout_and_dequant_fixture():
    z = np.load(os.path.join(G, "nvfp4.npz"))
    data, scale, gs = torch.from_numpy(z["data"]), torch.from_numpy(z["scale"]), float(z["gs"])
    deq = O.dequantize_nvfp4(data, scale, gs)
    ref = torch.from_numpy(z["deq_bf16"])
    assert torch.equal(deq.to(torch.bfloat16).float(), ref)
    r = torch.arange(300).view(-1, 1).expand(300, 8)
    c = torch.arange(8).view(1, -1).expand(300, 8)
    assert torch.equal(O.nvfp4_scale_offset(r, c, 8), torch.from_numpy(z["offsets"]))
    # the quantiser reproduces its own stored bytes and stays within half a step
    x = torch.from_numpy(z["x"])
    d2, s2, g2 = O.quantize_nvfp4(x)
    assert torch.equal(d2, data) and torch.equal(s2, scale) and g2 == gs
    assert (deq - x).abs().max() < 0.6


def test_fp8_roundtrip():
    torch.manual_seed(1)
    x = torch.randn(4, 2, 128, 128)
    q8, s = O.quantize_fp8_per_tensor(x)
    assert q8.dtype == torch.float8_e4m3fn and abs(s - float(x.abs().max()) / 448) < 1e-9
    assert ((q8.float() * s - x).abs() <= 0.0625 * x.abs() + s).all()


def test_dense_equals_sparse_with_full_lists():
    torch.manual_seed(2)
    qo, kv = [40, 130], [300, 130]
    ind = O.page_indptr(kv)
    kp = torch.randn(ind[-1], 2, 128, 128)
    vp = torch.randn(ind[-1], 2, 128, 128)
    q = torch.randn(sum(qo), 4, 128)
    table = torch.randperm(ind[-1]).int()
    idx = O.dense_block_indexes(qo, kv).unsqueeze(1).expand(-1, 2, -1).contiguous()
    o1, l1 = O.sparse_attention_paged(q, kp, vp, table, qo, kv, idx)
    o2, l2 = O.dense_attention_paged(q, kp, vp, table, qo, kv)
    assert torch.allclose(o1, o2, atol=1e-5) and torch.allclose(l1, l2, atol=1e-5)


def test_kv_append_oracle_matches_whole_tensor_quantisers():
    """The append restatement (explicit float32 arithmetic, scatter by slot) reproduces the stored NVFP4 bytes of
    the fixture -- whose layout the reference's own dequantiser pins -- and the per-tensor FP8 quantiser."""
    z = np.load(os.path.join(G, "nvfp4.npz"))
    x = torch.from_numpy(z["x"]).to(torch.bfloat16)                       # cache layout [pages, Hkv, 128, 128]
    pages, hkv = x.shape[0], x.shape[1]
    new = x.permute(0, 2, 1, 3).reshape(pages * 128, hkv, 128).contiguous()   # token-major rows
    perm = torch.randperm(pages * 128, generator=torch.Generator().manual_seed(3))
    slots = perm.int()                                                     # token i of `new[perm]` lives at slot perm[i]
    kc = torch.zeros(pages, hkv, 128, 64, dtype=torch.uint8)
    vc = torch.zeros_like(kc)
    ks = torch.zeros(pages * hkv * 128 * 8, dtype=torch.uint8)
    vs = torch.zeros_like(ks)
    gs = float(z["gs"])
    O.kv_append_nvfp4(new[perm], new[perm], kc, vc, ks, vs, slots, gs, gs)
    assert torch.equal(ks, torch.from_numpy(z["scale"])) and torch.equal(vs, ks) and torch.equal(vc, kc)
    # the append multiplies by the reciprocal where the whole-tensor quantiser divides: the codes may differ
    # where the quotient sits within an ulp of a rounding midpoint, by one grid step, and nowhere else
    gold = torch.from_numpy(z["data"])
    diff = kc != gold
    assert diff.float().mean() < 1e-3
    deq = O.dequantize_nvfp4(kc, ks, gs)
    ref = torch.from_numpy(z["deq_bf16"])
    step = O.dequantize_nvfp4(torch.full_like(kc, 0x22), ks, gs)          # code 2 everywhere: 1.0 * block scale
    assert ((deq - ref).abs() <= 2.0 * step + 1e-6).all()
    same = ~diff.repeat_interleave(2, dim=-1)
    assert torch.equal(deq.to(torch.bfloat16).float()[same], ref[same])
    # FP8, with skipped tokens: their rows keep the cache's previous bytes
    q8, s = O.quantize_fp8_per_tensor(x.float())
    k8 = torch.full((pages, hkv, 128, 128), 0x7f, dtype=torch.uint8)
    v8 = torch.full_like(k8, 0x7f)
    slots2 = slots.clone()
    slots2[::5] = -1
    O.kv_append_fp8(new[perm], new[perm], k8, v8, slots2, s, s)
    want = q8.view(torch.uint8).clone()
    skipped = perm[::5]
    want[skipped // 128, :, skipped % 128] = 0x7f
    assert torch.equal(k8, v8)
    off = (k8 != want)
    assert off.float().mean() < 1e-3 and (k8.int() - want.int()).abs().max() <= 1     # reciprocal vs division
    assert torch.equal(k8[skipped // 128, :, skipped % 128], want[skipped // 128, :, skipped % 128])


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
def test_fp4_indexer_fixture(fmt):
    """FP4 indexer oracle against the reference's own CPU scorer, dequantiser and scale-storage strides
    (python/fmha_sm100/cute/test_fp4_indexer.py:153-327, fp4_indexer_interface.py:220-249)."""
    z = np.load(os.path.join(G, "fp4_indexer.npz"))
    q, k = torch.from_numpy(z[f"{fmt}_q"]), torch.from_numpy(z[f"{fmt}_k"])
    qs, ks = torch.from_numpy(z[f"{fmt}_qs"]), torch.from_numpy(z[f"{fmt}_ks"])
    cu_q, cu_k, cu_p = (torch.from_numpy(z[n]) for n in ("cu_q", "cu_k", "cu_p"))
    kvi, off = torch.from_numpy(z[f"{fmt}_kvi"]), torch.from_numpy(z["off"])
    assert torch.equal(O.fp4_dequantize(q, qs, fmt), torch.from_numpy(z[f"{fmt}_deq_q"]))
    for name, causal, o in (("dense", False, None), ("causal", True, None), ("offset", True, off)):
        ref = torch.from_numpy(z[f"{fmt}_{name}"])
        got = O.fp4_indexer_block_scores(q, k, qs, ks, cu_q, cu_k, cu_p, kvi, fmt, causal=causal, qo_offset=o)
        assert got.shape == ref.shape
        fin = torch.isfinite(ref)
        assert torch.equal(fin, torch.isfinite(got))
        assert torch.allclose(got[fin], ref[fin], rtol=2e-6, atol=1e-3)      # float32 summation order only
    q_mma, k_mma = O.fp4_reorder_scales(qs, ks, fmt)
    assert torch.equal(q_mma, torch.from_numpy(z[f"{fmt}_qs_mma"]))
    assert torch.equal(k_mma, torch.from_numpy(z[f"{fmt}_ks_mma"]))
