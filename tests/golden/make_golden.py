"""Generate golden fixtures from the reference's OWN PyTorch code (CPU).

Run in a container that has the reference tree mounted:

    python tests/golden/make_golden.py /path/to/reference

It imports, unmodified, the reference oracles
  tests/regression/test_correctness.py   ref_tile_max_score, sdpa_ref
  tests/regression/test_sparse_attn.py   sparse_ref
  tests/integration/test_proxy_kv_e2e.py verify_topk_selection
  python/fmha_sm100/cute/test_sparse_atten.py  sparse_attention_ref
  python/fmha_sm100/cute/sparse_index_utils.py build_k2q_csr_torch_reference
  python/fmha_sm100/cute/quantize.py     dequantize_nvfp4_128x4_to_bf16
  python/fmha_sm100/cute/test_fp4_indexer.py       _reference_block_scores, _dequantize_public_fp4
  python/fmha_sm100/cute/fp4_indexer_interface.py  fp4_indexer_mma_scale_shape / _stride
runs them on small seeded inputs and stores inputs + outputs as .npz files
next to this script.  tests/test_oracle_golden.py replays the stored inputs
through oracle/msa_oracle.py and compares.  The reference tree is needed only
to (re)generate; the tests read the .npz files alone.
"""
import importlib.util
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle import msa_oracle as O  # noqa: E402


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def _np(t):
    if t.dtype == torch.bfloat16:
        return t.float().numpy()
    return t.numpy()


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "python"))
    sys.path.insert(0, os.path.join(ref_root, "python", "fmha_sm100", "cute"))
    tc = _load(os.path.join(ref_root, "tests/regression/test_correctness.py"), "ref_tc")
    ts = _load(os.path.join(ref_root, "tests/regression/test_sparse_attn.py"), "ref_ts")
    te = _load(os.path.join(ref_root, "tests/integration/test_proxy_kv_e2e.py"), "ref_te")
    import test_sparse_atten as tsa
    import sparse_index_utils as siu
    import quantize as rq

    # ---- 1. max score: ragged batch, GQA, causal with default and explicit offsets
    torch.manual_seed(11)
    qo_lens = [70, 128, 200]
    kv_lens = [300, 128, 457]
    Hq, Hkv, D = 4, 2, 128
    q = torch.randn(sum(qo_lens), Hq, D).to(torch.bfloat16)
    k = torch.randn(sum(kv_lens), Hkv, D).to(torch.bfloat16)
    max_k_tiles = 128
    ms_default = tc.ref_tile_max_score(q, k, torch.tensor(qo_lens), torch.tensor(kv_lens), Hkv, max_k_tiles,
                                       causal=True)
    offs = torch.tensor([100, 0, 250], dtype=torch.int32)
    ms_off = tc.ref_tile_max_score(q, k, torch.tensor(qo_lens), torch.tensor(kv_lens), Hkv, max_k_tiles,
                                   causal=True, qo_offset_tensor=offs)
    np.savez_compressed(os.path.join(HERE, "maxscore.npz"), q=_np(q), k=_np(k), qo_lens=qo_lens, kv_lens=kv_lens,
                        Hkv=Hkv, max_k_tiles=max_k_tiles, ms_default=ms_default[:, :4].numpy(),
                        ms_off=ms_off[:, :4].numpy(), offs=offs.numpy(),
                        tail_all_neg_inf=bool((ms_default[:, 4:] == float("-inf")).all()))

    # ---- 2. top-k: oracle choice must pass the reference's multiset verifier
    torch.manual_seed(12)
    H, K, T = 3, 128, 96
    ms = torch.randn(H, K, T)
    for t in range(T):                       # causal-like -inf frontier, some rows with < 16 finite
        ms[:, 1 + (t * 40) // T:, t] = float("-inf")
    ms[1, 3, 50:] = ms[1, 2, 50:]            # exact ties
    sel = O.topk_select(ms, 16, num_valid_pages=40)
    ok, max_diff, n_mis = te.verify_topk_selection(ms, sel, 16)
    ref_top = torch.sort(torch.topk(ms.permute(2, 0, 1), 16, dim=-1).values, dim=-1).values
    np.savez_compressed(os.path.join(HERE, "topk.npz"), ms=ms.numpy(), sel=sel.numpy(), verifier_ok=bool(ok),
                        max_diff=float(max_diff), n_mismatch=int(n_mis), ref_sorted_scores=ref_top.numpy())

    # ---- 3. sparse_ref (per-request block lists, identity table within the request)
    torch.manual_seed(13)
    qo_lens = [5, 33]
    kv_lens = [640, 1000]
    qo_offs = [kv_lens[i] - qo_lens[i] for i in range(2)]
    Hq, Hkv = 4, 2
    indptr = O.page_indptr(kv_lens)
    npages = indptr[-1]
    k_pages = torch.randn(npages, Hkv, 128, 128).to(torch.bfloat16)
    v_pages = torch.randn(npages, Hkv, 128, 128).to(torch.bfloat16)
    q = torch.randn(sum(qo_lens), Hq, 128).to(torch.bfloat16)
    blocks = [[[0, 2, 4], [1, 3, 4]], [[0, 3, 6, 7], [2, 5, 7]]]
    o_ref = ts.sparse_ref(q, k_pages, v_pages, qo_lens, indptr, blocks, Hq, Hkv, 128, qo_offs, 128, "cpu")
    np.savez_compressed(os.path.join(HERE, "sparse_ref.npz"), q=_np(q), k_pages=_np(k_pages), v_pages=_np(v_pages),
                        qo_lens=qo_lens, kv_lens=kv_lens, blocks0=np.array(blocks[0], dtype=object),
                        blocks1=np.array(blocks[1], dtype=object), out=_np(o_ref), allow_pickle=True)

    # ---- 4. sparse_attention_ref: per-token lists, causal with seqused_k, LSE
    torch.manual_seed(14)
    B, Sq, Sk, Hq, Hkv, topk = 2, 96, 512, 4, 2, 3
    q = torch.randn(B, Sq, Hq, 128).to(torch.bfloat16)
    k = torch.randn(B, Sk, Hkv, 128).to(torch.bfloat16)
    v = torch.randn(B, Sk, Hkv, 128).to(torch.bfloat16)
    seqused = torch.tensor([512, 400], dtype=torch.int32)
    q2k = torch.full((B, Hkv, Sq, topk), -1, dtype=torch.int32)
    g = torch.Generator().manual_seed(5)
    for b in range(B):
        for h in range(Hkv):
            for i in range(Sq):
                lim = i + int(seqused[b]) - Sq
                vis = lim // 128 + 1
                n = min(topk, vis) if (i % 7) else max(1, min(topk, vis) - 1)
                ch = torch.randperm(vis, generator=g)[:n].sort().values
                q2k[b, h, i, :n] = ch.to(torch.int32)
    out, lse = tsa.sparse_attention_ref(q, k, v, q2k, causal=True, seqused_k=seqused)
    np.savez_compressed(os.path.join(HERE, "sparse_attention_ref.npz"), q=_np(q), k=_np(k), v=_np(v),
                        q2k=q2k.numpy(), seqused=seqused.numpy(), out=out.numpy(), lse=lse.numpy())

    # ---- 5. FP8 unnormalised-P model of the reference (for the decode tolerance discussion)
    out8, lse8 = tsa.sparse_attention_ref(q, k, v, q2k, causal=True, seqused_k=seqused,
                                          p_dtype=torch.float8_e4m3fn)
    np.savez_compressed(os.path.join(HERE, "sparse_attention_ref_p8.npz"), out=out8.numpy(), lse=lse8.numpy())

    # ---- 6. k2q CSR
    cu_q = torch.tensor([0, Sq, 2 * Sq], dtype=torch.int32)
    cu_k = torch.tensor([0, Sk, 2 * Sk], dtype=torch.int32)
    q2k_flat = q2k.permute(1, 0, 2, 3).reshape(Hkv, B * Sq, topk).contiguous()
    rp, qi = siu.build_k2q_csr_torch_reference(q2k_flat, cu_q, cu_k, 128)
    np.savez_compressed(os.path.join(HERE, "k2q_csr.npz"), q2k=q2k_flat.numpy(), cu_q=cu_q.numpy(), cu_k=cu_k.numpy(),
                        row_ptr=rp.numpy(), q_indices=qi.numpy())

    # ---- 7. NVFP4 dequantisation + 128x4 scale layout (quantiser is this build's own)
    torch.manual_seed(15)
    x = torch.randn(3, 2, 128, 128).to(torch.bfloat16)
    data, sflat, gs = O.quantize_nvfp4(x)
    rows = 3 * 2 * 128
    qt = rq.Nvfp4QuantizedTensor(data=data.reshape(rows, 64), scale_128x4=sflat,
                                 global_scale=torch.tensor([gs], dtype=torch.float32),
                                 logical_scale_shape=(rows, 8), original_shape=(3, 2, 128, 128))
    deq = rq.dequantize_nvfp4_128x4_to_bf16(qt)
    r = torch.arange(300).view(-1, 1).expand(300, 8)
    c = torch.arange(8).view(1, -1).expand(300, 8)
    offs = rq.nvfp4_scale_128x4_offset(r, c, 8)
    np.savez_compressed(os.path.join(HERE, "nvfp4.npz"), x=_np(x), data=data.numpy(), scale=sflat.numpy(), gs=gs,
                        deq_bf16=_np(deq), offsets=offs.numpy())
    # ---- 8. FP4 indexer: the reference's own CPU scorer and scale-storage strides on seeded random inputs
    import fp4_indexer_interface as fii
    import test_fp4_indexer as tfi
    out = {}
    for fmt in ("nvfp4", "mxfp4"):
        g = torch.Generator().manual_seed(16)
        ql, kl, hq, hk = [70, 130], [300, 200], 4, 2
        groups = fii.normalize_fp4_format(fmt).scale_groups
        pages = [(x + 127) // 128 for x in kl]
        n_pages = sum(pages) + 1
        q = torch.randint(0, 256, (sum(ql), hq, 64), dtype=torch.uint8, generator=g)
        k = torch.randint(0, 256, (n_pages, hk, 128, 64), dtype=torch.uint8, generator=g)
        qs = tfi._random_scale((sum(ql), hq, groups), fmt=fmt, device=torch.device("cpu"), generator=g)
        ks = tfi._random_scale((n_pages, hk, 128, groups), fmt=fmt, device=torch.device("cpu"), generator=g)
        cu_q = torch.tensor([0, 70, 200], dtype=torch.int32)
        cu_k = torch.tensor([0, 300, 500], dtype=torch.int32)
        cu_p = torch.tensor([0, 3, 5], dtype=torch.int32)
        kvi = torch.randperm(n_pages, generator=g)[:5].to(torch.int32)
        off = torch.tensor([100, 60], dtype=torch.int32)
        out.update({f"{fmt}_q": q.numpy(), f"{fmt}_k": k.numpy(), f"{fmt}_qs": qs.view(torch.uint8).numpy(),
                    f"{fmt}_ks": ks.view(torch.uint8).numpy(), f"{fmt}_kvi": kvi.numpy()})
        for name, causal, o in (("dense", False, None), ("causal", True, None), ("offset", True, off)):
            out[f"{fmt}_{name}"] = tfi._reference_block_scores(q, k, qs, ks, cu_q, cu_k, cu_p, fmt=fmt, kv_indices=kvi,
                                                               causal=causal, qo_offset=o).numpy()
        out[f"{fmt}_deq_q"] = tfi._dequantize_public_fp4(q, qs, fmt=fmt).numpy()
        # the tiled scale storage, built from the reference's own shape / stride helpers
        for tag, src, mn, l in (("qs", qs.view(torch.uint8), sum(ql), hq),
                                ("ks", ks.view(torch.uint8).reshape(n_pages * hk, 128, groups).permute(1, 0, 2), 128,
                                 n_pages * hk)):
            shape = fii.fp4_indexer_mma_scale_shape(mn, l, fp4_format=fmt)
            stride = fii.fp4_indexer_mma_scale_stride(mn, l, fp4_format=fmt)
            nbytes = math.prod(fii.fp4_indexer_mma_scale_storage_shape(mn, l, fp4_format=fmt))
            flat = torch.zeros(nbytes, dtype=torch.uint8)
            view = torch.as_strided(flat, shape, stride)      # (32, 4, restM, 4, restG, L)
            for m in range(mn):
                for gi in range(groups):
                    view[m % 32, (m // 32) % 4, m // 128, gi % 4, gi // 4, :] = src[m, :, gi]
            out[f"{fmt}_{tag}_mma"] = flat.numpy()
    np.savez_compressed(os.path.join(HERE, "fp4_indexer.npz"), cu_q=cu_q.numpy(), cu_k=cu_k.numpy(), cu_p=cu_p.numpy(),
                        off=off.numpy(), **out)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python make_golden.py <checkout of MiniMax-AI/MSA>")
    main(sys.argv[1])
