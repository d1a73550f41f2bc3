"""KV-cache append kernels: bit-exact parity with the oracle restatement through the C ABI."""
import os

import numpy as np
import pytest
import torch

import msa_b200
from msa_b200 import kv_cache as KC
from oracle import msa_oracle as O

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")


def _new_rows(n, hkv, seed, spread=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, hkv, 128, generator=g)
    if spread:                       # rows of very different magnitude: small block scales, denormal e4m3 scales
        x = x * torch.logspace(-4, 1, n, base=10.0).view(n, 1, 1)
    x[0, 0, :16] = 0.0               # an all-zero block (block scale 0)
    x[1 % n, 0, 3] = -0.0
    return x.to(torch.bfloat16)


def _slots(n, pages, seed, skip=True):
    g = torch.Generator().manual_seed(seed)
    s = torch.randperm(pages * 128, generator=g)[:n].int()
    if skip and n > 4:
        s[3] = -1
        s[n - 1] = pages * 128       # out of range: skipped
    return s


@pytest.mark.parametrize("n,hkv,pages", [(1, 1, 1), (77, 2, 3), (640, 8, 9), (4096, 1, 40)])
def test_append_fp8_bit_exact(n, hkv, pages):
    k, v = _new_rows(n, hkv, n), _new_rows(n, hkv, n + 1)
    slots = _slots(n, pages, n + 2)
    ks, vs = float(k.float().abs().max()) / 448, float(v.float().abs().max()) / 448 * 0.5   # V saturates
    kc = torch.full((pages, hkv, 128, 128), 0x11, dtype=torch.uint8)
    vc = torch.full_like(kc, 0x22)
    kr, vr = kc.clone(), vc.clone()
    O.kv_append_fp8(k, v, kr, vr, slots, ks, vs)
    kd, vd = kc.cuda(), vc.cuda()
    KC.append_kv_fp8(k.cuda(), v.cuda(), kd, vd, slots.cuda(), ks, vs)
    assert torch.equal(kd.cpu(), kr) and torch.equal(vd.cpu(), vr)


@pytest.mark.parametrize("n,hkv,pages", [(1, 1, 1), (77, 2, 3), (640, 8, 9), (4096, 1, 40)])
def test_append_nvfp4_bit_exact(n, hkv, pages):
    k, v = _new_rows(n, hkv, 10 * n), _new_rows(n, hkv, 10 * n + 1, spread=False)
    slots = _slots(n, pages, n + 5)
    kg = KC.nvfp4_global_scale_from_amax(float(k.float().abs().max()))
    vg = KC.nvfp4_global_scale_from_amax(float(v.float().abs().max())) * 0.25    # block scales clamp at 448
    dev = torch.device("cuda")
    kd, vd, ksd, vsd = KC.alloc_nvfp4_cache(pages, hkv, dev)
    kr, vr, ksr, vsr = (t.cpu().clone() for t in (kd, vd, ksd, vsd))
    O.kv_append_nvfp4(k, v, kr, vr, ksr, vsr, slots, kg, vg)
    KC.append_kv_nvfp4(k.cuda(), v.cuda(), kd, vd, ksd, vsd, slots.cuda(), kg, vg)
    assert torch.equal(kd.cpu(), kr) and torch.equal(vd.cpu(), vr)
    assert torch.equal(ksd.cpu(), ksr) and torch.equal(vsd.cpu(), vsr)


def test_append_nvfp4_golden_fixture():
    """The stored fixture's scale bytes and layout (pinned by the reference's dequantiser) come out of the kernel."""
    z = np.load(os.path.join(G, "nvfp4.npz"))
    x = torch.from_numpy(z["x"]).to(torch.bfloat16)
    pages, hkv = x.shape[0], x.shape[1]
    new = x.permute(0, 2, 1, 3).reshape(pages * 128, hkv, 128).contiguous().cuda()
    slots = torch.arange(pages * 128, dtype=torch.int32, device="cuda")
    kd, vd, ksd, vsd = KC.alloc_nvfp4_cache(pages, hkv, new.device)
    gs = float(z["gs"])
    KC.append_kv_nvfp4(new, new, kd, vd, ksd, vsd, slots, gs, gs)
    assert torch.equal(ksd.cpu().reshape(-1), torch.from_numpy(z["scale"]).reshape(-1)) and torch.equal(vsd, ksd) and torch.equal(vd, kd)
    # codes: equal to the fixture except within an ulp of a rounding midpoint (reciprocal multiply here, division
    # in the whole-tensor quantiser that made the fixture), and equal to the oracle's append everywhere
    assert (kd.cpu() != torch.from_numpy(z["data"])).float().mean() < 1e-3
    kr, vr = torch.zeros_like(kd, device="cpu"), torch.zeros_like(kd, device="cpu")
    ksr, vsr = torch.zeros_like(ksd, device="cpu"), torch.zeros_like(ksd, device="cpu")
    O.kv_append_nvfp4(new.cpu(), new.cpu(), kr, vr, ksr, vsr, slots.cpu(), gs, gs)
    assert torch.equal(kd.cpu(), kr)


@pytest.mark.parametrize("n", [1, 7, 8, 4099, 1 << 20])
def test_absmax(n):
    g = torch.Generator().manual_seed(n)
    x = (torch.randn(n, generator=g) * 3).to(torch.bfloat16)
    got = KC.absmax_bf16(x.cuda())
    assert float(got.cpu()) == float(x.float().abs().max())
    # running maximum over two calls
    y = (torch.randn(n, generator=g) * 5).to(torch.bfloat16)
    KC.absmax_bf16(y.cuda(), out=got)
    assert float(got.cpu()) == max(float(x.float().abs().max()), float(y.float().abs().max()))


def test_append_then_attend_fp8():
    """Prefill K/V appended by the kernel, then sparse attention over the cache: the attention output equals the
    oracle's on the same cache bytes within the FP8 tolerance, and the cache equals the whole-tensor quantiser's."""
    torch.manual_seed(5)
    qo, kv, Hq, Hkv, topk = [256], [512], 8, 2, 4
    pages = 6
    k_new = torch.randn(kv[0], Hkv, 128).to(torch.bfloat16)
    v_new = torch.randn(kv[0], Hkv, 128).to(torch.bfloat16)
    table = torch.randperm(pages)[:4].int()
    pos = torch.arange(kv[0])
    slots = (table[pos // 128].long() * 128 + pos % 128).int()
    dev = torch.device("cuda")
    amax_k = float(KC.absmax_bf16(k_new.to(dev)).cpu())
    amax_v = float(KC.absmax_bf16(v_new.to(dev)).cpu())
    ks, vs = KC.fp8_scale_from_amax(amax_k), KC.fp8_scale_from_amax(amax_v)
    kc, vc = KC.alloc_fp8_cache(pages, Hkv, dev)
    KC.append_kv_fp8(k_new.to(dev), v_new.to(dev), kc, vc, slots.to(dev), ks, vs)
    q = torch.randn(qo[0], Hq, 128).to(torch.bfloat16)
    idx = torch.full((qo[0], Hkv, topk), -1, dtype=torch.int32)
    for t in range(qo[0]):
        vis = (kv[0] - qo[0] + t) // 128 + 1
        idx[t, :, :min(vis, topk)] = torch.arange(min(vis, topk), dtype=torch.int32)
    plan = msa_b200.fmha_sm100_plan(torch.tensor(qo), torch.tensor(kv), Hq, num_kv_heads=Hkv, page_size=128,
                                    kv_block_num=topk, sparse_kernel_mode="prefill")
    out, _ = msa_b200.fmha_sm100(q.to(dev), kc, vc, plan, kv_indices=table.to(dev), kv_block_indexes=idx.to(dev),
                                 k_scale=ks, v_scale=vs)
    ref, _ = O.sparse_attention_paged(q, kc.cpu(), vc.cpu(), table, qo, kv, idx, k_scale=ks, v_scale=vs)
    assert float((out.float().cpu() - ref).abs().max()) <= 6e-2          # FP8 K/V tolerance
    # the rows that were written equal the oracle's quantisation of the same rows
    kr = torch.zeros(pages, Hkv, 128, 128, dtype=torch.uint8)
    vr = torch.zeros_like(kr)
    O.kv_append_fp8(k_new, v_new, kr, vr, slots, ks, vs)
    assert torch.equal(kc.cpu().view(torch.uint8), kr) and torch.equal(vc.cpu().view(torch.uint8), vr)


def test_append_rejects_bad_arguments():
    dev = torch.device("cuda")
    k = torch.zeros(4, 2, 128, dtype=torch.bfloat16, device=dev)
    kc, vc = KC.alloc_fp8_cache(1, 2, dev)
    slots = torch.arange(4, dtype=torch.int32, device=dev)
    with pytest.raises(msa_b200.MsaError):
        KC.append_kv_fp8(k, k, kc, vc, slots, 0.0, 1.0)                   # scale must be positive
    with pytest.raises(msa_b200.MsaError):
        KC.append_kv_fp8(k.float(), k.float(), kc, vc, slots, 1.0, 1.0)   # bf16 only
    with pytest.raises(msa_b200.MsaError):
        KC.append_kv_fp8(k, k, kc[:, :1], vc[:, :1], slots, 1.0, 1.0)     # head count mismatch
    with pytest.raises(msa_b200.MsaError):
        KC.append_kv_fp8(k, k, kc, vc, slots[:3], 1.0, 1.0)               # one slot per token
    KC.append_kv_fp8(k[:0], k[:0], kc, vc, slots[:0], 1.0, 1.0)           # empty batch is a no-op
