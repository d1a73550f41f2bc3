"""CPU checks: the C-ABI library loads and exports what include/msa_b200.h declares,
host-side planning logic, the quantisers and CSR helpers against the oracle.
No kernel is launched here."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import msa_b200
from msa_b200 import _lib, quant
from msa_b200.api import build_work_list
from msa_b200.sparse import build_k2q_csr, k2q_csr_to_q2k
from oracle import msa_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    hdr = open(os.path.join(ROOT, "include", "msa_b200.h")).read()
    names = set(re.findall(r"\b(msa_[a-z0-9_]+)\s*\(", hdr))
    assert {"msa_topk_select", "msa_fmha_fwd", "msa_decode_fwd", "msa_block_max", "msa_expand_block_lists"} <= names
    lib = msa_b200.get_lib()
    for n in sorted(names):
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert lib.msa_abi_version() == 4
    assert lib.msa_error_string(-3).decode().startswith("device-side wait")


def test_struct_layout_matches_header_sizes():
    # pointers 8 B, int64 8 B, int32/float 4 B: the ctypes mirror must not be smaller than the C struct
    assert ctypes.sizeof(_lib.FmhaArgs) % 8 == 0 and ctypes.sizeof(_lib.FmhaArgs) == 232
    assert ctypes.sizeof(_lib.DecodeArgs) == 144


def test_argument_validation_without_gpu():
    lib = msa_b200.get_lib()
    assert lib.msa_topk_select(None, 1, 16, 1, 16, 16, 0, 0, None, None) == -1
    assert lib.msa_fmha_fwd(None, None) == -1
    assert lib.msa_decode_fwd(None, None) == -1
    assert lib.msa_decode_workspace_bytes(32, 64, 8) == 32 * 64 * 8 * 130 * 4
    assert lib.msa_decode_workspace_bytes(32, 64, 1) == 0
    # block lists -> per-token lists: null pointers, a row that is not a multiple of four ints, unaligned buffers
    assert lib.msa_expand_block_lists(None, None, 1, 1, 16, None, None) == _lib.MSA_ERR_INVALID
    assert lib.msa_expand_block_lists(256, 512, 1, 1, 3, 1024, None) == _lib.MSA_ERR_UNSUPPORTED
    assert lib.msa_expand_block_lists(260, 512, 1, 1, 16, 1024, None) == _lib.MSA_ERR_INVALID
    assert lib.msa_expand_block_lists(256, 512, 0, 1, 16, 1024, None) == 0      # no blocks: nothing to do


def test_fp8_pv_precision_setting():
    """The module-level choice behind msa_fmha_args.fp8_p_f16: two modes, restored by the context manager."""
    assert msa_b200.get_fp8_pv_precision() == "e4m3"
    with msa_b200.fp8_pv_precision("f16"):
        assert msa_b200.get_fp8_pv_precision() == "f16"
        with msa_b200.fp8_pv_precision("e4m3"):
            assert msa_b200.get_fp8_pv_precision() == "e4m3"
        assert msa_b200.get_fp8_pv_precision() == "f16"
    assert msa_b200.get_fp8_pv_precision() == "e4m3"
    assert msa_b200.set_fp8_pv_precision("f16") == "e4m3" and msa_b200.set_fp8_pv_precision("e4m3") == "f16"
    with pytest.raises(ValueError):
        msa_b200.set_fp8_pv_precision("bf16")
    assert "fp8_p_f16" in [f[0] for f in _lib.FmhaArgs._fields_]


def test_no_cpu_fallback():
    q = torch.zeros(4, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(msa_b200.MsaError):
        msa_b200.sparse_topk_select(torch.zeros(1, 16, 4), 16)
    with pytest.raises((msa_b200.MsaError, RuntimeError, AssertionError)):
        plan = msa_b200.fmha_sm100_plan(torch.tensor([4]), torch.tensor([4]), 2)
        msa_b200.fmha_sm100(q, q, q, plan)


def test_work_list_covers_every_tile_once_heaviest_first():
    qo, kv = [300, 1, 128, 0, 129], [1000, 500, 128, 64, 129]
    off = [k - q for q, k in zip(qo, kv)]
    w = build_work_list(qo, kv, off, True)
    seen = set()
    starts = np.concatenate([[0], np.cumsum(qo)])
    for b, tok0, rows, loc, kl, qoff, base, _ in w.tolist():
        assert kl == kv[b] and qoff == off[b] and base == sum((k + 127) // 128 for k in kv[:b])
        assert 1 <= rows <= 128 and loc % 128 == 0 and tok0 == starts[b] + loc
        assert (b, loc) not in seen
        seen.add((b, loc))
    assert len(seen) == sum((q + 127) // 128 for q in qo)
    cost = [(min(kv[b], loc + rows + off[b]) + 127) // 128 for b, _, rows, loc, *_ in w.tolist()]
    assert cost == sorted(cost, reverse=True)


def test_quantisers_match_oracle():
    torch.manual_seed(3)
    x = torch.randn(3, 2, 128, 128).to(torch.bfloat16)
    d, s, g = O.quantize_nvfp4(x)
    q = quant.quantize_bf16_to_nvfp4_128x4(x)
    assert torch.equal(d, q.data) and torch.equal(s.reshape(-1), q.scale_128x4.reshape(-1)) and q.scale_128x4.dim() == 2 and abs(g - float(q.global_scale)) < 1e-9
    assert torch.equal(O.dequantize_nvfp4(d, s, g), quant.dequantize_nvfp4_128x4(q))
    a, sa = quant.quantize_fp8_per_tensor(x)
    b, sb = O.quantize_fp8_per_tensor(x)
    assert sa == sb and torch.equal(a.view(torch.uint8), b.view(torch.uint8))


def test_csr_roundtrip_against_reference_fixture():
    z = np.load(os.path.join(ROOT, "tests", "golden", "k2q_csr.npz"))
    q2k = torch.from_numpy(z["q2k"])
    cu_q, cu_k = torch.from_numpy(z["cu_q"]), torch.from_numpy(z["cu_k"])
    rp, qi = build_k2q_csr(q2k, cu_q, cu_k, 128)
    assert torch.equal(rp, torch.from_numpy(z["row_ptr"])) and torch.equal(qi, torch.from_numpy(z["q_indices"]))
    back = k2q_csr_to_q2k(rp, qi, q2k.shape[2], cu_q, [512, 512], 128)
    assert torch.equal(back.permute(1, 0, 2), q2k)
    # ragged case against the oracle restatement
    torch.manual_seed(0)
    cu_q2, cu_k2 = torch.tensor([0, 5, 5, 40]), torch.tensor([0, 300, 428, 1428])
    q2k2 = torch.full((2, 40, 4), -1, dtype=torch.int32)
    for h in range(2):
        for t in range(40):
            nb = 3 if t < 5 else 8
            n = min(nb, int(torch.randint(0, 5, (1,))))
            q2k2[h, t, :n] = torch.randperm(nb)[:n].sort().values.int()
    rp2, qi2 = build_k2q_csr(q2k2, cu_q2, cu_k2, 128)
    rp3, qi3 = O.build_k2q_csr(q2k2, cu_q2.tolist(), cu_k2.tolist(), 128)
    assert torch.equal(rp2, rp3) and torch.equal(qi2, qi3)
    assert torch.equal(k2q_csr_to_q2k(rp2, qi2, 4, cu_q2, [300, 128, 1000], 128).permute(1, 0, 2), q2k2)


def test_header_is_plain_c(tmp_path):
    """include/msa_b200.h compiles as C99 and its structs have the sizes the ctypes mirror assumes."""
    import shutil
    import subprocess
    if shutil.which("gcc") is None:
        pytest.skip("no gcc")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = tmp_path / "hdr.c"
    src.write_text('#include "msa_b200.h"\n#include <stdio.h>\n'
                   'int main(void) { printf("%zu %zu\\n", sizeof(msa_fmha_args), sizeof(msa_decode_args)); return 0; }\n')
    exe = tmp_path / "hdr"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I", os.path.join(root, "include"),
                    str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert int(out[0]) == ctypes.sizeof(_lib.FmhaArgs) and int(out[1]) == ctypes.sizeof(_lib.DecodeArgs)


def _validate(qo, kv, total_q, kv_rows, paged, kvi, lists, Hq=4, Hkv=2):
    a = _lib.ValidateArgs()
    ql, kl = np.asarray(qo, np.int32), np.asarray(kv, np.int32)
    a.batch, a.qo_lens, a.kv_lens = len(qo), ql.ctypes.data, kl.ctypes.data
    a.total_q, a.kv_rows, a.paged = total_q, kv_rows, paged
    keep = [ql, kl]
    if kvi is not None:
        kvi = np.ascontiguousarray(kvi, np.int32)
        keep.append(kvi)
        a.kv_indices, a.n_kv_indices = kvi.ctypes.data, kvi.size
    if lists is not None:
        lists = np.ascontiguousarray(lists, np.int32)
        keep.append(lists)
        a.kv_block_indexes, a.list_heads, a.topk = lists.ctypes.data, lists.shape[1], lists.shape[2]
    a.num_qo_heads, a.num_kv_heads = Hq, Hkv
    where = ctypes.c_int64(-7)
    rc = msa_b200.get_lib().msa_validate_inputs(ctypes.byref(a), ctypes.byref(where))
    return rc, where.value


def test_validator_rejects_each_broken_rule_before_any_launch():
    """msa_validate_inputs on host arrays: every rule of the index contract (reference api.py:128-263),
    with the first offending element."""
    qo, kv = [3, 2], [300, 129]                       # 3 + 2 pages
    good = np.full((5, 2, 4), -1, np.int32)
    good[:3, :, :3] = [0, 1, 2]
    good[3:, :, :2] = [0, 1]
    table = np.arange(5, dtype=np.int32)[::-1]
    assert _validate(qo, kv, 5, 5, 1, table, good) == (0, -1)
    assert _validate(qo, kv, 5, 5, 1, table, None) == (0, -1)
    assert _validate(qo, kv, 6, 5, 1, table, good)[0] == -101                      # q rows
    assert _validate(qo, kv, 5, 428, 0, None, good)[0] == -102                     # ragged K/V rows
    assert _validate(qo, kv, 5, 429, 0, None, good)[0] == 0
    assert _validate(qo, kv, 5, 5, 1, table[:4], good)[0] == -103                  # short kv_indices
    bad_t = table.copy()
    bad_t[3] = 5
    assert _validate(qo, kv, 5, 5, 1, bad_t, good) == (-104, 3)                    # page outside the pool
    bad_t[3] = -1
    assert _validate(qo, kv, 5, 5, 1, bad_t, good) == (-104, 3)
    assert _validate(qo, kv, 5, 5, 1, table, good[:, :1].repeat(3, 1))[0] == -105  # heads neither Hkv nor Hq
    for value, at, code in ((-2, (1, 0, 1), -106),        # below -1
                            (1, (4, 1, 3), -107),         # valid entry after the -1 tail started
                            (3, (2, 1, 2), -108),         # >= the request's 3 pages
                            (2, (3, 0, 1), -108),         # >= the second request's 2 pages
                            (0, (0, 1, 1), -109)):        # not strictly ascending
        bad = good.copy()
        bad[at] = value
        flat = (at[0] * 2 + at[1]) * 4 + at[2]
        assert _validate(qo, kv, 5, 5, 1, table, bad) == (code, flat), (value, at)
    # rule order: a -2 anywhere is reported before an ordering fault earlier in the tensor
    bad = good.copy()
    bad[0, 0, 1] = 0
    bad[4, 1, 0] = -2
    assert _validate(qo, kv, 5, 5, 1, table, bad)[0] == -106
    # the Python wrapper raises AssertionError with the rule's text
    plan = {"qo_lens_host": qo, "kv_lens_host": kv, "num_qo_heads": 4, "num_kv_heads": 2}
    from msa_b200.api import _validate_fmha_inputs
    q = torch.zeros(5, 4, 128)
    k = torch.zeros(5, 2, 128, 128)
    _validate_fmha_inputs(q, k, k, plan, torch.from_numpy(table.copy()), torch.from_numpy(good), True)
    bad = good.copy()
    bad[2, 1, 2] = 3
    with pytest.raises(AssertionError, match="out of range"):
        _validate_fmha_inputs(q, k, k, plan, torch.from_numpy(table.copy()), torch.from_numpy(bad), True)
    with pytest.raises(AssertionError, match="page pool"):
        _validate_fmha_inputs(q, k[:4], k[:4], plan, torch.from_numpy(table.copy()), torch.from_numpy(good), True)


def test_planner_through_the_c_abi():
    """msa_plan: tile list, page-table offsets, decode metadata and split choice."""
    from msa_b200.api import _host_plan
    work, indptr, tr, tp, splits = _host_plan([2, 1], [300, 1000], None, True, True, 16, 2, kv_block_num=8,
                                              num_kv_splits=-1, num_sms=148, decode=True)
    assert indptr.tolist() == [0, 3, 11] and tr.tolist() == [0, 0, 1] and tp.tolist() == [298, 299, 999]
    assert work.shape == (2, 8) and work[0].tolist() == [1, 2, 1, 0, 1000, 999, 3, 0]
    assert 1 <= splits <= 8
    # forced split counts are clamped to the list length; non-causal sees every key
    assert _host_plan([1], [500], None, True, True, 8, 8, kv_block_num=4, num_kv_splits=9, decode=True)[4] == 4
    assert _host_plan([3], [500], None, False, True, 8, 8, kv_block_num=4, decode=True)[3].tolist() == [499] * 3
    # 157 pages in one list: a split count is still found (entries per split may exceed 64)
    s = _host_plan([1] * 2, [20000] * 2, None, True, True, 16, 2, kv_block_num=157, num_sms=148, decode=True)[4]
    assert 2 <= s <= 64
    with pytest.raises(msa_b200.MsaError):
        _host_plan([1], [-5], None, True, True)
    # KV splits of a dense tile: 3 entries over pages [0,3) [3,6) [6,8), output rows offset by split * total_q,
    # kv_len cut at the end of each range; a split past the visible pages walks nothing
    w = _host_plan([5], [1000], None, True, True, 8, 8, dense_kv_splits=3)[0]
    recs = sorted(w.tolist(), key=lambda r: r[7])
    assert [(r[2] & 1023, r[2] >> 10, r[4], r[7]) for r in recs] == [(5, 0, 384, 0), (5, 3, 768, 5), (5, 6, 1000, 10)]
    w = _host_plan([2], [200], None, True, True, 8, 8, dense_kv_splits=4)[0]
    recs = sorted(w.tolist(), key=lambda r: r[7])
    assert [(r[2] >> 10, r[4]) for r in recs] == [(0, 128), (1, 200), (2, 200), (2, 200)] and len(recs) == 4


def test_c_program_plans_and_validates_through_the_header(tmp_path):
    """A plain C caller: include/msa_b200.h + libmsa_b200.so, no Python, no GPU."""
    import shutil
    import subprocess
    if shutil.which("gcc") is None:
        pytest.skip("no gcc")
    msa_b200.get_lib()
    src = tmp_path / "plan.c"
    src.write_text(r'''
#include <stdio.h>
#include <stdlib.h>
#include "msa_b200.h"
int main(void) {
  const int32_t qo[2] = {200, 1}, kv[2] = {1000, 4000};
  msa_plan_desc d = {0};
  d.batch = 2; d.qo_lens = qo; d.kv_lens = kv; d.qo_offset = NULL; d.causal = 1; d.paged = 1;
  d.num_qo_heads = 8; d.num_kv_heads = 2; d.kv_block_num = 16; d.num_kv_splits = -1; d.num_sms = 148;
  int32_t n_work = 0; int64_t total_q = 0, total_pages = 0;
  if (msa_plan_sizes(&d, &n_work, &total_q, &total_pages) != MSA_OK) return 1;
  int32_t* work = malloc((size_t)n_work * 8 * sizeof(int32_t));
  int32_t indptr[3], splits = 0;
  int32_t* treq = malloc((size_t)total_q * sizeof(int32_t));
  int32_t* tpos = malloc((size_t)total_q * sizeof(int32_t));
  if (msa_plan(&d, work, indptr, treq, tpos, &splits) != MSA_OK) return 2;
  int32_t* table = malloc((size_t)total_pages * sizeof(int32_t));
  for (int64_t i = 0; i < total_pages; ++i) table[i] = (int32_t)(total_pages - 1 - i);
  msa_validate_args v = {0};
  v.batch = 2; v.qo_lens = qo; v.kv_lens = kv; v.total_q = total_q; v.kv_rows = total_pages; v.paged = 1;
  v.kv_indices = table; v.n_kv_indices = total_pages; v.num_qo_heads = 8; v.num_kv_heads = 2;
  int64_t where = 0;
  int ok = msa_validate_inputs(&v, &where);
  table[5] = (int32_t)total_pages;
  int bad = msa_validate_inputs(&v, &where);
  printf("%d %lld %lld %d %d %d %d %d %d %lld %s\n", n_work, (long long)total_q, (long long)total_pages, indptr[2],
         work[0], tpos[200], splits, ok, bad, (long long)where, msa_error_string(bad));
  return 0;
}
''')
    exe = tmp_path / "plan"
    libdir = os.path.join(ROOT, "msa_b200")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                    "-L", libdir, "-l:libmsa_b200.so", f"-Wl,-rpath,{libdir}"], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split(maxsplit=10)
    assert out[:4] == ["3", "201", "40", "40"]
    assert out[4] == "1" and out[5] == "3999"       # heaviest tile first: the decode token over 4000 keys
    assert 1 <= int(out[6]) <= 16 and out[7] == "0" and out[8] == "-104" and out[9] == "5"
    assert "page pool" in out[10]


def test_alias_package_exposes_the_reference_names():
    """`import fmha_sm100` (the reference's package name) serves the same public names from this library."""
    import fmha_sm100
    from fmha_sm100 import sparse as fs
    assert fmha_sm100.fmha_sm100 is msa_b200.fmha_sm100 and fmha_sm100.fmha_sm100_plan is msa_b200.fmha_sm100_plan
    assert fmha_sm100.sparse_topk_select is msa_b200.sparse_topk_select
    assert fmha_sm100.sparse_atten_func is msa_b200.sparse_atten_func          # lazy attribute
    for n in ("sparse_atten_nvfp4_kv_func", "sparse_decode_atten_func", "SparseDecodePagedAttentionWrapper",
              "build_k2q_csr", "quantize_kv_bf16_to_nvfp4_128x4"):
        assert hasattr(fs, n)
    import inspect
    sig = inspect.signature(msa_b200.SparseDecodePagedAttentionWrapper.plan)
    for kw in ("page_table", "seqused_k", "seqlen_q", "max_seqlen_k", "q2k_indices", "num_qo_heads", "num_kv_heads",
               "head_dim", "enable_cuda_graph", "max_grid_size", "fixed_split_size", "disable_split_kv"):
        assert kw in sig.parameters, kw
    sig = inspect.signature(msa_b200.SparseDecodePagedAttentionWrapper.run)
    for kw in ("softmax_scale", "return_softmax_lse", "out", "lse"):
        assert kw in sig.parameters, kw


def test_score_work_lists_tile_rows_splits_and_fill_flags():
    """Work lists of the score-only pass: 256-row entries, 16-token entries for 16 packed heads, page-range splits,
    and the entry of every query tile that is flagged to write the -inf tail."""
    from msa_b200.api import _flag_fill_entries, _host_plan
    w = _host_plan([600], [1000], None, True, True, 8, 8, tile_rows=256)[0]
    assert sorted(r[2] for r in w.tolist()) == [88, 256, 256] and all(r[7] == 0 for r in w.tolist())
    assert _flag_fill_entries(w, True) and all(r[7] == 1 for r in w.tolist())
    # decode-like: 8 tokens per request in 16-token entries, three page ranges each
    w = _host_plan([8, 8], [5000, 3000], None, True, True, 64, 4, tile_rows=16, dense_kv_splits=3)[0]
    assert w.shape[0] == 6 and {r[2] & 1023 for r in w.tolist()} == {8}
    assert _flag_fill_entries(w, True)
    top = {}
    for r in w.tolist():
        top.setdefault(r[0], []).append((r[2] >> 10, r[7]))
    for req, lst in top.items():
        lst.sort()
        assert [f for _, f in lst] == [0, 0, 1]          # only the highest page range writes the tail
    # a query tile that sees no key at all (more queries than keys): no entry runs for it -> pre-fill needed
    w = _host_plan([400], [100], None, True, True, 1, 1, tile_rows=256)[0]
    assert not _flag_fill_entries(w, True)
    # invalid sizes are refused by the planner
    with pytest.raises(msa_b200.MsaError):
        _host_plan([10], [10], None, True, True, 1, 1, tile_rows=512)


def test_fp4_indexer_names_and_scale_layout_helpers():
    """The FP4 indexer module and its alias import on a machine without a GPU; the storage helpers agree with the
    oracle's offset formula (python/fmha_sm100/cute/fp4_indexer_interface.py:220-249)."""
    import fmha_sm100.fp4_indexer_interface as fii
    from oracle import msa_oracle as O
    assert fii.fp4_indexer_block_scores is msa_b200.fp4_indexer_block_scores
    for fmt, groups in (("nvfp4", 8), ("mxfp4", 4)):
        mn, l = 300, 5
        shape = fii.fp4_indexer_mma_scale_shape(mn, l, fp4_format=fmt)
        stride = fii.fp4_indexer_mma_scale_stride(mn, l, fp4_format=fmt)
        store = fii.fp4_indexer_mma_scale_storage_shape(mn, l, fp4_format=fmt)
        assert shape == (32, 4, 3, 4, (groups + 3) // 4, l) and store == (l, 3, (groups + 3) // 4, 32, 4, 4)
        for m, g, ll in ((0, 0, 0), (37, 3, 2), (299, groups - 1, 4), (128, 1, 1)):
            idx = (m % 32, (m // 32) % 4, m // 128, g % 4, g // 4, ll)
            assert sum(i * s_ for i, s_ in zip(idx, stride)) == O.fp4_mma_scale_offset(m, g, ll, mn, groups)
    with pytest.raises(ValueError):
        fii.fp4_indexer_mma_scale_shape(1, 1, fp4_format="fp4")


def test_plan_cache_does_not_survive_its_tensors():
    """Plans cached per (cu_seqlens, ...) tensors: an in-place update misses, and so does another tensor object with
    the same address, version and shape (what an allocator hands out after the original was freed)."""
    from msa_b200.api import TensorKeyedCache
    c = TensorKeyedCache(2)
    a, b = torch.tensor([0, 5, 9]), torch.tensor([0, 7])
    assert c.get((a, b, None), (1,)) is None
    c.put((a, b, None), (1,), "plan1")
    assert c.get((a, b, None), (1,)) == "plan1" and c.get((a, b, None), (2,)) is None
    a.add_(1)
    assert c.get((a, b, None), (1,)) is None
    c.put((a, b, None), (1,), "plan2")
    assert c.get((a.view_as(a), b, None), (1,)) is None      # same storage and version, different tensor object
    c.put((b,), (), "x")
    c.put((torch.tensor([1]),), (), "y")                      # capacity 2: the oldest entry is dropped
    assert c.get((a, b, None), (1,)) is None
