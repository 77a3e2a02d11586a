"""CPU-only tests: the C ABI loads and exports every declared symbol, the host plan agrees with the oracle's
chunk table, argument errors come back as codes, and the Python-side adapters behave like the reference's."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from oracle import moba_oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from moba_b200 import _lib

    header = open(os.path.join(ROOT, "include", "moba_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(moba_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/moba_b200.h but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert lib.moba_version() >= 100


@pytest.mark.parametrize("cu,chunk,topk", [
    ([0, 1024, 4096], 512, 3),
    ([0, 198, 389, 433, 512], 128, 3),
    ([0, 29, 47, 300], 96, 2),
    ([0, 131072], 4096, 12),
    ([0, 5, 5, 700], 100, 4),
])
def test_plan_matches_oracle_chunk_table(cu, chunk, topk):
    from moba_b200 import ops

    plan = ops.get_plan(cu, chunk, topk, "cpu")
    tab = orc.chunk_table(cu, chunk)
    np.testing.assert_array_equal(plan.table("chunk_start").numpy(), tab["cu_chunk"])
    assert plan.info.n_chunks == len(tab["chunk_seq"])
    assert plan.info.n_filtered == len(tab["filtered"])
    assert plan.info.rows_per_head == (orc.rows_per_head(cu, chunk, topk) if plan.kk > 0 else 0)
    assert plan.kk == max(0, min(topk - 1, max((b - a + chunk - 1) // chunk for a, b in zip(cu, cu[1:])) - 1))
    first = plan.table("chunk_seq_first").numpy()
    last = plan.table("chunk_seq_last").numpy()
    seq_first = tab["seq_first_chunk"]
    for c, b in enumerate(tab["chunk_seq"]):
        assert first[c] == seq_first[b] and last[c] == seq_first[b + 1] - 1
    # query tiles never straddle chunks and cover every token once
    qs, qc = plan.table("qtile_start").numpy(), plan.table("qtile_chunk").numpy()
    covered = 0
    for s, c in zip(qs, qc):
        assert tab["cu_chunk"][c] <= s < tab["cu_chunk"][c + 1]
        covered += min(128, tab["cu_chunk"][c + 1] - s)
    assert covered == cu[-1]
    # upper bound on gathered tiles
    assert plan.info.max_work_tiles_per_head >= plan.info.rows_per_head // 128


def test_config3_counts():
    from moba_b200 import ops

    plan = ops.get_plan([0, 131072], 4096, 12, "cpu")
    assert (plan.info.n_chunks, plan.info.n_filtered, plan.kk) == (32, 31, 11)
    assert plan.info.rows_per_head == 1171456


def test_bad_arguments_return_codes():
    from moba_b200 import _lib

    info = _lib.PlanInfo()
    arr = (ctypes.c_int32 * 3)(0, 10, 5)
    assert _lib.lib.moba_plan_sizes(arr, 2, 4, 2, ctypes.byref(info)) == -2          # decreasing cu_seqlens
    assert b"decreases" in _lib.lib.moba_last_error_string()
    arr = (ctypes.c_int32 * 2)(1, 10)
    assert _lib.lib.moba_plan_sizes(arr, 1, 4, 2, ctypes.byref(info)) == -2          # does not start at 0
    arr = (ctypes.c_int32 * 2)(0, 10)
    assert _lib.lib.moba_plan_sizes(arr, 1, 0, 2, ctypes.byref(info)) == -1          # chunk size 0
    assert _lib.lib.moba_plan_sizes(arr, 1, 4, 0, ctypes.byref(info)) == -1          # top-k 0
    assert _lib.lib.moba_plan_sizes(None, 1, 4, 2, ctypes.byref(info)) == -1         # null pointer
    with pytest.raises(_lib.MobaError):
        _lib.call("moba_plan_sizes", arr, 0, 4, 2, ctypes.byref(info))


def test_calc_chunks_matches_reference_layout():
    from moba_b200 import calc_chunks

    cu = torch.tensor([0, 198, 389, 433, 512], dtype=torch.int32)
    cu_chunk, filtered, n_filtered, chunk_to_batch = calc_chunks(cu, 128)
    assert cu_chunk.tolist() == [0, 128, 198, 326, 389, 433, 512]
    assert filtered.tolist() == [0, 2] and n_filtered == 2
    assert chunk_to_batch.tolist() == [0, 0, 1, 1, 2, 3]


def test_public_api_surface():
    import inspect

    import moba_b200

    sig = inspect.signature(moba_b200.moba_attn_varlen)
    assert list(sig.parameters) == ["q", "k", "v", "cu_seqlens", "max_seqlen", "moba_chunk_size", "moba_topk"]
    cfg = moba_b200.MoBAConfig(moba_chunk_size=4096, moba_topk=12)
    assert (cfg.moba_chunk_size, cfg.moba_topk) == (4096, 12)
    assert list(inspect.signature(moba_b200.moba_layer).parameters)[:6] == [
        "moba_impl", "moba_config", "module", "query", "key", "value"]


def test_cpu_tensors_are_rejected():
    from moba_b200 import moba_attn_varlen

    q = torch.zeros(16, 1, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        moba_attn_varlen(q, q, q, torch.tensor([0, 16], dtype=torch.int32), 16, 8, 2)


def test_register_moba_and_layout_helpers():
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS

    import moba_b200
    from moba_b200.wrapper import fa_to_hf, hf_to_fa

    moba_b200.register_moba(moba_b200.MoBAConfig(512, 3))
    assert "moba" in ALL_ATTENTION_FUNCTIONS
    x = torch.arange(2 * 3 * 5 * 4, dtype=torch.float32).view(2, 3, 5, 4)
    y = hf_to_fa(x)
    assert y.shape == (10, 3, 4)
    assert torch.equal(fa_to_hf(y, 2), x)


def test_decode_branch_matches_dense_causal():
    """q_len != kv_len goes to dense causal attention aligned to the end of the keys (moba/wrapper.py:76-82)."""
    from moba_b200 import MoBAConfig, moba_layer

    class M(torch.nn.Module):
        is_causal = True

    torch.manual_seed(0)
    q = torch.randn(2, 4, 3, 16)
    k = torch.randn(2, 2, 7, 16)
    v = torch.randn(2, 2, 7, 16)
    out, w = moba_layer(None, MoBAConfig(4, 2), M(), q, k, v, scaling=0.25)
    assert w is None and out.shape == (2, 3, 4, 16)
    kk, vv = k.repeat_interleave(2, 1), v.repeat_interleave(2, 1)
    s = torch.einsum("bhqd,bhkd->bhqk", q, kk) * 0.25
    mask = torch.arange(7)[None, :] <= (torch.arange(3)[:, None] + 4)
    s = s.masked_fill(~mask, float("-inf"))
    ref = torch.einsum("bhqk,bhkd->bhqd", s.softmax(-1), vv).transpose(1, 2)
    torch.testing.assert_close(out, ref, atol=1e-5, rtol=1e-5)


def test_register_moba_registers_both_reference_keys(monkeypatch):
    """moba/__init__.py:9-11 registers "moba" and "moba_naive"; the second forwards to the reference package's dense
    oracle and says so clearly when that package is not importable."""
    import builtins

    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS

    import moba_b200

    moba_b200.register_moba(moba_b200.MoBAConfig(512, 3))
    assert "moba" in ALL_ATTENTION_FUNCTIONS and "moba_naive" in ALL_ATTENTION_FUNCTIONS
    real_import = builtins.__import__

    def no_reference(name, *a, **k):
        if name.startswith("moba.") or name == "moba":
            raise ImportError("no reference package")
        return real_import(name, *a, **k)

    monkeypatch.setattr(builtins, "__import__", no_reference)
    with pytest.raises(RuntimeError, match='attn_implementation="moba"'):
        moba_b200._moba_naive_impl()


def test_plans_are_shared_by_value_and_wrapper_cu_seqlens_by_identity():
    from moba_b200 import ops
    from moba_b200.wrapper import _cu_seqlens

    a = ops.get_plan([0, 100, 356], 64, 3, "cpu")
    b = ops.get_plan(torch.tensor([0, 100, 356], dtype=torch.int32), 64, 3, "cpu")
    assert a is b                                              # equal values: one plan, one table upload
    assert ops.get_plan([0, 100, 356], 64, 4, "cpu") is not a
    t1 = _cu_seqlens(3, 40, torch.device("cpu"))
    assert t1.tolist() == [0, 40, 80, 120] and t1.dtype == torch.int32
    assert _cu_seqlens(3, 40, torch.device("cpu")) is t1       # every layer call sees the same tensor

    class NoReadBack(torch.Tensor):
        pass

    t = torch.tensor([0, 128, 256], dtype=torch.int32)
    ops.register_cu_seqlens(t, [0, 128, 256])
    calls = []
    orig = torch.Tensor.cpu
    try:
        torch.Tensor.cpu = lambda self, *a, **k: calls.append(1) or orig(self, *a, **k)
        p = ops.get_plan(t, 128, 2, "cpu")
    finally:
        torch.Tensor.cpu = orig
    assert not calls and p.info.total_tokens == 256            # registered host values: no read-back of the tensor


def test_decode_branch_rejects_more_queries_than_keys():
    from moba_b200 import MoBAConfig, moba_layer

    class M(torch.nn.Module):
        is_causal = True

    q, k = torch.randn(1, 2, 5, 16), torch.randn(1, 2, 3, 16)
    with pytest.raises(ValueError, match="kv_len >= q_len"):
        moba_layer(None, MoBAConfig(4, 2), M(), q, k, k)


def test_host_numa_nodes_reads_sysfs():
    """The NUMA nodes bench.py reports beside the copy rates: every node that has CPUs, with CPU ids as integers;
    together they cover the CPUs this process may run on (an empty dict only where sysfs has no node directory)."""
    import os

    from moba_b200.host_io import host_numa_nodes

    nodes = host_numa_nodes()
    if not os.path.isdir("/sys/devices/system/node"):
        assert nodes == {}
        return
    assert nodes and all(isinstance(n, int) and cpus and all(isinstance(c, int) for c in cpus)
                         for n, cpus in nodes.items())
    assert os.sched_getaffinity(0) <= set().union(*nodes.values())
