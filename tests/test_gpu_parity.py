"""GPU parity tests: every call goes through the C ABI of libmoba_b200.so (via the ctypes binding) and is
compared with the CPU oracle on the same seeded inputs, and with the committed reference fixtures."""
import numpy as np
import pytest
import torch

from oracle import moba_oracle as orc
from tests import helpers as H

pytestmark = pytest.mark.gpu

TORCH_DT = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}


def t2n(t):
    return t.detach().float().cpu().numpy()


def to_dev(x, dev, dtype="bf16"):
    return torch.from_numpy(np.ascontiguousarray(x)).to(dev).to(TORCH_DT[dtype])


def run_api(q, k, v, d_out, cu, chunk, topk, dev, dtype="bf16"):
    from moba_b200.moba_efficient import check_kernel_status, moba_attn_varlen

    tq, tk, tv = (to_dev(x, dev, dtype).requires_grad_() for x in (q, k, v))
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    out = moba_attn_varlen(tq, tk, tv, cu_t, max(b - a for a, b in zip(cu, cu[1:])), chunk, topk)
    out.backward(to_dev(d_out, dev, dtype))
    check_kernel_status(dev)
    return t2n(out), t2n(tq.grad), t2n(tk.grad), t2n(tv.grad)


def check_against_oracle(q, k, v, d_out, cu, chunk, topk, dev, dtype="bf16", tag=""):
    got = run_api(q, k, v, d_out, cu, chunk, topk, dev, dtype)
    want = orc.moba_attn_varlen_oracle(q, k, v, cu, None, chunk, topk, dtype, d_out=d_out)
    for name, g, w in zip(("out", "dq", "dk", "dv"), got, want):
        H.assert_parity(f"{tag}{name}", g, w)
    return got


# ------------------------------------------------------------------------------------------ building blocks
@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("mode", [0, 1, 2, 4, 5])
def test_umma_selftest(cuda_device, mode, dtype):
    from moba_b200 import ops

    torch.manual_seed(mode)
    a = torch.randn(128, 128, device=cuda_device).to(TORCH_DT[dtype])
    b = torch.randn(128, 128, device=cuda_device).to(TORCH_DT[dtype])
    c = ops.selftest_umma(mode, a, b)
    ref = a.float() @ (b.float().T if mode in (0, 4) else b.float())
    if mode == 5:       # both operands MN-major, 64 result columns
        ref = torch.zeros_like(ref)
        ref[:, :64] = a.float().T @ b.float()[:, :64]
    if mode == 4:       # plus a ninth k-step from thread-written tiles without swizzle
        ref = ref + a[:, :16].float() @ b[:, :16].float().T
    assert (c - ref).abs().max().item() < 1e-3


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
def test_umma_pair_selftest(cuda_device, dtype):
    """256-row instructions over a pair of CTAs: each CTA's half of the rows, of the keys (S) and of the value
    columns (O) must land where a plain matrix product puts them."""
    from moba_b200 import ops

    torch.manual_seed(7)
    q = torch.randn(256, 128, device=cuda_device).to(TORCH_DT[dtype])
    k = torch.randn(128, 128, device=cuda_device).to(TORCH_DT[dtype])
    v = torch.randn(128, 128, device=cuda_device).to(TORCH_DT[dtype])
    s, o = ops.selftest_umma_pair(q, k, v)
    s_ref = q.float() @ k.float().T
    assert (s - s_ref).abs().max().item() < 1e-3
    p = (s * 0.0625).to(TORCH_DT[dtype]).float()          # what the kernel hands to the second product
    o_ref = p @ v.float()
    assert (o - o_ref).abs().max().item() < 2e-3


@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
def test_pool_keys_bit_exact_on_fixture_shapes(cuda_device, dtype):
    from moba_b200 import ops

    (k,) = H.make_inputs(3, 1000, 3, dtype, n=1)
    cu = [0, 130, 131, 700, 1000]
    for chunk in (64, 96, 128, 512):
        plan = ops.get_plan(cu, chunk, 3, cuda_device)
        got = t2n(ops.pool_keys(to_dev(k, cuda_device, dtype), plan))
        want = orc.pool_keys(k, cu, chunk, dtype)
        # same fp32 sum up to order; the rounding to `dtype` can flip on a half-ulp tie
        ulp = {"bf16": 2.0 ** -8, "f16": 2.0 ** -11, "f32": 2.0 ** -22}[dtype]
        assert np.abs(got - want).max() <= ulp * max(1.0, np.abs(want).max())
        if dtype != "f32":      # fp32 means differ in the last bits with the summation order
            assert (got != want).mean() < 1e-3


@pytest.mark.parametrize("name", H.SMALL_CASES)
def test_selection_and_lists_match_reference(cuda_device, name):
    """Top-k sets identical to the reference's (pairs with fp32 gate scores within 1e-3 relative excluded),
    and the index lists / row map are consistent with the selection."""
    from moba_b200 import ops

    fx = H.load_small(name)
    cu, chunk, topk = fx["cu_seqlens"], fx["chunk"], fx["topk"]
    q, k = to_dev(fx["q"], cuda_device), to_dev(fx["k"], cuda_device)
    S, heads, _ = q.shape
    plan = ops.get_plan(cu, chunk, topk, cuda_device)
    kmean = ops.pool_keys(k, plan)
    sel, scores, tile_cnt = ops.gate_topk(q, kmean, plan, want_scores=True)
    list_off, work_off, list_tok, row_of = ops.build_lists(plan, heads, sel, tile_cnt)
    torch.cuda.synchronize()
    sel_n = sel.cpu().numpy()
    first = plan.table("chunk_seq_first").numpy()
    cs = plan.table("chunk_start").numpy()
    tok_chunk = np.searchsorted(cs, np.arange(S), side="right") - 1
    local = np.where(sel_n >= 0, sel_n - first[tok_chunk][:, None, None], -1)

    def score_of(s, h, c):
        b = max(i for i in range(len(cu) - 1) if cu[i] <= s)
        return float(fx[f"scores{b}"][h, s - cu[b], c])

    n_exact, n_tie, n_bad = H.compare_selections(local, fx["sel"].astype(np.int64), score_of)
    assert n_bad == 0, (n_exact, n_tie, n_bad)
    assert n_tie <= 0.01 * S * heads

    lo, lt, ro, wo = (x.cpu().numpy() for x in (list_off, list_tok, row_of, work_off))
    R = plan.rows_total(heads)
    assert lo[-1] == R
    assert wo[-1] <= plan.info.max_work_tiles_per_head * heads
    for e in range(plan.info.n_chunks * heads):
        c, h = divmod(e, heads)
        want = np.nonzero((sel_n[:, h, :] == c).any(-1))[0]
        np.testing.assert_array_equal(lt[lo[e]:lo[e + 1]], want)      # ascending token order
        assert wo[e + 1] - wo[e] == -(-len(want) // 128)
    rows = ro[sel_n >= 0]
    assert len(np.unique(rows)) == len(rows) == R
    assert (ro[sel_n < 0] == -1).all()
    ss, hh, jj = np.nonzero(sel_n >= 0)
    np.testing.assert_array_equal(lt[ro[ss, hh, jj]], ss)


# ------------------------------------------------------------------------------------------ fixtures
@pytest.mark.parametrize("name", H.SMALL_CASES)
def test_forward_backward_vs_reference_fixture(cuda_device, name):
    fx = H.load_small(name)
    got = check_against_oracle(fx["q"], fx["k"], fx["v"], fx["d_out"], fx["cu_seqlens"], fx["chunk"], fx["topk"],
                               cuda_device, tag=name + ":")
    # the reference's stored outputs are themselves bf16-rounded: its own test tolerances (tests/test_moba_attn.py:85-100)
    for nm, g in zip(("out", "dq", "dk", "dv"), got):
        d = np.abs(g - fx[nm])
        assert d.max() < 4e-2 and d.mean() < 4e-4, (nm, d.max(), d.mean())


def test_config1_fp32_inputs(cuda_device):
    """cu_seqlens=[0,1024,4096], 4 heads, fp32 N(0,1) seed 0, chunk 512, top-k 3, forward + backward."""
    fx, inputs = H.load_config1()
    torch.manual_seed(0)
    q, k, v, d_out = (torch.randn(4096, 4, 128).numpy() for _ in range(4))
    cu = fx["cu_seqlens"]
    got = check_against_oracle(q, k, v, d_out, cu, 512, 3, cuda_device, dtype="f32", tag="config1:")
    if inputs is not None:
        rows = fx["rows"]
        for nm, g in zip(("out", "dq", "dk", "dv"), got):
            H.assert_parity("config1-fixture:" + nm, g[rows], fx[nm])
    # identical block selection on fp32 inputs
    from moba_b200 import ops
    plan = ops.get_plan(cu, 512, 3, cuda_device)
    tq, tk = to_dev(q, cuda_device, "f32"), to_dev(k, cuda_device, "f32")
    sel, _, _ = ops.gate_topk(tq, ops.pool_keys(tk, plan), plan)
    sel_n = sel.cpu().numpy()
    first = plan.table("chunk_seq_first").numpy()
    tok_chunk = np.searchsorted(plan.table("chunk_start").numpy(), np.arange(4096), side="right") - 1
    local = np.where(sel_n >= 0, sel_n - first[tok_chunk][:, None, None], -1)
    _, scores, _ = orc.select_all(q, k, cu, 512, 3, "f32")

    def score_of(s, h, c):
        b = 0 if s < cu[1] else 1
        return float(scores[b][h, s - cu[b], c])

    n_exact, n_tie, n_bad = H.compare_selections(local, fx["sel"].astype(np.int64), score_of)
    assert n_bad == 0 and n_tie <= 40, (n_exact, n_tie, n_bad)


# ------------------------------------------------------------------------------------------ the reference's grid
@pytest.mark.parametrize("batch", [1, 4, 7])
@pytest.mark.parametrize("head", [1, 2, 4, 8])
@pytest.mark.parametrize("seqlen", [512, 1024, 2048])
@pytest.mark.parametrize("moba_chunk_size", [128, 256, 1024])
@pytest.mark.parametrize("moba_topk", [2, 3, 4])
def test_reference_grid(cuda_device, batch, head, seqlen, moba_chunk_size, moba_topk):
    """The parameter grid of the reference's differential test (tests/test_moba_attn.py:37-42), bf16, ragged
    cu_seqlens, forward + backward against the oracle."""
    seed = hash((batch, head, seqlen, moba_chunk_size, moba_topk)) % 1000
    q, k, v, d_out = H.make_inputs(seed, seqlen, head)
    cu = H.ragged_cu(0, seqlen, batch)
    check_against_oracle(q, k, v, d_out, cu, moba_chunk_size, moba_topk, cuda_device)


# ------------------------------------------------------------------------------------------ corner cases
@pytest.mark.parametrize("case", [
    dict(S=200, cu=[0, 200], chunk=256, topk=3),              # sequence shorter than a chunk (no candidates)
    dict(S=700, cu=[0, 700], chunk=128, topk=1),              # top-k 1: plain causal attention over the sequence
    dict(S=777, cu=[0, 777], chunk=100, topk=3),              # chunk and length not multiples of the tile
    dict(S=640, cu=[0, 640], chunk=64, topk=12),              # top-k larger than the number of past chunks
    dict(S=900, cu=[0, 300, 300, 900], chunk=128, topk=3),    # an empty sequence inside the batch
    dict(S=515, cu=[0, 1, 2, 130, 515], chunk=128, topk=2),   # one-token sequences
    dict(S=1024, cu=[0, 1024], chunk=512, topk=2),            # two chunks, one slot
    dict(S=1536, cu=[0, 1536], chunk=48, topk=5),             # many small chunks (32 per sequence)
])
def test_corner_cases(cuda_device, case):
    q, k, v, d_out = H.make_inputs(11, case["S"], 2)
    check_against_oracle(q, k, v, d_out, case["cu"], case["chunk"], case["topk"], cuda_device)


def test_expert_nobody_selects(cuda_device):
    """Keys of chunk 1 are pushed far away from every query, so its (chunk, head) list stays empty."""
    q, k, v, d_out = H.make_inputs(5, 1024, 1)
    k[128:256] = orc.round_bf16(-np.abs(k[128:256]) - 2.0)
    q[:] = orc.round_bf16(np.abs(q))
    from moba_b200 import ops
    plan = ops.get_plan([0, 1024], 128, 3, cuda_device)
    sel, _, _ = ops.gate_topk(to_dev(q, cuda_device), ops.pool_keys(to_dev(k, cuda_device), plan), plan)
    assert not (sel[384:] == 1).any()      # queries with more than two candidates never keep chunk 1
    check_against_oracle(q, k, v, d_out, [0, 1024], 128, 3, cuda_device)


def test_fp16_inputs(cuda_device):
    q, k, v, d_out = H.make_inputs(21, 1024, 2, "f16")
    check_against_oracle(q, k, v, d_out, [0, 400, 1024], 128, 3, cuda_device, dtype="f16")


def test_strided_inputs(cuda_device):
    """q, k, v as views of one packed [S, 3, H, D] tensor (row stride 3*H*D)."""
    from moba_b200.moba_efficient import moba_attn_varlen

    q, k, v, d_out = H.make_inputs(22, 768, 2)
    qkv = torch.stack([to_dev(x, cuda_device) for x in (q, k, v)], dim=1).requires_grad_()
    cu = torch.tensor([0, 768], dtype=torch.int32, device=cuda_device)
    out = moba_attn_varlen(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, 768, 128, 3)
    out.backward(to_dev(d_out, cuda_device))
    want = orc.moba_attn_varlen_oracle(q, k, v, [0, 768], None, 128, 3, "bf16", d_out=d_out)
    H.assert_parity("out", t2n(out), want[0])
    for i, nm in enumerate(("dq", "dk", "dv")):
        H.assert_parity(nm, t2n(qkv.grad[:, i]), want[i + 1])


def test_bitwise_run_to_run_determinism(cuda_device):
    q, k, v, d_out = H.make_inputs(31, 2048, 4)
    cu = H.ragged_cu(3, 2048, 3)
    a = run_api(q, k, v, d_out, cu, 128, 4, cuda_device)
    b = run_api(q, k, v, d_out, cu, 128, 4, cuda_device)
    for x, y in zip(a, b):
        assert np.array_equal(x, y)




@pytest.mark.parametrize("duplex", [True, False])
@pytest.mark.parametrize("groups", [1, 3, 8])
def test_host_entry_point_matches_device_call(cuda_device, groups, duplex):
    """moba_attn_varlen_host (pinned host tensors, head groups pipelined over copy and compute streams, with both
    copy directions at once or one at a time) returns bit for bit what moba_attn_varlen returns on device tensors:
    heads are independent."""
    from moba_b200 import moba_attn_varlen_host

    q, k, v, d_out = H.make_inputs(51, 1536, 6)
    cu = [0, 500, 1536]
    want = run_api(q, k, v, d_out, cu, 128, 3, cuda_device)
    hq, hk, hv, hdo = (torch.from_numpy(x).to(torch.bfloat16).pin_memory() for x in (q, k, v, d_out))
    cu_t = torch.tensor(cu, dtype=torch.int32, device=cuda_device)
    stats = {}
    out, grads = moba_attn_varlen_host(hq, hk, hv, cu_t, 1036, 128, 3, d_out=hdo, head_groups=groups,
                                       device=cuda_device, duplex=duplex, stats=stats)
    for name, g, w in zip(("out", "dq", "dk", "dv"), (out,) + tuple(grads), want):
        assert np.array_equal(g.float().numpy(), w), name
    assert sum(stats["slices"]) == 6 and len(stats["timeline"]) == len(stats["slices"])
    if not duplex:      # every copy-in ends before the first copy-out begins
        assert max(t[1] for t in stats["timeline"]) <= min(t[4] for t in stats["timeline"]) + 1e-3
    fwd_only = moba_attn_varlen_host(hq, hk, hv, cu_t, 1036, 128, 3, head_groups=groups, device=cuda_device,
                                     duplex=duplex)
    assert np.array_equal(fwd_only.float().numpy(), want[0])


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
def test_large_logits(cuda_device, dtype):
    """Scores with a standard deviation of ~36 (softmax close to one-hot, log-sum-exp in the hundreds): the range
    handling of the running maximum, of the merged statistics and of the lse / delta operands of the backward."""
    q, k, v, d_out = H.make_inputs(61, 1024, 2, dtype)
    q = orc.round_dtype(6.0 * q, dtype)
    k = orc.round_dtype(6.0 * k, dtype)
    cu = [0, 300, 1024]
    got = run_api(q, k, v, d_out, cu, 128, 3, cuda_device, dtype)
    want = orc.moba_attn_varlen_oracle(q, k, v, cu, None, 128, 3, dtype, d_out=d_out)
    # Gradients reach magnitudes of 20-30 here and every entry is a sum of terms of that size, each carrying the
    # 2^-9 rounding of P / dS to 16 bit (as in the reference's flash kernels): the error scales with the
    # tensor's magnitude, so the bound is 1 % of max|ref| (+ the usual 2e-2) instead of the flat bound of the
    # other tests.
    for name, g, w in zip(("out", "dq", "dk", "dv"), got, want):
        assert np.isfinite(g).all(), name
        diff = np.abs(g - w)
        bound = 2e-2 + 1e-2 * np.abs(w).max()
        assert diff.max() <= bound, f"{name}: max {diff.max():.4g} > {bound:.4g}"
        assert diff.mean() <= 4e-3, f"{name}: mean-abs {diff.mean():.4g}"


@pytest.mark.parametrize("dtype,S,cu,chunk", [
    ("bf16", 4396, [0, 1500, 4396], 64),          # up to 45 candidate chunks
    ("f16", 4396, [0, 1500, 4396], 64),
    ("bf16", 20000, [0, 20000], 64),              # 312 chunks: two rounds of 256 candidates on the tensor pipe
])
def test_gate_tensor_pipe_matches_fma(cuda_device, dtype, S, cu, chunk):
    """The tensor-pipe gate (16-bit q) and the fp32-FMA gate differ only in the order of the fp32 additions:
    scores agree to ~1e-6 relative, selections are identical except where two candidates tie within 1e-3."""
    from moba_b200 import ops

    q, k, _, _ = H.make_inputs(71, S, 2, dtype)
    tq, tk = to_dev(q, cuda_device, dtype), to_dev(k, cuda_device, dtype)
    plan = ops.get_plan(cu, chunk, 5, cuda_device)
    kmean = ops.pool_keys(tk, plan)
    sel_a, sc_a, cnt_a = ops.gate_topk(tq, kmean, plan, want_scores=True)
    sel_b, sc_b, cnt_b = ops.gate_topk(tq, kmean, plan, want_scores=True, fma=True)
    # the two kernels list a row's chunks in different orders (ascending chunk id / best first): compare by chunk
    ord_a, ord_b = sel_a.sort(dim=-1), sel_b.sort(dim=-1)
    sel_a, sc_a = ord_a.values, sc_a.gather(-1, ord_a.indices)
    sel_b, sc_b = ord_b.values, sc_b.gather(-1, ord_b.indices)
    same = (sel_a == sel_b).all(dim=-1)
    fin = torch.isfinite(sc_b) & same[..., None]
    assert torch.equal(torch.isfinite(sc_b), torch.isfinite(sc_a))
    assert ((sc_a - sc_b)[fin].abs() <= 1e-5 * (1 + sc_b[fin].abs())).all()
    assert same.float().mean().item() > 0.999
    # rows that differ: the candidates not shared by both selections score within 1e-3 relative of each other
    for s_i, h_i in torch.nonzero(~same).tolist():
        a, b = set(sel_a[s_i, h_i].tolist()), set(sel_b[s_i, h_i].tolist())
        only = sorted((a ^ b) - {-1})
        sc = (tq[s_i, h_i].float()[None, :] * kmean[only, h_i]).sum(-1)
        assert (sc.max() - sc.min()).item() <= 1e-3 * sc.abs().max().item(), (s_i, h_i, only, sc.tolist())
    if bool(same.all()):
        assert torch.equal(cnt_a, cnt_b)


@pytest.mark.parametrize("head_dim", [64, 96, 32])
def test_smaller_head_dims(cuda_device, head_dim):
    """head_dim below the 128-column tile width: the call pads with zero columns and keeps head_dim^-0.5
    (moba/moba_efficient.py:86), so the result is that of the reference at that head dim."""
    rng = np.random.RandomState(head_dim)
    S, heads, chunk, topk = 1100, 2, 128, 3
    cu = [0, 500, 1100]
    q, k, v, d_out = (orc.round_bf16(rng.randn(S, heads, head_dim).astype(np.float32)) for _ in range(4))
    got = check_against_oracle(q, k, v, d_out, cu, chunk, topk, cuda_device, tag=f"D{head_dim}:")
    assert got[0].shape == (S, heads, head_dim) and got[3].shape == (S, heads, head_dim)


def test_unsupported_head_dims_are_refused(cuda_device):
    from moba_b200 import moba_attn_varlen

    cu = torch.tensor([0, 256], dtype=torch.int32, device=cuda_device)
    for d in (256, 100):
        x = torch.zeros(256, 1, d, dtype=torch.bfloat16, device=cuda_device)
        with pytest.raises(ValueError, match="head_dim"):
            moba_attn_varlen(x, x, x, cu, 256, 64, 2)


@pytest.mark.parametrize("chunk,topk", [(256, 3), (1024, 4), (4096, 3)])
def test_dq_kernel_forms_give_the_same_bits(cuda_device, chunk, topk):
    """The dQ kernel's two forms (one query tile per CTA; a persistent CTA per SM walking its tiles, several rounds
    each here) run the same arithmetic in the same order: dq_self and part_dq are bit for bit the same, on a ragged
    batch with partial tiles."""
    from moba_b200 import ops

    dev = cuda_device
    lens = [5000, 37, 12288 + 77, 128, 20000]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    S, H = cu[-1], 3
    g = torch.Generator(device=dev).manual_seed(11)
    q, k, v, d_out = (torch.randn(S, H, 128, generator=g, device=dev).to(torch.bfloat16) for _ in range(4))
    plan = ops.get_plan(cu, chunk, topk, dev)
    status = ops.new_status(dev)
    sel, _, tile_cnt = ops.gate_topk(q, ops.pool_keys(k, plan), plan, status=status)
    list_off, work_off, list_tok, row_of = ops.build_lists(plan, H, sel, tile_cnt, status=status)
    lists = (list_off, work_off, list_tok)
    out, lse, part_o, part_lse = ops.attn_fwd(q, k, v, plan, lists, status)
    ops.merge_fwd(out, lse, plan, part_o, part_lse, row_of)
    delta = ops.bwd_delta(out, d_out)
    gathered = ops.gather_rows(q, d_out, plan, lists, lse, delta)
    got = {}
    for form in ("tile", "persistent"):
        dq_self, part_dq = ops.attn_bwd_dq(q, k, v, d_out, plan, lists, lse, delta, status, gathered=gathered, form=form)
        got[form] = (dq_self, part_dq[: plan.rows_total(H)])
    ops.check_status(status)
    assert torch.equal(got["tile"][0], got["persistent"][0])
    assert torch.equal(got["tile"][1], got["persistent"][1])
    assert got["tile"][0].abs().max().item() > 0


def test_tile_records_equal_the_offset_search(cuda_device):
    """The list kernels find a work tile's list either from its record (moba_tile_records) or by searching the work
    offsets: forward partials, list-ordered copies and dq partials are the same bits either way."""
    from moba_b200 import ops

    dev = cuda_device
    lens = [3000, 129, 9000, 64, 16384]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    S, H, chunk, topk = cu[-1], 3, 1024, 4
    g = torch.Generator(device=dev).manual_seed(5)
    q, k, v, d_out = (torch.randn(S, H, 128, generator=g, device=dev).to(torch.bfloat16) for _ in range(4))
    plan = ops.get_plan(cu, chunk, topk, dev)
    status = ops.new_status(dev)
    sel, _, tile_cnt = ops.gate_topk(q, ops.pool_keys(k, plan), plan, status=status)
    list_off, work_off, list_tok, row_of = ops.build_lists(plan, H, sel, tile_cnt, status=status)
    rec = ops.tile_records(plan, H, list_off, work_off)
    # the records against the tables they come from
    wo, lo = work_off.cpu().numpy(), list_off.cpu().numpy()
    r = rec.cpu().numpy()
    n_tiles = int(wo[-1])
    assert (r[n_tiles:, 2] == 0).all() and (r[:n_tiles, 2] > 0).all()
    e = np.searchsorted(wo, np.arange(n_tiles), side="right") - 1
    assert (r[:n_tiles, 0] == e % H).all()
    assert (r[:n_tiles, 1] == lo[e] + (np.arange(n_tiles) - wo[e]) * 128).all()
    assert (r[:n_tiles, 2] == np.minimum(128, lo[e + 1] - r[:n_tiles, 1])).all()
    n = plan.rows_total(H)
    res = {}
    for name, lists in (("search", (list_off, work_off, list_tok)), ("records", (list_off, work_off, list_tok, rec))):
        out, lse, part_o, part_lse = ops.attn_fwd(q, k, v, plan, lists, status)
        out2, lse2 = out.clone(), lse.clone()
        ops.merge_fwd(out2, lse2, plan, part_o, part_lse, row_of)
        delta = ops.bwd_delta(out2, d_out)
        gathered = ops.gather_rows(q, d_out, plan, lists, lse2, delta)
        dqs = [ops.attn_bwd_dq(q, k, v, d_out, plan, lists, lse2, delta, status, gathered=gathered, form=f)
               for f in ("tile", "persistent")]
        res[name] = [part_o[:n], part_lse[:n], gathered[0][:n], gathered[1][:n], gathered[2][:n], gathered[3][:n]] + \
                    [t for dq_self, part_dq in dqs for t in (dq_self, part_dq[:n])]
    ops.check_status(status)
    for a_, b_ in zip(res["search"], res["records"]):
        assert torch.equal(a_, b_)


def test_random_shapes_kernel_forms_and_lookups_agree(cuda_device):
    """Seeded random ragged batches (chunk 64..4096, one to six sequences with lengths off every tile boundary,
    grouped-query K / V, both 16-bit types): the record and search lookups and the two dQ kernel forms give the same
    bits for every tensor of the forward and the backward, and all of them are finite."""
    import random

    from moba_b200 import ops

    dev = cuda_device
    rnd = random.Random(1234)
    n_checked = 0
    for it in range(60):
        nseq = rnd.randint(1, 6)
        chunk = rnd.choice([64, 96, 128, 192, 256, 512, 1024, 2048, 4096])
        topk = rnd.randint(2, 6)
        lens = [rnd.randint(1, 6 * chunk + 300) for _ in range(nseq)]
        if rnd.random() < 0.2:
            lens[rnd.randrange(nseq)] = rnd.randint(1, 40)
        hkv, rep = rnd.choice([1, 1, 2, 3]), rnd.choice([1, 1, 2, 4])
        Hq = hkv * rep
        dt = rnd.choice([torch.bfloat16, torch.bfloat16, torch.float16])
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        S = cu[-1]
        g = torch.Generator(device=dev).manual_seed(it)
        q, d_out = (torch.randn(S, Hq, 128, generator=g, device=dev).to(dt) for _ in range(2))
        k, v = (torch.randn(S, hkv, 128, generator=g, device=dev).to(dt) for _ in range(2))
        plan = ops.get_plan(cu, chunk, topk, dev)
        if plan.kk == 0:
            continue
        status = ops.new_status(dev)
        sel, _, tile_cnt = ops.gate_topk(q, ops.pool_keys(k, plan), plan, status=status)
        list_off, work_off, list_tok, row_of = ops.build_lists(plan, Hq, sel, tile_cnt, status=status)
        rec = ops.tile_records(plan, Hq, list_off, work_off)
        n = plan.rows_total(Hq)
        res = {}
        for name, lists in (("search", (list_off, work_off, list_tok)),
                            ("records", (list_off, work_off, list_tok, rec))):
            out, lse, part_o, part_lse = ops.attn_fwd(q, k, v, plan, lists, status)
            ops.merge_fwd(out, lse, plan, part_o, part_lse, row_of)
            delta = ops.bwd_delta(out, d_out)
            gathered = ops.gather_rows(q, d_out, plan, lists, lse, delta)
            dk, dv = ops.attn_bwd_dkdv(q, k, v, d_out, plan, lists, lse, delta, status, gathered=gathered)
            tensors = [out, lse, part_o[:n], part_lse[:n], dk, dv] + [t[:n] for t in gathered]
            for form in ("tile", "persistent"):
                dq_self, part_dq = ops.attn_bwd_dq(q, k, v, d_out, plan, lists, lse, delta, status,
                                                   gathered=gathered, form=form)
                tensors += [dq_self, part_dq[:n]]
            res[name] = tensors
        ops.check_status(status)
        tag = f"case {it}: lens={lens} chunk={chunk} topk={topk} H={Hq}/{hkv} {dt}"
        for i, (a_, b_) in enumerate(zip(res["search"], res["records"])):
            assert torch.equal(a_, b_), f"{tag}: tensor {i} differs between the lookups"
        a_ = res["search"]
        assert torch.equal(a_[-4], a_[-2]) and torch.equal(a_[-3], a_[-1]), f"{tag}: dQ forms differ"
        for i in (0, 4, 5, -2, -1):
            assert torch.isfinite(a_[i].float()).all().item(), f"{tag}: tensor {i} is not finite"
        n_checked += 1
    assert n_checked >= 50
