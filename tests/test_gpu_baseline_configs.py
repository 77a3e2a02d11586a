"""Parity at the sizes the benchmark reports numbers for.

* 32768 tokens x 1 head, chunk 2048 (and the chunk 512 of the reference's tests/test_moba_speedup.py:84), top-k 3:
  small enough for the full numpy oracle -- out, dq, dk, dv and the block selection of every query.
* the varlen training batch (16 ragged sequences, 630272 tokens, chunk 512, top-k 3) on a 2-head cut, the
  1M-token prefill on one GPU's 4-query-head / 1-key-value-head share (forward), and the 131072-token layer with
  the grouped-query head mapping on an 8-query-head / 2-key-value-head cut: a dense oracle is impossible there
  (tests/sparse_ref.py), so the selection of EVERY query is compared with an fp32 restatement of the gate, the
  index lists and the row map are checked against the selection, and sampled rows of out / dq / dk / dv are
  compared with fp32 arithmetic over exactly the keys / queries the MoBA rule prescribes.
"""
import numpy as np
import pytest
import torch

from oracle import moba_oracle as orc
from tests import helpers as H
from tests import sparse_ref as R

pytestmark = pytest.mark.gpu


def _varlen_lengths(seed=0, n=16):
    import random

    rnd = random.Random(seed)
    return [512 * rnd.randint(8, 128) for _ in range(n)]


def _randn_heads(S, heads, seed, dev, off_chunks=0, off_std=0.0, chunk=0):
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(S, heads, 128, generator=g, device=dev)
    if off_std > 0:
        off = torch.randn(off_chunks, heads, 128, generator=g, device=dev) * off_std
        x = x + off.repeat_interleave(chunk, dim=0)[:S]
    return x.to(torch.bfloat16)


@pytest.mark.parametrize("chunk", [2048, 512])
def test_32k_single_head_against_full_oracle(cuda_device, chunk):
    from moba_b200 import ops
    from moba_b200.moba_efficient import check_kernel_status, moba_attn_varlen

    S, topk = 32768, 3
    q, k, v, d_out = H.make_inputs(2, S, 1, "bf16")
    cu = [0, S]
    tq, tk, tv = (torch.from_numpy(x).to(cuda_device).to(torch.bfloat16).requires_grad_() for x in (q, k, v))
    out = moba_attn_varlen(tq, tk, tv, torch.tensor(cu, dtype=torch.int32, device=cuda_device), S, chunk, topk)
    out.backward(torch.from_numpy(d_out).to(cuda_device).to(torch.bfloat16))
    check_kernel_status(cuda_device)
    kmean, scores, masks = orc.select_all(q, k, cu, chunk, topk, "bf16")
    want = orc.moba_attn_varlen_oracle(q, k, v, cu, None, chunk, topk, "bf16", d_out=d_out)
    for name, g, w in zip(("out", "dq", "dk", "dv"), (out, tq.grad, tk.grad, tv.grad), want):
        H.assert_parity(f"chunk{chunk}:{name}", g.detach().float().cpu().numpy(), w)
    # block selection of every query: identical sets up to near ties of the fp32 gate
    plan = ops.get_plan(cu, chunk, topk, cuda_device)
    sel, _, _ = ops.gate_topk(tq.detach(), ops.pool_keys(tk.detach(), plan), plan)
    sel_n = np.sort(sel.cpu().numpy(), axis=-1)                           # one sequence: global id == local id
    ref = np.full_like(sel_n, -1)
    m = masks[0]                                                          # [H, S, n]
    for s in range(S):
        c = np.nonzero(m[0, s])[0]
        ref[s, 0, sel_n.shape[2] - len(c):] = c
    sc = scores[0]
    n_exact, n_tie, n_bad = H.compare_selections(sel_n, ref, lambda s, h, c: float(sc[h, s, c]))
    assert n_bad == 0 and n_tie <= 1e-3 * S, (n_exact, n_tie, n_bad)


def test_varlen_training_batch_two_head_cut(cuda_device):
    """16 ragged sequences (lengths 512 * U{8..128}, seeded as in bench.py), chunk 512, top-k 3: 1231 chunks, up
    to 125 candidates per query -- the hardest list-building case."""
    from moba_b200 import ops
    from moba_b200.moba_efficient import check_kernel_status, moba_attn_varlen

    dev = cuda_device
    lens = _varlen_lengths()
    assert sum(lens) == 630272
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    S, heads, chunk, topk = cu[-1], 2, 512, 3
    q, k, v, d_out = (_randn_heads(S, heads, 40 + i, dev) for i in range(4))
    qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    out = moba_attn_varlen(qr, kr, vr, cu_t, max(lens), chunk, topk)
    out.backward(d_out)
    check_kernel_status(dev)

    lay = R.Layout(cu, chunk, dev)
    plan = ops.get_plan(cu, chunk, topk, dev)
    assert plan.info.n_chunks == 1231
    kmean = ops.pool_keys(k, plan)
    R.check_pooled_keys(kmean, k, lay)
    ref_mask, gate = R.reference_selection(q, k, lay, topk, kmean_kernel=kmean)
    sel, _, tile_cnt = ops.gate_topk(q, kmean, plan)
    got_mask = R.kernel_selection(sel, lay)
    R.assert_same_selection(got_mask, ref_mask, gate, lay, topk)
    list_off, work_off, list_tok, row_of = ops.build_lists(plan, heads, sel, tile_cnt)
    R.check_lists(plan, heads, sel, list_off, work_off, list_tok, row_of)

    rng = np.random.RandomState(4)
    # sampled rows, plus the first / last token of the batch and tokens around sequence and chunk borders
    rows = [(int(rng.randint(0, S)), int(rng.randint(0, heads))) for _ in range(40)]
    rows += [(0, 0), (S - 1, 1), (cu[1] - 1, 0), (cu[1], 1), (cu[5] + 511, 0), (cu[5] + 512, 1), (cu[-2], 0)]
    R.check_query_rows(rows, q, k, v, d_out, out.detach(), qr.grad, got_mask, lay)
    keys = [(int(rng.randint(0, S)), int(rng.randint(0, heads))) for _ in range(10)]
    keys += [(0, 0), (S - 1, 1), (cu[3], 0), (cu[3] + 511, 1)]
    R.check_key_rows(keys, q, k, v, d_out, out.detach(), kr.grad, vr.grad, got_mask, lay)


def test_one_million_token_prefill_share(cuda_device):
    """One GPU's share of the 1M-token prefill: 4 query heads on 1 key/value head, chunk 4096, top-k 12, forward.
    256 chunks: the gate works in two rounds of candidates, the lists cover 8192 (chunk, head) experts."""
    from moba_b200 import ops
    from moba_b200.moba_efficient import check_kernel_status, moba_attn_varlen

    dev = cuda_device
    S, heads, chunk, topk = 1048576, 4, 4096, 12
    q = _randn_heads(S, heads, 51, dev)
    k = _randn_heads(S, 1, 52, dev, off_chunks=S // chunk, off_std=0.5, chunk=chunk)
    v = _randn_heads(S, 1, 53, dev)
    cu = [0, S]
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    with torch.no_grad():
        out = moba_attn_varlen(q, k, v, cu_t, S, chunk, topk)             # grouped-query K / V, unexpanded
    check_kernel_status(dev)
    lay = R.Layout(cu, chunk, dev)
    plan = ops.get_plan(cu, chunk, topk, dev)
    kmean = ops.pool_keys(k, plan)
    R.check_pooled_keys(kmean, k, lay)
    sel, _, tile_cnt = ops.gate_topk(q, kmean, plan)
    got_mask = R.kernel_selection(sel, lay)
    ref_mask, gate = R.reference_selection(q, k, lay, topk, rep=heads, kmean_kernel=kmean)
    R.assert_same_selection(got_mask, ref_mask, gate, lay, topk)
    del ref_mask, gate
    list_off, work_off, list_tok, row_of = ops.build_lists(plan, heads, sel, tile_cnt)
    R.check_lists(plan, heads, sel, list_off, work_off, list_tok, row_of)
    rng = np.random.RandomState(5)
    rows = [(int(rng.randint(0, S)), int(rng.randint(0, heads))) for _ in range(40)]
    rows += [(0, 0), (S - 1, 3), (chunk, 1), (255 * chunk - 1, 2), (255 * chunk, 0)]
    R.check_query_rows(rows, q, k, v, None, out, None, got_mask, lay, rep=heads)
    # the same call on expanded K / V (what moba/wrapper.py:59-61 feeds the reference) gives the same bits
    with torch.no_grad():
        out_x = moba_attn_varlen(q, k.expand(S, heads, 128).contiguous(), v.expand(S, heads, 128).contiguous(), cu_t,
                                 S, chunk, topk)
    check_kernel_status(dev)
    assert torch.equal(out, out_x)


def test_128k_layer_grouped_query_mapping(cuda_device):
    """The 131072-token layer with the 32-query-head / 8-key-value-head mapping on an 8 / 2 cut (four query heads
    per key/value head), forward + backward: K / V expanded before the call (what the benchmark times) against
    sampled fp32 rows, and the unexpanded grouped-query call against the expanded one."""
    from moba_b200 import ops
    from moba_b200.moba_efficient import check_kernel_status, moba_attn_varlen

    dev = cuda_device
    S, heads, kv_heads, chunk, topk = 131072, 8, 2, 4096, 12
    rep = heads // kv_heads
    q = _randn_heads(S, heads, 31, dev)
    k = _randn_heads(S, kv_heads, 32, dev, off_chunks=S // chunk, off_std=0.5, chunk=chunk)
    v = _randn_heads(S, kv_heads, 33, dev)
    d_out = _randn_heads(S, heads, 34, dev)
    cu = [0, S]
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    kx, vx = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    qr, kr, vr = (t.clone().requires_grad_() for t in (q, kx, vx))
    out = moba_attn_varlen(qr, kr, vr, cu_t, S, chunk, topk)
    out.backward(d_out)
    check_kernel_status(dev)

    lay = R.Layout(cu, chunk, dev)
    plan = ops.get_plan(cu, chunk, topk, dev)
    kmean = ops.pool_keys(k, plan)
    R.check_pooled_keys(kmean, k, lay)
    sel, _, _ = ops.gate_topk(q, kmean, plan)
    got_mask = R.kernel_selection(sel, lay)
    ref_mask, gate = R.reference_selection(q, k, lay, topk, rep=rep, kmean_kernel=kmean)
    R.assert_same_selection(got_mask, ref_mask, gate, lay, topk)
    del ref_mask, gate
    rng = np.random.RandomState(6)
    rows = [(int(rng.randint(0, S)), int(rng.randint(0, heads))) for _ in range(32)] + [(0, 0), (S - 1, 7), (chunk, 5)]
    R.check_query_rows(rows, q, kx, vx, d_out, out.detach(), qr.grad, got_mask, lay)
    keys = [(int(rng.randint(0, S)), int(rng.randint(0, heads))) for _ in range(6)] + [(0, 0), (S - 1, 6)]
    R.check_key_rows(keys, q, kx, vx, d_out, out.detach(), kr.grad, vr.grad, got_mask, lay)

    # grouped-query call on the unexpanded K / V: out and dq bit for bit, dk / dv = sums over each group
    qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
    out_g = moba_attn_varlen(qg, kg, vg, cu_t, S, chunk, topk)
    out_g.backward(d_out)
    check_kernel_status(dev)
    assert torch.equal(out_g, out) and torch.equal(qg.grad, qr.grad)
    keys_g = [(int(rng.randint(0, S)), int(rng.randint(0, kv_heads))) for _ in range(4)] + [(S - 1, 1)]
    R.check_key_rows(keys_g, q, k, v, d_out, out.detach(), kg.grad, vg.grad, got_mask, lay, rep=rep)
