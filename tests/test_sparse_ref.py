"""Pins tests/sparse_ref.py (the sampled-row checker used where a dense oracle is impossible) to the numpy oracle
on a small ragged batch, on the CPU: same selection, and its per-row fp32 arithmetic reproduces the oracle's
out / dq / dk / dv far inside the parity tolerance."""
import numpy as np
import torch

from oracle import moba_oracle as orc
from tests import helpers as H
from tests import sparse_ref as R


def test_sparse_ref_reproduces_the_oracle(monkeypatch):
    cu, chunk, topk, heads = [0, 300, 301, 1100, 1500], 128, 3, 2
    S = cu[-1]
    q, k, v, d_out = H.make_inputs(11, S, heads, "bf16")
    out, dq, dk, dv = orc.moba_attn_varlen_oracle(q, k, v, cu, None, chunk, topk, "bf16", d_out=d_out)
    _, _, masks = orc.select_all(q, k, cu, chunk, topk, "bf16")
    tq, tk, tv, tdo = (torch.from_numpy(x).to(torch.bfloat16) for x in (q, k, v, d_out))
    lay = R.Layout(cu, chunk, torch.device("cpu"))
    mask, gate = R.reference_selection(tq, tk, lay, topk)
    for b, (t0, t1) in enumerate(zip(cu, cu[1:])):
        m = np.transpose(masks[b], (1, 0, 2))                      # [S_b, H, n_b]
        got = mask[t0:t1, :, :m.shape[2]].numpy()
        assert (got == m).all() and not mask[t0:t1, :, m.shape[2]:].any()
    R.assert_same_selection(mask, mask, gate, lay, topk)

    def tight(name, got, want):
        assert np.abs(np.asarray(got) - np.asarray(want)).max() < 2e-4, name

    monkeypatch.setattr(H, "assert_row_parity", tight)
    rows = [(s, h) for s in (0, 127, 128, 299, 300, 301, 700, 1099, 1100, 1499) for h in range(heads)]
    to = lambda x: torch.from_numpy(np.ascontiguousarray(x))
    R.check_query_rows(rows, tq, tk, tv, tdo, to(out), to(dq), mask, lay)
    R.check_key_rows(rows, tq, tk, tv, tdo, to(out), to(dk), to(dv), mask, lay)
    # grouped-query form: 2 query heads on 1 key/value head == the oracle on expanded K / V
    k1, v1 = k[:, :1], v[:, :1]
    kx, vx = np.repeat(k1, 2, axis=1), np.repeat(v1, 2, axis=1)
    out, dq, dk, dv = orc.moba_attn_varlen_oracle(q, kx, vx, cu, None, chunk, topk, "bf16", d_out=d_out)
    tk1, tv1 = (torch.from_numpy(np.ascontiguousarray(x)).to(torch.bfloat16) for x in (k1, v1))
    mask, gate = R.reference_selection(tq, tk1, lay, topk, rep=2)
    R.check_query_rows(rows, tq, tk1, tv1, tdo, to(out), to(dq), mask, lay, rep=2)
    R.check_key_rows([(s, 0) for s, _ in rows[::2]], tq, tk1, tv1, tdo, to(out), to(dk.sum(1, keepdims=True)),
                     to(dv.sum(1, keepdims=True)), mask, lay, rep=2)
