"""Failure paths of the kernels, exercised without faulting or hanging the GPU: a bounded wait that runs out is
reported through the status word and leaves the context usable; an index buffer with an out-of-range entry is
skipped and reported, not dereferenced."""
import numpy as np
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_is_reported(cuda_device):
    from moba_b200 import _lib, ops

    status = ops.new_status(cuda_device)
    ops.check_status(status)                                       # clean word: no error
    ops.selftest_wait_timeout(status, limit_ns=1_000_000, n_ctas=8)
    with pytest.raises(_lib.MobaError) as err:
        ops.check_status(status)
    assert err.value.code == -4                                    # MOBA_ERR_DEVICE
    assert int(status.item()) == 1                                 # 1 = a bounded wait expired
    # the context is still healthy and the tensor memory was released: a kernel that allocates all 512 columns
    # per SM (the backward tiles) and a tile product run right after it
    status.zero_()
    a = torch.randn(128, 128, device=cuda_device).to(torch.bfloat16)
    b = torch.randn(128, 128, device=cuda_device).to(torch.bfloat16)
    c = ops.selftest_umma(0, a, b)
    assert (c - a.float() @ b.float().T).abs().max().item() < 1e-3
    from moba_b200.moba_efficient import check_kernel_status, moba_attn_varlen

    q, k, v, d_out = (torch.from_numpy(x).to(cuda_device).to(torch.bfloat16) for x in H.make_inputs(5, 1024, 2))
    q.requires_grad_()
    out = moba_attn_varlen(q, k, v, torch.tensor([0, 1024], dtype=torch.int32, device=cuda_device), 1024, 128, 3)
    out.backward(d_out)
    check_kernel_status(cuda_device)
    assert torch.isfinite(q.grad.float()).all()


def test_out_of_range_selection_is_skipped_and_reported(cuda_device):
    """A sel buffer holding a chunk id that is not a candidate of its query (the gate never writes one) must not
    be used as an index: the slot counts as empty and the status word becomes 2."""
    from moba_b200 import _lib, ops

    S, heads, chunk, topk = 1024, 2, 128, 3
    (q, k) = (torch.from_numpy(x).to(cuda_device).to(torch.bfloat16) for x in H.make_inputs(6, S, heads, n=2))
    plan = ops.get_plan([0, S], chunk, topk, cuda_device)
    sel, _, tile_cnt = ops.gate_topk(q, ops.pool_keys(k, plan), plan)
    good = ops.build_lists(plan, heads, sel.clone(), tile_cnt.clone())
    bad = sel.clone()
    bad[700, 1, 0] = 1_000_000                                     # far outside the chunk table
    bad[900, 0, 1] = 7                                             # own chunk of token 900: not a candidate
    status = ops.new_status(cuda_device)
    list_off, work_off, list_tok, row_of = ops.build_lists(plan, heads, bad, tile_cnt.clone(), status=status)
    with pytest.raises(_lib.MobaError):
        ops.check_status(status)
    assert int(status.item()) == 2
    assert int(row_of[700, 1, 0]) == -1 and int(row_of[900, 0, 1]) == -1
    # untouched slots keep rows inside the row space
    keep = torch.ones_like(row_of, dtype=torch.bool)
    keep[700, 1, 0] = keep[900, 0, 1] = False
    r = row_of[keep & (bad >= 0)]
    assert int(r.min()) >= 0 and int(r.max()) < plan.rows_total(heads)
    assert good[0].shape == list_off.shape
