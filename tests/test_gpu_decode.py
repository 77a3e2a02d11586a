"""Decode-phase dense attention (moba_decode_attn behind moba_layer's q_len != kv_len branch, the stand-in for the
flash_attn_func call of moba/wrapper.py:76-82) against the CPU oracle, and both against flash_attn_func itself."""
import numpy as np
import pytest
import torch

from oracle import moba_oracle as orc
from tests import helpers as H
from tests.test_gpu_parity import TORCH_DT, t2n

pytestmark = pytest.mark.gpu


class _Causal(torch.nn.Module):
    is_causal = True


def _inputs(seed, B, Hq, Hkv, Lq, Lk, dtype, dev, spread=1.0):
    rng = np.random.RandomState(seed)
    q = orc.round_dtype((rng.randn(B, Hq, Lq, 128) * spread).astype(np.float32), dtype)
    k = orc.round_dtype(rng.randn(B, Hkv, Lk, 128).astype(np.float32), dtype)
    v = orc.round_dtype(rng.randn(B, Hkv, Lk, 128).astype(np.float32), dtype)
    return (q, k, v), tuple(torch.from_numpy(x).to(dev).to(TORCH_DT[dtype]) for x in (q, k, v))


@pytest.mark.parametrize("B,Hq,Hkv,Lq,Lk,dtype", [
    (1, 4, 1, 1, 1000, "bf16"),        # one new token, grouped heads, length not a multiple of the key tile
    (2, 8, 2, 1, 4096, "bf16"),
    (1, 32, 8, 1, 20000, "bf16"),      # a Llama-3.1-8B layer's head counts; several key ranges per head
    (2, 4, 4, 3, 517, "bf16"),         # a few positions at once: the causal mask inside the last keys
    (1, 8, 1, 5, 300, "f16"),          # 40 rows share one key/value head: three row blocks
    (1, 2, 2, 7, 7, "bf16"),           # q_len == kv_len handled too (plain causal attention)
    (3, 2, 1, 1, 1, "f16"),            # a single key
    (1, 4, 2, 2, 70000, "bf16"),       # long cache
])
def test_decode_matches_oracle(cuda_device, B, Hq, Hkv, Lq, Lk, dtype):
    from moba_b200 import ops

    (q, k, v), (tq, tk, tv) = _inputs(7, B, Hq, Hkv, Lq, Lk, dtype, cuda_device)
    scale = 128 ** -0.5
    got = t2n(ops.decode_attn(tq, tk, tv, scale))
    want = orc.decode_attention(q, k, v, scale, dtype)
    assert got.shape == (B, Lq, Hq, 128)
    H.assert_parity("out", got, want)


def test_decode_peaked_softmax_and_scale(cuda_device):
    """Large logits (a few keys dominate) and a caller-supplied scale."""
    from moba_b200 import ops

    (q, k, v), (tq, tk, tv) = _inputs(8, 1, 4, 2, 2, 3000, "bf16", cuda_device, spread=6.0)
    got = t2n(ops.decode_attn(tq, tk, tv, 0.2))
    want = orc.decode_attention(q, k, v, 0.2, "bf16")
    H.assert_parity("out", got, want)


def test_decode_strided_cache_views(cuda_device):
    """K / V as the first kv_len positions of a longer preallocated cache, q as a transposed view."""
    from moba_b200 import ops

    B, Hq, Hkv, Lq, Lk, cap = 2, 4, 2, 1, 777, 1024
    (q, k, v), (tq, tk, tv) = _inputs(9, B, Hq, Hkv, Lq, Lk, "bf16", cuda_device)
    cache_k = torch.zeros(B, Hkv, cap, 128, dtype=torch.bfloat16, device=cuda_device)
    cache_v = torch.full_like(cache_k, 3.0)
    cache_k[:, :, :Lk], cache_v[:, :, :Lk] = tk, tv
    q_view = tq.transpose(1, 2).contiguous().transpose(1, 2)          # [B, Lq, Hq, D] memory
    got = t2n(ops.decode_attn(q_view, cache_k[:, :, :Lk], cache_v[:, :, :Lk], 128 ** -0.5))
    H.assert_parity("out", got, orc.decode_attention(q, k, v, 128 ** -0.5, "bf16"))


def test_moba_layer_decode_branch_runs_the_kernel(cuda_device):
    from moba_b200 import MoBAConfig, moba_attn_varlen, moba_layer, ops

    (q, k, v), (tq, tk, tv) = _inputs(10, 2, 8, 2, 1, 2500, "bf16", cuda_device)
    rec = []
    ops.set_timing(rec)
    try:
        with torch.no_grad():
            out, w = moba_layer(moba_attn_varlen, MoBAConfig(512, 3), _Causal(), tq, tk, tv, scaling=128 ** -0.5)
    finally:
        ops.set_timing(None)
    assert w is None and [name for name, _, _ in rec] == ["decode_attn"]
    H.assert_parity("out", t2n(out), orc.decode_attention(q, k, v, 128 ** -0.5, "bf16"))


def test_decode_argument_errors(cuda_device):
    from moba_b200 import ops

    q = torch.zeros(1, 4, 2, 128, dtype=torch.bfloat16, device=cuda_device)
    k = torch.zeros(1, 3, 16, 128, dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(Exception):
        ops.decode_attn(q, k, k)                   # 3 key/value heads do not divide 4
    k1 = torch.zeros(1, 2, 1, 128, dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(Exception):
        ops.decode_attn(q, k1, k1)                 # fewer keys than query positions


@pytest.mark.parametrize("B,Hq,Hkv,Lq,Lk,dtype", [
    (1, 4, 1, 1, 1000, "bf16"), (2, 8, 2, 1, 4096, "bf16"), (2, 4, 4, 3, 517, "bf16"), (1, 8, 1, 5, 300, "f16"),
    (1, 2, 2, 7, 7, "bf16"), (1, 32, 8, 1, 20000, "bf16"),
])
def test_decode_oracle_and_kernel_against_flash_attn_func(cuda_device, B, Hq, Hkv, Lq, Lk, dtype):
    """Pins the decode branch to the call the reference makes there: flash_attn_func(query, key, value, dropout,
    scaling, True) on [batch, len, heads, dim] tensors (moba/wrapper.py:79-82), run here on the installed flash-attn.
    Both the numpy restatement (oracle.decode_attention) and the kernel are compared with its output. Skips when
    flash-attn cannot run on this GPU."""
    from moba_b200 import ops

    try:
        from flash_attn import flash_attn_func
    except ImportError:
        pytest.skip("flash-attn is not installed")
    (q, k, v), (tq, tk, tv) = _inputs(9, B, Hq, Hkv, Lq, Lk, dtype, cuda_device)
    scale = 128 ** -0.5
    try:
        ref = flash_attn_func(tq.transpose(1, 2), tk.transpose(1, 2), tv.transpose(1, 2), 0.0, scale, True)
        torch.cuda.synchronize()
    except RuntimeError as e:
        pytest.skip(f"flash-attn cannot run here: {str(e).splitlines()[0]}")
    ref = t2n(ref)                                                   # [B, Lq, Hq, 128]
    want = orc.decode_attention(q, k, v, scale, dtype)
    assert np.abs(want - ref).max() < 1e-2 and np.abs(want - ref).mean() < 5e-4      # the oracle restates that call
    got = t2n(ops.decode_attn(tq, tk, tv, scale))
    H.assert_parity("kernel vs flash_attn_func", got, ref)


@pytest.mark.parametrize("B,Hq,Hkv,Lq,Lk", [(2, 4, 2, 3, 517), (1, 8, 1, 1, 1000), (1, 2, 2, 7, 7), (1, 4, 4, 130, 400)])
def test_decode_branch_under_autograd_runs_on_the_kernels(cuda_device, monkeypatch, B, Hq, Hkv, Lq, Lk):
    """q_len != kv_len with gradients (moba/wrapper.py:76-82 is differentiable through flash_attn_func): the layer
    runs the attention tile kernels as two merged parts, no library attention; out and the gradients of query, key
    and value against an fp64 evaluation of bottom-right aligned causal attention."""
    from moba_b200 import MoBAConfig, check_kernel_status, moba_layer
    from moba_b200.wrapper import _decode_attention

    (q, k, v), (tq, tk, tv) = _inputs(11, B, Hq, Hkv, Lq, Lk, "bf16", cuda_device)
    tq, tk, tv = (t.requires_grad_() for t in (tq, tk, tv))

    def no_sdpa(*a, **kw):
        raise AssertionError("the decode branch fell back to torch's attention")

    monkeypatch.setattr(torch.nn.functional, "scaled_dot_product_attention", no_sdpa)
    if Lq != Lk:
        out, _ = moba_layer(None, MoBAConfig(64, 3), _Causal(), tq, tk, tv, scaling=128 ** -0.5)
    else:       # the layer treats q_len == kv_len as prefill; the decode function itself also covers it
        out = _decode_attention(tq, tk, tv, None)
    g = torch.Generator(device=cuda_device).manual_seed(3)
    d_out = torch.randn(out.shape, generator=g, device=cuda_device).to(torch.bfloat16)
    out.backward(d_out)
    check_kernel_status(cuda_device)
    assert out.shape == (B, Lq, Hq, 128)

    rq, rk, rv = (t.detach().double().requires_grad_() for t in (tq, tk, tv))
    rep = Hq // Hkv
    s = torch.einsum("bhqd,bhkd->bhqk", rq, rk.repeat_interleave(rep, 1)) * 128 ** -0.5
    mask = torch.arange(Lk, device=cuda_device)[None, :] <= (torch.arange(Lq, device=cuda_device)[:, None] + (Lk - Lq))
    ref = torch.einsum("bhqk,bhkd->bqhd", s.masked_fill(~mask, float("-inf")).softmax(-1), rv.repeat_interleave(rep, 1))
    ref.backward(d_out.double())
    H.assert_parity("out", t2n(out), ref.detach().float().cpu().numpy())
    for name, got, want in (("dq", tq.grad, rq.grad), ("dk", tk.grad, rk.grad), ("dv", tv.grad, rv.grad)):
        H.assert_parity(name, t2n(got) / rep ** 0.5, want.float().cpu().numpy() / rep ** 0.5)
