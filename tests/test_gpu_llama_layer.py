"""The HuggingFace attention-interface adapter on the GPU: moba_layer (mirror of moba/wrapper.py:29-84) with
grouped-query K / V handed to the kernels unexpanded, and a random-init Llama (the stand-in for
examples/llama.py, whose checkpoint needs a network) whose attention runs through register_moba."""
import numpy as np
import pytest
import torch

from oracle import moba_oracle as orc
from tests import helpers as H
from tests.test_gpu_grouped_query import assert_group_grad, expand, group_sum
from tests.test_gpu_parity import t2n, to_dev

pytestmark = pytest.mark.gpu


class _Causal(torch.nn.Module):
    is_causal = True


@pytest.mark.parametrize("batch,memory", [(1, "bhsd"), (2, "bshd"), (2, "bhsd")])
def test_moba_layer_prefill_grouped_kv(cuda_device, batch, memory):
    """[batch, heads, len, dim] tensors as HuggingFace passes them: `bshd` = transposed views of [batch, len,
    heads, dim] memory (the projections' layout), `bhsd` = contiguous (what a key/value cache returns)."""
    from moba_b200 import MoBAConfig, check_kernel_status, moba_attn_varlen, moba_layer

    S, heads, kv_heads, chunk, topk = 512, 4, 2, 128, 3
    q, d_out = H.make_inputs(51, batch * S, heads, n=2)
    k, v = H.make_inputs(52, batch * S, kv_heads, n=2)

    def hf(x):                       # [batch * S, h, D] -> [batch, h, S, D] in the requested memory layout
        t = to_dev(x, cuda_device).view(batch, S, x.shape[1], 128)
        t = t.transpose(1, 2).contiguous() if memory == "bhsd" else t.transpose(1, 2)
        return t.requires_grad_()

    tq, tk, tv = hf(q), hf(k), hf(v)
    out, weights = moba_layer(moba_attn_varlen, MoBAConfig(chunk, topk), _Causal(), tq, tk, tv)
    assert weights is None and out.shape == (batch * S, heads, 128)
    out.backward(to_dev(d_out, cuda_device))
    check_kernel_status(cuda_device)
    cu = [i * S for i in range(batch + 1)]
    want = orc.moba_attn_varlen_oracle(q, expand(k, 2), expand(v, 2), cu, None, chunk, topk, "bf16", d_out=d_out)

    def fa(g):                       # gradient [batch, h, S, D] -> [batch * S, h, D]
        return t2n(g.transpose(1, 2).reshape(batch * S, -1, 128))

    H.assert_parity("out", t2n(out), want[0])
    H.assert_parity("dq", fa(tq.grad), want[1])
    assert_group_grad("dk", fa(tk.grad), group_sum(want[2], 2), 2)
    assert_group_grad("dv", fa(tv.grad), group_sum(want[3], 2), 2)


def test_llama_random_init_through_register_moba(cuda_device):
    """A random-init Llama (4 query heads, 2 key/value heads, head_dim 128) with attn_implementation "moba". With
    top-k at least the number of chunks every query attends all of its past, so the logits and the parameter
    gradients must agree with the model's own dense causal attention."""
    from transformers import LlamaConfig, LlamaForCausalLM

    import moba_b200

    moba_b200.register_moba(moba_b200.MoBAConfig(64, 8))
    cfg = LlamaConfig(vocab_size=128, hidden_size=512, intermediate_size=256, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=512)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg).to(cuda_device).to(torch.bfloat16)
    ids = torch.randint(0, 128, (2, 256), device=cuda_device)

    def run(impl):
        model.config._attn_implementation = impl
        model.zero_grad(set_to_none=True)
        res = model(input_ids=ids, labels=ids)
        res.loss.backward()
        grads = {n: p.grad.detach().float().clone() for n, p in model.named_parameters() if "self_attn" in n}
        return res.logits.detach().float(), float(res.loss), grads

    logits_m, loss_m, grads_m = run("moba")
    moba_b200.check_kernel_status(cuda_device)
    logits_d, loss_d, grads_d = run("sdpa")
    assert np.isfinite(loss_m) and abs(loss_m - loss_d) < 2e-2
    torch.testing.assert_close(logits_m, logits_d, atol=5e-2, rtol=5e-2)
    for name, g in grads_m.items():
        ref = grads_d[name]
        assert torch.isfinite(g).all(), name
        assert (g - ref).abs().max() <= 5e-2 * max(float(ref.abs().max()), 1e-3) + 1e-4, name


def test_batched_layout_is_read_in_place(cuda_device, monkeypatch):
    """[batch, heads, len, dim]-contiguous tensors with batch > 1 (where the reference's hf_to_fa copies): the layer
    hands the kernels views of the caller's memory, and the result and the gradients are bit for bit those of the
    call on the copied [batch * len, heads, dim] tensors."""
    from moba_b200 import MoBAConfig, check_kernel_status, moba_attn_varlen, moba_efficient, moba_layer
    from moba_b200.wrapper import hf_to_fa

    B, S, heads, kv_heads, chunk, topk = 3, 640, 4, 2, 128, 3
    g = torch.Generator(device=cuda_device).manual_seed(5)
    query = torch.randn(B, heads, S, 128, generator=g, device=cuda_device).to(torch.bfloat16).requires_grad_()
    key = torch.randn(B, kv_heads, S, 128, generator=g, device=cuda_device).to(torch.bfloat16).requires_grad_()
    value = torch.randn(B, kv_heads, S, 128, generator=g, device=cuda_device).to(torch.bfloat16).requires_grad_()
    d_out = torch.randn(B * S, heads, 128, generator=g, device=cuda_device).to(torch.bfloat16)

    seen = []
    real_forward = moba_efficient._forward

    def spy(q, k, v, *a, **kw):
        seen.append((q.untyped_storage().data_ptr(), k.untyped_storage().data_ptr(), v.untyped_storage().data_ptr()))
        return real_forward(q, k, v, *a, **kw)

    monkeypatch.setattr(moba_efficient, "_forward", spy)
    out, _ = moba_layer(moba_attn_varlen, MoBAConfig(chunk, topk), _Causal(), query, key, value)
    out.backward(d_out)
    check_kernel_status(cuda_device)
    want_ptrs = (query.untyped_storage().data_ptr(), key.untyped_storage().data_ptr(), value.untyped_storage().data_ptr())
    assert len(seen) == B and all(p == want_ptrs for p in seen)          # the kernels saw the caller's memory
    monkeypatch.setattr(moba_efficient, "_forward", real_forward)

    q2, k2, v2 = (hf_to_fa(t.detach()).contiguous().requires_grad_() for t in (query, key, value))
    cu = torch.tensor([i * S for i in range(B + 1)], dtype=torch.int32, device=cuda_device)
    out2 = moba_attn_varlen(q2, k2, v2, cu, S, chunk, topk)
    out2.backward(d_out)
    check_kernel_status(cuda_device)
    assert torch.equal(out, out2)
    for got, ref in ((query.grad, q2.grad), (key.grad, k2.grad), (value.grad, v2.grad)):
        assert torch.equal(hf_to_fa(got), ref)
