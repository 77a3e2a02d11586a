"""HuggingFace attention-interface adapter (mirrors MoonshotAI/MoBA moba/wrapper.py:7-84)."""
from typing import Callable, Optional, Tuple

import torch

from .config import MoBAConfig


def hf_to_fa(x: torch.Tensor):
    """[batch, heads, seqlen, head_dim] -> [batch * seqlen, heads, head_dim] (moba/wrapper.py:7-15)."""
    return x.permute(0, 2, 1, 3).reshape(-1, x.shape[1], x.shape[3])


def _reshape_is_view(x: torch.Tensor) -> bool:
    """Whether hf_to_fa(x) is a view of x (no copy): true for transposed views of [batch, len, heads, dim] memory."""
    b, h, s, d = x.shape
    st = x.permute(0, 2, 1, 3).stride()                 # strides of [batch, len, heads, dim]
    return b == 1 or st[0] == s * st[1]                 # batch and len merge into one dimension


def fa_to_hf(x: torch.Tensor, batch: int):
    """[batch * seqlen, heads, head_dim] -> [batch, heads, seqlen, head_dim] (moba/wrapper.py:18-26)."""
    return x.view(batch, -1, x.shape[1], x.shape[2]).permute(0, 2, 1, 3)


_CU_CACHE = {}


def _cu_seqlens(batch, kv_len, device):
    """cumsum([0] + [kv_len] * batch) as an int32 tensor on `device` (moba/wrapper.py:62-66), made once per
    (batch, kv_len, device): every layer of a model then hands the same tensor to the attention call, whose plan
    cache works by tensor identity, and the host values are registered with it so that planning never reads the
    device tensor back."""
    key = (int(batch), int(kv_len), str(device))
    t = _CU_CACHE.get(key)
    if t is None:
        values = [i * int(kv_len) for i in range(int(batch) + 1)]
        t = torch.tensor(values, dtype=torch.int32, device=device)
        if t.is_cuda:
            from . import ops

            ops.register_cu_seqlens(t, values)
        if len(_CU_CACHE) >= 64:
            _CU_CACHE.clear()
        _CU_CACHE[key] = t
    return t


def _decode_attention(query, key, value, scaling):
    """Dense causal attention for the decode phase (q_len != kv_len), bottom-right aligned as the reference's
    flash_attn_func(..., causal=True) call (moba/wrapper.py:76-82); returns [batch, q_len, heads, dim].

    16-bit CUDA tensors with head_dim 128 that need no gradient run the library's decode kernel
    (moba_decode_attn: K / V streamed once, grouped-query heads sharing the tiles); with gradients (and the default
    scale) the attention tile kernels run it as two merged parts (_decode_attention_autograd). Anything else --
    other head dims, fp32, CPU tensors, a caller-chosen scale under autograd -- is outside what the kernels cover
    and goes through torch's scaled-dot-product attention."""
    b, hq, lq, d = query.shape
    hkv, lk = key.shape[1], key.shape[2]
    needs_grad = torch.is_grad_enabled() and (query.requires_grad or key.requires_grad or value.requires_grad)
    kernel_ok = (query.is_cuda and d == 128 and lk >= lq and query.dtype in (torch.bfloat16, torch.float16)
                 and key.dtype == query.dtype and value.dtype == query.dtype)
    if kernel_ok and not needs_grad:
        from . import ops
        from .moba_efficient import _status_word

        return ops.decode_attn(query, key, value, scaling, status=_status_word(query.device))
    if kernel_ok and hq % hkv == 0 and (scaling is None or abs(float(scaling) - d ** -0.5) < 1e-7):
        return _decode_attention_autograd(query, key, value)
    if lk < lq:
        raise ValueError(f"decode needs kv_len >= q_len (got q_len {lq}, kv_len {lk}): the causal mask is aligned to "
                         "the end of the keys, so earlier query positions would see no key at all")
    qi = torch.arange(lq, device=query.device)[:, None] + (lk - lq)
    ki = torch.arange(lk, device=query.device)[None, :]
    mask = ki <= qi
    out = torch.nn.functional.scaled_dot_product_attention(query, key, value, attn_mask=mask, scale=scaling,
                                                           enable_gqa=hkv != hq)
    return out.transpose(1, 2)


def _decode_attention_autograd(query, key, value):
    """The decode step with gradients, on the attention tile kernels (no library attention): bottom-right aligned
    causal attention of q_len positions over kv_len keys is the two-part attention MixedAttention computes --
    part 1, causal attention of the queries over the last q_len keys; part 2, full attention of the same queries over
    the kv_len - q_len keys before them, one (batch, query head) pair per key/value segment -- merged by their
    log-sum-exps. The operands are cut and regrouped with differentiable torch ops, so the gradients reach query,
    key and value through autograd. Returns [batch, q_len, q_heads, dim] like the inference kernel."""
    from .moba_efficient import MixedAttention

    b, hq, lq, d = query.shape
    hkv, lk = key.shape[1], key.shape[2]
    rep, dev = hq // hkv, query.device
    q1 = query.permute(0, 2, 1, 3).reshape(b * lq, hq, d)                                   # tokens (batch, l)
    k_tail = key[:, :, lk - lq:].repeat_interleave(rep, dim=1) if rep > 1 else key[:, :, lk - lq:]
    v_tail = value[:, :, lk - lq:].repeat_interleave(rep, dim=1) if rep > 1 else value[:, :, lk - lq:]
    k1 = k_tail.permute(0, 2, 1, 3).reshape(b * lq, hq, d)
    v1 = v_tail.permute(0, 2, 1, 3).reshape(b * lq, hq, d)
    cu_self = torch.arange(b + 1, device=dev, dtype=torch.int32) * lq
    n_pre = lk - lq
    e = b * hq                                                                              # (batch, head) segments
    if n_pre > 0:
        moba_q = query.reshape(e * lq, 1, d)                                                # rows (batch, head, l)
        k_pre = key[:, :, :n_pre].repeat_interleave(rep, dim=1) if rep > 1 else key[:, :, :n_pre]
        v_pre = value[:, :, :n_pre].repeat_interleave(rep, dim=1) if rep > 1 else value[:, :, :n_pre]
        moba_kv = torch.stack((k_pre.reshape(e * n_pre, 1, d), v_pre.reshape(e * n_pre, 1, d)), dim=1)
        cu_q = torch.arange(e + 1, device=dev, dtype=torch.int32) * lq
        cu_kv = torch.arange(e + 1, device=dev, dtype=torch.int32) * n_pre
        bi = torch.arange(b, device=dev).view(b, 1, 1)
        hi = torch.arange(hq, device=dev).view(1, hq, 1)
        li = torch.arange(lq, device=dev).view(1, 1, lq)
        sh = ((bi * lq + li) * hq + hi).reshape(-1)                                         # target (token, head) row
    else:
        moba_q = query.new_zeros((0, 1, d))
        moba_kv = query.new_zeros((0, 2, 1, d))
        cu_q = cu_kv = torch.zeros(1, device=dev, dtype=torch.int32)
        sh = torch.zeros(0, device=dev, dtype=torch.int64)
    out = MixedAttention.apply(q1.contiguous(), k1.contiguous(), v1.contiguous(), cu_self, moba_q.contiguous(),
                               moba_kv, cu_q, cu_kv, lq, max(n_pre, 1), sh)
    return out.view(b, lq, hq, d)


def moba_layer(
    moba_impl: Callable,
    moba_config: MoBAConfig,
    module: torch.nn.Module,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    *args,
    dropout: float = 0.0,
    scaling: Optional[float] = None,
    **kwargs,
) -> Tuple[torch.Tensor, None]:
    """
    Args:
        query (torch.Tensor): [batch, q_heads, q_len, head_dim]
        key (torch.Tensor): [batch, kv_heads, kv_len, head_dim]
        value (torch.Tensor): [batch, kv_heads, kv_len, head_dim]

    Returns:
        attn_output (torch.Tensor): [batch * q_len, q_heads, head_dim] in prefill (the reference leaves this
            layout, moba/wrapper.py:83), [batch, q_len, q_heads, head_dim] in decode
        attn_weights (None): not needed
    """
    assert module.is_causal
    batch, q_heads, q_len, head_dim = query.shape
    _, kv_heads, kv_len, _ = key.shape
    if q_len == kv_len:
        # prefill phase: as the reference, `scaling` and the attention mask are not used here.
        # hf_to_fa is a view (no copy) when the tensors are transposed views of [batch, len, heads, dim] memory,
        # which is what the HuggingFace Llama attention passes (modeling_llama.py projects to [batch, len,
        # heads * dim] and transposes), and for batch 1 in any layout; any other layout is read in place per sequence.
        if batch > 1 and head_dim == 128 and getattr(moba_impl, "supports_grouped_kv", False) and not all(
                _reshape_is_view(t) for t in (query, key, value)):
            # [batch, heads, len, dim]-contiguous memory (a key/value cache): hf_to_fa would copy all three tensors.
            # This package's implementation reads them in place, one call per sequence (moba_attn_batched).
            from .moba_efficient import moba_attn_batched

            return moba_attn_batched(query, key, value, moba_config.moba_chunk_size, moba_config.moba_topk), None
        query = hf_to_fa(query)
        key = hf_to_fa(key)
        value = hf_to_fa(value)
        if not getattr(moba_impl, "supports_grouped_kv", False):
            # moba/wrapper.py:59-61: expand K / V to the query head count for implementations that need it
            kv_replicas = q_heads // kv_heads
            key = torch.repeat_interleave(key, kv_replicas, dim=1)
            value = torch.repeat_interleave(value, kv_replicas, dim=1)
        cu_seqlens_k = _cu_seqlens(batch, kv_len, query.device)
        out = moba_impl(
            q=query,
            k=key,
            v=value,
            cu_seqlens=cu_seqlens_k,
            max_seqlen=kv_len,
            moba_chunk_size=moba_config.moba_chunk_size,
            moba_topk=moba_config.moba_topk,
        )
    else:
        out = _decode_attention(query, key, value, scaling)
    return out, None
