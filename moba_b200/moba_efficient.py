"""Drop-in for MoonshotAI/MoBA ``moba/moba_efficient.py``: same names, same argument meaning.

``moba_attn_varlen(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk)`` is the public entry
(moba/moba_efficient.py:270-278). All device work happens in libmoba_b200.so (sm_100a kernels); torch only
owns the buffers. There is no flash-attn dependency and no CPU path.
"""
import torch

from . import ops

_STATUS = {}


def _status_word(device):
    """Per-device error word in pinned host memory that kernels write through its device mapping when a
    bounded wait expires. Reading it costs no synchronisation, so it is checked at the start of every
    call (an error therefore surfaces at the next call, or at `check_kernel_status()`)."""
    key = torch.device(device).index or 0
    if key not in _STATUS:
        _STATUS[key] = torch.zeros(1, dtype=torch.int32, pin_memory=True)
    st = _STATUS[key]
    code = int(st[0])
    if code != 0:
        st[0] = 0
        raise RuntimeError(f"a moba_b200 kernel reported status {code} (1 = bounded wait expired, 2 = bad index)")
    return st


def check_kernel_status(device=None):
    """Synchronise `device` and raise if any kernel launched so far reported an error."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    torch.cuda.synchronize(device)
    _status_word(device)


def calc_chunks(cu_seqlen, moba_chunk_size):
    """Chunk metadata, as the reference's calc_chunks returns it (moba/moba_efficient.py:14-64):
    (cu_chunk int32 [n+1], filtered_chunk_indices int64 [F], num_filtered_chunk, chunk_to_batch int32 [n]).
    The tensors live on cu_seqlen's device."""
    plan = ops.get_plan(cu_seqlen, moba_chunk_size, 2, cu_seqlen.device if cu_seqlen.is_cuda else "cpu")
    dev = cu_seqlen.device
    cu_chunk = plan.table("chunk_start").to(torch.int32).to(dev)
    first = plan.table("chunk_seq_first")
    last = plan.table("chunk_seq_last")
    idx = torch.arange(plan.info.n_chunks)
    filtered = idx[idx != last.to(torch.int64)].to(torch.int64).to(dev)
    seq_first_sorted = torch.unique(first)
    chunk_to_batch = (torch.searchsorted(seq_first_sorted, first, right=True) - 1).to(torch.int32)
    # sequences of length zero own no chunk; count them so batch indices stay those of cu_seqlens
    lens = torch.tensor(plan.cu_host[1:]) - torch.tensor(plan.cu_host[:-1])
    nonempty = torch.nonzero(lens > 0).flatten()
    chunk_to_batch = nonempty[chunk_to_batch.long()].to(torch.int32).to(dev) if len(nonempty) else chunk_to_batch.to(dev)
    return cu_chunk, filtered, int(filtered.numel()), chunk_to_batch


class _Context:
    """What forward keeps for backward: the plan, the query lists and the merged softmax statistics."""

    __slots__ = ("plan", "lists", "row_of", "lse", "gate_dtype", "scale")


def _compute_dtype(t):
    return t.dtype if t.dtype in (torch.bfloat16, torch.float16) else torch.bfloat16


def _as_compute(t):
    dt = _compute_dtype(t)
    t = t if t.dtype == dt else t.to(dt)
    return t if (t.stride(2) == 1 and t.stride(1) % 8 == 0 and t.stride(0) % 8 == 0) else t.contiguous()


def _share_strides(q, k, v):
    """k and v always share strides; q shares them too unless k / v carry fewer heads (grouped-query)."""
    if k.shape[1] != q.shape[1]:
        return (q, k, v) if v.stride() == k.stride() else (q, k.contiguous(), v.contiguous())
    if k.stride() == q.stride() and v.stride() == q.stride():
        return q, k, v
    return q.contiguous(), k.contiguous(), v.contiguous()


def _forward(q, k, v, cu_seqlens, moba_chunk_size, moba_topk, out=None, scale=0.0):
    """Runs pool -> gate/top-k -> lists -> attention tiles -> merge. Returns (out in q.dtype, context). `out`:
    optional contiguous [S, H, D] buffer of the compute dtype that receives the result; `scale`: softmax scale
    (0 = 128^-0.5; tensors of a smaller head dim arrive zero-padded to 128 columns with their own head_dim^-0.5)."""
    if k.shape != v.shape or k.shape[0] != q.shape[0] or k.shape[2] != q.shape[2] or k.shape[1] < 1 \
            or q.shape[1] % k.shape[1] != 0:
        raise ValueError("k and v must have the shape of q, or the same shape with a head count that divides "
                         f"q's; got {tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    if q.dtype != k.dtype or q.dtype != v.dtype:
        raise ValueError("q, k, v must have the same dtype")
    if moba_topk < 1 or moba_chunk_size < 1:
        raise ValueError("moba_topk and moba_chunk_size must be >= 1")
    dev = q.device
    status = _status_word(dev)
    plan = ops.get_plan(cu_seqlens, moba_chunk_size, moba_topk, dev)
    if plan.info.total_tokens != q.shape[0]:
        raise ValueError(f"cu_seqlens ends at {plan.info.total_tokens} but q has {q.shape[0]} tokens")
    H = q.shape[1]
    ctx = _Context()
    ctx.gate_dtype = q.dtype
    lists, row_of = (None, None, None), None
    if plan.kk > 0:
        # gate in the caller's dtype: the pooled key is rounded to it (moba/moba_efficient.py:335-340)
        qg = q if q.stride(2) == 1 else q.contiguous()
        kg = k if k.stride(2) == 1 else k.contiguous()
        kmean = ops.pool_keys(kg, plan)
        sel, _, tile_cnt = ops.gate_topk(qg, kmean, plan, status=status)
        list_off, work_off, list_tok, row_of = ops.build_lists(plan, H, sel, tile_cnt, status=status)
        lists = (list_off, work_off, list_tok, ops.tile_records(plan, H, list_off, work_off))
    else:
        # moba_topk == 1 or every sequence is a single chunk: plain causal attention over whole sequences
        # (moba/moba_efficient.py:314-321) = self-chunk attention with one chunk per sequence
        longest = max((b - a for a, b in zip(plan.cu_host, plan.cu_host[1:])), default=1)
        plan = ops.Plan(plan.cu_host, max(longest, 1), 1, dev)
    qc, kc, vc = _share_strides(_as_compute(q), _as_compute(k), _as_compute(v))
    out, lse, part_o, part_lse = ops.attn_fwd(qc, kc, vc, plan, lists, status, out=out, scale=scale)
    if plan.kk > 0:
        ops.merge_fwd(out, lse, plan, part_o, part_lse, row_of)
    ctx.plan, ctx.lists, ctx.row_of, ctx.lse, ctx.scale = plan, lists, row_of, lse, scale
    return out, (qc, kc, vc), ctx


def _backward(qc, kc, vc, out, d_out, ctx, grads_out=None):
    """dq, dk, dv in the compute dtype. No gradient flows through the selection
    (moba/moba_efficient.py:365-371 uses indices / booleans only). `grads_out`: optional contiguous (dq [S,H,D],
    dk, dv [S,H_kv,D]) buffers that receive the gradients."""
    status = _status_word(qc.device)
    plan = ctx.plan
    d_out = d_out if d_out.dtype == out.dtype else d_out.to(out.dtype)
    d_out = d_out.contiguous()
    delta = ops.bwd_delta(out, d_out)
    if d_out.stride() != qc.stride():
        # the tile kernels read d_out through q's strides: one strided copy of d_out, not three of q / k / v
        d_out = torch.empty_strided(qc.shape, qc.stride(), dtype=d_out.dtype, device=d_out.device).copy_(d_out)
    # the rows every (chunk, head) list names, copied into list order once for both backward kernels
    gathered = ops.gather_rows(qc, d_out, plan, ctx.lists, ctx.lse, delta) if plan.kk > 0 else (None,) * 4
    dk, dv = ops.attn_bwd_dkdv(qc, kc, vc, d_out, plan, ctx.lists, ctx.lse, delta, status, gathered=gathered,
                               out=grads_out[1:] if grads_out else None, scale=ctx.scale)
    dq_self, part_dq = ops.attn_bwd_dq(qc, kc, vc, d_out, plan, ctx.lists, ctx.lse, delta, status, gathered=gathered,
                                       scale=ctx.scale)
    dq = ops.merge_dq(dq_self, plan, part_dq, ctx.row_of, qc.dtype, out=grads_out[0] if grads_out else None)
    return dq, dk, dv


class _MobaAttnFunction(torch.autograd.Function):
    """Fused autograd function behind moba_attn_varlen: never materialises gathered Q or regrouped KV."""

    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, moba_chunk_size, moba_topk):
        D = q.shape[2]
        if D > ops._lib.HEAD_DIM or D % 8 != 0 or D < 8:
            raise ValueError(f"head_dim {D} is not supported: the kernels take a multiple of 8 up to {ops._lib.HEAD_DIM}")
        scale = 0.0
        if D < ops._lib.HEAD_DIM:
            # the tiles are 128 columns wide: zero columns change neither q . k nor the pooled keys' scores, and the
            # extra columns of v only produce zero columns of the result; the scale stays that of the real head dim
            pad = (0, ops._lib.HEAD_DIM - D)
            q, k, v = (torch.nn.functional.pad(t, pad) for t in (q, k, v))
            scale = D ** -0.5
        out, (qc, kc, vc), c = _forward(q, k, v, cu_seqlens, moba_chunk_size, moba_topk, scale=scale)
        ctx.save_for_backward(qc, kc, vc, out)
        ctx.moba = c
        ctx.in_dtype = q.dtype
        ctx.head_dim = D
        if D < ops._lib.HEAD_DIM:
            out = out[:, :, :D].contiguous()
        return out if out.dtype == q.dtype else out.to(q.dtype)

    @staticmethod
    def backward(ctx, d_out):
        qc, kc, vc, out = ctx.saved_tensors
        D = ctx.head_dim
        if D < ops._lib.HEAD_DIM:
            d_out = torch.nn.functional.pad(d_out, (0, ops._lib.HEAD_DIM - D))
        dq, dk, dv = _backward(qc, kc, vc, out, d_out, ctx.moba)
        if D < ops._lib.HEAD_DIM:
            dq, dk, dv = (g[:, :, :D].contiguous() for g in (dq, dk, dv))
        if ctx.in_dtype != dq.dtype:
            dq, dk, dv = dq.to(ctx.in_dtype), dk.to(ctx.in_dtype), dv.to(ctx.in_dtype)
        return dq, dk, dv, None, None, None


class _MobaLayerFunction(torch.autograd.Function):
    """moba_attn_varlen for a batch of equal-length sequences in the memory layout HuggingFace hands to an attention
    function, [batch, heads, len, dim] (contiguous: what a key/value cache returns), without the permute + reshape
    copies of moba/wrapper.py:56-58: sequences are independent in MoBA, so every batch element is one call on
    [len, heads, dim] views of the caller's tensors (strides dim and len * dim), writing straight into the packed
    [batch * len, heads, dim] output; the gradients land in [batch, len, heads, dim] buffers that are returned as
    [batch, heads, len, dim] views."""

    @staticmethod
    def forward(ctx, query, key, value, moba_chunk_size, moba_topk):
        B, H, S, D = query.shape
        Hkv = key.shape[1]
        dt = _compute_dtype(query)
        out = torch.empty((B * S, H, D), dtype=dt, device=query.device)
        cu = [0, S]
        saved, ctxs = [], []
        for b in range(B):
            o, (qc, kc, vc), c = _forward(query[b].transpose(0, 1), key[b].transpose(0, 1), value[b].transpose(0, 1),
                                          cu, moba_chunk_size, moba_topk, out=out[b * S:(b + 1) * S])
            saved += [qc, kc, vc]
            ctxs.append(c)
        ctx.save_for_backward(out, *saved)
        ctx.moba = ctxs
        ctx.shape = (B, H, Hkv, S, D)
        ctx.in_dtype = query.dtype
        return out if dt == query.dtype else out.to(query.dtype)

    @staticmethod
    def backward(ctx, d_out):
        out, *saved = ctx.saved_tensors
        B, H, Hkv, S, D = ctx.shape
        dq = torch.empty((B, S, H, D), dtype=out.dtype, device=out.device)
        dk = torch.empty((B, S, Hkv, D), dtype=out.dtype, device=out.device)
        dv = torch.empty((B, S, Hkv, D), dtype=out.dtype, device=out.device)
        for b in range(B):
            qc, kc, vc = saved[3 * b:3 * b + 3]
            _backward(qc, kc, vc, out[b * S:(b + 1) * S], d_out[b * S:(b + 1) * S], ctx.moba[b],
                      grads_out=(dq[b], dk[b], dv[b]))
        grads = [g.permute(0, 2, 1, 3) for g in (dq, dk, dv)]
        if ctx.in_dtype != out.dtype:
            grads = [g.to(ctx.in_dtype) for g in grads]
        return grads[0], grads[1], grads[2], None, None


def moba_attn_batched(query, key, value, moba_chunk_size, moba_topk):
    """MoBA attention of [batch, heads, len, dim] tensors (equal-length sequences, grouped-query key / value heads
    allowed) -> [batch * len, heads, dim], reading the tensors in place whatever their strides (innermost stride 1).
    Used by moba_layer when the reference's hf_to_fa reshape would have to copy."""
    for name, t in (("query", query), ("key", key), ("value", value)):
        if not isinstance(t, torch.Tensor) or t.dim() != 4:
            raise ValueError(f"{name} must be a [batch, heads, len, head_dim] tensor")
        if not t.is_cuda:
            raise RuntimeError(f"{name} is on {t.device}: moba_b200 runs on CUDA (sm_100a) only and has no CPU fallback")
    return _MobaLayerFunction.apply(query, key, value, int(moba_chunk_size), int(moba_topk))


def _host_list(t):
    return [int(x) for x in (t.detach().cpu().tolist() if isinstance(t, torch.Tensor) else t)]


def _one_chunk_plan(cu_host, dev, what):
    """Plan in which every segment of cu_host is one chunk of one sequence."""
    lens = [b - a for a, b in zip(cu_host, cu_host[1:])]
    if any(n <= 0 for n in lens):
        raise ValueError(f"{what} holds an empty or negative-length segment")
    return ops.Plan(cu_host, max(lens, default=1), 1, dev)


class MixedAttention(torch.autograd.Function):
    """The reference's two-part attention on operands the caller has already gathered
    (moba/moba_efficient.py:67-267), with the same eleven arguments and the same gradients
    (dq, dk, dv, None, d_moba_q, d_moba_kv, None x 5):

    * part 1: causal attention of q over k, v inside each segment of self_attn_cu_seqlen;
    * part 2: full attention of moba_q rows [cu_q[e], cu_q[e+1]) over moba_kv rows [cu_kv[e], cu_kv[e+1]);
    * row i of part 2 is merged into row moba_q_sh_indices[i] of the flattened [S*H] part-1 result by the
      log-sum-exp rule; backward runs both parts with the merged out / lse.

    moba_attn_varlen does not go through this class (it never materialises moba_q / moba_kv); the class is for
    callers that built those tensors themselves. It runs the same tile kernels: part 1 as the own-chunk launch,
    part 2 as the list launch over a one-head view in which every kv segment is a chunk and the query lists are
    the identity. A flattened row may be the target of at most 32 part-2 rows. max_seqlen and moba_chunk_size
    are launch hints in the reference and unused here. The three cu_seqlen tensors are read on the host."""

    @staticmethod
    def forward(ctx, q, k, v, self_attn_cu_seqlen, moba_q, moba_kv, moba_cu_seqlen_q, moba_cu_seqlen_kv,
                max_seqlen, moba_chunk_size, moba_q_sh_indices):
        del max_seqlen, moba_chunk_size
        if not q.is_cuda:
            raise RuntimeError("MixedAttention runs on CUDA (sm_100a) only and has no CPU fallback")
        if q.dtype not in (torch.bfloat16, torch.float16):
            raise ValueError("MixedAttention takes bf16 / fp16 tensors, as the flash kernels it replaces do")
        S, H, D = q.shape
        dev = q.device
        status = _status_word(dev)
        none3 = (None, None, None)
        # ---- part 1
        plan_self = _one_chunk_plan(_host_list(self_attn_cu_seqlen), dev, "self_attn_cu_seqlen")
        if plan_self.info.total_tokens != S:
            raise ValueError(f"self_attn_cu_seqlen ends at {plan_self.info.total_tokens} but q has {S} tokens")
        qc, kc, vc = _share_strides(_as_compute(q), _as_compute(k), _as_compute(v))
        out, lse, _, _ = ops.attn_fwd(qc, kc, vc, plan_self, none3, status, parts=1)
        # ---- part 2
        R = moba_q.shape[0]
        idx = moba_q_sh_indices.to(torch.int64)
        mq = moba_q.reshape(R, 1, D).contiguous()
        mk = moba_kv[:, 0].reshape(-1, 1, D).contiguous()
        mv = moba_kv[:, 1].reshape(-1, 1, D).contiguous()
        g = None
        if R > 0:
            cu_q, cu_kv = _host_list(moba_cu_seqlen_q), _host_list(moba_cu_seqlen_kv)
            if len(cu_q) != len(cu_kv) or cu_q[-1] != R or cu_kv[-1] != mk.shape[0] or idx.numel() != R:
                raise ValueError("moba_cu_seqlen_q / moba_cu_seqlen_kv / moba_q_sh_indices do not match moba_q / moba_kv")
            base = _one_chunk_plan(cu_kv, dev, "moba_cu_seqlen_kv")
            tiles = [0]
            for a, b in zip(cu_q, cu_q[1:]):
                if b < a:
                    raise ValueError("moba_cu_seqlen_q must not decrease")
                tiles.append(tiles[-1] + (b - a + 127) // 128)
            view = ops.PlanView(base, 1, R, tiles[-1])
            lists = (torch.tensor(cu_q, dtype=torch.int32, device=dev),
                     torch.tensor(tiles, dtype=torch.int32, device=dev),
                     torch.arange(R, dtype=torch.int32, device=dev))
            _, _, part_o, part_lse = ops.attn_fwd(mq, mk, mv, view, lists, status, parts=2)
            # slots of every flattened (token, head) row: the part-2 rows that merge into it, -1 = none
            counts = torch.bincount(idx, minlength=S * H)
            kmax = int(counts.max())
            if kmax > 32:
                raise ValueError(f"a row is the target of {kmax} moba_q rows; at most 32 are supported")
            order = torch.argsort(idx, stable=True)
            sorted_idx = idx[order]
            rank = torch.arange(R, device=dev) - (torch.cumsum(counts, 0) - counts)[sorted_idx]
            row_of = torch.full((S * H, kmax), -1, dtype=torch.int32, device=dev)
            row_of[sorted_idx, rank] = order.to(torch.int32)
            merge_view = ops.PlanView(plan_self, kmax, R, 0)
            ops.merge_fwd(out, lse, merge_view, part_o, part_lse, row_of)
            g = (view, lists)
        ctx.save_for_backward(out, lse, qc, kc, vc, mq, mk, mv, idx)
        ctx.moba = (plan_self, g)
        return out

    @staticmethod
    def backward(ctx, d_output):
        out, lse, qc, kc, vc, mq, mk, mv, idx = ctx.saved_tensors
        plan_self, g = ctx.moba
        S, H, D = out.shape
        status = _status_word(out.device)
        none3 = (None, None, None)
        d_out = (d_output if d_output.dtype == out.dtype else d_output.to(out.dtype)).contiguous()
        if d_out.stride() != qc.stride():
            qc, kc, vc = qc.contiguous(), kc.contiguous(), vc.contiguous()
        delta = ops.bwd_delta(out, d_out)
        dk, dv = ops.attn_bwd_dkdv(qc, kc, vc, d_out, plan_self, none3, lse, delta, status, parts=1)
        dq_self, _ = ops.attn_bwd_dq(qc, kc, vc, d_out, plan_self, none3, lse, delta, status, parts=1)
        dq = dq_self.to(out.dtype)
        R = mq.shape[0]
        if g is None:
            dmq = torch.zeros_like(mq)
            dmkv = torch.zeros((mk.shape[0], 2, 1, D), dtype=out.dtype, device=out.device)
            return dq, dk, dv, None, dmq, dmkv, None, None, None, None, None
        view, lists = g
        # merged statistics of the rows part 2 came from, in part-2 row order
        dog = d_out.view(-1, D).index_select(0, idx)
        lse_g = lse.view(-1).index_select(0, idx)
        delta_g = delta.view(-1).index_select(0, idx)
        do3, lse2, delta2 = dog.view(R, 1, D), lse_g.view(R, 1), delta_g.view(R, 1)
        rows = (mq.view(R, D), dog, lse_g, delta_g)
        dmk, dmv = ops.attn_bwd_dkdv(mq, mk, mv, do3, view, lists, lse2, delta2, status, parts=2, gathered=rows)
        _, part_dq = ops.attn_bwd_dq(mq, mk, mv, do3, view, lists, lse2, delta2, status, parts=2, gathered=rows)
        dmq = part_dq.to(out.dtype).view(R, 1, D)
        dmkv = torch.stack((dmk, dmv), dim=1)
        return dq, dk, dv, None, dmq, dmkv, None, None, None, None, None


def moba_attn_varlen(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cu_seqlens: torch.Tensor,
    max_seqlen: int,
    moba_chunk_size: int,
    moba_topk: int,
) -> torch.Tensor:
    """MoBA attention over packed variable-length sequences (signature of moba/moba_efficient.py:270-278).

    Args:
        q, k, v: [seqlen, head, head_dim] CUDA tensors, bf16 / fp16 (fp32 is accepted: the gate runs on the fp32
            values, the attention tiles on a bf16 copy). head_dim 128 is the native tile width; a smaller head_dim
            (a multiple of 8) runs on zero-padded copies with its own head_dim^-0.5, so 64 costs what 128 does. Beyond the reference, k and v may
            carry fewer heads than q (grouped-query attention, at most 16 query heads per key/value head): query
            head h then reads key/value head h // (heads of q // heads of k), the result equals the call with
            k.repeat_interleave(...) / v.repeat_interleave(...) (what moba/wrapper.py:59-61 feeds the reference),
            and dk / dv come back summed over each group
        cu_seqlens: cumulative sequence lengths, int32, starts at 0, ends at seqlen
        max_seqlen: longest sequence; a launch hint in the reference, unused here
        moba_chunk_size, moba_topk: block size and number of attended blocks (own block included)

    Returns:
        attn_output [seqlen, head, head_dim], dtype of q
    """
    del max_seqlen
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not isinstance(t, torch.Tensor) or t.dim() != 3:
            raise ValueError(f"{name} must be a [seqlen, head, head_dim] tensor")
        if not t.is_cuda:
            raise RuntimeError(f"{name} is on {t.device}: moba_b200 runs on CUDA (sm_100a) only and has no CPU fallback")
    return _MobaAttnFunction.apply(q, k, v, cu_seqlens, int(moba_chunk_size), int(moba_topk))


# moba_layer (moba_b200/wrapper.py) passes grouped-query K / V through unexpanded to implementations that say so
moba_attn_varlen.supports_grouped_kv = True
