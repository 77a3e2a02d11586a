"""CPU oracle for the MoBA attention path -- TEST INFRASTRUCTURE, not product code.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this module; the
product package (moba_b200) never does and has no CPU path.

What is restated (numpy, fp32 arithmetic, file:line in MoonshotAI/MoBA):
  * chunk_table        calc_chunks, moba/moba_efficient.py:14-64 (per-sequence chunk alignment, short tail)
  * pool_keys          per-chunk key mean rounded to the input dtype, moba/moba_naive.py:46-50 and
                       moba/moba_efficient.py:335-340
  * gate_scores/select fp32 q . mean, own / future chunks excluded, top-(k-1) past chunks,
                       moba/moba_naive.py:53-73 and moba/moba_efficient.py:341-371
  * forward_dense      the dense-mask softmax of moba/moba_naive.py:74-93, literally (O(S^2) per sequence)
  * forward / backward the same function evaluated block-sparsely: every (key chunk, head) is attended by
                       the queries that selected it, partial results are joined with a log-sum-exp merge
                       (the algebra of MixedAttention, moba/moba_efficient.py:118-168 and :185-267)
  * decode_attention   the dense decode step of moba/wrapper.py:76-82, flash_attn_func(q, k, v, dropout, scaling,
                       causal=True): flash-attn (2.6.3 in the reference's requirements.txt) is a third-party
                       dependency that is not part of the reference checkout, so its published definition is
                       restated -- softmax(scale * q k^T) v with the causal mask aligned to the bottom-right corner
                       (query i of q_len sees keys 0 .. kv_len - q_len + i), grouped-query heads sharing key/value
                       head h // (q_heads // kv_heads). The reference holds no test or fixture for its decode branch; this
                       function is pinned instead against flash_attn_func itself, run on the GPU from the installed
                       flash-attn package (tests/test_gpu_decode.py), and is unpinned where that cannot run.

Parity pin: tests/test_oracle_golden.py checks every function here against fixtures produced by running
the reference's own moba_attn_varlen_naive (tests/golden/make_golden.py is the generating script).

Semantics note: with moba_topk == 1, or when no sequence has more than one chunk, the efficient reference
returns plain causal attention over whole sequences (moba/moba_efficient.py:314-321) while moba_naive keeps
attention inside the own chunk. `forward`/`backward` follow the efficient path (it is the one the product
replaces); `forward_dense` follows moba_naive. They agree whenever moba_topk >= 2.
"""
import math

import numpy as np


# ----------------------------------------------------------------------------- dtype rounding helpers
def round_bf16(x):
    """Round fp32 to the nearest bfloat16 (ties to even) and return it widened back to fp32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    out = rounded.astype(np.uint32).view(np.float32)
    return np.where(np.isfinite(x), out, x).astype(np.float32)


def round_dtype(x, dtype):
    """dtype: 'bf16', 'f16' or 'f32' -- the element type the reference was handed."""
    if dtype == "bf16":
        return round_bf16(x)
    if dtype == "f16":
        return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)
    if dtype == "f32":
        return np.asarray(x, dtype=np.float32)
    raise ValueError(f"unknown dtype {dtype!r}")


# ----------------------------------------------------------------------------- chunk metadata
def chunk_table(cu_seqlens, chunk_size):
    """Per-sequence chunking (moba/moba_efficient.py:14-64).

    Returns dict with: cu_chunk [n+1] (token offset of every chunk), chunk_seq [n] (sequence of every
    chunk), seq_first_chunk [batch+1] (first global chunk id of every sequence), filtered [F] (chunks that
    are not the last of their sequence).
    """
    cu = [int(x) for x in cu_seqlens]
    cu_chunk, chunk_seq, seq_first, filtered = [0], [], [0], []
    for b in range(len(cu) - 1):
        t0, t1 = cu[b], cu[b + 1]
        nb = (t1 - t0 + chunk_size - 1) // chunk_size
        for c in range(nb):
            cu_chunk.append(min(t0 + (c + 1) * chunk_size, t1))
            chunk_seq.append(b)
            if c + 1 < nb:
                filtered.append(len(chunk_seq) - 1)
        seq_first.append(len(chunk_seq))
    return {
        "cu_chunk": np.asarray(cu_chunk, dtype=np.int64),
        "chunk_seq": np.asarray(chunk_seq, dtype=np.int64),
        "seq_first_chunk": np.asarray(seq_first, dtype=np.int64),
        "filtered": np.asarray(filtered, dtype=np.int64),
    }


def effective_topk(cu_seqlens, chunk_size, moba_topk):
    """min(moba_topk - 1, number of filtered chunks) (moba/moba_efficient.py:314)."""
    tab = chunk_table(cu_seqlens, chunk_size)
    return min(moba_topk - 1, len(tab["filtered"]))


def rows_per_head(cu_seqlens, chunk_size, moba_topk):
    """Number of (query, selected chunk) pairs per head: a query in the c-th chunk picks min(c, k-1)."""
    cu = [int(x) for x in cu_seqlens]
    total = 0
    for b in range(len(cu) - 1):
        n = cu[b + 1] - cu[b]
        nb = (n + chunk_size - 1) // chunk_size
        for c in range(nb):
            cs = min(chunk_size, n - c * chunk_size)
            total += cs * min(c, moba_topk - 1)
    return total


def selected_pairs(cu_seqlens, chunk_size, moba_topk):
    """(query, key) pairs per head on which attention is evaluated: causal own chunk + selected chunks."""
    cu = [int(x) for x in cu_seqlens]
    pairs = 0
    for b in range(len(cu) - 1):
        n = cu[b + 1] - cu[b]
        nb = (n + chunk_size - 1) // chunk_size
        for c in range(nb):
            cs = min(chunk_size, n - c * chunk_size)
            pairs += cs * (cs + 1) // 2 + chunk_size * cs * min(c, moba_topk - 1)
    return pairs


# ----------------------------------------------------------------------------- pooling and gate
def pool_keys(k, cu_seqlens, chunk_size, dtype):
    """Mean key of every chunk, rounded to `dtype` as the reference's .mean() does. k: [S,H,D] fp32 values
    that are representable in `dtype`. Returns [n,H,D] fp32."""
    tab = chunk_table(cu_seqlens, chunk_size)
    cu_chunk = tab["cu_chunk"]
    n = len(cu_chunk) - 1
    out = np.zeros((n,) + k.shape[1:], dtype=np.float32)
    for c in range(n):
        blk = k[cu_chunk[c]:cu_chunk[c + 1]].astype(np.float32)
        out[c] = round_dtype(blk.sum(axis=0, dtype=np.float32) * np.float32(1.0 / blk.shape[0]), dtype)
    return out


def gate_scores(q, kmean, cu_seqlens, chunk_size):
    """fp32 gate scores of every query against the chunks of its own sequence.

    Returns a list over sequences of arrays [H, S_b, n_b]; entries for the own and future chunks are -inf
    (moba/moba_efficient.py:352-360: a chunk is visible only to queries at or after its end)."""
    tab = chunk_table(cu_seqlens, chunk_size)
    out = []
    for b in range(len(cu_seqlens) - 1):
        t0, t1 = int(cu_seqlens[b]), int(cu_seqlens[b + 1])
        c0, c1 = int(tab["seq_first_chunk"][b]), int(tab["seq_first_chunk"][b + 1])
        qb = q[t0:t1].astype(np.float32)                      # [S_b, H, D]
        g = np.einsum("shd,nhd->hsn", qb, kmean[c0:c1].astype(np.float32)).astype(np.float32)
        pos = np.arange(t1 - t0)
        own = pos // chunk_size                                # chunk of every query
        future = np.arange(c1 - c0)[None, :] >= own[:, None]   # own chunk and later ones
        g[:, future] = -np.inf
        out.append(g)
    return out


def select_chunks(scores, moba_topk):
    """Top-(moba_topk-1) visible chunks per (head, query). scores: one [H,S_b,n_b] array. Returns a boolean
    mask of the same shape. Ties go to the lower chunk index (the reference leaves tie order to
    torch.topk)."""
    H, S, n = scores.shape
    kk = min(moba_topk - 1, n)
    mask = np.zeros(scores.shape, dtype=bool)
    if kk <= 0:
        return mask
    order = np.argsort(-scores, axis=-1, kind="stable")[..., :kk]
    picked = np.take_along_axis(scores, order, axis=-1)
    hh, ss, _ = np.meshgrid(np.arange(H), np.arange(S), np.arange(kk), indexing="ij")
    ok = np.isfinite(picked)
    mask[hh[ok], ss[ok], order[ok]] = True
    return mask


def select_all(q, k, cu_seqlens, chunk_size, moba_topk, dtype):
    """Pooling + gate + selection. Returns (kmean, list of score arrays, list of boolean masks)."""
    kmean = pool_keys(k, cu_seqlens, chunk_size, dtype)
    scores = gate_scores(q, kmean, cu_seqlens, chunk_size)
    masks = [select_chunks(s, moba_topk) for s in scores]
    return kmean, scores, masks


# ----------------------------------------------------------------------------- dense restatement of moba_naive
def forward_dense(q, k, v, cu_seqlens, chunk_size, moba_topk, dtype):
    """moba/moba_naive.py:34-93 literally: [H,S_b,S_b] additive mask, fp32 softmax. Returns fp32 [S,H,D]."""
    q = np.asarray(q, dtype=np.float32)
    k = np.asarray(k, dtype=np.float32)
    v = np.asarray(v, dtype=np.float32)
    scale = np.float32(q.shape[-1] ** -0.5)
    out = np.zeros_like(q)
    for b in range(len(cu_seqlens) - 1):
        t0, t1 = int(cu_seqlens[b]), int(cu_seqlens[b + 1])
        n = t1 - t0
        if n == 0:
            continue
        qb, kb, vb = q[t0:t1], k[t0:t1], v[t0:t1]
        nb = math.ceil(n / chunk_size)
        kmean = np.stack([
            round_dtype(kb[i * chunk_size:min(n, (i + 1) * chunk_size)].sum(axis=0, dtype=np.float32)
                        * np.float32(1.0 / (min(n, (i + 1) * chunk_size) - i * chunk_size)), dtype)
            for i in range(nb)])
        gate = np.einsum("shd,nhd->hsn", qb, kmean).astype(np.float32)
        for i in range(nb):
            gate[:, :(i + 1) * chunk_size, i] = -np.inf
            gate[:, i * chunk_size:(i + 1) * chunk_size, i] = np.inf
        kk = min(moba_topk, nb)
        order = np.argsort(-gate, axis=-1, kind="stable")[..., :kk]
        need = np.zeros(gate.shape, dtype=bool)
        np.put_along_axis(need, order, True, axis=-1)
        thr = np.take_along_axis(gate, order, axis=-1).min(axis=-1, keepdims=True)
        need &= gate >= thr
        add = np.where(need, np.float32(0), np.float32(-np.inf))
        add = np.repeat(add, chunk_size, axis=-1)[:, :, :n]
        add[:, np.triu_indices(n, 1)[0], np.triu_indices(n, 1)[1]] = -np.inf
        qk = (np.einsum("xhd,yhd->hxy", qb, kb) + add) * scale
        qk -= qk.max(axis=-1, keepdims=True)
        p = np.exp(qk)
        p /= p.sum(axis=-1, keepdims=True)
        out[t0:t1] = np.einsum("hxy,yhd->xhd", p, vb)
    return out


# ----------------------------------------------------------------------------- block-sparse forward / backward
def _blocks(cu_seqlens, chunk_size):
    """Yield (b, t0, t1, c0, n_chunks) per sequence."""
    tab = chunk_table(cu_seqlens, chunk_size)
    for b in range(len(cu_seqlens) - 1):
        yield (b, int(cu_seqlens[b]), int(cu_seqlens[b + 1]), int(tab["seq_first_chunk"][b]),
               int(tab["seq_first_chunk"][b + 1] - tab["seq_first_chunk"][b]))


def _full_causal(cu_seqlens):
    return max(int(cu_seqlens[i + 1]) - int(cu_seqlens[i]) for i in range(len(cu_seqlens) - 1)) if len(cu_seqlens) > 1 else 1


def forward(q, k, v, cu_seqlens, chunk_size, moba_topk, dtype, masks=None):
    """Block-sparse evaluation. Returns (out fp32 [S,H,D], lse fp32 [S,H] natural log, masks).

    Own chunk: causal softmax pieces; every selected chunk: full pieces; merged per query with the
    log-sum-exp rule of moba/moba_efficient.py:118-168 (here in one pass, in fp32/fp64)."""
    q = np.asarray(q, dtype=np.float32)
    k = np.asarray(k, dtype=np.float32)
    v = np.asarray(v, dtype=np.float32)
    S, H, D = q.shape
    scale = D ** -0.5
    if effective_topk(cu_seqlens, chunk_size, moba_topk) <= 0:
        chunk_size = max(_full_causal(cu_seqlens), 1)          # plain causal attention over sequences
        masks = None
        moba_topk = 1
    if masks is None:
        _, _, masks = select_all(q, k, cu_seqlens, chunk_size, moba_topk, dtype)
    m_run = np.full((S, H), -np.inf, dtype=np.float64)
    l_run = np.zeros((S, H), dtype=np.float64)
    acc = np.zeros((S, H, D), dtype=np.float64)

    def absorb(rows, h, s_blk, v_blk):
        # s_blk [nq, nk] scaled scores (may hold -inf), v_blk [nk, D]
        m_new = np.maximum(m_run[rows, h], s_blk.max(axis=1))
        alpha = np.exp(m_run[rows, h] - m_new)
        p = np.exp(s_blk - m_new[:, None])
        l_run[rows, h] = l_run[rows, h] * alpha + p.sum(axis=1)
        acc[rows, h] = acc[rows, h] * alpha[:, None] + p @ v_blk
        m_run[rows, h] = m_new

    for b, t0, t1, c0, nb in _blocks(cu_seqlens, chunk_size):
        n = t1 - t0
        for h in range(H):
            for c in range(nb):
                a0, a1 = t0 + c * chunk_size, min(t0 + (c + 1) * chunk_size, t1)
                rows = np.arange(a0, a1)
                s_own = (q[a0:a1, h].astype(np.float64) @ k[a0:a1, h].astype(np.float64).T) * scale
                s_own[np.triu_indices(a1 - a0, 1)] = -np.inf
                absorb(rows, h, s_own, v[a0:a1, h].astype(np.float64))
                if c + 1 < nb:      # this chunk as a selected block for later queries
                    sel_rows = t0 + np.nonzero(masks[b][h, :, c])[0]
                    if len(sel_rows):
                        s_blk = (q[sel_rows, h].astype(np.float64) @ k[a0:a1, h].astype(np.float64).T) * scale
                        absorb(sel_rows, h, s_blk, v[a0:a1, h].astype(np.float64))
    out = (acc / l_run[..., None]).astype(np.float32)
    lse = (m_run + np.log(l_run)).astype(np.float32)
    return out, lse, masks


def backward(q, k, v, cu_seqlens, chunk_size, moba_topk, dtype, out, lse, d_out, masks):
    """Gradients of `forward` w.r.t. q, k, v (no gradient through the selection or the pooled keys,
    moba/moba_efficient.py:365-371). Uses the merged out / lse exactly as MixedAttention.backward hands them
    to both flash backward calls (moba/moba_efficient.py:208-264). Returns fp32 (dq, dk, dv)."""
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    v = np.asarray(v, dtype=np.float64)
    d_out = np.asarray(d_out, dtype=np.float64)
    S, H, D = q.shape
    scale = D ** -0.5
    if effective_topk(cu_seqlens, chunk_size, moba_topk) <= 0:
        chunk_size = max(_full_causal(cu_seqlens), 1)
    delta = (d_out * np.asarray(out, dtype=np.float64)).sum(axis=-1)      # [S,H]
    lse = np.asarray(lse, dtype=np.float64)
    dq = np.zeros_like(q)
    dk = np.zeros_like(k)
    dv = np.zeros_like(v)

    def block(rows, h, a0, a1, causal):
        s = (q[rows, h] @ k[a0:a1, h].T) * scale
        p = np.exp(s - lse[rows, h][:, None])
        if causal:
            p[np.triu_indices(a1 - a0, 1)] = 0.0
        dv[a0:a1, h] += p.T @ d_out[rows, h]
        dp = d_out[rows, h] @ v[a0:a1, h].T
        ds = p * (dp - delta[rows, h][:, None]) * scale
        dq[rows, h] += ds @ k[a0:a1, h]
        dk[a0:a1, h] += ds.T @ q[rows, h]

    for b, t0, t1, c0, nb in _blocks(cu_seqlens, chunk_size):
        for h in range(H):
            for c in range(nb):
                a0, a1 = t0 + c * chunk_size, min(t0 + (c + 1) * chunk_size, t1)
                block(np.arange(a0, a1), h, a0, a1, True)
                if c + 1 < nb and masks is not None:
                    sel_rows = t0 + np.nonzero(masks[b][h, :, c])[0]
                    if len(sel_rows):
                        block(sel_rows, h, a0, a1, False)
    return dq.astype(np.float32), dk.astype(np.float32), dv.astype(np.float32)


def moba_attn_varlen_oracle(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk, dtype="bf16",
                            d_out=None):
    """Same argument order as the reference entry points. Returns out, or (out, dq, dk, dv) with d_out."""
    del max_seqlen  # a launch hint in the reference (moba/moba_efficient.py:96-97); unused by moba_naive too
    out, lse, masks = forward(q, k, v, cu_seqlens, moba_chunk_size, moba_topk, dtype)
    if d_out is None:
        return out
    # exact gradient of the fp32 softmax, as autograd computes it through moba_naive
    dq, dk, dv = backward(q, k, v, cu_seqlens, moba_chunk_size, moba_topk, dtype, out, lse, d_out, masks)
    return out, dq, dk, dv


def selection_sets(masks):
    """Flatten a list of [H,S_b,n_b] masks into a set of (sequence, head, local token, local chunk)."""
    res = set()
    for b, m in enumerate(masks):
        hh, ss, cc = np.nonzero(m)
        res.update(zip([b] * len(hh), hh.tolist(), ss.tolist(), cc.tolist()))
    return res


def decode_attention(query, key, value, scaling, dtype="bf16"):
    """query [B, Hq, Lq, D], key / value [B, Hkv, Lk, D] (fp32 arrays holding `dtype` values) ->
    [B, Lq, Hq, D] rounded to `dtype` (the layout flash_attn_func returns, moba/wrapper.py:76-82)."""
    B, Hq, Lq, D = query.shape
    Hkv, Lk = key.shape[1], key.shape[2]
    rep = Hq // Hkv
    out = np.zeros((B, Lq, Hq, D), dtype=np.float32)
    allowed = np.arange(Lk)[None, :] <= (np.arange(Lq)[:, None] + (Lk - Lq))
    for b in range(B):
        for h in range(Hq):
            s = (query[b, h].astype(np.float64) @ key[b, h // rep].astype(np.float64).T) * scaling
            s = np.where(allowed, s, -np.inf)
            p = np.exp(s - s.max(axis=1, keepdims=True))
            p /= p.sum(axis=1, keepdims=True)
            out[b, :, h] = (p @ value[b, h // rep].astype(np.float64)).astype(np.float32)
    return round_dtype(out, dtype)
