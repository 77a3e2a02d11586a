"""Test infrastructure for sizes where a dense oracle is impossible: an fp32 torch restatement of the MoBA rule
that works on packed variable-length batches and is evaluated (a) for the block selection of every query and (b)
for sampled query rows (out, dq) and sampled key rows (dk, dv) only.

What it restates (file:line in MoonshotAI/MoBA): the pooled key rounded to the input dtype and the fp32 gate
(moba/moba_efficient.py:335-347), candidates = earlier chunks of the same sequence (:355-360), top-(k-1)
(:365-371), attention over own chunk (causal) + selected chunks with scale D^-0.5 (:86-116), ordinary attention
gradients with no gradient through the selection (:208-264). Runs on the test's CUDA device with torch ops only;
nothing here is used by the product package.
"""
import numpy as np
import torch

from tests import helpers as H


class Layout:
    """Per-token tables of a packed batch: sequence start / end, first token of the own chunk, local chunk index."""

    def __init__(self, cu, chunk, dev):
        self.cu, self.chunk, self.dev = [int(x) for x in cu], int(chunk), dev
        S = self.cu[-1]
        self.S = S
        lens = [b - a for a, b in zip(self.cu, self.cu[1:])]
        self.n_local = [-(-n // chunk) for n in lens]                 # chunks per sequence
        self.n_max = max(self.n_local, default=0)
        seq = torch.repeat_interleave(torch.arange(len(lens), device=dev), torch.tensor(lens, device=dev))
        starts = torch.tensor(self.cu[:-1], device=dev)
        self.seq_start = starts[seq]
        self.seq_end = torch.tensor(self.cu[1:], device=dev)[seq]
        pos = torch.arange(S, device=dev) - self.seq_start
        self.c_loc = pos // chunk                                     # local chunk index of every token
        self.chunk_first = self.seq_start + self.c_loc * chunk        # first token of the token's own chunk
        # global chunk id of (sequence, local chunk 0)
        first = np.concatenate([[0], np.cumsum(self.n_local)])[:-1]
        self.seq_chunk0 = torch.tensor(first, device=dev)[seq]


def check_pooled_keys(kmean_kernel, k, lay):
    """The kernel's pooled keys [n_chunks, H_kv, D] (fp32 holding values of k.dtype) against torch's .mean() of the
    full chunks: the same fp32 sum up to its order, so an entry may differ by one rounding step of k.dtype where
    the sum falls next to a rounding boundary -- rarely (< 1e-3 of the entries)."""
    c = 0
    n_bad = n_all = 0
    for b, (t0, t1) in enumerate(zip(lay.cu, lay.cu[1:])):
        nc = lay.n_local[b] - 1
        if nc > 0:
            want = k[t0:t0 + nc * lay.chunk].view(nc, lay.chunk, k.shape[1], k.shape[2]).mean(dim=1).float()
            got = kmean_kernel[c:c + nc]
            ulp = 2.0 ** -7 if k.dtype == torch.bfloat16 else 2.0 ** -10
            assert bool(((got - want).abs() <= ulp * want.abs().clamp(min=2.0 ** -20)).all())
            n_bad += int((got != want).sum())
            n_all += want.numel()
        c += lay.n_local[b]
    assert n_bad <= 1e-3 * max(n_all, 1), (n_bad, n_all)


def reference_selection(q, k, lay, topk, rep=1, kmean_kernel=None):
    """mask [S, H, n_max] bool over LOCAL chunk ids, and the fp32 gate [S, H, n_max] (-inf where not a
    candidate). k may carry H / rep heads (query head h reads key head h // rep). With kmean_kernel (the pooling
    kernel's output, checked by check_pooled_keys) the gate is evaluated on exactly the pooled keys the gate kernel
    saw: a pooled key that rounds the other way on a half-ulp tie moves a score by ~1e-3 absolute, which is not
    what the selection comparison is about."""
    S, Hq, D = q.shape
    dev = q.device
    mask = torch.zeros((S, Hq, lay.n_max), dtype=torch.bool, device=dev)
    gate = torch.full((S, Hq, lay.n_max), float("-inf"), dtype=torch.float32, device=dev)
    B = lay.chunk
    for b, (t0, t1) in enumerate(zip(lay.cu, lay.cu[1:])):
        n_b = lay.n_local[b]
        if n_b <= 1:
            continue
        nc = n_b - 1                                                  # candidate chunks: all full-size
        if kmean_kernel is not None:
            c0 = sum(lay.n_local[:b])
            kmean = kmean_kernel[c0:c0 + nc].float()
        else:
            kmean = k[t0:t0 + nc * B].view(nc, B, k.shape[1], D).mean(dim=1).float()   # rounded to k.dtype first
        if rep > 1:
            kmean = kmean.repeat_interleave(rep, dim=1)
        for h0 in range(0, Hq, 4):                                    # a few heads at a time bounds the memory
            hs = slice(h0, min(h0 + 4, Hq))
            g = torch.einsum("nhd,shd->shn", kmean[:, hs], q[t0:t1, hs].float())
            own = lay.c_loc[t0:t1][:, None, None]
            g = g.masked_fill(torch.arange(nc, device=dev)[None, None, :] >= own, float("-inf"))
            kk = min(topk - 1, nc)
            if kk > 0:
                val, idx = torch.topk(g, kk, dim=-1)
                m = torch.zeros_like(g, dtype=torch.bool).scatter_(-1, idx, torch.isfinite(val))
                mask[t0:t1, hs, :nc] = m
            gate[t0:t1, hs, :nc] = g
    return mask, gate


def kernel_selection(sel, lay):
    """sel [S, H, kk] global chunk ids (-1 = empty) -> mask [S, H, n_max] over local chunk ids."""
    S, Hq, kk = sel.shape
    local = torch.where(sel >= 0, sel - lay.seq_chunk0[:, None, None].to(sel.dtype), torch.full_like(sel, lay.n_max))
    got = torch.zeros((S, Hq, lay.n_max + 1), dtype=torch.bool, device=sel.device)
    got.scatter_(-1, local.long(), torch.ones_like(local, dtype=torch.bool))
    return got[..., :lay.n_max]


def assert_same_selection(got, ref, gate, lay, topk, max_tie_frac=1e-3):
    """Identical sets, except queries where the chunks only one side picked score within 1e-3 relative."""
    S, Hq, _ = got.shape
    diff_q = (got != ref).any(-1)
    n_diff = int(diff_q.sum())
    if n_diff:
        for s_i, h_i in diff_q.nonzero()[:200].tolist():
            a = gate[s_i, h_i][got[s_i, h_i] & ~ref[s_i, h_i]].sort().values
            b = gate[s_i, h_i][ref[s_i, h_i] & ~got[s_i, h_i]].sort().values
            assert len(a) == len(b), (s_i, h_i)
            rel = (a - b).abs() / torch.maximum(a.abs(), b.abs()).clamp(min=1e-30)
            assert (rel < H.TIE_REL).all(), (s_i, h_i, a.tolist(), b.tolist())
    assert n_diff <= max_tie_frac * S * Hq, n_diff
    want_n = torch.clamp(lay.c_loc, max=topk - 1)[:, None].expand(S, Hq)
    assert int((got.sum(-1) != want_n).sum()) == 0            # every query picked min(c, k-1) chunks
    return n_diff


def _key_index(s_i, h_i, mask, lay):
    dev = mask.device
    t0 = int(lay.seq_start[s_i])
    own0 = int(lay.chunk_first[s_i])
    parts = [torch.arange(t0 + c * lay.chunk, t0 + (c + 1) * lay.chunk, device=dev)
             for c in mask[s_i, h_i].nonzero().flatten().tolist()]
    parts.append(torch.arange(own0, s_i + 1, device=dev))
    return torch.cat(parts)


def check_query_rows(rows, q, k, v, d_out, out, dq, mask, lay, rep=1):
    """out (and dq when given) of the sampled (token, head) rows against fp32 arithmetic over the keys the rule
    prescribes, with the selection the kernel made."""
    scale = q.shape[-1] ** -0.5
    for s_i, h_i in rows:
        hk = h_i // rep
        idx = _key_index(s_i, h_i, mask, lay)
        kf, vf = k[idx, hk].float(), v[idx, hk].float()
        sc = (kf @ q[s_i, h_i].float()) * scale
        p = torch.softmax(sc, 0)
        o_ref = p @ vf
        H.assert_row_parity(f"out[{s_i},{h_i}]", out[s_i, h_i].float().cpu().numpy(), o_ref.cpu().numpy())
        if dq is not None:
            do = d_out[s_i, h_i].float()
            dp = vf @ do
            delta = (do * o_ref).sum()
            dq_ref = ((p * (dp - delta)) * scale) @ kf
            H.assert_row_parity(f"dq[{s_i},{h_i}]", dq[s_i, h_i].float().cpu().numpy(), dq_ref.cpu().numpy())


def _lse_of(qs, h_i, q, k, mask, lay, hk):
    """fp32 log-sum-exp of the queries qs (all of one sequence) of head h_i over their prescribed keys."""
    dev = q.device
    scale = q.shape[-1] ** -0.5
    t0 = int(lay.seq_start[qs[0]])
    n_b = int(lay.c_loc[int(lay.seq_end[qs[0]]) - 1]) + 1
    m = torch.full((len(qs),), float("-inf"), device=dev)
    acc = torch.zeros(len(qs), device=dev)
    qf = q[qs, h_i].float()
    own_c = lay.c_loc[qs]
    for cc in range(n_b):
        sel_c = mask[qs, h_i, cc] if cc < mask.shape[2] else torch.zeros_like(own_c, dtype=torch.bool)
        rows_c = (sel_c | (own_c == cc)).nonzero().flatten()
        if len(rows_c) == 0:
            continue
        k0 = t0 + cc * lay.chunk
        k1 = min(k0 + lay.chunk, int(lay.seq_end[qs[0]]))
        sc = (qf[rows_c] @ k[k0:k1, hk].float().T) * scale
        is_own = own_c[rows_c] == cc
        causal = torch.arange(k0, k1, device=dev)[None, :] > qs[rows_c][:, None]
        sc = sc.masked_fill(is_own[:, None] & causal, float("-inf"))
        m_new = torch.maximum(m[rows_c], sc.max(1).values)
        acc[rows_c] = acc[rows_c] * torch.exp(m[rows_c] - m_new) + torch.exp(sc - m_new[:, None]).sum(1)
        m[rows_c] = m_new
    return m + torch.log(acc)


def check_key_rows(rows, q, k, v, d_out, out, dk, dv, mask, lay, rep=1):
    """dk / dv of the sampled (token, key/value head) rows: sums over every query (of every query head of the
    group) that attends the key, probabilities from a per-query fp32 log-sum-exp."""
    scale = q.shape[-1] ** -0.5
    dev = q.device
    for t_i, hk in rows:
        c = int(lay.c_loc[t_i])
        t0, t1 = int(lay.seq_start[t_i]), int(lay.seq_end[t_i])
        own_end = min(int(lay.chunk_first[t_i]) + lay.chunk, t1)
        dk_ref = torch.zeros(q.shape[-1], device=dev)
        dv_ref = torch.zeros(q.shape[-1], device=dev)
        for h_i in range(hk * rep, (hk + 1) * rep):
            later = mask[t0:t1, h_i, c].nonzero().flatten() + t0 if c < mask.shape[2] else torch.zeros(0, dtype=torch.long, device=dev)
            qs = torch.cat([torch.arange(t_i, own_end, device=dev), later])
            lse_q = _lse_of(qs, h_i, q, k, mask, lay, hk)
            qf, dof, of = q[qs, h_i].float(), d_out[qs, h_i].float(), out[qs, h_i].float()
            p = torch.exp((qf @ k[t_i, hk].float()) * scale - lse_q)
            dv_ref += p @ dof
            delta = (dof * of).sum(-1)
            dk_ref += ((p * (dof @ v[t_i, hk].float() - delta)) * scale) @ qf
        # the bound grows with the number of rounded summands (one per query head of the group)
        H.assert_row_parity(f"dv[{t_i},{hk}]", dv[t_i, hk].float().cpu().numpy() / rep ** 0.5, dv_ref.cpu().numpy() / rep ** 0.5)
        H.assert_row_parity(f"dk[{t_i},{hk}]", dk[t_i, hk].float().cpu().numpy() / rep ** 0.5, dk_ref.cpu().numpy() / rep ** 0.5)


def check_lists(plan, heads, sel, list_off, work_off, list_tok, row_of):
    """Index lists and row map against the selection, on the device: row count, ascending tokens inside every
    (chunk, head) list, list membership == selection, row_of inverse of list_tok."""
    dev = sel.device
    S, Hq, kk = sel.shape
    E = plan.info.n_chunks * heads
    R = plan.rows_total(heads)
    lo = list_off.long()
    assert int(lo[E]) == R
    lens = lo[1:] - lo[:-1]
    assert int((work_off[1:].long() - work_off[:-1].long() - (lens + 127) // 128).abs().sum()) == 0
    # expert of every row
    row_e = torch.repeat_interleave(torch.arange(E, device=dev), lens)
    lt = list_tok.long()
    inside = torch.ones(R, dtype=torch.bool, device=dev)
    inside[lo[:-1][lens > 0]] = False                                # first row of every non-empty list
    assert bool((lt[1:][inside[1:]] > lt[:-1][inside[1:]]).all())    # ascending tokens inside a list
    # every (token, head, slot) with a chunk owns exactly the row (expert = chunk * H + head) that names its token
    ss, hh, jj = (sel >= 0).nonzero(as_tuple=True)
    rows = row_of[ss, hh, jj].long()
    assert len(rows) == R and int(rows.min()) >= 0 and int(rows.max()) < R
    assert len(torch.unique(rows)) == R
    assert bool((lt[rows] == ss).all())
    assert bool((row_e[rows] == sel[ss, hh, jj].long() * heads + hh).all())
    assert bool((row_of[sel < 0] == -1).all())
