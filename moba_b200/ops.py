"""Thin torch-facing wrappers over the C ABI: one function per kernel group.

torch supplies device memory and the current stream; every computation happens in libmoba_b200.so.
"""
import ctypes
from collections import OrderedDict

import torch

from . import _lib
from ._lib import PlanInfo, call

_DTYPES = {torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_F16, torch.float32: _lib.DTYPE_F32}


# Optional per-kernel-group timing: when a list is installed with `set_timing(list)`, every wrapper below
# appends (name, start_event, end_event) recorded on the current stream around its launch(es).
_TIMING = None


def set_timing(records):
    """Install (or with None remove) the list that receives (name, start, end) CUDA event triples."""
    global _TIMING
    _TIMING = records


class _timed:
    def __init__(self, name, device):
        self.name, self.device = name, device

    def __enter__(self):
        if _TIMING is not None:
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record(torch.cuda.current_stream(self.device))
        return self

    def __exit__(self, *exc):
        if _TIMING is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record(torch.cuda.current_stream(self.device))
            _TIMING.append((self.name, self.start, end))
        return False


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _dev_index(t):
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def _check_shd(name, t):
    if t.dim() != 3 or t.shape[2] != _lib.HEAD_DIM:
        raise ValueError(f"{name} must be [seqlen, heads, {_lib.HEAD_DIM}], got {tuple(t.shape)}")
    if t.stride(2) != 1:
        raise ValueError(f"{name} must have unit stride in the last dimension")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor: moba_b200 has no CPU path")
    if t.dtype not in _DTYPES:
        raise ValueError(f"{name} has unsupported dtype {t.dtype}")


class Plan:
    """Chunk plan for one (cu_seqlens, chunk size, top-k): sizes on the host, integer tables on the device.

    Plays the role of calc_chunks (MoonshotAI/MoBA moba/moba_efficient.py:14-64)."""

    def __init__(self, cu_host, chunk_size, topk, device):
        self.cu_host = [int(x) for x in cu_host]
        self.chunk_size = int(chunk_size)
        self.topk = int(topk)
        self.device = torch.device(device)
        batch = len(self.cu_host) - 1
        arr = (ctypes.c_int32 * (batch + 1))(*self.cu_host)
        self.info = PlanInfo()
        call("moba_plan_sizes", arr, batch, self.chunk_size, self.topk, ctypes.byref(self.info))
        meta = torch.empty(max(self.info.meta_ints, 1), dtype=torch.int32, pin_memory=self.device.type == "cuda")
        call("moba_plan_fill", arr, batch, self.chunk_size, self.topk, ctypes.byref(self.info),
             ctypes.c_void_p(meta.data_ptr()))
        self.meta_host = meta          # pinned and kept alive by the plan: the upload below is asynchronous
        self.meta = meta.to(self.device, non_blocking=True) if self.device.type == "cuda" else meta

    def table(self, name):
        """Host view of one integer table (for tests)."""
        i = self.info
        spans = {
            "chunk_start": (i.off_chunk_start, i.n_chunks + 1),
            "chunk_seq_first": (i.off_chunk_seq_first, i.n_chunks),
            "chunk_seq_last": (i.off_chunk_seq_last, i.n_chunks),
            "qtile_chunk": (i.off_qtile_chunk, i.n_qtiles),
            "qtile_start": (i.off_qtile_start, i.n_qtiles),
            "qtile_cand_off": (i.off_qtile_cand_off, i.n_qtiles + 1),
            "chunk_qtile_first": (i.off_chunk_qtile_first, i.n_chunks + 1),
        }
        off, n = spans[name]
        return self.meta_host[off:off + n]

    @property
    def kk(self):
        return self.info.kk

    def rows_total(self, H):
        return self.info.rows_per_head * H


class PlanView:
    """A plan whose integer tables are another plan's and whose list sizes are given by the caller: used when
    the query lists do not come from gate_topk / build_lists (pre-gathered queries, MoonshotAI/MoBA
    moba/moba_efficient.py:67-127)."""

    def __init__(self, base, kk, rows_per_head, max_work_tiles_per_head):
        self.base = base
        self.meta = base.meta
        self.meta_host = base.meta_host
        self.device = base.device
        self.info = PlanInfo.from_buffer_copy(base.info)
        self.info.kk = int(kk)
        self.info.rows_per_head = int(rows_per_head)
        self.info.max_work_tiles_per_head = int(max_work_tiles_per_head)

    @property
    def kk(self):
        return self.info.kk

    def rows_total(self, H):
        return self.info.rows_per_head * H


_PLAN_CACHE = OrderedDict()        # (tensor identity, version, chunk, topk, device) -> (tensor, plan)
_PLAN_BY_VALUE = OrderedDict()     # (cu_seqlens values, chunk, topk, device) -> plan
_PLAN_CACHE_MAX = 16
_CU_HOST = {}                      # id(tensor) -> (weak reference, host values) registered by the tensor's maker


def register_cu_seqlens(tensor, values):
    """Tells get_plan the host values of a cu_seqlens tensor whose maker knows them (the layer wrapper builds
    cu_seqlens from batch and kv_len), so that no device-to-host copy is needed to plan for it."""
    import weakref

    key = id(tensor)
    _CU_HOST[key] = (weakref.ref(tensor, lambda _: _CU_HOST.pop(key, None)), tuple(int(x) for x in values))


def _plan_for_values(values, chunk_size, topk, device):
    key = (tuple(values), int(chunk_size), int(topk), str(device))
    plan = _PLAN_BY_VALUE.get(key)
    if plan is None:
        plan = Plan(values, chunk_size, topk, device)
        _PLAN_BY_VALUE[key] = plan
        while len(_PLAN_BY_VALUE) > _PLAN_CACHE_MAX:
            _PLAN_BY_VALUE.popitem(last=False)
    else:
        _PLAN_BY_VALUE.move_to_end(key)
    return plan


def get_plan(cu_seqlens, chunk_size, topk, device):
    """Plan for a cu_seqlens tensor (device or host) or a list. Plans are cached twice: by tensor identity and
    version, as the reference caches calc_chunks by tensor identity (moba/moba_efficient.py:14), and by the
    values themselves, so that equal batches share one plan (and one upload of its tables) whatever tensor
    carries them. A device tensor whose values were not registered (register_cu_seqlens) is copied to the host
    once per identity."""
    if isinstance(cu_seqlens, torch.Tensor):
        key = (id(cu_seqlens), cu_seqlens._version, int(chunk_size), int(topk), str(device))
        hit = _PLAN_CACHE.get(key)
        if hit is not None and hit[0] is cu_seqlens:
            _PLAN_CACHE.move_to_end(key)
            return hit[1]
        if cu_seqlens.dtype not in (torch.int32, torch.int64) or cu_seqlens.dim() != 1 or cu_seqlens.numel() < 2:
            raise ValueError("cu_seqlens must be a 1-D int32 tensor with at least two entries")
        known = _CU_HOST.get(id(cu_seqlens))
        if known is not None and known[0]() is cu_seqlens and cu_seqlens._version == 0:
            values = known[1]
        else:
            values = cu_seqlens.detach().cpu().tolist()
        plan = _plan_for_values(values, chunk_size, topk, device)
        _PLAN_CACHE[key] = (cu_seqlens, plan)
        while len(_PLAN_CACHE) > _PLAN_CACHE_MAX:
            _PLAN_CACHE.popitem(last=False)
        return plan
    return _plan_for_values([int(x) for x in cu_seqlens], chunk_size, topk, device)


def new_status(device):
    return torch.zeros(1, dtype=torch.int32, device=device)


def check_status(status):
    call("moba_check_status", _ptr(status), _dev_index(status), _stream(status.device))


def _kv_layout(q, k, v):
    """None when k / v are laid out like q, else the moba_kv_layout of grouped-query k / v ([S, H_kv, D] with
    H_kv dividing the head count of q; k and v must share strides)."""
    if v.shape != k.shape or v.stride() != k.stride():
        raise ValueError("k and v must share shape and strides")
    H, Hkv = q.shape[1], k.shape[1]
    if Hkv == H and k.stride() == q.stride():
        return None
    if Hkv < 1 or H % Hkv != 0:
        raise ValueError(f"the key/value head count {Hkv} must divide the query head count {H}")
    return ctypes.pointer(_lib.KvLayout(Hkv, 0, k.stride(0), k.stride(1)))


# ------------------------------------------------------------------------------------------- kernels
def pool_keys(k, plan):
    """kmean [n_chunks, H, D] fp32: per-chunk key mean rounded to k.dtype."""
    _check_shd("k", k)
    H = k.shape[1]
    ws = torch.empty(max(_lib.lib.moba_pool_ws_floats(ctypes.byref(plan.info), H), 1), dtype=torch.float32,
                     device=k.device)
    kmean = torch.empty((plan.info.n_chunks, H, _lib.HEAD_DIM), dtype=torch.float32, device=k.device)
    with _timed("pool_keys", k.device):
        call("moba_pool_keys", _ptr(k), _DTYPES[k.dtype], H, k.stride(0), k.stride(1), ctypes.byref(plan.info),
             _ptr(plan.meta), _ptr(ws), _ptr(kmean), _dev_index(k), _stream(k.device))
    return kmean


def gate_topk(q, kmean, plan, want_scores=False, status=None, fma=False):
    """Returns (sel [S,H,kk] int32 global chunk ids, scores or None, tile_cnt).

    16-bit q is scored on the tensor pipe (needs a status word for its bounded waits: `status`, or a fresh one
    that is checked before returning); fp32 q, or fma=True, takes the fp32-FMA kernel."""
    _check_shd("q", q)
    S, H, _ = q.shape
    if kmean.dim() != 3 or H % kmean.shape[1] != 0 or not kmean.is_contiguous():
        raise ValueError("kmean must be a contiguous [n_chunks, H_kv, 128] tensor with H_kv dividing the heads of q")
    kk = plan.kk
    sel = torch.empty((S, H, kk), dtype=torch.int32, device=q.device)
    scores = torch.empty((S, H, kk), dtype=torch.float32, device=q.device) if want_scores else None
    tile_cnt = torch.empty(max(plan.info.cand_per_head * H, 1), dtype=torch.int32, device=q.device)
    own_status = None
    if not fma and status is None and q.dtype in (torch.bfloat16, torch.float16):
        own_status = status = new_status(q.device)
    with _timed("gate_topk", q.device):
        call("moba_gate_topk", _ptr(q), _DTYPES[q.dtype], H, q.stride(0), q.stride(1), _ptr(kmean),
             kmean.shape[1], ctypes.byref(plan.info), _ptr(plan.meta), _ptr(sel), _ptr(scores), _ptr(tile_cnt),
             _ptr(None if fma else status), _dev_index(q), _stream(q.device))
    if own_status is not None:
        check_status(own_status)
    return sel, scores, tile_cnt


def build_lists(plan, H, sel, tile_cnt, status=None):
    """Returns (list_off [E+1], work_off [E+1], list_tok [R*H], row_of [S,H,kk]); E = n_chunks*H. A chunk id in
    `sel` that is not a candidate of its query is skipped and reported through `status` (2 = bad index)."""
    dev = sel.device
    E = plan.info.n_chunks * H
    list_off = torch.empty(E + 1, dtype=torch.int32, device=dev)
    work_off = torch.empty(E + 1, dtype=torch.int32, device=dev)
    list_tok = torch.empty(max(plan.rows_total(H), 1), dtype=torch.int32, device=dev)
    row_of = torch.empty_like(sel)
    with _timed("build_lists", dev):
        call("moba_build_lists", H, ctypes.byref(plan.info), _ptr(plan.meta), _ptr(sel), _ptr(tile_cnt),
             _ptr(list_off), _ptr(work_off), _ptr(list_tok), _ptr(row_of), _ptr(status), _dev_index(sel),
             _stream(dev))
    return list_off, work_off, list_tok, row_of


def tile_records(plan, H, list_off, work_off):
    """[max_work_tiles * H, 8] int32: one record per 128-row work tile of the list part (head, first row, rows, first
    key token, keys), so that the tile kernels start from one load instead of a search through work_off. Optional:
    a `lists` tuple may carry it as its fourth element."""
    n = max(int(plan.info.max_work_tiles_per_head) * H, 1)
    rec = torch.empty((n, 8), dtype=torch.int32, device=list_off.device)
    with _timed("build_lists", list_off.device):
        call("moba_tile_records", H, ctypes.byref(plan.info), _ptr(plan.meta), _ptr(list_off), _ptr(work_off),
             _ptr(rec), _dev_index(list_off), _stream(list_off.device))
    return rec


def _split_lists(lists):
    """(list_off, work_off, list_tok, tile_rec or None) from a 3- or 4-element `lists` tuple."""
    if len(lists) == 4:
        return lists
    return (*lists, None)


def attn_fwd(q, k, v, plan, lists, status, parts=3, out=None, scale=0.0):
    """Self-chunk causal attention -> (out, lse); gathered rows -> (part_o, part_lse).

    parts: 3 both, 1 own-chunk part only, 2 list part only (buffers of the other part are left unwritten).
    out: optional contiguous [S, H, D] tensor to receive the result (allocated when None)."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        _check_shd(n, t)
    S, H, D = q.shape
    kv = _kv_layout(q, k, v)
    list_off, work_off, list_tok, tile_rec = _split_lists(lists)
    if out is None:
        out = torch.empty((S, H, D), dtype=q.dtype, device=q.device)
    elif out.shape != (S, H, D) or out.dtype != q.dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous [S, H, D] tensor of q's dtype")
    lse = torch.empty((S, H), dtype=torch.float32, device=q.device)
    R = max(plan.rows_total(H), 1)
    part_o = torch.empty((R, D), dtype=q.dtype, device=q.device)
    part_lse = torch.empty(R, dtype=torch.float32, device=q.device)
    with _timed("attn_fwd", q.device):
        call("moba_attn_fwd", _ptr(q), _ptr(k), _ptr(v), _DTYPES[q.dtype], H, q.stride(0), q.stride(1), kv,
             ctypes.byref(plan.info), _ptr(plan.meta), _ptr(list_off), _ptr(work_off), _ptr(list_tok), _ptr(tile_rec),
             _ptr(out), _ptr(lse), _ptr(part_o), _ptr(part_lse), parts, float(scale), _ptr(status), _dev_index(q),
             _stream(q.device))
    return out, lse, part_o, part_lse


def merge_fwd(out, lse, plan, part_o, part_lse, row_of):
    H = out.shape[1]
    with _timed("merge_fwd", out.device):
        call("moba_merge_fwd", _ptr(out), _ptr(lse), _DTYPES[out.dtype], H, ctypes.byref(plan.info), _ptr(part_o),
             _ptr(part_lse), _ptr(row_of), _dev_index(out), _stream(out.device))


def bwd_delta(out, d_out):
    S, H, _ = out.shape
    delta = torch.empty((S, H), dtype=torch.float32, device=out.device)
    with _timed("bwd_delta", out.device):
        call("moba_bwd_delta", _ptr(out), _ptr(d_out), _DTYPES[out.dtype], H, S, _ptr(delta), _dev_index(out),
             _stream(out.device))
    return delta


def gather_rows(q, d_out, plan, lists, lse, delta):
    """List-ordered copies of q / d_out rows and of their lse / delta: (qg, dog [R*H,128], lse_g, delta_g [R*H])."""
    S, H, D = q.shape
    list_off, work_off, list_tok, tile_rec = _split_lists(lists)
    R = max(plan.rows_total(H), 1)
    qg = torch.empty((R, D), dtype=q.dtype, device=q.device)
    dog = torch.empty((R, D), dtype=q.dtype, device=q.device)
    lse_g = torch.empty(R, dtype=torch.float32, device=q.device)
    delta_g = torch.empty(R, dtype=torch.float32, device=q.device)
    if plan.kk > 0:
        with _timed("gather_rows", q.device):
            call("moba_gather_rows", _ptr(q), _ptr(d_out), _ptr(lse), _ptr(delta), _DTYPES[q.dtype], H, q.stride(0),
                 q.stride(1), ctypes.byref(plan.info), _ptr(list_off), _ptr(work_off), _ptr(list_tok), _ptr(tile_rec),
                 _ptr(qg), _ptr(dog), _ptr(lse_g), _ptr(delta_g), _dev_index(q), _stream(q.device))
    return qg, dog, lse_g, delta_g


def attn_bwd_dkdv(q, k, v, d_out, plan, lists, lse, delta, status, parts=3, gathered=None, out=None, scale=0.0):
    """dk, dv [S_k, H_kv, D] (summed over the query heads that share a key/value head). `gathered` = (qg, dog,
    lse_g, delta_g) when the caller already holds the rows in list order (else they are produced here by
    gather_rows)."""
    H, D = q.shape[1], q.shape[2]
    kv = _kv_layout(q, k, v)
    list_off = lists[0]
    if gathered is None:
        gathered = gather_rows(q, d_out, plan, lists, lse, delta) if (parts & 2 and plan.kk > 0) else (None,) * 4
    qg, dog, lse_g, delta_g = gathered
    if out is not None:
        dk, dv = out              # contiguous [S_k, H_kv, D] buffers of the caller
    else:
        dk = torch.empty((k.shape[0], k.shape[1], D), dtype=q.dtype, device=q.device)
        dv = torch.empty((k.shape[0], k.shape[1], D), dtype=q.dtype, device=q.device)
    with _timed("attn_bwd_dkdv", q.device):
        call("moba_attn_bwd_dkdv", _ptr(q), _ptr(k), _ptr(v), _ptr(d_out), _DTYPES[q.dtype], H, q.stride(0),
             q.stride(1), kv, ctypes.byref(plan.info), _ptr(plan.meta), _ptr(list_off), _ptr(qg), _ptr(dog), _ptr(lse_g),
             _ptr(delta_g), _ptr(lse), _ptr(delta), _ptr(dk), _ptr(dv), parts, float(scale), _ptr(status), _dev_index(q),
             _stream(q.device))
    return dk, dv


_DQ_FORMS = {None: 0, "tile": 0x10, "persistent": 0x20}


def attn_bwd_dq(q, k, v, d_out, plan, lists, lse, delta, status, parts=3, gathered=None, scale=0.0, form=None):
    """Unrounded dq pieces: (dq_self [S,H,D] fp32, part_dq [R*H, D] fp32). `gathered` = (qg, dog, lse_g, delta_g),
    the rows in list order (gather_rows); produced here when not given. `form` names one of the kernel's two forms
    ("tile": one query tile per CTA, "persistent": one CTA per SM walking its tiles; same bits either way) instead of
    leaving the choice to the chunk size."""
    S, H, D = q.shape
    kv = _kv_layout(q, k, v)
    list_off, work_off, list_tok, tile_rec = _split_lists(lists)
    if gathered is None:
        gathered = gather_rows(q, d_out, plan, lists, lse, delta) if (parts & 2 and plan.kk > 0) else (None,) * 4
    qg, dog, lse_g, delta_g = gathered
    dq_self = torch.empty((S, H, D), dtype=torch.float32, device=q.device)
    part_dq = torch.empty((max(plan.rows_total(H), 1), D), dtype=torch.float32, device=q.device)
    with _timed("attn_bwd_dq", q.device):
        call("moba_attn_bwd_dq", _ptr(q), _ptr(k), _ptr(v), _ptr(d_out), _DTYPES[q.dtype], H, q.stride(0),
             q.stride(1), kv, ctypes.byref(plan.info), _ptr(plan.meta), _ptr(list_off), _ptr(work_off), _ptr(list_tok),
             _ptr(tile_rec), _ptr(qg), _ptr(dog), _ptr(lse_g), _ptr(delta_g), _ptr(lse), _ptr(delta), _ptr(dq_self),
             _ptr(part_dq),
             parts | _DQ_FORMS[form], float(scale), _ptr(status), _dev_index(q), _stream(q.device))
    return dq_self, part_dq


def merge_dq(dq_self, plan, part_dq, row_of, dtype, out=None):
    """dq [S,H,D] in `dtype`: fp32 sum of the self piece and the gathered pieces, rounded once."""
    S, H, D = dq_self.shape
    dq = out if out is not None else torch.empty((S, H, D), dtype=dtype, device=dq_self.device)
    with _timed("merge_dq", dq.device):
        call("moba_merge_dq", _ptr(dq), _DTYPES[dtype], H, ctypes.byref(plan.info), _ptr(dq_self), _ptr(part_dq),
             _ptr(row_of), _dev_index(dq), _stream(dq.device))
    return dq


def decode_attn(query, key, value, scaling=None, status=None):
    """Dense causal attention of [batch, q_heads, q_len, 128] queries over a [batch, kv_heads, kv_len, 128] cache,
    the mask aligned to the end of the keys; returns [batch, q_len, q_heads, 128]. 16-bit CUDA tensors only."""
    if query.dim() != 4 or key.dim() != 4 or key.shape != value.shape:
        raise ValueError("query / key / value must be [batch, heads, len, 128] with key.shape == value.shape")
    B, Hq, Lq, D = query.shape
    _, Hkv, Lk, _ = key.shape
    if D != _lib.HEAD_DIM or key.shape[3] != D or key.shape[0] != B:
        raise ValueError(f"head_dim must be {_lib.HEAD_DIM} and the batch sizes equal")
    if not query.is_cuda or query.dtype not in (torch.bfloat16, torch.float16) or key.dtype != query.dtype \
            or value.dtype != query.dtype:
        raise ValueError("decode_attn takes bf16 / fp16 CUDA tensors of one dtype")

    def evenly_spaced(t):            # innermost stride 1, 16-byte rows, (batch, head) pairs at one pitch
        return (t.stride(3) == 1 and t.stride(2) % 8 == 0 and t.stride(1) % 8 == 0
                and (t.shape[0] == 1 or t.stride(0) == t.shape[1] * t.stride(1)))

    if query.stride(3) != 1 or any(query.stride(i) % 8 for i in range(3)):
        query = query.contiguous()
    if not evenly_spaced(key) or not evenly_spaced(value) or key.stride() != value.stride():
        key, value = key.contiguous(), value.contiguous()
    scale = float(scaling) if scaling is not None else D ** -0.5
    dev = query.device
    out = torch.empty((B, Lq, Hq, D), dtype=query.dtype, device=dev)
    ws = torch.empty(max(_lib.lib.moba_decode_ws_floats(B, Hq, Hkv, Lq, Lk), 1), dtype=torch.float32, device=dev)
    own = status is None
    if own:
        status = new_status(dev)
    with _timed("decode_attn", dev):
        call("moba_decode_attn", _ptr(query), _ptr(key), _ptr(value), _DTYPES[query.dtype], B, Hq, Hkv, Lq, Lk,
             query.stride(0), query.stride(1), query.stride(2), key.stride(1), key.stride(2), scale, _ptr(out),
             _ptr(ws), _ptr(status), _dev_index(query), _stream(dev))
    if own:
        check_status(status)
    return out


def copy_heads(dst, src, stream):
    """dst[...] = src[...] between a pinned host tensor and a device tensor, both [S, h, D] views (heads sliced
    out of a wider tensor are fine), as one pitched copy on `stream`."""
    S, h, D = src.shape
    if dst.shape != src.shape or dst.dtype != src.dtype:
        raise ValueError("copy_heads needs equal shapes and dtypes")
    e = src.element_size()
    for t in (dst, src):
        if t.stride(2) != 1 or t.stride(1) != D:
            raise ValueError("copy_heads needs [S, h, D] views with contiguous heads")
    to_device = dst.is_cuda
    dev = dst.device if to_device else src.device
    call("moba_memcpy_2d", _ptr(dst), dst.stride(0) * e, _ptr(src), src.stride(0) * e, h * D * e, S,
         1 if to_device else 0, dev.index or 0, ctypes.c_void_p(stream.cuda_stream))


def selftest_umma(mode, a, b):
    """C = A*B^T (mode 0) or A*B (modes 1, 2) for 128x128 16-bit tiles; returns fp32 [128,128]."""
    c = torch.zeros((128, 128), dtype=torch.float32, device=a.device)
    status = new_status(a.device)
    call("moba_selftest_umma", mode, _ptr(a), _ptr(b), _ptr(c), _DTYPES[a.dtype], _ptr(status), _dev_index(a),
         _stream(a.device))
    check_status(status)
    return c


def selftest_umma_pair(q, k, v):
    """S = Q K^T and O = (S / 16, rounded to 16 bit) V for q [256,128], k, v [128,128], computed by a pair of CTAs
    with 256-row instructions; returns fp32 (S, O), [256,128] each."""
    s_out = torch.zeros((256, 128), dtype=torch.float32, device=q.device)
    o_out = torch.zeros((256, 128), dtype=torch.float32, device=q.device)
    status = new_status(q.device)
    call("moba_selftest_umma_pair", _ptr(q), _ptr(k), _ptr(v), _ptr(s_out), _ptr(o_out), _DTYPES[q.dtype],
         _ptr(status), _dev_index(q), _stream(q.device))
    check_status(status)
    return s_out, o_out


def selftest_wait_timeout(status, limit_ns=1_000_000, n_ctas=4):
    """Launches CTAs that wait on a barrier nothing arrives on; the waits run out after limit_ns and set `status`
    (a zeroed device word) to 1. The kernel frees its tensor memory and returns."""
    call("moba_selftest_wait_timeout", int(limit_ns), int(n_ctas), _ptr(status), _dev_index(status),
         _stream(status.device))
