"""MoBA attention for tensors that live in (pinned) host memory.

Heads are independent in MoBA (MoonshotAI/MoBA moba/moba_efficient.py works per head throughout), so a layer
whose q, k, v (and d_out) start on the host can be cut into head groups and pipelined: while the kernels of
group g run, the copy engines bring in group g + 1 and take the results of group g - 1 back. With PCIe moving
~50 GB/s per direction and the kernels needing ~3 ms per head at 128K tokens, the copies hide almost completely
behind the compute; issued back to back on one stream they add 40 % to a step.

`moba_attn_varlen_host` is the same operator as `moba_attn_varlen` (same argument meaning) with host tensors in
and host tensors out; it also peaks at 1 / head_groups of the device memory for intermediates.
"""
import time

import torch

from . import ops
from .moba_efficient import moba_attn_varlen


def _pinned(t, name):
    if t.device.type != "cpu":
        raise ValueError(f"{name} must be a host tensor")
    if not t.is_pinned():
        raise ValueError(f"{name} must be in pinned host memory (tensor.pin_memory()) for asynchronous copies")


def bind_host_to_device_numa(device):
    """Restricts the calling process to the CPUs of the NUMA node the GPU hangs off (read from sysfs), so that the
    pinned host buffers it allocates afterwards and the copy threads sit next to the GPU's PCIe root: with one
    process per GPU on a two-socket host, half the processes otherwise stream their tensors across the socket
    interconnect. Returns the node number, or None when the topology cannot be read (nothing is changed then)."""
    import os

    try:
        props = torch.cuda.get_device_properties(torch.device(device))
        bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                a, _, b = part.partition("-")
                cpus.update(range(int(a), int(b or a) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except (OSError, ValueError, AttributeError):
        return None


def host_numa_nodes():
    """{node: set of CPUs} for the NUMA nodes of this host that have CPUs (from sysfs); empty if unreadable."""
    import glob
    import os

    nodes = {}
    try:
        for path in glob.glob("/sys/devices/system/node/node[0-9]*"):
            with open(os.path.join(path, "cpulist")) as f:
                text = f.read().strip()
            cpus = set()
            for part in text.split(",") if text else []:
                a, _, b = part.partition("-")
                cpus.update(range(int(a), int(b or a) + 1))
            if cpus:
                nodes[int(os.path.basename(path)[4:])] = cpus
    except (OSError, ValueError):
        return {}
    return nodes


def moba_attn_varlen_host(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk, d_out=None, out=None,
                          grads=None, head_groups=4, device=None, out_device=None, stats=None, duplex=True):
    """MoBA attention (and, with d_out, its backward) on pinned host tensors [seqlen, head, head_dim].

    Args:
        q, k, v, d_out: pinned host tensors, bf16 / fp16; d_out=None runs the forward only. k and v may carry
            fewer heads than q (grouped-query attention); dk / dv then have their shape
        cu_seqlens: int32 cumulative sequence lengths on `device` (as for moba_attn_varlen)
        out: pinned host tensor to receive the output (allocated when None)
        grads: (dq, dk, dv) pinned host tensors to receive the gradients (allocated when None and d_out is given)
        head_groups: number of head slices in flight one after the other (clamped to the key/value head count);
            with more than one, the first and the last slice are additionally cut down to one key/value head
        duplex: True -- two staging sets, copy-in of slice g + 1 and copy-out of slice g - 1 run beside the kernels of
            slice g on two copy streams (both directions of the link at once). False -- every slice has its own
            staging set, all copy-ins are queued first and the copy-outs follow them on the same stream, so the link
            carries one direction at a time: for hosts on which many GPUs copy at once and simultaneous reads and
            writes of host memory slow each other down (measured with eight ranks on one host)
        out_device: optional device tensor [seqlen, head, head_dim] that also receives the output (e.g. to feed
            a collective); written on the current stream
        stats: optional dict; receives "h2d" and "d2h", lists of (bytes, milliseconds) per head slice measured with
            events on the two copy streams (the achieved copy rates of the slices), "timeline" (per slice, milliseconds
            from the start of the call at which its copy-in, kernels and copy-out begin and end on the device) and
            "host_issue_ms" (host time until everything was enqueued)
    Returns:
        out, or (out, (dq, dk, dv)) when d_out is given. The results are complete when this function returns.
    """
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    for name, t in (("q", q), ("k", k), ("v", v)):
        _pinned(t, name)
    if d_out is not None:
        _pinned(d_out, "d_out")
    S, H, D = q.shape
    Hkv = k.shape[1]
    if k.shape != v.shape or k.shape[0] != S or k.shape[2] != D or Hkv < 1 or H % Hkv != 0:
        raise ValueError("k and v must be [seqlen, kv_heads, head_dim] with kv_heads dividing the heads of q")
    rep = H // Hkv                      # grouped-query K / V: head slices are cut between key/value heads
    backward = d_out is not None
    if out is None:
        out = torch.empty_like(q).pin_memory()
    if backward and grads is None:
        grads = (torch.empty_like(q).pin_memory(), torch.empty_like(k).pin_memory(), torch.empty_like(v).pin_memory())
    groups = max(1, min(int(head_groups), Hkv))
    kv_bounds = [Hkv * g // groups for g in range(groups + 1)]
    if groups > 1:
        # Nothing hides the copy-in of the first slice and the copy-out of the last one: make those two slices one
        # key/value head wide (a slice computes ~4x longer than it copies, so the second slice still arrives in time)
        if kv_bounds[1] - kv_bounds[0] > 1:
            kv_bounds.insert(1, kv_bounds[0] + 1)
        if kv_bounds[-1] - kv_bounds[-2] > 1:
            kv_bounds.insert(len(kv_bounds) - 1, kv_bounds[-1] - 1)
        groups = len(kv_bounds) - 1
    bounds = [b * rep for b in kv_bounds]

    compute = torch.cuda.current_stream(device)
    s_in = torch.cuda.Stream(device)
    s_out = torch.cuda.Stream(device) if duplex else s_in
    s_in.wait_stream(compute)
    # input staging buffers: two sets (group g + 1 is copied in while group g computes), or one per group
    n_sets = 2 if duplex else groups
    width = max(b - a for a, b in zip(bounds, bounds[1:]))
    srcs = (q, k, v, d_out) if backward else (q, k, v)
    is_kv = (False, True, True, False)
    stage = [[torch.empty((S, width // rep if kv else width, D), dtype=q.dtype, device=device)
              for kv in is_kv[:len(srcs)]] for _ in range(n_sets)]
    ev_in = [torch.cuda.Event() for _ in range(groups)]
    ev_done = [torch.cuda.Event() for _ in range(groups)]
    timed = stats is not None
    t_in = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(groups)] if timed else None
    t_out = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(groups)] if timed else None
    t_run = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(groups)] if timed else None
    if timed:
        t_base = torch.cuda.Event(enable_timing=True)
        t_base.record(compute)
        host_t0 = time.perf_counter()
    n_in = [0] * groups
    n_out = [0] * groups

    def copy_in(g):
        with torch.cuda.stream(s_in):
            if g >= n_sets:
                s_in.wait_event(ev_done[g - n_sets])     # the staging set is free again
            if timed:
                t_in[g][0].record(s_in)
            for dst, src, kv in zip(stage[g % n_sets], srcs, is_kv):
                h0, h1 = (kv_bounds[g], kv_bounds[g + 1]) if kv else (bounds[g], bounds[g + 1])
                ops.copy_heads(dst[:, : h1 - h0], src[:, h0:h1], s_in)
                n_in[g] += S * (h1 - h0) * D * src.element_size()
            if timed:
                t_in[g][1].record(s_in)
            ev_in[g].record(s_in)

    for g in range(1 if duplex else groups):
        copy_in(g)
    for g in range(groups):
        if duplex and g + 1 < groups:
            copy_in(g + 1)
        h0, h1 = bounds[g], bounds[g + 1]
        k0, k1 = kv_bounds[g], kv_bounds[g + 1]
        compute.wait_event(ev_in[g])
        if timed:
            t_run[g][0].record(compute)
        ins = [t[:, : (k1 - k0) if kv else (h1 - h0)] for t, kv in zip(stage[g % n_sets], is_kv)]
        if backward:
            tq, tk, tv = (t.detach().requires_grad_() for t in ins[:3])
            o = moba_attn_varlen(tq, tk, tv, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk)
            o.backward(ins[3])
            results = [(out, o.detach(), h0, h1), (grads[0], tq.grad, h0, h1), (grads[1], tk.grad, k0, k1),
                       (grads[2], tv.grad, k0, k1)]
        else:
            with torch.no_grad():
                o = moba_attn_varlen(ins[0], ins[1], ins[2], cu_seqlens, max_seqlen, moba_chunk_size, moba_topk)
            results = [(out, o, h0, h1)]
        if out_device is not None:
            out_device[:, h0:h1].copy_(results[0][1])
        if timed:
            t_run[g][1].record(compute)
        ev_done[g].record(compute)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[g])
            if timed:
                t_out[g][0].record(s_out)
            for dst, src, a, b in results:
                src.record_stream(s_out)
                ops.copy_heads(dst[:, a:b], src if src.is_contiguous() else src.contiguous(), s_out)
                n_out[g] += src.numel() * src.element_size()
            if timed:
                t_out[g][1].record(s_out)
    compute.wait_stream(s_out)
    compute.wait_stream(s_in)
    for buf in (b for bufs in stage for b in bufs):
        buf.record_stream(s_in)
    if timed:
        stats["host_issue_ms"] = (time.perf_counter() - host_t0) * 1e3
    torch.cuda.current_stream(device).synchronize()
    if timed:
        stats["timeline"] = [[round(t_base.elapsed_time(e), 2) for pair in (t_in[g], t_run[g], t_out[g]) for e in pair]
                             for g in range(groups)]
        stats["h2d"] = [(n_in[g], t_in[g][0].elapsed_time(t_in[g][1])) for g in range(groups)]
        stats["d2h"] = [(n_out[g], t_out[g][0].elapsed_time(t_out[g][1])) for g in range(groups)]
        stats["slices"] = [b - a for a, b in zip(bounds, bounds[1:])]
    return (out, grads) if backward else out
