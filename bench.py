"""Benchmark of the MoBA attention layer (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 3]

Workload (N = 1 and N > 1): a Llama-3.1-8B attention-layer shape -- one 131072-token sequence, 32 query heads,
8 KV heads repeated to 32, head_dim 128, bf16 N(0,1) with a per-chunk key offset ~ N(0, 0.5), chunk 4096,
top-k 12, forward + backward. Seeded synthetic tensors stand in for real activations. With N GPUs the 32 heads
are split N ways (strong scaling); ranks exchange nothing on the data path except the forward output, which
is all-gathered over NCCL.

Prints ONE JSON line (rank 0). `value` = selected-block FLOPs (14 * D * pairs) / step time, inputs resident
in HBM; `e2e` = the same through moba_attn_varlen_host with host (pinned) tensors in and out, the copies inside
the timed region (head groups pipelined: copy engines and kernels overlap);
`roofline` = the dominant kernel group against the measured dense bf16 peak; `cpu_baseline` = the reference's own
moba_attn_varlen_naive (installed unmodified under baseline/_ref by baseline/install_reference.sh; pure torch) on
this box's host cores over a bounded sample of the workload -- the numpy port in oracle/ only if that install is
missing, and the line says which (`kind`). `--impl reference` times that CPU function alone, with all host threads,
on the same metric and unit. `checksums` = CRC32 of the bf16 bits of a few heads of out (after the head re-layout of
the gathered output when N > 1) and of rank 0's first head of dq / dk / dv: equal across N = 1 / 2 / 4 / 8.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D = 128
CONFIGS = {
    # name: (lengths, heads, kv_heads, chunk, topk, key_offset_std, backward)
    2: dict(lens=[32768], heads=1, kv_heads=1, chunk=2048, topk=3, off_std=0.0, backward=True),
    3: dict(lens=[131072], heads=32, kv_heads=8, chunk=4096, topk=12, off_std=0.5, backward=True),
    # a slice of config 3 (same chunk / top-k, 4 heads, 32768 tokens) small enough for an ncu capture
    30: dict(lens=[32768], heads=4, kv_heads=1, chunk=4096, topk=12, off_std=0.5, backward=True),
    31: dict(lens=[131072], heads=4, kv_heads=1, chunk=4096, topk=12, off_std=0.5, backward=True),
    # varlen training batch: 16 sequences, lengths 512 * randint(8, 128) from random.Random(0)
    4: dict(lens=None, heads=32, kv_heads=32, chunk=512, topk=3, off_std=0.0, backward=True),
    # a 2-head slice of it, small enough for an ncu capture
    41: dict(lens=None, heads=2, kv_heads=2, chunk=512, topk=3, off_std=0.0, backward=True),
    # 1M-token prefill, forward only (meant for 8 GPUs, 4 heads each); 51 = one GPU's share of it
    5: dict(lens=[1048576], heads=32, kv_heads=8, chunk=4096, topk=12, off_std=0.5, backward=False),
    51: dict(lens=[1048576], heads=4, kv_heads=1, chunk=4096, topk=12, off_std=0.5, backward=False),
    # decode step of the layer wrapper (dense attention of one new token over the cache, grouped-query heads): not
    # the headline metric -- a bandwidth line for the decode kernel; 60 = a smaller cache for an ncu capture
    6: dict(decode=True, batch=8, heads=32, kv_heads=8, q_len=1, kv_len=32768),
    60: dict(decode=True, batch=2, heads=32, kv_heads=8, q_len=1, kv_len=32768),
}


def _varlen_lengths(seed=0, n=16):
    import random

    rnd = random.Random(seed)
    return [512 * rnd.randint(8, 128) for _ in range(n)]      # 630272 tokens, longest sequence 64000


CONFIGS[4]["lens"] = _varlen_lengths()
CONFIGS[41]["lens"] = _varlen_lengths()


def selected_pairs(lens, chunk, topk):
    pairs = 0
    for n in lens:
        nb = (n + chunk - 1) // chunk
        for c in range(nb):
            cs = min(chunk, n - c * chunk)
            pairs += cs * (cs + 1) // 2 + chunk * cs * min(c, topk - 1)
    return pairs


_RESULT_STREAM = None


def claim_stdout():
    """stdout carries exactly one JSON line. Libraries print there too (NCCL's version banner is a plain printf on
    file descriptor 1), so descriptor 1 is pointed at stderr for the rest of the run and the result line goes to a
    duplicate of the original stdout."""
    global _RESULT_STREAM
    sys.stdout.flush()
    _RESULT_STREAM = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)


def emit(line):
    out = _RESULT_STREAM if _RESULT_STREAM is not None else sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def read_traffic_table():
    """(chunk, top-k, lengths, kernel) -> DRAM bytes per head and launch, from profiles/dram_traffic_per_head.txt
    (lines: kernel chunk topk tokens bytes_per_head; '#' starts a comment). Empty when the file is missing."""
    table = {}
    path = os.path.join(ROOT, "profiles", "dram_traffic_per_head.txt")
    if os.path.exists(path):
        with open(path) as f:
            for line in f:
                fields = line.split("#")[0].split()
                if len(fields) == 5:
                    table[(int(fields[1]), int(fields[2]), (int(fields[3]),), fields[0])] = float(fields[4])
    return table


# ----------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_uuid):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        cmd = ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"]
        if gpu_uuid:
            cmd.insert(1, f"--id={gpu_uuid}")
        try:
            self.proc = subprocess.Popen(cmd, stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for nm, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        self.file.close()
        os.unlink(self.file.name)
        if sm:
            sm.sort()
            out.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=max(smax), reasons=sorted(reasons), samples=len(sm))
        return out


# ----------------------------------------------------------------------------------------------- inputs
def make_inputs(cfg_id, cfg, head_lo, head_hi, device):
    """q, k, v, d_out [S, heads_local, 128] bf16 for heads [head_lo, head_hi). Values depend only on the head
    index (per-head generators), so any head sharding sees identical numbers. K/V come from kv_heads heads,
    each repeated heads/kv_heads times (the repeat_interleave of the reference's wrapper)."""
    import torch

    S = sum(cfg["lens"])
    rep = cfg["heads"] // cfg["kv_heads"]
    n = head_hi - head_lo
    q = torch.empty((S, n, D), dtype=torch.bfloat16, device=device)
    k = torch.empty_like(q)
    v = torch.empty_like(q)
    d_out = torch.empty_like(q)
    n_chunks = sum((l + cfg["chunk"] - 1) // cfg["chunk"] for l in cfg["lens"])
    kv_cache = {}
    for i, h in enumerate(range(head_lo, head_hi)):
        g = torch.Generator(device=device).manual_seed(1000 * cfg_id + h)
        q[:, i] = torch.randn(S, D, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        d_out[:, i] = torch.randn(S, D, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        kvh = h // rep
        if kvh not in kv_cache:
            gk = torch.Generator(device=device).manual_seed(1000 * cfg_id + 500 + kvh)
            kk = torch.randn(S, D, generator=gk, device=device, dtype=torch.float32)
            vv = torch.randn(S, D, generator=gk, device=device, dtype=torch.float32)
            if cfg["off_std"] > 0:
                off = torch.randn(n_chunks, D, generator=gk, device=device, dtype=torch.float32) * cfg["off_std"]
                pos = 0
                c = 0
                for l in cfg["lens"]:
                    for c0 in range(0, l, cfg["chunk"]):
                        c1 = min(c0 + cfg["chunk"], l)
                        kk[pos + c0:pos + c1] += off[c]
                        c += 1
                    pos += l
            kv_cache = {kvh: (kk.to(torch.bfloat16), vv.to(torch.bfloat16))}
        k[:, i], v[:, i] = kv_cache[kvh]
    return q, k, v, d_out


# ----------------------------------------------------------------------------------------------- CPU arm
def _cpu_inputs(cfg_id, cfg, tokens):
    """First `tokens` tokens of one head of the workload's value distribution, as fp32 numpy arrays holding bf16
    values (seeded; the same numbers for the reference function and for the numpy port)."""
    import numpy as np
    from oracle import moba_oracle as orc

    rng = np.random.RandomState(1000 * cfg_id)
    q, k, v, d_out = (orc.round_bf16(rng.randn(tokens, 1, D).astype(np.float32)) for _ in range(4))
    if cfg["off_std"] > 0:
        nb = (tokens + cfg["chunk"] - 1) // cfg["chunk"]
        off = rng.randn(nb, 1, D).astype(np.float32) * cfg["off_std"]
        k = orc.round_bf16(k + np.repeat(off, cfg["chunk"], axis=0)[:tokens])
    return q, k, v, d_out


def cpu_sample(cfg_id, cfg, tokens, threads):
    """Times the reference's CPU implementation of the path, moba_attn_varlen_naive (forward + backward through
    torch autograd), on the first `tokens` tokens of one head of the workload; the numpy port of the same function
    when the reference is not installed under baseline/_ref. Returns (tflops, seconds, description, kind)."""
    from baseline import reference as ref

    q, k, v, d_out = _cpu_inputs(cfg_id, cfg, tokens)
    pairs = selected_pairs([tokens], cfg["chunk"], cfg["topk"])
    flops = (14 if cfg["backward"] else 4) * D * pairs
    what = (f"fwd{'+bwd' if cfg['backward'] else ''}, first {tokens} tokens of 1 head of the workload "
            f"(chunk {cfg['chunk']}, top-k {cfg['topk']}), {threads} threads")
    if ref.available():
        import torch

        naive = ref.load_naive()
        torch.set_num_threads(threads)
        tq, tk, tv, tdo = (torch.from_numpy(x).to(torch.bfloat16) for x in (q, k, v, d_out))
        if cfg["backward"]:
            tq.requires_grad_(), tk.requires_grad_(), tv.requires_grad_()
        cu = torch.tensor([0, tokens], dtype=torch.int32)
        t0 = time.perf_counter()
        out = naive(tq, tk, tv, cu, tokens, cfg["chunk"], cfg["topk"])
        if cfg["backward"]:
            out.backward(tdo)
        secs = time.perf_counter() - t0
        return flops / secs / 1e12, secs, "reference moba_attn_varlen_naive (torch, fp32 math on bf16 inputs) " + what, "reference"

    from oracle import moba_oracle as orc

    try:
        from threadpoolctl import threadpool_limits
    except ImportError:
        threadpool_limits = None

    def run():
        t0 = time.perf_counter()
        orc.moba_attn_varlen_oracle(q, k, v, [0, tokens], tokens, cfg["chunk"], cfg["topk"], "bf16",
                                    d_out=d_out if cfg["backward"] else None)
        return time.perf_counter() - t0

    if threadpool_limits is not None:
        with threadpool_limits(limits=threads):
            secs = run()
    else:
        secs = run()
    return flops / secs / 1e12, secs, "numpy port of moba_attn_varlen_naive (baseline/_ref not installed) " + what, "port"


def cpu_sample_bounded(cfg_id, cfg, tokens, threads, min_seconds=10.0, max_repeats=16):
    """cpu_sample repeated until it has run for at least min_seconds (10-30 s of CPU work whatever the number of
    host cores): the token count stays bounded by the dense function's O(tokens^2) memory, the duration by the
    repeats. Returns (tflops over all repeats, total seconds, description, kind)."""
    total, n = 0.0, 0
    flops_s = 0.0
    while n < max_repeats and (n == 0 or total < min_seconds):
        tf, secs, desc, kind = cpu_sample(cfg_id, cfg, tokens, threads)
        flops_s += tf * secs
        total += secs
        n += 1
    return flops_s / total, total, desc + (f", run {n} times" if n > 1 else ""), kind


def cpu_sample_tokens(cfg):
    """Bounded sample: the dense reference function needs O(tokens^2) fp32 per head (1 GB per [tokens, tokens]
    tensor at 16384 tokens); cpu_sample_bounded repeats it up to the wanted duration."""
    return min(16384, sum(cfg["lens"]) if len(cfg["lens"]) == 1 else max(cfg["lens"]))


def run_reference_arm(args, cfg_id, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    tokens = cpu_sample_tokens(cfg)
    for _ in range(args.warmup):
        cpu_sample(cfg_id, cfg, min(tokens, 4096), threads)
    vals, secs = [], []
    for _ in range(args.steps):
        tf, s_, desc, kind = cpu_sample_bounded(cfg_id, cfg, tokens, threads)
        vals.append(tf)
        secs.append(s_)
    value = sum(vals) / len(vals)
    line = {
        "impl": "reference", "metric": "moba_layer_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * sum(secs) / len(secs), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg_id, cfg, args.gpus),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": desc},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "the reference's GPU path needs flash-attn kernels; this arm times its own CPU implementation "
                "(moba_naive) on the host cores over a bounded sample: each step is the sample named in "
                "cpu_baseline.sample, not the whole workload",
    }
    emit(line)


def workload_config(cfg_id, cfg, n_gpus):
    return {
        "workload": f"config{cfg_id}: {len(cfg['lens'])} sequence(s), {sum(cfg['lens'])} tokens, {cfg['heads']} heads "
                    f"({cfg['kv_heads']} KV heads repeated), head_dim {D}, chunk {cfg['chunk']}, top-k {cfg['topk']}, "
                    f"forward{'+backward' if cfg['backward'] else ''}",
        "tokens": sum(cfg["lens"]), "heads": cfg["heads"], "kv_heads": cfg["kv_heads"], "head_dim": D,
        "moba_chunk_size": cfg["chunk"], "moba_topk": cfg["topk"],
        "parallelism": f"head-parallel x{n_gpus}" if n_gpus > 1 else "single GPU",
        "l2_policy": "inputs_exceed_l2",
    }


# ----------------------------------------------------------------------------------------------- GPU arm
def run_ours(args, cfg_id, cfg):
    import torch
    import torch.distributed as dist

    from moba_b200 import ops
    from moba_b200.host_io import moba_attn_varlen_host
    from moba_b200.moba_efficient import check_kernel_status, moba_attn_varlen

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run --nproc-per-node N")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    # the pinned host buffers of the end-to-end leg should sit on the GPU's NUMA node (one process per GPU)
    from moba_b200.host_io import bind_host_to_device_numa, host_numa_nodes

    numa_node = None if args.no_numa_bind else bind_host_to_device_numa(dev)
    if world > 1:
        # keep stdout to the one JSON line: NCCL's version / info banner goes to a file instead
        os.environ.setdefault("NCCL_DEBUG_FILE", os.path.join(tempfile.gettempdir(), "nccl_debug.%h.%p.log"))
        dist.init_process_group("nccl", device_id=dev)
    H = cfg["heads"]
    if H % world != 0:
        raise SystemExit(f"{H} heads do not split over {world} GPUs")
    hl = H // world
    S = sum(cfg["lens"])
    q, k, v, d_out = make_inputs(cfg_id, cfg, rank * hl, (rank + 1) * hl, dev)
    q.requires_grad_()
    k.requires_grad_()
    v.requires_grad_()
    cu_list = [0]
    for l in cfg["lens"]:
        cu_list.append(cu_list[-1] + l)
    cu = torch.tensor(cu_list, dtype=torch.int32, device=dev)
    out_all = torch.empty((world * S, hl, D), dtype=torch.bfloat16, device=dev) if world > 1 else None

    # forward-only runs on several GPUs: two head groups, so that the output gather of the first overlaps the
    # kernels of the second (with a backward pass the gather overlaps that instead)
    split = world > 1 and not cfg["backward"] and hl >= 2
    groups = [(0, hl // 2), (hl // 2, hl)] if split else [(0, hl)]
    out_grp = [torch.empty((world * S, b - a, D), dtype=torch.bfloat16, device=dev) for a, b in groups] if split else None

    def step():
        q.grad = k.grad = v.grad = None
        if split:
            works = []
            for g, (a, b) in enumerate(groups):
                with torch.no_grad():
                    o = moba_attn_varlen(q[:, a:b], k[:, a:b], v[:, a:b], cu, max(cfg["lens"]), cfg["chunk"], cfg["topk"])
                works.append(dist.all_gather_into_tensor(out_grp[g], o, async_op=True))
            for w in works:
                w.wait()
            return o
        out = moba_attn_varlen(q, k, v, cu, max(cfg["lens"]), cfg["chunk"], cfg["topk"])
        work = dist.all_gather_into_tensor(out_all, out.detach(), async_op=True) if world > 1 else None
        if cfg["backward"]:
            out.backward(d_out)
        if work is not None:
            work.wait()
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(args.warmup):
        step()
    check_kernel_status(dev)
    barrier()

    # ---- timed region: device-resident inputs ------------------------------------------------------
    uuid = None
    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(dev).uuid)
    except Exception:
        pass
    sampler = ClockSampler(uuid) if rank == 0 else None
    records = []
    ops.set_timing(records)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ops.set_timing(None)
    ms_total = e0.elapsed_time(e1)
    check_kernel_status(dev)
    clocks = sampler.stop() if sampler else None
    t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps

    per_kernel = {}
    for name, a, b in records:
        per_kernel.setdefault(name, []).append(a.elapsed_time(b))
    kernel_ms = {n: sum(x) / args.steps for n, x in per_kernel.items()}      # per step (a kernel may run twice)

    # ---- end to end: host tensors in, host tensors out -----------------------------------------------
    e2e = None
    if not args.no_e2e:
        hq, hk, hv, hdo = (t_.detach().to("cpu").pin_memory() for t_ in (q, k, v, d_out))
        ho = torch.empty_like(hq).pin_memory()
        hgrads = [torch.empty_like(hq).pin_memory() for _ in range(3)] if cfg["backward"] else []

        out_dev = torch.empty((S, hl, D), dtype=torch.bfloat16, device=dev) if world > 1 else None

        copy_stats = {}
        # eight ranks copying in both directions at once slow each other down on the host side (measured: a slice
        # copy takes 3-5x longer while the other direction is busy); one direction at a time is faster there
        duplex = args.copy_order == "duplex" or (args.copy_order == "auto" and world < 8)

        def e2e_step(stats=None):
            # host tensors in, host tensors out, through the package's host entry point: head groups are
            # pipelined so that the H2D / D2H copies of one group overlap with the kernels of another
            moba_attn_varlen_host(hq, hk, hv, cu, max(cfg["lens"]), cfg["chunk"], cfg["topk"],
                                  d_out=hdo if cfg["backward"] else None, out=ho,
                                  grads=tuple(hgrads) if cfg["backward"] else None, head_groups=args.head_groups,
                                  device=dev, out_device=out_dev, stats=stats, duplex=duplex)
            if world > 1:
                dist.all_gather_into_tensor(out_all, out_dev)

        e2e_steps = max(1, min(args.steps, 3))
        e2e_step(copy_stats)          # untimed first call, with the per-slice copy rates recorded
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(e2e_steps):
            e2e_step()
        s1.record()
        barrier()
        te = torch.tensor([s0.elapsed_time(s1)], dtype=torch.float64, device=dev)
        own_ms = float(te.item()) / e2e_steps
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_ms = float(te.item()) / e2e_steps
        steady = {}
        if world > 1:
            e2e_step(steady)          # one more untimed call: the device timeline of a step in steady state
            barrier()
        nbytes = hq.numel() * 2
        e2e = dict(ms=e2e_ms, h2d=4 * nbytes if cfg["backward"] else 3 * nbytes,
                   d2h=(4 if cfg["backward"] else 1) * nbytes)
        if copy_stats:
            def rate(key):
                return [round(b / ms / 1e6, 1) if ms > 0 else None for b, ms in copy_stats[key]]

            e2e["copy_rates"] = {"head_slices": copy_stats["slices"], "h2d_gbs_per_slice": rate("h2d"),
                                 "d2h_gbs_per_slice": rate("d2h"), "host_numa_node": numa_node,
                                 "host_numa_nodes": {str(n): len(c) for n, c in sorted(host_numa_nodes().items())}}
        if world > 1:
            # every rank's own end-to-end time and slowest slice copies: the ranks share the host's memory system
            mine = {"ms": round(own_ms, 2)}
            if copy_stats:
                mine["h2d_min_gbs"] = min((x for x in e2e["copy_rates"]["h2d_gbs_per_slice"] if x), default=None)
                mine["d2h_min_gbs"] = min((x for x in e2e["copy_rates"]["d2h_gbs_per_slice"] if x), default=None)
            if steady:
                # [copy-in begin, end, kernels begin, end, copy-out begin, end] per head slice, ms from the call
                mine["timeline_ms"] = steady["timeline"]
                mine["host_issue_ms"] = round(steady["host_issue_ms"], 2)
            mine["copy_order"] = "duplex" if duplex else "in-first"
            mine["numa_node"] = numa_node
            per_rank = [None] * world
            dist.all_gather_object(per_rank, mine)
            e2e["per_rank"] = per_rank
    check_kernel_status(dev)

    # ---- checksums (outside every timed region): equal bits at every N ---------------------------------
    import zlib

    from moba_b200 import head_parallel

    def head_crc(t, h):
        return zlib.crc32(t[:, h].contiguous().view(torch.int16).cpu().numpy().tobytes())

    last = step()
    full = head_parallel.gather_heads(last.detach()) if world > 1 else last.detach()      # [S, H, D], heads in order
    checksums = {f"out_h{h}": head_crc(full, h) for h in sorted({0, H // 2 - 1 if H > 1 else 0, H - 1})}
    if cfg["backward"]:
        checksums.update(dq_h0=head_crc(q.grad, 0), dk_h0=head_crc(k.grad, 0), dv_h0=head_crc(v.grad, 0))
    del full, last

    secondary = None
    if args.config == 3 and not args.no_secondary:
        q = k = v = d_out = out_all = None
        torch.cuda.empty_cache()
        secondary = measure_prefill_1m(world, rank, dev)

    if rank == 0:
        peaks = read_peaks()
        pairs = selected_pairs(cfg["lens"], cfg["chunk"], cfg["topk"]) * H
        flops = (14 if cfg["backward"] else 4) * D * pairs
        value = flops / (ms_step * 1e-3) / 1e12
        pairs_local = pairs // world
        # executed tile products per kernel group: the forward runs 2 products per (query tile, key tile) pair, the
        # key/value-side backward 4 (S^T, dP^T, dV, dK) and the query-side backward 3 (S, dP, dQ): the split
        # backward recomputes S and dP, so it executes 14 D pairs where 10 D pairs are counted
        group_flops = {"attn_fwd": 4 * D * pairs_local, "attn_bwd_dkdv": 8 * D * pairs_local,
                       "attn_bwd_dq": 6 * D * pairs_local}
        dom = max((n for n in group_flops if n in kernel_ms), key=lambda n: kernel_ms[n], default=None)
        roofline = None
        if dom:
            ach = group_flops[dom] / (kernel_ms[dom] * 1e-3) / 1e12
            peak = peaks["bf16_tflops_sustained"]
            # DRAM bytes per launch: measured per head on a 4-head slice of this workload (one ncu capture per
            # kernel, listed in the traffic table next to the profiles); proportional to the heads a launch covers
            traffic = None
            per_head = read_traffic_table().get((cfg["chunk"], cfg["topk"], tuple(cfg["lens"]), dom))
            if per_head is not None:
                traffic = per_head * (H // world)
            roofline = {"kernel": dom, "bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s",
                        "frac": ach / peak, "traffic": traffic, "peak_source": peaks["source"] + " (sustained bf16)",
                        "ms_per_launch_group": kernel_ms[dom]}
        threads = os.cpu_count() or 1
        if args.no_cpu_baseline:
            cpu = None
        else:
            tf, secs, desc, kind = cpu_sample_bounded(cfg_id, cfg, cpu_sample_tokens(cfg), threads)
            cpu = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": desc,
                   "seconds": secs}
        line = {
            "metric": "moba_layer_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(cfg_id, cfg, world),
            "frac_of_bf16_peak": value / (world * peaks["bf16_tflops_sustained"]),
            "kernel_ms": kernel_ms, "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
            "gpu_launches": len(records) and args.steps * launches_per_step(cfg, world),
            "checksums": checksums,
        }
        if world > 1:
            line["config"]["timed_gather_layout"] = ("rank-major [N, S, H/N, D] as the collective lands it; the "
                                                     "[S, H, D] re-layout is applied for `checksums` only")
        if secondary:
            line["secondary"] = secondary
        if e2e:
            line["e2e"] = {"value": flops / (e2e["ms"] * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e["ms"],
                           "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"]}
            if "copy_rates" in e2e:
                line["e2e"]["copy_rates_rank0"] = e2e["copy_rates"]
            if "per_rank" in e2e:
                line["e2e"]["per_rank"] = e2e["per_rank"]
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def measure_prefill_1m(world, rank, dev, steps=3, warmup=1):
    """The 1M-token forward-only configuration (config 5: 1048576 tokens, 32 heads from 8 KV heads, chunk 4096,
    top-k 12) beside the headline line, so that its curve over N is visible too: every rank runs its 32 / N heads in
    groups of at most 4 and all-gathers each group's output (NCCL) while the next group computes."""
    import torch
    import torch.distributed as dist

    from moba_b200.moba_efficient import check_kernel_status, moba_attn_varlen

    cfg = CONFIGS[5]
    S, H = sum(cfg["lens"]), cfg["heads"]
    hl = H // world
    q, k, v, _ = make_inputs(5, cfg, rank * hl, (rank + 1) * hl, dev)
    cu = torch.tensor([0, S], dtype=torch.int32, device=dev)
    gw = min(4, hl)
    groups = [(a, min(a + gw, hl)) for a in range(0, hl, gw)]
    gathered = [torch.empty((world * S, b - a, D), dtype=torch.bfloat16, device=dev) for a, b in groups[:2]] if world > 1 else None

    def step():
        works = []
        for g, (a, b) in enumerate(groups):
            with torch.no_grad():
                o = moba_attn_varlen(q[:, a:b], k[:, a:b], v[:, a:b], cu, S, cfg["chunk"], cfg["topk"])
            if world > 1:
                if len(works) >= 2:
                    works.pop(0).wait()
                works.append(dist.all_gather_into_tensor(gathered[g % 2], o, async_op=True))
        for w in works:
            w.wait()

    for _ in range(warmup):
        step()
    check_kernel_status(dev)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    check_kernel_status(dev)
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / steps
    flops = 4 * D * selected_pairs(cfg["lens"], cfg["chunk"], cfg["topk"]) * H
    return {"metric": "moba_layer_fwd_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "ms_per_step": ms, "steps": steps, "warmup": warmup, "n_gpus": world, "scaling": "strong",
            "config": workload_config(5, cfg, world)}


def run_decode(args, cfg_id, cfg):
    """One step = one decode attention call (K / V of the whole cache read once, larger than L2)."""
    import torch

    from moba_b200 import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, Hq, Hkv, Lq, Lk = cfg["batch"], cfg["heads"], cfg["kv_heads"], cfg["q_len"], cfg["kv_len"]
    g = torch.Generator(device=dev).manual_seed(0)
    q = torch.randn(B, Hq, Lq, D, device=dev, dtype=torch.bfloat16, generator=g)
    k = torch.randn(B, Hkv, Lk, D, device=dev, dtype=torch.bfloat16, generator=g)
    v = torch.randn(B, Hkv, Lk, D, device=dev, dtype=torch.bfloat16, generator=g)
    status = ops.new_status(dev)
    for _ in range(max(args.warmup, 3)):
        ops.decode_attn(q, k, v, None, status=status)
    torch.cuda.synchronize()
    sampler = ClockSampler(None)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        ops.decode_attn(q, k, v, None, status=status)
    t1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ops.check_status(status)
    ms = t0.elapsed_time(t1) / args.steps
    peaks = read_peaks()
    kv_bytes = 2 * B * Hkv * Lk * D * 2
    gbs = kv_bytes / ms / 1e6
    emit({
        "metric": "decode attention: key/value cache bytes read per second", "value": gbs, "unit": "GB/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"config{cfg_id}: decode, batch {B}, {Hq} query / {Hkv} key-value heads, q_len {Lq}, "
                               f"cache of {Lk} positions, head_dim {D}; inputs ({kv_bytes >> 20} MiB) larger than L2"},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"]},
        "gpu_launches": 2 * args.steps, "clocks": clocks})


def launches_per_step(cfg, world):
    """Kernels of libmoba_b200.so launched per step: pool 2, gate 1, lists 4 (scan, offsets, fill, tile records),
    forward tiles 2, merge 1, and in backward delta 1, row gather 1, dK/dV 1, dQ 2, dq merge 1. A forward-only run on
    several GPUs works in two head groups (twice the forward launches)."""
    hl = cfg["heads"] // world
    if world > 1 and not cfg["backward"] and hl >= 2:
        return 20
    return 10 + (6 if cfg["backward"] else 0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=3, choices=sorted(CONFIGS))
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--head-groups", type=int, default=8, help="head slices pipelined in the end-to-end leg")
    ap.add_argument("--copy-order", choices=["auto", "duplex", "in-first"], default="auto",
                    help="end-to-end leg: host<->device copies in both directions at once (duplex) or all copy-ins "
                         "before the copy-outs (in-first); auto = in-first from 8 ranks per host up")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-numa-bind", action="store_true", help="leave the process's CPU affinity alone")
    ap.add_argument("--no-secondary", action="store_true", help="skip the 1M-token forward-only line (config 3 runs)")
    args = ap.parse_args()
    claim_stdout()
    cfg = CONFIGS[args.config]
    if cfg.get("decode"):
        if args.impl == "reference" or args.gpus != 1:
            raise SystemExit("the decode configurations run on one GPU with --impl ours only")
        run_decode(args, args.config, cfg)
    elif args.impl == "reference":
        run_reference_arm(args, args.config, cfg)
    else:
        run_ours(args, args.config, cfg)


if __name__ == "__main__":
    main()
