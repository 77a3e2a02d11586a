"""Head-parallel run on 2 GPUs (NCCL) against the single-GPU result, bit for bit: every rank computes its half of
the heads (forward + backward), the outputs are gathered through head_parallel.gather_heads (all-gather + head
re-layout), and rank 0 compares the gathered [S, H, D] output and its own heads of dq / dk / dv with the same call
on all heads on one GPU. Skips when fewer than 2 GPUs are visible."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(dev, S, heads, kv_heads):
    g = torch.Generator(device="cpu").manual_seed(17)
    q = torch.randn(S, heads, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(S, kv_heads, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(S, kv_heads, 128, generator=g).to(torch.bfloat16)
    d_out = torch.randn(S, heads, 128, generator=g).to(torch.bfloat16)
    return [t.to(dev) for t in (q, k, v, d_out)]


def _run(q, k, v, d_out, cu, chunk, topk):
    from moba_b200.moba_efficient import check_kernel_status, moba_attn_varlen

    q, k, v = (t.clone().requires_grad_() for t in (q, k, v))
    out = moba_attn_varlen(q, k, v, cu, int((cu[1:] - cu[:-1]).max()), chunk, topk)
    out.backward(d_out)
    check_kernel_status(q.device)
    return out.detach(), q.grad, k.grad, v.grad


def _worker(rank, world, port, result):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from moba_b200.head_parallel import gather_heads, shard_heads

    S, heads, kv_heads, chunk, topk = 6144, 8, 4, 512, 4
    q, k, v, d_out = _inputs(dev, S, heads, kv_heads)
    cu = torch.tensor([0, 1000, 2536, S], dtype=torch.int32, device=dev)
    ql, kl, vl, dl = (shard_heads(t, rank, world).contiguous() for t in (q, k, v, d_out))
    out_l, dq_l, dk_l, dv_l = _run(ql, kl, vl, dl, cu, chunk, topk)
    out = gather_heads(out_l)
    ok = True
    if rank == 0:
        out1, dq1, dk1, dv1 = _run(q, k, v, d_out, cu, chunk, topk)
        ok = (torch.equal(out, out1) and torch.equal(dq_l, shard_heads(dq1, 0, world))
              and torch.equal(dk_l, shard_heads(dk1, 0, world)) and torch.equal(dv_l, shard_heads(dv1, 0, world)))
    result.put((rank, bool(ok)))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_head_parallel_equals_single_gpu():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
        assert p.exitcode == 0
    got = dict(result.get(timeout=10) for _ in range(world))
    assert got == {0: True, 1: True}
