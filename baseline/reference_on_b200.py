"""Runs the reference's own GPU path -- moba.moba_efficient.moba_attn_varlen on flash-attn kernels, installed
unmodified under baseline/_ref, with the two private flash-attn names rebound for the installed flash-attn
(baseline/reference.py) -- on this GPU: first one tiny call (does it run at all?), then its forward + backward time on
the shapes the reference's own speed test uses and on a 4-head cut of the 131072-token layer, by the method of the
reference's tests/test_moba_speedup.py:45-76 (3 warm-up + 10 timed iterations, wall clock around a device
synchronise), with this package timed the same way beside it and the largest difference between the two results.

    python -m baseline.reference_on_b200 [--probe] [--out reference_on_b200.json]

Prints one JSON object; {"unavailable": "<reason>"} when the reference cannot run here. Test / benchmark
infrastructure: nothing in the product package imports it.
"""
import argparse
import json
import os
import sys
import time
import traceback

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _inputs(S, heads, chunk, off_std, seed, dev):
    import torch

    g = torch.Generator(device=dev).manual_seed(seed)
    q, k, v, d_out = (torch.randn(S, heads, 128, generator=g, device=dev) for _ in range(4))
    if off_std > 0:
        off = torch.randn((S + chunk - 1) // chunk, heads, 128, generator=g, device=dev) * off_std
        k = k + off.repeat_interleave(chunk, dim=0)[:S]
    return [t.to(torch.bfloat16) for t in (q, k, v, d_out)]


def _time(fn, q, k, v, d_out, cu, max_seqlen, chunk, topk, warmup=3, iters=10):
    import torch

    q, k, v = (t.clone().requires_grad_() for t in (q, k, v))
    for _ in range(warmup):
        o = fn(q, k, v, cu, max_seqlen, moba_chunk_size=chunk, moba_topk=topk)
        torch.autograd.backward(o, d_out)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(iters):
        q.grad = k.grad = v.grad = None
        o = fn(q, k, v, cu, max_seqlen, moba_chunk_size=chunk, moba_topk=topk)
        torch.autograd.backward(o, d_out)
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) / iters * 1e3
    return ms, (o.detach(), q.grad, k.grad, v.grad)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--probe", action="store_true", help="only the tiny call")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    result = {}
    try:
        import torch

        from baseline import reference as ref

        if not ref.available():
            raise RuntimeError("baseline/_ref holds no reference install (baseline/install_reference.sh)")
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        ref_fn = ref.load_efficient()
        from moba_b200.moba_efficient import check_kernel_status, moba_attn_varlen as our_fn

        def compare(a, b):
            return {n: float((x.float() - y.float()).abs().max()) for n, x, y in zip(("out", "dq", "dk", "dv"), a, b)}

        # ---- tiny call: ragged batch, both implementations, difference inside the reference's own test tolerance
        S, heads, chunk, topk = 1024, 2, 128, 3
        q, k, v, d_out = _inputs(S, heads, chunk, 0.0, 1, dev)
        cu = torch.tensor([0, 300, S], dtype=torch.int32, device=dev)
        _, r = _time(ref_fn, q, k, v, d_out, cu, S - 300, chunk, topk, warmup=1, iters=1)
        _, o = _time(our_fn, q, k, v, d_out, cu, S - 300, chunk, topk, warmup=1, iters=1)
        check_kernel_status(dev)
        result["probe"] = {"runs": True, "max_abs_diff": compare(o, r), "flash_attn": __import__("flash_attn").__version__,
                           "gpu": torch.cuda.get_device_name(dev)}
        if not args.probe:
            cases = [("32768 tokens x 1 head, chunk 2048, top-k 3", 32768, 1, 2048, 3, 0.0),
                     ("32768 tokens x 1 head, chunk 512, top-k 3 (the reference speed test's shape)", 32768, 1, 512, 3, 0.0),
                     ("131072 tokens x 4 heads, chunk 4096, top-k 12 (4-head cut of the benchmark layer)", 131072, 4, 4096, 12, 0.5)]
            result["cases"] = []
            for name, S, heads, chunk, topk, off in cases:
                q, k, v, d_out = _inputs(S, heads, chunk, off, 2, dev)
                cu = torch.tensor([0, S], dtype=torch.int32, device=dev)
                ms_ref, r = _time(ref_fn, q, k, v, d_out, cu, S, chunk, topk)
                ms_our, o = _time(our_fn, q, k, v, d_out, cu, S, chunk, topk)
                check_kernel_status(dev)
                pairs = sum(min(chunk, S - c * chunk) * (min(chunk, S - c * chunk) + 1) // 2 + chunk * min(chunk, S - c * chunk) * min(c, topk - 1)
                            for c in range((S + chunk - 1) // chunk)) * heads
                flops = 14 * 128 * pairs
                result["cases"].append({"case": name, "reference_ms": ms_ref, "moba_b200_ms": ms_our,
                                        "reference_tflops": flops / ms_ref / 1e9, "moba_b200_tflops": flops / ms_our / 1e9,
                                        "max_abs_diff": compare(o, r)})
                del q, k, v, d_out, r, o
                torch.cuda.empty_cache()
    except Exception as e:                      # the reference cannot run here: say why, exit 0
        result = {"unavailable": f"{type(e).__name__}: {e}".splitlines()[0][:400],
                  "traceback_tail": traceback.format_exc().splitlines()[-6:]}
    text = json.dumps(result)
    print(text)
    if args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        with open(args.out, "w") as f:
            f.write(text + "\n")


if __name__ == "__main__":
    main()
