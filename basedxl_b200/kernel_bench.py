"""Time one library kernel in isolation (CUDA events on the launching stream, L2
flushed between launches) and print one JSON line with its achieved rate.

    python -m basedxl_b200.kernel_bench gemm --M 2048 --K 1280 --N 10240
    python -m basedxl_b200.kernel_bench conv --B 2 --Cin 640 --Cout 640 --H 64 --W 64
    python -m basedxl_b200.kernel_bench attention --B 2 --heads 10 --Lq 4096 --Lslot 4096 --slots 1
    python -m basedxl_b200.kernel_bench groupnorm --B 2 --C 1280 --H 32 --W 32          # two-launch form
    python -m basedxl_b200.kernel_bench groupnorm_fused --B 2 --C 1280 --H 32 --W 32    # one-launch form

The same command line is what the profiler captures are taken on (few launches,
small device footprint).
"""
from __future__ import annotations

import argparse
import json
import statistics

import torch

from . import _lib, ops


def _time(fn, iters: int, warmup: int, flush: bool = True) -> float:
    dev = torch.device("cuda", torch.cuda.current_device())
    buf = torch.empty(256 << 20, device=dev, dtype=torch.uint8) if flush else None
    stream = torch.cuda.current_stream()
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        if buf is not None:
            buf.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        fn()
        e1.record(stream)
        e1.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    return statistics.median(ts)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "conv", "attention", "groupnorm", "groupnorm_fused", "geglu", "layernorm"])
    for n, d in [("M", 2048), ("K", 1280), ("N", 1280), ("B", 2), ("Cin", 640), ("Cout", 640), ("C", 1280), ("H", 64), ("W", 64),
                 ("heads", 10), ("Lq", 4096), ("Lslot", 4096), ("slots", 1), ("stride", 1), ("iters", 10), ("warmup", 3),
                 ("bn", 0), ("split", 0), ("pair", -1)]:
        ap.add_argument(f"--{n}", type=int, default=d)
    ap.add_argument("--no-flush", action="store_true")
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    l = _lib.lib()
    if a.bn or a.split or a.pair >= 0:
        _lib.check(l.bxl_debug_force_tiles(a.bn, a.split, a.pair), l, kernels=0)
    g = torch.Generator(device="cuda").manual_seed(0)
    rn = lambda *s: torch.randn(*s, device=dev, generator=g).half()
    if a.kernel == "gemm":
        x, w, o = rn(a.M, a.K), rn(a.N, a.K), torch.empty(a.M, a.N, device=dev, dtype=torch.float16)
        fn = lambda: ops.gemm(x, w, out=o)
        work, unit, desc = 2.0 * a.M * a.N * a.K, "TFLOP/s", {"M": a.M, "K": a.K, "N": a.N}
    elif a.kernel == "conv":
        x = rn(a.B, a.H, a.W, a.Cin)
        wp = ops.conv_weight_pack(rn(a.Cout, a.Cin, 3, 3))
        o = torch.empty(a.B, a.H // a.stride, a.W // a.stride, a.Cout, device=dev, dtype=torch.float16)
        fn = lambda: ops.conv3x3(x, wp, None, stride=a.stride, out=o)
        work = 2.0 * 9 * a.Cin * a.Cout * a.B * (a.H // a.stride) * (a.W // a.stride)
        unit, desc = "TFLOP/s", {"B": a.B, "Cin": a.Cin, "Cout": a.Cout, "H": a.H, "W": a.W, "stride": a.stride}
    elif a.kernel == "attention":
        C = a.heads * 64
        q = rn(a.B, a.Lq, C)
        slots = [rn(a.B, a.Lslot, 2 * C) for _ in range(a.slots)]
        o = torch.empty_like(q)
        fn = lambda: ops.attention(q, slots, a.heads, out=o)
        work = 4.0 * a.B * a.heads * a.Lq * a.Lslot * a.slots * 64
        unit, desc = "TFLOP/s", {"B": a.B, "heads": a.heads, "Lq": a.Lq, "Lkv": a.Lslot * a.slots}
    elif a.kernel == "groupnorm":
        x = rn(a.B, a.H, a.W, a.C)
        gamma, beta = rn(a.C), rn(a.C)
        y = torch.empty_like(x)

        def fn():
            m = ops.groupnorm_stats(x, 32)
            ops.groupnorm_apply(x, 32, 1e-5, gamma, beta, m, silu=True, out=y)

        work, unit, desc = 2.0 * x.numel() * 2, "GB/s", {"B": a.B, "C": a.C, "H": a.H, "W": a.W, "launches": 2}
    elif a.kernel == "groupnorm_fused":
        x = rn(a.B, a.H, a.W, a.C)
        gamma, beta = rn(a.C), rn(a.C)
        y = torch.empty_like(x)
        mom = torch.empty(2, a.B, 32, device=dev, dtype=torch.float32)
        fn = lambda: ops.groupnorm_fused(x, 32, 1e-5, gamma, beta, silu=True, fresh_out=mom, out=y)
        work, unit, desc = 2.0 * x.numel() * 2, "GB/s", {"B": a.B, "C": a.C, "H": a.H, "W": a.W, "launches": 1}
    elif a.kernel == "geglu":
        h = rn(a.M, 2 * a.N)
        fn = lambda: ops.geglu(h)
        work, unit, desc = 3.0 * a.M * a.N * 2, "GB/s", {"rows": a.M, "F": a.N}
    else:
        x, gamma, beta = rn(a.M, a.C), rn(a.C), rn(a.C)
        fn = lambda: ops.layernorm(x, gamma, beta, 1e-5)
        work, unit, desc = 2.0 * a.M * a.C * 2, "GB/s", {"rows": a.M, "C": a.C}
    us = _time(fn, a.iters, a.warmup, flush=not a.no_flush)
    _lib.device_status()
    rate = work / us / (1e6 if unit == "TFLOP/s" else 1e3)
    print(json.dumps({"kernel": a.kernel, **desc, "us": round(us, 2), "rate": round(rate, 1), "unit": unit,
                      "l2": "flushed" if not a.no_flush else "warm"}))


if __name__ == "__main__":
    main()
