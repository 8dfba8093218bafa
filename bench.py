"""Benchmark of the SDXL 1024^2 UNet denoising loop.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One JSON line on stdout (rank 0).  A *step* is one denoising step of the loop:
UNet forward on the CFG batch of 2 (split over the ranks as the reference's
config does: CFG halves first, then H-strips), guidance combine, Euler update.
``value`` is seconds per 50-step image = 50 x the mean step time, with every
input resident in device memory; a timed region of K = 50 steps started from a
fresh image contains the reference's 5 synchronous warm-up steps followed by 45
displaced steps, like a real image.  ``e2e`` is the same figure measured through
``BasedXLPipeline.__call__`` with pinned HOST conditioning / latents in and the
final latent copied back out inside the timed region.

``--impl reference`` times the reference's CPU path instead: the same UNet graph
evaluated by stock PyTorch fp32 operators on all host cores (the reference has no
CPU implementation other than its PyTorch modules on CPU tensors).  A step of that
arm is one full-size UNet forward on the CFG batch of 2 - the same configuration
as the accelerated arm, no extrapolation over the problem size.

Synthetic data throughout: N(0,1) latents and conditioning, seed-0 random
weights of the SDXL architecture.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

IMAGE_STEPS = 50
METRIC = "sdxl_1024_50step_unet_s_per_image"  # the name carries the configured resolution, see metric_name()


def metric_name(height: int) -> str:
    return f"sdxl_{height}_50step_unet_s_per_image"
UNIT = "s/image"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"tflops_burst": p["bf16_tflops"], "tflops_sustained": p["bf16_tflops_sustained"], "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"tflops_burst": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """SM clock, power and clock-event reasons of one GPU, sampled while the timed region runs.
    Reads through NVML every 20 ms from a thread of this process (read-only queries); falls back
    to an `nvidia-smi -lms 50` child if the NVML binding is missing.  Only samples taken between
    `mark_begin()` and `mark_end()` are reported."""

    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    REASON_BITS = (("sw_power_cap", 0x4), ("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40))

    def __init__(self, device):
        self.device = device
        self.gpu_index = device.index if device.index is not None else 0
        self.proc = None
        self.nvml = None
        self.samples: list[tuple] = []   # (monotonic time, sm MHz, max MHz, watts, [reasons])
        self.t_begin = self.t_end = None
        self._stop = threading.Event()

    def _nvml_handle(self):
        import pynvml

        pynvml.nvmlInit()
        try:
            uuid = str(torch.cuda.get_device_properties(self.device).uuid)
            uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            try:
                h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except TypeError:
                h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        except Exception:
            h = pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)
        return pynvml, h

    def start(self):
        try:
            self.nvml = self._nvml_handle()
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
            self.thread = threading.Thread(target=self._read_smi, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _poll_nvml(self):
        nv, h = self.nvml
        mx = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
        reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self._stop.is_set():
            try:
                sm = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                watts = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
                mask = int(reasons_fn(h))
                self.samples.append((time.monotonic(), sm, mx, watts, [n for n, bit in self.REASON_BITS if mask & bit]))
            except Exception:
                pass
            self._stop.wait(0.02)

    def _read_smi(self):
        for line in self.proc.stdout:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm, mx, watts = float(f[1]), float(f[2]), float(f[3])
            except ValueError:
                continue
            names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
            self.samples.append((time.monotonic(), sm, mx, watts, [n for n, v in zip(names, f[5:9]) if v.lower().startswith("active")]))

    def mark_begin(self):
        self.t_begin = time.monotonic()

    def mark_end(self):
        self.t_end = time.monotonic()

    def stop(self) -> dict:
        self._stop.set()
        if self.nvml is None and self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source (NVML binding and nvidia-smi unavailable)"]}
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        else:
            self.thread.join(timeout=1.0)
        lo = self.t_begin if self.t_begin is not None else -1e30
        hi = self.t_end if self.t_end is not None else 1e30
        inside = [x for x in self.samples if lo <= x[0] <= hi]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        reasons = sorted({r for x in inside for r in x[4]})
        return {"sm_mhz": statistics.median(x[1] for x in inside), "sm_max_mhz": max(x[2] for x in inside), "reasons": reasons,
                "power_w_max": max(x[3] for x in inside), "samples": len(inside), "source": "nvml" if self.nvml else "nvidia-smi"}


# --------------------------------------------------------------------------- synthetic inputs
def synthetic_inputs(height, width, pin: bool):
    g = torch.Generator().manual_seed(1234)
    t = {
        "latents": torch.randn(1, 4, height // 8, width // 8, generator=g),
        "prompt_embeds": torch.randn(1, 77, 2048, generator=g),
        "negative_prompt_embeds": torch.randn(1, 77, 2048, generator=g),
        "pooled_prompt_embeds": torch.randn(1, 1280, generator=g),
        "negative_pooled_prompt_embeds": torch.randn(1, 1280, generator=g),
    }
    if pin:
        t = {k: v.pin_memory() for k, v in t.items()}
    return t


# --------------------------------------------------------------------------- GEMM kernel roofline
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "gemm_linear_traffic.txt")


def measured_traffic():
    """DRAM bytes per launch of the GEMM kernel from the committed profiler capture (a text
    summary under profiles/: ``key: value`` lines).  None if the summary is absent."""
    if not os.path.exists(TRAFFIC_FILE):
        return None
    kv = {}
    with open(TRAFFIC_FILE) as f:
        for ln in f:
            if ":" in ln and not ln.startswith("#"):
                k, v = ln.split(":", 1)
                kv[k.strip()] = v.strip()
    try:
        return {"bytes_per_launch": float(kv["dram_bytes_read"]) + float(kv["dram_bytes_write"]), "case": kv["case"],
                "algorithmic_bytes": float(kv["algorithmic_bytes"]), "capture": "profiles/gemm_linear_traffic.txt"}
    except (KeyError, ValueError):
        return None


def linear_shapes(n_strips: int, height: int, width: int, batch: int):
    """(tokens, K, N, launches per UNet forward) of the linear layers one rank runs."""
    hw = (height // 8) * (width // 8) // n_strips
    b = batch
    return [
        (b * hw // 4, 640, 640, 40), (b * hw // 4, 640, 1920, 10), (b * hw // 4, 640, 5120, 10), (b * hw // 4, 2560, 640, 10),
        (b * hw // 16, 1280, 1280, 192), (b * hw // 16, 1280, 3840, 60), (b * hw // 16, 1280, 10240, 60), (b * hw // 16, 5120, 1280, 60),
    ]


def gemm_kernel_roofline(device, n_strips: int, height: int, width: int, peaks) -> dict:
    """The dominant kernel (the tcgen05 GEMM: 64 % of the loop's FLOPs at 1024^2) over the UNet's
    own linear-layer shapes.  For every shape a chain of launches cycles through enough operand
    sets (activations, weights, outputs) to exceed the 126 MB L2 several times over, so every
    launch reads its operands from HBM as in the real loop (5 GB of weights per step).  The
    chain is captured into a CUDA graph and REPLAYED, as the UNet step is, so the host's launch
    cost is not in the figure; it is timed with CUDA events on the replaying stream and divided
    by the number of launches.  ``achieved`` = sum of algorithmic FLOPs (2*M*N*K) / sum of launch
    durations, weighted by launches per forward."""
    from basedxl_b200 import _lib, ops

    b = 2 if n_strips == 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1 else 1
    stream = torch.cuda.current_stream()
    tot_flops = tot_ms = 0.0
    per_shape = []
    l = _lib.lib()
    _lib.check(l.bxl_set_static_weights(1), l, kernels=0)  # as inside a UNet step: B operands are weights
    try:
        for (M, K, N, count) in linear_shapes(n_strips, height, width, b):
            set_bytes = 2 * (M * K + N * K + M * N)
            n_sets = max(4, min(48, (512 << 20) // set_bytes + 1))  # >= 512 MB cycled through
            a = [torch.randn(M, K, device=device).half() for _ in range(n_sets)]
            w = [torch.randn(N, K, device=device).half() for _ in range(n_sets)]
            out = [torch.empty(M, N, device=device, dtype=torch.float16) for _ in range(n_sets)]
            for i in range(n_sets):
                ops.gemm(a[i], w[i], out=out[i])
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(n_sets):
                    ops.gemm(a[i], w[i], out=out[i])
            graph.replay()
            times = []
            for _ in range(5):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                graph.replay()
                e1.record(stream)
                e1.synchronize()
                times.append(e0.elapsed_time(e1) / n_sets)
            ms = statistics.median(times)
            fl = 2.0 * M * N * K
            per_shape.append({"M": M, "K": K, "N": N, "launches_per_forward": count, "us": round(ms * 1e3, 2), "tflops": round(fl / ms / 1e9, 1)})
            tot_flops += fl * count
            tot_ms += ms * count
            graph.reset()
            del graph, a, w, out
    finally:
        _lib.check(l.bxl_set_static_weights(0), l, kernels=0)
    achieved = tot_flops / tot_ms / 1e9
    return {
        "bound": "tensor", "kernel": "gemm_conv_kernel (linear layers)", "achieved": round(achieved, 1),
        "peak": peaks["tflops_burst"], "peak_kind": f"{peaks['source']} burst (kernel timed alone)", "unit": "TFLOP/s",
        "frac": round(achieved / peaks["tflops_burst"], 4),
        "timing": "device: chains of launches replayed from a CUDA graph, CUDA events on the replaying stream",
        "l2": "operand sets cycled, > 512 MB per shape (larger than L2)",
        "traffic": measured_traffic(),
        "per_shape": per_shape,
    }


# --------------------------------------------------------------------------- CPU baseline (oracle port)
def cpu_unet(state_dict=None):
    from basedxl_b200.sdxl_unet import UNet2DConditionModel, sdxl_config
    from oracle.torch_layers import TorchLayers

    torch.manual_seed(0)
    with torch.device("meta"):
        m = UNet2DConditionModel(sdxl_config(), layers=TorchLayers)
    m = m.to_empty(device="cpu").eval()
    if state_dict is not None:
        m.load_state_dict({k: v.float().cpu() for k, v in state_dict.items()})
    else:
        with torch.no_grad():
            for p in m.parameters():
                p.uniform_(-0.02, 0.02)
    return m


def cpu_forward_seconds(model, latent_hw: int, batch: int = 2) -> float:
    g = torch.Generator().manual_seed(7)
    x = torch.randn(batch, 4, latent_hw, latent_hw, generator=g)
    ehs = torch.randn(batch, 77, 2048, generator=g)
    added = {"text_embeds": torch.randn(batch, 1280, generator=g), "time_ids": torch.tensor([[1024.0, 1024, 0, 0, 1024, 1024]] * batch)}
    t0 = time.perf_counter()
    with torch.no_grad():
        model(x, torch.tensor(999.0), ehs, added_cond_kwargs=added)
    return time.perf_counter() - t0


def run_reference_arm(args):
    """The reference's CPU path: stock PyTorch fp32 modules on all host cores, one full-size
    UNet forward (CFG batch 2) per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # a launcher for several ranks pins OMP_NUM_THREADS=1; this arm is one process on the whole host
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    model = cpu_unet()
    hw = args.height // 8
    for _ in range(args.warmup_reference):
        cpu_forward_seconds(model, hw)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_forward_seconds(model, hw)
    per_step = (time.perf_counter() - t0) / args.steps
    value = per_step * IMAGE_STEPS
    sample = (f"per step: one UNet forward, CFG batch 2, {hw}x{hw} latent (the full-size workload), fp32, stock PyTorch CPU "
              f"operators on {torch.get_num_threads()} threads; {args.steps} steps timed, s/image = {IMAGE_STEPS} x mean step")
    line = {
        "impl": "reference", "metric": metric_name(args.height), "value": round(value, 2), "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(per_step * 1e3, 1), "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args), "arm": "CPU path of the reference: PyTorch modules on host cores",
                   "warmup_steps_run": args.warmup_reference},
        "cpu_baseline": {"value": round(value, 2), "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 2), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- per-operator workload
def _chain_us(launch, n_sets: int, reps: int = 5) -> float:
    """Device time per launch of ``launch(i)``, i cycling through ``n_sets`` operand sets: the chain is captured
    into a CUDA graph, replayed, and timed with CUDA events on the replaying stream."""
    stream = torch.cuda.current_stream()
    for i in range(n_sets):
        launch(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(n_sets):
            launch(i)
    graph.replay()
    times = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        graph.replay()
        e1.record(stream)
        e1.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3 / n_sets)
    graph.reset()
    return statistics.median(times)


def _cpu_seconds(fn, reps: int = 2) -> float:
    fn()
    t0 = time.perf_counter()
    for _ in range(reps):
        fn()
    return (time.perf_counter() - t0) / reps


def run_ops_workload(args):
    """The isolated-operator configurations: the five matmul shapes (fp16 operands and the split-operand fp32
    product, error against an fp64 product by the reference's error-study method) and the patched operators at
    2 / 4 / 8 strips (3x3 convolution 2x640x64x64, GroupNorm 2x1280x32x32 with 32 groups, self-attention 10 heads x 64
    on 2x4096x640; stale = current + N(0, 0.01)); for each the device time of this rank's launch, its rate against
    the measured peak, and the time of the reference's CPU path (PyTorch operators on the host cores) beside it."""
    from basedxl_b200 import _lib, ops
    from oracle import matmul as om
    from oracle import patched_ops as po

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = load_peaks()
    torch.set_num_threads(os.cpu_count() or 1)
    cores = torch.get_num_threads()
    sets = lambda nbytes: max(4, min(48, (512 << 20) // max(1, nbytes) + 1))
    out = {"metric": "isolated operator configurations", "workload": "ops", "n_gpus": 1, "dtype": "f16", "data": "synthetic",
           "peaks": peaks, "cpu_cores": cores,
           "timing": "device: chains over operand sets > L2 replayed from a CUDA graph, CUDA events; CPU: wall clock, PyTorch fp32 operators"}
    # ---- matmul shapes
    mm = []
    for (M, K, N) in [(8192, 640, 640), (8192, 640, 5120), (2048, 1280, 1280), (2048, 1280, 10240), (16384, 320, 320)]:
        torch.manual_seed(0)
        a32, b32 = torch.randn(M, K), torch.randn(K, N)
        a16, b16 = a32.half(), b32.half()
        n = sets(2 * (M * K + K * N + M * N))
        A = [a16.to(dev) for _ in range(n)]
        Bm = [b16.to(dev) for _ in range(n)]
        C = [torch.empty(M, N, device=dev, dtype=torch.float16) for _ in range(n)]
        us16 = _chain_us(lambda i: ops.gemm(A[i], Bm[i], out=C[i], b_is_kn=True), n)
        y16 = C[0].cpu()
        del A, Bm, C
        a32d, b32d = a32.to(dev), b32.to(dev)
        y32 = ops.gemm_split_f32(a32d, b32d).cpu()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ts = []
        for _ in range(5):
            e0.record(); ops.gemm_split_f32(a32d, b32d); e1.record(); e1.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        us32 = statistics.median(ts)
        exp16, exp32 = om.matmul_fp64(a16, b16), om.matmul_fp64(a32, b32)
        sub = slice(0, 512)  # the model of the reference's fp16 accumulator is evaluated on a row block
        e_ref = om.error_table(exp16[sub], om.matmul_fp16_accumulate(a16[sub], b16, block_k=32, model="block"))
        e_16, e_32 = om.error_table(exp16, y16), om.error_table(exp32, y32)
        cpu_s = _cpu_seconds(lambda: a32 @ b32)
        fl = 2.0 * M * N * K
        mm.append({"M": M, "K": K, "N": N,
                   "fp16_operands": {"us": round(us16, 2), "tflops": round(fl / us16 / 1e6, 1), "frac_of_burst_peak": round(fl / us16 / 1e6 / peaks["tflops_burst"], 3),
                                     "max_abs_err": e_16["max"], "l1_err": e_16["l1"], "rel_err_median": e_16["rel_median"]},
                   "split_fp32_operands": {"us_incl_split_kernels_host_launched": round(us32, 2), "max_abs_err": e_32["max"], "l1_err": e_32["l1"],
                                           "rel_err_median": e_32["rel_median"]},
                   "reference_fp16_accumulator_model": {"rows": 512, "max_abs_err": e_ref["max"], "l1_err": e_ref["l1"], "rel_err_median": e_ref["rel_median"]},
                   "cpu_fp32_matmul_s": round(cpu_s, 4)})
    out["matmul"] = mm
    _lib.device_status()
    # ---- patched operators, per strip count
    gen = torch.Generator().manual_seed(0)
    x_c = torch.randn(2, 640, 64, 64, generator=gen).half()
    w_c = (torch.randn(640, 640, 3, 3, generator=gen) / (9 * 640) ** 0.5).half()
    b_c = torch.randn(640, generator=gen).half()
    x_g = torch.randn(2, 1280, 32, 32, generator=gen).half()
    ga, be = torch.randn(1280, generator=gen).half(), torch.randn(1280, generator=gen).half()
    q_a, kv_a = torch.randn(2, 4096, 640, generator=gen).half(), torch.randn(2, 4096, 1280, generator=gen).half()
    nhwc = lambda t: t.permute(0, 2, 3, 1).contiguous()
    conv, gn, att = [], [], []
    wp = ops.conv_weight_pack(w_c.to(dev))
    for n_strips in (2, 4, 8):
        i = n_strips // 2
        # conv: this rank's strip, stale halo rows from its neighbours
        hs = 64 // n_strips
        xs = nhwc(x_c)[:, i * hs:(i + 1) * hs]
        nset = sets(2 * (xs.numel() + w_c.numel() + 2 * hs * 64 * 640))
        X = [xs.to(dev) for _ in range(nset)]
        W = [wp.clone() for _ in range(nset)]
        top = nhwc(x_c)[:, i * hs - 1:i * hs].to(dev)
        bot = nhwc(x_c)[:, (i + 1) * hs:(i + 1) * hs + 1].to(dev) if (i + 1) * hs < 64 else None  # last strip: image edge
        Y = [torch.empty(2, hs, 64, 640, device=dev, dtype=torch.float16) for _ in range(nset)]
        bd = b_c.to(dev)
        us = _chain_us(lambda k: ops.conv3x3(X[k], W[k], bd, top=top, bot=bot, out=Y[k]), nset)
        fl = 2.0 * 9 * 640 * 640 * 2 * hs * 64
        xf, wf, bf = x_c.float(), w_c.float(), b_c.float()
        strips = torch.chunk(xf, n_strips, 2)
        stale = [po.conv2d_boundary(t, 1) for t in strips]
        cpu_s = _cpu_seconds(lambda: po.conv2d_pp(strips[i], wf, bf, 1, 1, stale, i, n_strips))
        conv.append({"strips": n_strips, "strip_shape": [2, 640, hs, 64], "us": round(us, 2), "tflops": round(fl / us / 1e6, 1),
                     "frac_of_burst_peak": round(fl / us / 1e6 / peaks["tflops_burst"], 3), "cpu_s": round(cpu_s, 4)})
        del X, W, Y
        # GroupNorm + SiLU, stale moments, one launch
        hg = 32 // n_strips
        xg = nhwc(x_g)[:, i * hg:(i + 1) * hg].contiguous()
        nset = sets(4 * xg.numel())
        Xg = [xg.to(dev) for _ in range(nset)]
        Yg = [torch.empty_like(Xg[0]) for _ in range(nset)]
        gstrips = torch.chunk(x_g.float(), n_strips, 2)
        mom = [po.groupnorm_moments(t, 32) for t in gstrips]
        peers = [m.reshape(2, 2, 32).float().contiguous().to(dev) for m in mom]
        gad, bed = ga.to(dev), be.to(dev)
        us = _chain_us(lambda k: ops.groupnorm_fused(Xg[k], 32, 1e-5, gad, bed, peers, i, ops.MODE_STALE, silu=True, out=Yg[k]), nset)
        nbytes = 2.0 * xg.numel() * 2
        cpu_s = _cpu_seconds(lambda: torch.nn.functional.silu(po.groupnorm_pp(gstrips[i], 32, 1e-5, ga.float(), be.float(), mom, i, "stale")))
        gn.append({"strips": n_strips, "strip_shape": [2, 1280, hg, 32], "us": round(us, 2), "gbps": round(nbytes / us / 1e3, 1),
                   "frac_of_hbm_peak": round(nbytes / us / 1e3 / peaks["hbm_gbs"], 4), "algorithmic_bytes": nbytes, "cpu_s": round(cpu_s, 5)})
        del Xg, Yg
        # self-attention core: this strip's queries against all strips' K/V slots
        ls = 4096 // n_strips
        qs = q_a[:, i * ls:(i + 1) * ls].contiguous()
        nset = sets(2 * (qs.numel() * 2 + kv_a.numel()))
        Q = [qs.to(dev) for _ in range(nset)]
        KV = [[kv_a[:, j * ls:(j + 1) * ls].contiguous().to(dev) for j in range(n_strips)] for _ in range(nset)]
        O = [torch.empty_like(Q[0]) for _ in range(nset)]
        us = _chain_us(lambda k: ops.attention(Q[k], KV[k], 10, out=O[k]), nset)
        fl = 4.0 * 2 * 10 * ls * 4096 * 64
        qf, kvf = qs.float(), kv_a.float()
        cpu_s = _cpu_seconds(lambda: po._sdpa_heads(qf, kvf, 10))
        att.append({"strips": n_strips, "queries": ls, "keys": 4096, "us": round(us, 2), "tflops": round(fl / us / 1e6, 1),
                    "frac_of_burst_peak": round(fl / us / 1e6 / peaks["tflops_burst"], 3), "cpu_s": round(cpu_s, 4)})
        del Q, KV, O
    _lib.device_status()
    out["conv3x3_2x640x64x64"], out["groupnorm_silu_2x1280x32x32"], out["self_attention_2x4096x640_h10"] = conv, gn, att
    print(json.dumps(out), flush=True)


# --------------------------------------------------------------------------- main arm
def workload_name(args) -> str:
    return (f"SDXL {args.height}x{args.width} UNet loop: latent 1x4x{args.height // 8}x{args.width // 8}, CFG batch 2, guidance 5.0, "
            f"50 Euler steps, 5 synchronous steps then displaced")


def comm_summary(pipe, cfg, step_ms):
    """What a rank exchanges per step (bytes from the registered tensors), over which transport,
    and the measured device time of synchronous and displaced steps."""
    cm = pipe.unet.comm_manager
    n = cfg.n_device_per_batch
    sync_steps = cfg.warmup_steps + 1
    med = lambda v: round(statistics.median(v), 3) if v else None
    out = {
        "output_assembly": "peer stores + flag barrier (bxl_comm_exchange)" if pipe.unet.world_peer is not None else "nccl all_gather",
        "sync_step_ms": med(step_ms[:sync_steps]), "displaced_step_ms": med(step_ms[sync_steps:]),
    }
    if cm is not None and cm.numel:
        slot = cm.numel * 2  # fp16 staging slot of this rank: halo rows, GroupNorm moments, K/V of all patched layers
        gathers = -(-len(cm.starts) // cfg.comm_checkpoint)
        out.update({
            "strips_per_image": n, "exchanged_tensors": len(cm.starts), "slot_bytes": slot,
            "displaced_step": {"transport": "nccl all_gather on the communication stream, joined one step later", "gathers": gathers,
                               "bytes_sent_per_rank": slot, "bytes_received_per_rank": slot * (n - 1)},
            "sync_step": {"transport": "peer stores + flag barrier, one kernel per layer (bxl_comm_exchange)" if cm.peer is not None
                          else "blocking nccl all_gather per layer", "exchanges": len(cm.starts), "bytes_pushed_per_rank": slot * (n - 1)},
        })
        # NVLink time of the displaced exchange at the measured peer-copy rate, against the step it hides behind
        nvlink_ms = slot * (n - 1) / 770e9 * 1e3
        out["displaced_step"]["nvlink_ms_at_770GBps"] = round(nvlink_ms, 3)
    return out


def run_b200_arm(args):
    from basedxl_b200 import _lib
    from basedxl_b200.flops import unet_flops
    from basedxl_b200.model import BasedXLPipeline
    from basedxl_b200.sdxl_unet import sdxl_config
    from basedxl_b200.utils import BasedXLConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    cfg = BasedXLConfig(height=args.height, width=args.width, patch_parallelism=True, use_cfg=True, warmup_steps=4)
    rank, dev = cfg.rank, torch.device(cfg.device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    torch.cuda.set_device(dev)
    peaks = load_peaks()
    pipe = BasedXLPipeline.from_config(cfg, seed=0)
    if not args.no_graph:
        pipe.unet.enable_cuda_graph()
    host = synthetic_inputs(args.height, args.width, pin=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    stream = torch.cuda.current_stream()
    steps_total = max(IMAGE_STEPS, args.steps)

    def timed_image(lat, ehs, added):
        """Steps 0..K-1 of a fresh image on device-resident inputs: (max-over-ranks ms, launches, latents)."""
        pipe.unet.reset()
        launches0 = _lib.launches
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        out = pipe.denoise(lat, ehs, added, steps_total, 5.0, first_step=0, last_step=args.steps)
        e1.record(stream)
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)), _lib.launches - launches0, out

    # ---- device-resident loop -------------------------------------------------
    lat, ehs, added = pipe.prepare_inputs(**host)
    pipe.unet.reset()
    # Untimed warm-up.  One GPU: W steps (the first one captures the step graph).  Several GPUs: a
    # complete image of at least K steps, so that everything an image does once per process - the
    # eager first step, the capture of the synchronous-step and displaced-step graphs, NCCL's
    # channel set-up on their first replay, the allocator's growth - lies outside the timed region.
    warm_steps = max(args.warmup, 3)
    if world > 1:
        warm_steps = max(warm_steps, args.steps, cfg.warmup_steps + 2)
    pipe.denoise(lat, ehs, added, steps_total, 5.0, first_step=0, last_step=min(warm_steps, steps_total))
    sampler = ClockSampler(dev)
    sampler.start()
    barrier()
    sampler.mark_begin()
    ms_total, launches, out = timed_image(lat, ehs, added)
    sampler.mark_end()
    clocks = sampler.stop()
    ms_second, _, out2 = timed_image(lat, ehs, added)
    # per-step device times of one more image (diagnostic: synchronous vs displaced steps)
    step_ms = []
    if world > 1:
        pipe.unet.reset()
        barrier()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        cur = lat
        for i in range(args.steps):
            evs[i].record(stream)
            cur = pipe.denoise(cur, ehs, added, steps_total, 5.0, first_step=i, last_step=i + 1)
        evs[args.steps].record(stream)
        barrier()
        step_ms = [evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps)]
    _lib.device_status()
    assert torch.isfinite(out).all(), "non-finite latents"
    # the same image twice: the loop (graph replay included) must be deterministic
    repeat_err = float((out2.float() - out.float()).norm() / out.float().norm())
    ms_per_step = ms_total / args.steps
    value = ms_per_step * IMAGE_STEPS / 1e3

    # ---- end to end through the public API, host buffers in, latent out ----------
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    res = pipe(host["prompt_embeds"], host["pooled_prompt_embeds"], host["negative_prompt_embeds"],
               host["negative_pooled_prompt_embeds"], num_inference_steps=steps_total, guidance_scale=5.0, latents=host["latents"],
               last_step=args.steps)
    final = res.latents.to("cpu", non_blocking=False)
    e1.record(stream)
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1))
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = final.numel() * final.element_size()
    e2e_value = e2e_ms / args.steps * IMAGE_STEPS / 1e3
    # the public call ran the same steps on the same inputs as the device-resident loop
    e2e_err = float((final.float() - out.float().cpu()).norm() / out.float().norm().cpu())

    # ---- roofline of the dominant kernel ----------------------------------------------
    n_strips = cfg.n_device_per_batch
    roof = gemm_kernel_roofline(dev, n_strips, args.height, args.width, peaks)
    flops_image = unet_flops(sdxl_config(), args.height // 8, args.width // 8, 2) * IMAGE_STEPS
    loop_tflops = flops_image / value / 1e12
    roof["loop"] = {"algorithmic_tflop_per_image": round(flops_image / 1e12, 1), "achieved_tflops_all_gpus": round(loop_tflops, 1),
                    "frac_of_sustained_peak_x_gpus": round(loop_tflops / (peaks["tflops_sustained"] * world), 4)}

    # ---- CPU baseline on the host cores (rank 0, N = 1 only) --------------------------------
    cpu = None
    if world == 1 and not args.skip_cpu:
        torch.set_num_threads(os.cpu_count() or 1)
        model = cpu_unet(pipe.unet.model.state_dict())
        secs = cpu_forward_seconds(model, args.height // 8)
        cpu = {"value": round(secs * IMAGE_STEPS, 1), "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
               "sample": f"one UNet forward (CFG batch 2, {args.height // 8}x{args.width // 8} latent, fp32, stock PyTorch CPU operators) = 1/{IMAGE_STEPS} image, {secs:.1f} s; x{IMAGE_STEPS}"}
        del model

    if rank == 0:
        par = "1 gpu" if world == 1 else (f"cfg2 x {n_strips} strips" if n_strips > 1 else "cfg2")
        line = {
            "metric": metric_name(args.height), "value": round(value, 4), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 3), "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": workload_name(args),
                       "parallelism": par, "l2": "activations and weights per step (5 GB of fp16 weights) exceed L2; no explicit flush in the loop",
                       "warmup_steps_run": warm_steps},
            "clocks": clocks, "gpu_launches": launches, "cuda_graph": bool(pipe.unet.cuda_graph),
            "e2e": {"value": round(e2e_value, 4), "unit": UNIT, "h2d_bytes_per_step": h2d // args.steps, "d2h_bytes_per_step": d2h // args.steps,
                    "rel_l2_vs_device_resident_run": e2e_err},
            "second_image": {"ms_per_step": round(ms_second / args.steps, 3), "rel_l2_vs_first": repeat_err},
            "roofline": roof,
        }
        if world > 1:
            line["comm"] = comm_summary(pipe, cfg, step_ms)
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    shutdown(pipe, world)


def shutdown(pipe, world):
    """Release the captured graphs, then the process group, then return so that the interpreter
    exits normally.  A watchdog turns a stalled tear-down into a loud non-zero exit instead of
    a hang."""
    sys.stdout.flush()

    def stalled():
        sys.stderr.write("bench.py: tear-down did not finish within 60 s (graph release / process-group destruction stalled)\n")
        sys.stderr.flush()
        os._exit(3)

    watchdog = threading.Timer(60.0, stalled)
    watchdog.daemon = True
    watchdog.start()
    pipe.unet.release_graph()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    watchdog.cancel()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="timed steps (default: 50; reference arm: 10 full-size CPU forwards)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--height", type=int, default=1024)
    ap.add_argument("--width", type=int, default=1024)
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from Python instead of replaying a CUDA graph")
    ap.add_argument("--skip-cpu", action="store_true", help="omit the cpu_baseline leg")
    ap.add_argument("--workload", default="loop", choices=["loop", "ops"],
                    help="loop: the denoising loop (the benchmark line); ops: the isolated matmul / conv / GroupNorm / attention configurations")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    args.warmup_reference = args.warmup
    if args.workload == "ops":
        run_ops_workload(args)
        return
    if args.impl == "reference":
        if args.steps is None:
            args.steps = 10  # default run: ten full-size CPU forwards, a couple of minutes
        run_reference_arm(args)
    else:
        if args.steps is None:
            args.steps = IMAGE_STEPS
        run_b200_arm(args)


if __name__ == "__main__":
    main()
