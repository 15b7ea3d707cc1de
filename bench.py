"""Benchmark of the fused attention forward + backward path.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (one "step"): causal softmax attention forward + backward at the Llama-3.1-8B GQA shape
B=8, Hq=32, Hkv=8, S=8192, D=DV=128, fp16, synthetic N(0,1) inputs.  FLOPs follow the reference's
convention (attention_engine/benchmark/bench_utils.py:1185-1188): forward 4*B*Hq*S^2*D/2, backward
2.5x that.  With N GPUs the B=8 workload is sharded by batch rows over the ranks (8 / N rows each; independent
(batch, kv-group) units, no collective on the data path): strong scaling, value = flops of the whole workload /
max-over-ranks time.  ``--scaling weak`` runs the whole workload on every rank instead (value = N * flops / time).

One JSON line is printed by rank 0.  ``--impl reference`` times the reference's naive PyTorch path
(restated in oracle/attention_oracle.py) on the host cores on a bounded slice of the same workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(B=8, Hq=32, Hkv=8, S=8192, D=128)
METRIC = "attention fwd+bwd throughput, Llama-3.1-8B GQA S=8K causal"


def flops_fwd(B, Hq, S, D):
    return 4.0 * B * Hq * S * S * D / 2


def max_over_ranks(value: float, device=None) -> float:
    """Largest ``value`` over all ranks of the default process group (the identity without one)."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def aggregate_throughput(work_per_rank: float, ms_local: float, world: int, device=None) -> tuple:
    """Every rank does ``work_per_rank`` (its shard under strong scaling, a full copy under weak scaling); the job's
    throughput is the total work over the slowest rank's time.  Returns (units per second, that time in ms)."""
    ms = max_over_ranks(ms_local, device)
    return world * work_per_rank / (ms / 1e3), ms


def shard_batch(total: int, world: int, scaling: str) -> int:
    """Batch rows per rank: the stated workload split over the ranks (strong), or all of it on each (weak)."""
    if scaling == "weak" or world == 1:
        return total
    if total % world:
        raise SystemExit(f"--gpus {world} does not divide the workload's {total} batch rows")
    return total // world


def read_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """SM clock and throttle reasons while the timed region runs: an NVML polling thread (a sample every 10 ms from
    the first millisecond on); falls back to an nvidia-smi child process where NVML cannot be loaded.  Read-only."""

    _REASONS = (("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40),
                ("sw_power_cap", 0x4))

    def __init__(self, index: int):
        import threading
        self.sm, self.mx, self.reasons = [], [], set()
        self.p = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.mx.append(float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)))
            get_reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons

            def poll():
                while not self._stop.is_set():
                    try:
                        self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                        r = int(get_reasons(h))
                        for name, bit in self._REASONS:
                            if r & bit:
                                self.reasons.add(name)
                    except Exception:
                        pass
                    self._stop.wait(0.01)

            self._thread = threading.Thread(target=poll, daemon=True)
            self._thread.start()
        except Exception:
            q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                 "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
            try:
                self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms",
                                           "100", "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                                          text=True)
            except OSError:
                self.p = None

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
            return {"sm_mhz": statistics.median(self.sm) if self.sm else None,
                    "sm_max_mhz": max(self.mx) if self.mx else None, "samples": len(self.sm),
                    "reasons": sorted(self.reasons), "source": "nvml"}
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock sampling unavailable"]}
        self.p.terminate()
        try:
            out, _ = self.p.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
            out, _ = self.p.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons), "source": "nvidia-smi"}


def cpu_sample(n_slices: int, threads: int):
    """The naive fp32 PyTorch reference (oracle port) on ``n_slices`` (batch, kv-group) slices of the workload:
    each slice is 4 q-heads x S=8192 against one kv-head, forward + backward."""
    import torch
    from oracle import attention_oracle as orc
    torch.set_num_threads(threads)
    S, D, g = CFG["S"], CFG["D"], CFG["Hq"] // CFG["Hkv"]
    gen = torch.Generator().manual_seed(0)
    t = 0.0
    for _ in range(n_slices):
        q = torch.randn(1, S, g, D, generator=gen).to(torch.float16)
        k = torch.randn(1, S, 1, D, generator=gen).to(torch.float16)
        v = torch.randn(1, S, 1, D, generator=gen).to(torch.float16)
        d_o = torch.randn(1, S, g, D, generator=gen).to(torch.float16)
        t0 = time.perf_counter()
        orc.fwd_bwd(lambda a, b, c: orc.softmax_attention(a, b, c, True), (q, k, v), d_o)
        t += time.perf_counter() - t0
    fl = 3.5 * flops_fwd(1, g, S, D) * n_slices
    return fl / t / 1e12, t


def run_reference(args, rank, world):
    if rank != 0:
        return
    import torch
    threads = os.cpu_count() or 1
    times = []
    for i in range(args.warmup + args.steps):
        tf, t = cpu_sample(4, threads)
        if i >= args.warmup:
            times.append(t)
    g = CFG["Hq"] // CFG["Hkv"]
    fl = 4 * 3.5 * flops_fwd(1, g, CFG["S"], CFG["D"])
    ms = 1e3 * sum(times) / len(times)
    value = fl / (ms / 1e3) / 1e12
    sample = "4 of 64 (batch, kv-group) slices per step: 4 q-heads x S=8192 x D=128 vs one kv-head, fwd+bwd, fp32"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "llama3.1-8b-gqa causal softmax attention fwd+bwd, B=8 Hq=32 Hkv=8 S=8192 D=128 fp16"},
            "cpu_baseline": {"value": value, "unit": "TFLOPS", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# kernel -> (batch of the capture, dram__bytes_read.sum + dram__bytes_write.sum of one launch) at Hq=32, Hkv=8,
# S=8192, D=128, from ncu captures on one B200 (the summaries under profiles/ name the commands)
NCU_DRAM_BYTES = {"ae_attn_fwd": (2, 301.5e6), "ae_attn_bwd_dq": (2, 450.9e6), "ae_attn_bwd_dkv": (2, 396.6e6),
                  "ae_attn_bwd_prep": (2, 273.6e6), "ae_attn_bwd_fused": (1, 436.7e6)}


def time_events(torch, fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def run_other(args):
    """The benchmark's other configurations, one JSON line each (single GPU): cfg3 sigmoid / relu attention
    (B=4, H=32, S=4096, D=128, bf16, non-causal, fwd+bwd), cfg4 Mamba2 SSD (B=8, L=8192, 80 heads, P=64, N=128, bf16,
    fwd+bwd) and cfg5 MLA decode (B=128, H=128, S=8192, fp16, scale 1/sqrt(192))."""
    import math
    import torch
    from attentionengine_b200 import examples as helpers
    from oracle import attention_oracle as orc
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    peaks, which = read_peaks()
    wl = args.workload
    sampler = ClockSampler(0)
    if wl in ("cfg3_sigmoid", "cfg3_relu"):
        B, H, S, D, dt = 4, 32, 4096, 128, torch.bfloat16
        eng = (helpers.sigmoid_engine(B, H, S, D, dt, False) if wl == "cfg3_sigmoid"
               else helpers.relu_engine(B, H, S, D, dt, False, post_scale=1.0 / S))
        q, k, v, d_o = (torch.randn(B, S, H, D, device=dev, dtype=dt) for _ in range(4))
        q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
        custom = (torch.tensor([-math.log(S)], device=dev),) if wl == "cfg3_sigmoid" else ()

        def step():
            q.grad = k.grad = v.grad = None
            eng(q, k, v, *custom).backward(d_o)
        ms = time_events(torch, step, args.steps, args.warmup)
        eng.check_status()
        work = 3.5 * 4.0 * B * H * S * S * D
        value, unit, bound, peak = work / ms / 1e9, "TFLOPS", "tensor", float(peaks.get("bf16_tflops", 1590.0))
        desc = f"{wl[5:]} attention fwd+bwd, B=4 H=32 S=4096 D=128 bf16 non-causal"
        # forward; per batch range of the one-pass backward the main kernel and the dQ cast, and the delta pre-pass where
        # the functor needs it (the ranges apply when no custom tensor is indexed by the batch)
        from attentionengine_b200.attn_engine import attn_bwd as _ab
        n_rng = _ab._batch_parts(B, H, S, dev)  # the sigmoid bias is one scalar: no batch index
        launches = (1 + n_rng * (2 + int(eng.lowered.uses_doosum))) * args.steps
        g = torch.Generator().manual_seed(0)
        qs, ks, vs, ds = (torch.randn(1, S, 2, D, generator=g).to(dt) for _ in range(4))
        fn = ((lambda a, b, c: orc.sigmoid_attention(a, b, c, bias=-math.log(S))) if wl == "cfg3_sigmoid"
              else (lambda a, b, c: orc.relu_attention(a, b, c, post_scale=1.0 / S)))
        t0 = time.perf_counter()
        for _ in range(4):
            orc.fwd_bwd(fn, (qs, ks, vs), ds)
        tc = time.perf_counter() - t0
        cpu = {"value": 4 * 3.5 * 4.0 * 2 * S * S * D / tc / 1e12, "unit": "TFLOPS", "cores": os.cpu_count(), "kind": "port",
               "sample": "4 x (1 batch row, 2 of 32 heads), fwd+bwd, fp32 torch"}
    elif wl == "cfg4":
        B, H, T, DK, DV, dt = args.batch or 8, 80, 8192, 128, 64, torch.bfloat16
        eng = helpers.mamba2_engine(B, H, T, DK, DV, dt, d_skip=True)
        x = torch.randn(B, H, T, DV, device=dev, dtype=dt, requires_grad=True)
        Bm = torch.randn(B, 1, T, DK, device=dev, dtype=dt, requires_grad=True)
        Cm = torch.randn(B, 1, T, DK, device=dev, dtype=dt, requires_grad=True)
        dts = torch.nn.functional.softplus(torch.randn(B, H, T, device=dev) - 4).requires_grad_()
        A = (-torch.exp(torch.rand(H, device=dev) * math.log(16.0))).view(1, H).requires_grad_()
        dtb = dts.detach().to(dt).requires_grad_()
        Dsk = torch.randn(1, H, device=dev).requires_grad_()
        d_o = torch.randn(B, H, T, DV, device=dev, dtype=dt)
        leaves = (x, Bm, Cm, dts, A, dtb, Dsk)

        def step():
            for t_ in leaves:
                t_.grad = None
            eng(Cm, Bm, x, dts, A, dtb, Dsk).backward(d_o)
        ms = time_events(torch, step, args.steps, args.warmup)
        eng.check_status()
        Q = 256
        fwd = (2 * Q * Q * DK + 2 * Q * Q * DV + 4 * Q * DK * DV) * (T // Q) * H * B
        work = 3.5 * fwd
        value, unit, bound, peak = work / ms / 1e9, "TFLOPS", "tensor", float(peaks.get("bf16_tflops", 1590.0))
        desc = ("Mamba2 SSD fwd+bwd with D_skip (v_mod and the skip inside the scan kernel, their backward inside the reverse pass, decay mod eager torch), B=8 L=8192 H=80 P=64 N=128 ngroups=1 bf16; FLOPs by "
                "the chunk-256 convention, fwd (2Q^2N+2Q^2P+4QNP) per chunk and head, bwd counted as 2.5x fwd")
        desc = desc.replace("B=8 ", f"B={B} ")
        # the MMAs the two scan kernels issue, at the chunk size they run (128): forward q k^T, q h, k^T v', P v; reverse
        # pass three 128^3 products and six 128 x 128 x 64 ones per chunk and head
        executed = 2.0 * 128 * 128 * ((128 + 3 * DV) + (3 * 128 + 6 * DV)) * (-(-T // 128)) * H * B
        extra = {"executed_tflops_chunk128": executed / ms / 1e9,
                 "note": "value counts FLOPs by the chunk-256 convention; executed_tflops_chunk128 counts the tensor-core products issued"}
        launches = 7 * args.steps  # scan (row scale, skip, decay scale and the chunk states inside); per batch half: reverse pass (their gradients inside) and two head sums
        from oracle.linear_oracle import linear_scan
        xs, dt_s, As, Bs, Cs = helpers.mamba2_inputs(1, 2, 1024, DK, DV, dt, seed=0)
        t0 = time.perf_counter()
        l2 = [t_.double().requires_grad_() for t_ in (Cs, Bs, xs * dt_s[..., None].to(dt), dt_s * As.view(1, -1, 1))]
        linear_scan(*l2).sum().backward()
        tc = time.perf_counter() - t0
        f_s = (2 * Q * Q * DK + 2 * Q * Q * DV + 4 * Q * DK * DV) * (1024 // Q) * 2
        cpu = {"value": 3.5 * f_s / tc / 1e12, "unit": "TFLOPS", "cores": os.cpu_count(), "kind": "port",
               "sample": "step-by-step recurrence, 1 batch row x 2 heads x 1024 steps, fwd+bwd, fp64 torch"}
    elif wl == "cfg5":
        B, H, S, dt = args.batch or 128, 128, 8192, torch.float16
        eng = helpers.mla_engine(B, H, S, dt, 1 / math.sqrt(192))
        q = torch.randn(B, 1, H, 512, device=dev, dtype=dt)
        q_pe = torch.randn(B, 1, H, 64, device=dev, dtype=dt)
        kv = torch.randn(B, S, 1, 512, device=dev, dtype=dt)
        k_pe = torch.randn(B, S, 1, 64, device=dev, dtype=dt)
        ms = time_events(torch, lambda: eng(q, q_pe, kv, k_pe), args.steps, args.warmup)
        eng.check_status()
        work = (B * S * 576 + B * H * 576 + B * H * 512) * 2.0
        value, unit, bound, peak = work / ms / 1e6, "GB/s", "hbm", float(peaks.get("hbm_gbs", 6650.0))
        desc = f"MLA decode, B={B} H=128 Skv=8192 D=512+64 DV=512 fp16, scale 1/sqrt(192)"
        launches = (1 if eng._mla.last_num_split == 1 else 2) * args.steps
        g = torch.Generator().manual_seed(0)
        qs, ps = torch.randn(4, H, 512, generator=g).to(dt), torch.randn(4, H, 64, generator=g).to(dt)
        kvs, kps = torch.randn(4, S, 1, 512, generator=g).to(dt), torch.randn(4, S, 1, 64, generator=g).to(dt)
        t0 = time.perf_counter()
        for _ in range(3):
            orc.mla_decode(qs, ps, kvs, kps, scale=1 / math.sqrt(192))
        tc = time.perf_counter() - t0
        cpu = {"value": 3 * (4 * S * 576 + 4 * H * 576 + 4 * H * 512) * 2.0 / tc / 1e9, "unit": "GB/s", "cores": os.cpu_count(),
               "kind": "port", "sample": "3 x 4 of 128 batch rows, fp32 torch"}
    elif wl == "gqa_decode":
        # the shape of the reference's attn_script/gqa_inference.py (H=32, 8 kv heads, S=8192, D=128, fp16, one query
        # position) at batch 16 by default: K + V = 537 MB per step, larger than L2 (batch 1 is 33.5 MB and L2-resident)
        B, Hq, Hkv, S, D, dt = args.batch or 16, 32, 8, 8192, 128, torch.float16
        eng = helpers.decode_engine(B, Hq, Hkv, 1, S, D, dt)
        q = torch.randn(B, 1, Hq, D, device=dev, dtype=dt)
        k = torch.randn(B, S, Hkv, D, device=dev, dtype=dt)
        v = torch.randn(B, S, Hkv, D, device=dev, dtype=dt)
        ms = time_events(torch, lambda: eng(q, k, v), args.steps, args.warmup)
        eng.check_status()
        work = (2 * B * S * Hkv * D + 2 * B * Hq * D) * 2.0
        value, unit, bound, peak = work / ms / 1e6, "GB/s", "hbm", float(peaks.get("hbm_gbs", 6650.0))
        desc = f"GQA decode (split-KV + combine), B={B} Hq=32 Hkv=8 Skv=8192 D=128 fp16, {eng._decode.last_num_split} splits"
        launches = (1 if eng._decode.last_num_split == 1 else 2) * args.steps
        g = torch.Generator().manual_seed(0)
        qs = torch.randn(2, 1, Hq, D, generator=g).to(dt)
        ks, vs = torch.randn(2, S, Hkv, D, generator=g).to(dt), torch.randn(2, S, Hkv, D, generator=g).to(dt)
        t0 = time.perf_counter()
        for _ in range(5):
            orc.softmax_attention(qs, ks, vs, False)
        tc = time.perf_counter() - t0
        cpu = {"value": 5 * (2 * 2 * S * Hkv * D + 2 * 2 * Hq * D) * 2.0 / tc / 1e9, "unit": "GB/s", "cores": os.cpu_count(),
               "kind": "port", "sample": "5 x 2 batch rows, fp32 torch"}
    else:
        raise SystemExit(f"unknown workload {wl}")
    clocks = sampler.stop()
    ach = value
    cfg_extra = locals().get("extra", {})
    line = {"metric": desc, "value": value, "unit": unit, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if "fp16" not in desc else "f16", "data": "synthetic",
            "config": {"workload": wl, "l2": "inputs larger than L2", **cfg_extra}, "clocks": clocks, "e2e": None,
            "gpu_launches": launches,
            "roofline": {"bound": bound, "achieved": ach, "peak": peak, "unit": "TFLOP/s" if unit == "TFLOPS" else "GB/s",
                         "frac": ach / peak, "peak_source": f"{which}", "traffic": None, "kernel": "whole step"},
            "cpu_baseline": cpu}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end pass (profiling runs)")
    ap.add_argument("--workload", default="cfg2", help="cfg2 (the headline, default) | cfg3_sigmoid | cfg3_relu | cfg4 | cfg5 | gqa_decode")
    ap.add_argument("--batch", type=int, default=None,
                    help="batch size; default = the benchmark's (8; cfg5: 128). Smaller values are for ncu captures")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="N > 1: split the workload's batch rows over the ranks (strong) or replicate it (weak)")
    ap.add_argument("--bwd", default=None, choices=["fused", "split"], help="backward form (default: the package's)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.workload != "cfg2":
        if rank == 0:
            run_other(args)
        return

    import ctypes as C

    import torch
    import torch.distributed as dist
    from attentionengine_b200 import examples as helpers
    from attentionengine_b200 import runtime as rt
    from attentionengine_b200.attn_engine import attn_bwd as ab

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    Hq, Hkv, S, D = (CFG[k] for k in ("Hq", "Hkv", "S", "D"))
    B_total = args.batch or CFG["B"]
    B = shard_batch(B_total, world, args.scaling)
    mode = args.bwd or ab.DEFAULT_MODE
    dt = torch.float16
    eng = helpers.softmax_engine(B, Hq, Hkv, S, D, D, dt, True)
    eng.bwd_mode = mode
    kern = eng.kernels.bwd_fused if mode == "fused" else eng.kernels.bwd  # compile / load before timing

    gen = torch.Generator(device="cpu").manual_seed(1234 + rank)
    host = {}
    for name, shape in (("q", (B, S, Hq, D)), ("k", (B, S, Hkv, D)), ("v", (B, S, Hkv, D)), ("do", (B, S, Hq, D))):
        t = torch.empty(shape, dtype=dt).pin_memory()
        # fill in chunks to bound host memory for the fp32 temporaries
        for b in range(B):
            t[b].copy_(torch.randn(shape[1:], generator=gen).to(dt))
        host[name] = t
    q, k, v, d_o = (host[n].to(dev, non_blocking=True) for n in ("q", "k", "v", "do"))
    q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
    torch.cuda.synchronize()

    def step_resident():
        q.grad = k.grad = v.grad = None
        o = eng(q, k, v)
        o.backward(d_o)
        return o

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        step_resident()
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step_resident()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop() if sampler else None
    eng.check_status()
    fl_step = 3.5 * flops_fwd(B, Hq, S, D)  # this rank's share
    per_s, ms = aggregate_throughput(fl_step, ms, world, dev)
    value = per_s / 1e12

    # ---- end to end: host buffers in, host buffers out, through the public operator call ----------
    # One operator call per batch row; the row's H2D copies, its forward + backward and its D2H copies run on
    # three streams, so copies of neighbouring rows overlap the kernels.  The same loop without the operator call
    # gives the time the copies alone need on this host (`copy_only_ms`): the floor of any end-to-end figure.
    out_host = {n: torch.empty_like(host[n]).pin_memory() for n in ("q", "k", "v", "do")}
    eng1 = helpers.softmax_engine(1, Hq, Hkv, S, D, D, dt, True)
    eng1.bwd_mode = mode
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    main_s = torch.cuda.current_stream(dev)

    def step_e2e(compute=True):
        for bi in range(B):
            with torch.cuda.stream(s_in):
                qd = host["q"][bi:bi + 1].to(dev, non_blocking=True)
                kd = host["k"][bi:bi + 1].to(dev, non_blocking=True)
                vd = host["v"][bi:bi + 1].to(dev, non_blocking=True)
                dod = host["do"][bi:bi + 1].to(dev, non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(s_in)
            main_s.wait_event(ready)
            for t_ in (qd, kd, vd, dod):
                t_.record_stream(main_s)
            if compute:
                qd.requires_grad_(); kd.requires_grad_(); vd.requires_grad_()
                o = eng1(qd, kd, vd)
                o.backward(dod)
                res = (o.detach(), qd.grad, kd.grad, vd.grad)
            else:
                res = (dod, qd, kd, vd)
            done = torch.cuda.Event()
            done.record(main_s)
            s_out.wait_event(done)
            with torch.cuda.stream(s_out):
                for t_ in res:
                    t_.record_stream(s_out)
                out_host["do"][bi:bi + 1].copy_(res[0], non_blocking=True)
                out_host["q"][bi:bi + 1].copy_(res[1], non_blocking=True)
                out_host["k"][bi:bi + 1].copy_(res[2], non_blocking=True)
                out_host["v"][bi:bi + 1].copy_(res[3], non_blocking=True)
        main_s.wait_stream(s_out)

    def time_e2e(compute, n):
        step_e2e(compute)
        barrier()
        e0.record()
        for _ in range(n):
            step_e2e(compute)
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1) / n, dev)

    n_e2e = 0 if args.no_e2e else max(1, min(args.steps, 3))
    e2e = None
    if n_e2e:
        ms_e2e = time_e2e(True, n_e2e)
        ms_copy = time_e2e(False, n_e2e)
        io_bytes = sum(host[n].numel() * 2 for n in host)
        e2e = {"value": world * fl_step / (ms_e2e / 1e3) / 1e12, "unit": "TFLOPS", "ms_per_step": ms_e2e,
               "copy_only_ms": ms_copy, "h2d_bytes_per_step": io_bytes, "d2h_bytes_per_step": io_bytes,
               "gpu_launches": 4 * B * n_e2e,
               "how": "per batch row: H2D, operator call + backward, D2H on three streams; copy_only_ms = the same "
                      "loop without the operator call (the host-link floor); bytes are per rank"}
        eng1.check_status()

    # ---- per-kernel times (CUDA events on the launching stream) and the roofline of the longest one -----
    kernels = {}
    if rank == 0:
        o, finals = eng._launch_fwd(q.detach(), k.detach(), v.detach(), ())

        def time_call(fn, n=3):
            fn()
            torch.cuda.synchronize()
            a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(n):
                fn()
            b_.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b_) / n

        gemm = flops_fwd(B, Hq, S, D) / 2  # one S x S x D contraction over the causal half
        kernels["ae_attn_fwd"] = {"ms": time_call(lambda: eng._launch_fwd(q.detach(), k.detach(), v.detach(), ())),
                                  "flops": 2 * gemm}
        # backward launches one by one, through the C ABI
        L = rt.lib()
        p = rt.AttnBwdParams()
        qd, kd, vd = q.detach(), k.detach(), v.detach()
        dq, dk, dv = torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)
        delta = torch.empty(B, Hq, S, dtype=torch.float32, device=dev)
        p.q, p.k, p.v, p.o, p.d_o = qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), d_o.data_ptr()
        p.dq, p.dk, p.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
        s3 = ab._s3
        p.q_stride, p.k_stride, p.v_stride, p.o_stride, p.do_stride = s3(qd), s3(kd), s3(vd), s3(o), s3(d_o)
        p.dq_stride, p.dk_stride, p.dv_stride = s3(dq), s3(dk), s3(dv)
        p.final_rowscales[0] = finals[0].data_ptr()
        p.delta = delta.data_ptr()
        p.B, p.Hq, p.Hkv, p.Sq, p.Skv = B, Hq, Hkv, S, S
        p.status = eng._get_status(dev).data_ptr()
        st = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        kernels["ae_attn_bwd_prep"] = {"ms": time_call(lambda: rt.check(L.ae_launch_attn_bwd_prep(kern.prep.handle, C.byref(p), st))),
                                       "flops": 0.0, "bytes": 2.0 * B * S * Hq * D * 2 + B * Hq * S * 4}
        if mode == "fused":
            acc = torch.empty(B, S, Hq, D, dtype=torch.float32, device=dev)
            p.dq_accum = acc.data_ptr()
            # the launcher clears the fp32 accumulator on the stream before the kernel: that clear is inside this time
            kernels["ae_attn_bwd_fused"] = {"ms": time_call(lambda: rt.check(L.ae_launch_attn_bwd_fused(kern.fused.handle, C.byref(p), st))),
                                            "flops": 5 * gemm, "executed_flops": 5 * gemm}
            kernels["ae_attn_bwd_dq_cast"] = {"ms": time_call(lambda: rt.check(L.ae_launch_attn_bwd_dq_cast(kern.cast.handle, C.byref(p), st))),
                                              "flops": 0.0, "bytes": B * S * Hq * D * 6.0}
        else:
            kernels["ae_attn_bwd_dq"] = {"ms": time_call(lambda: rt.check(L.ae_launch_attn_bwd_dq(kern.dq.handle, C.byref(p), st))),
                                         "flops": 1 * gemm, "executed_flops": 3 * gemm}
            kernels["ae_attn_bwd_dkv"] = {"ms": time_call(lambda: rt.check(L.ae_launch_attn_bwd_dkv(kern.dkv.handle, C.byref(p), st))),
                                          "flops": 4 * gemm, "executed_flops": 4 * gemm}
        eng.check_status()

    if rank == 0:
        peaks, which = read_peaks()
        dom = max((n for n in kernels if kernels[n]["flops"] > 0), key=lambda n: kernels[n]["ms"])
        ach = kernels[dom]["flops"] / (kernels[dom]["ms"] / 1e3) / 1e12
        peak = float(peaks.get("bf16_tflops", 1590.0))
        roofline = {"bound": "tensor", "kernel": dom, "achieved": ach, "peak": peak, "unit": "TFLOP/s",
                    "frac": ach / peak, "peak_source": f"{which} cuBLAS bf16 burst",
                    # DRAM bytes per launch of that kernel (dram__bytes_read.sum + dram__bytes_write.sum of one ncu
                    # capture at the batch size of NCU_DRAM_BYTES), scaled by the batch, to which it is proportional
                    "traffic": (NCU_DRAM_BYTES[dom][1] * (B / NCU_DRAM_BYTES[dom][0])) if dom in NCU_DRAM_BYTES else None,
                    "whole_step_frac": value / world / peak,
                    "kernels": {n: {"ms": round(d["ms"], 4), "tflops": round(d["flops"] / (d["ms"] / 1e3) / 1e12, 1)}
                                for n, d in kernels.items()}}
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            tf, t = cpu_sample(16, threads)
            cpu = {"value": tf, "unit": "TFLOPS", "cores": threads, "kind": "port", "seconds": round(t, 2),
                   "sample": "16 of 64 (batch, kv-group) slices: 4 q-heads x S=8192 x D=128 vs one kv-head, fwd+bwd, fp32 torch"}
        # fwd, then per batch range of the one-pass backward: prep, fused, cast | fwd, prep, dQ pass, dK/dV pass
        from attentionengine_b200.attn_engine import attn_bwd as _ab
        n_launch = ((1 + 3 * _ab._batch_parts(B, 32, 8192, dev)) if mode == "fused" else 4) * args.steps
        line = {"metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": args.scaling,
                "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": {"workload": f"llama3.1-8b-gqa causal softmax attention fwd+bwd, B={B_total} Hq=32 Hkv=8 S=8192 D=128 fp16",
                           "per_gpu_batch": B, "backward": mode,
                           "l2": f"inputs ({1.34 * B / 8:.2f} GB per rank and step) larger than L2",
                           "flops_per_step": fl_step * world, "frac_of_nominal_fp16_peak": value / world / 2250.0},
                "clocks": clocks, "e2e": e2e, "gpu_launches": n_launch, "roofline": roofline,
                "cpu_baseline": cpu}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
