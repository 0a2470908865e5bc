#!/usr/bin/env python
"""Benchmark of the FRAC chunked-scan forward at the 135M layer shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the hot path over one batch of synthetic input: the composed
frac_scan forward (u, c, kappa, rho -> h) followed by the skip-mix + gated-RMSNorm epilogue.
Workload at every N: batch 8 x 24 heads (192 sequences), L 8192, R 64, M 128, chunk 256,
bf16 u/c/kappa/z, fp32 rho, per GPU (weak scaling: every rank owns one such batch; the scan
partitions by batch x head, so there is no data-path collective).

Prints ONE JSON line on rank 0.  `--impl reference` times the CPU restatement of the
reference's pure-PyTorch scan (oracle/frac_oracle.py) on the host cores instead.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "frac-ssm-kernels_b200"))

import torch  # noqa: E402

CFG = dict(batch=8, L=8192, H=24, R=64, M=128, T=256)
METRIC = "frac_scan fwd tokens/s (all GPUs) at the 135M layer shape"


def algorithmic_bytes(BH, L, R, M, with_init=False):
    """Scan-level bytes the problem must move: bf16 u, c, kappa, h; fp32 rho; fp32 final state
    (the reference's own accounting, benchmarks/benchmark_frac_scan.py:52-61)."""
    return BH * L * (2 * R + 2 * M + 2 * M + 4 * M + 2 * R) + BH * R * M * 4 * (2 if with_init else 1)


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def device_inputs(dev, seed):
    """Layer-level synthetic inputs with the stated distributions, generated on the device:
    x, Bt, Ct, z ~ N(0,1) bf16; dt = softplus(N(0,1) - 4); A = -exp(U[0, ln 16]); D ~ N(0,1);
    alpha ~ U(0.3, 0.9) per head; mapped to (u, c, kappa, rho) as oracle.layer_inputs does."""
    b, L, H, R, M = CFG["batch"], CFG["L"], CFG["H"], CFG["R"], CFG["M"]
    g = torch.Generator(device=dev).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, device=dev, generator=g)
    x = rn(b, L, H, R).bfloat16()
    z = rn(b, L, H * R).bfloat16()
    dt = torch.nn.functional.softplus(rn(b, L, H) - 4.0)
    A = -torch.exp(torch.rand(H, device=dev, generator=g) * math.log(16.0))
    D = rn(H)
    alpha = 0.3 + 0.6 * torch.rand(H, device=dev, generator=g)
    log_tau = torch.linspace(0.0, math.log(65536.0), M, device=dev)
    rate = (-A) ** (1.0 / alpha)
    prior = -alpha[:, None] * log_tau[None, :]                      # [H, M]
    u = x.permute(0, 2, 1, 3).reshape(b * H, L, R).contiguous()
    c = torch.empty(b * H, L, M, device=dev, dtype=torch.bfloat16)
    kappa = torch.empty_like(c)
    rho = torch.empty(b * H, L, M, device=dev, dtype=torch.float32)
    for bi in range(b):                                             # bound the float32 temporaries
        Bt = rn(L, 1, M).bfloat16().float()
        Ct = rn(L, 1, M).bfloat16().float()
        r = torch.exp(-dt[bi][..., None] * rate[None, :, None] / log_tau.exp()).clamp(1e-6, 1 - 1e-6)
        cw = torch.softmax(prior + Ct, dim=-1)
        ww = torch.softmax(prior + Bt, dim=-1)
        sl = slice(bi * H, (bi + 1) * H)
        rho[sl] = r.permute(1, 0, 2)
        c[sl] = cw.permute(1, 0, 2).bfloat16()
        kappa[sl] = ((1 - r) * ww).permute(1, 0, 2).bfloat16()
    Dhr = D[:, None].expand(H, R).contiguous()
    w = torch.ones(H * R, device=dev, dtype=torch.bfloat16)
    return dict(u=u, c=c, kappa=kappa, rho=rho, x_conv=x.reshape(b, L, H * R), z=z, D=Dhr, w=w)


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML in a thread of this
    process (light; about every 10 ms), or `nvidia-smi -lms 100` when NVML cannot be loaded."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None
        self.sm, self.mx, self.reasons = [], None, set()
        self._stop, self._thread, self._nvml = threading.Event(), None, None

    def _nvml_loop(self):
        nv, h = self._nvml
        names = (("hw_slowdown", nv.nvmlClocksThrottleReasonHwSlowdown),
                 ("hw_thermal_slowdown", nv.nvmlClocksThrottleReasonHwThermalSlowdown),
                 ("sw_thermal_slowdown", nv.nvmlClocksThrottleReasonSwThermalSlowdown),
                 ("sw_power_cap", nv.nvmlClocksThrottleReasonSwPowerCap))
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for name, bit in names:
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                break
            self._stop.wait(0.005)

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[self.index]) if visible and visible.split(",")[0].isdigit() else self.index
            h = nv.nvmlDeviceGetHandleByIndex(phys)
            self.mx = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            self._nvml = (nv, h)
            # first queries are slow (lazy set-up inside NVML): make them before the timed region
            nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
            nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
            self._thread = threading.Thread(target=self._nvml_loop, daemon=True)
            self._thread.start()
            return
        except Exception:
            self._nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def reset(self):
        """Forget the samples taken so far (called at the start of the timed region)."""
        self.sm, self.rows, self.reasons = [], [], set()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([f.strip() for f in line.split(",")])

    def stop(self):
        if self._nvml is not None:
            self._stop.set()
            self._thread.join(timeout=1.0)
            return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.mx,
                    "reasons": sorted(self.reasons), "samples": len(self.sm), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source available"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx = float(r[2])
            except (ValueError, IndexError):
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi"}


def host_threads():
    """Use every host core this process may run on, whatever OMP_NUM_THREADS says (torch.distributed.run
    exports OMP_NUM_THREADS=1 to its workers, which would throttle the CPU arm tenfold); returns the count."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def cpu_baseline_sample(slabs, threads=None):
    """Time the CPU restatement of the reference scan on `slabs` (batch, head) rows of the workload
    (working precision: bf16 inputs, as the reference's upcast=False).  Returns tokens/s and a note."""
    from oracle import frac_oracle as O

    if threads:
        torch.set_num_threads(threads)
    H, L, R, M, T = CFG["H"], CFG["L"], CFG["R"], CFG["M"], CFG["T"]
    u, c, kappa, rho, _ = O.scan_inputs(slabs, L, R, M, dtype=torch.bfloat16, gen="model_like", seed=0)
    O.frac_scan_slabs(u[:1, :1024], c[:1, :1024], kappa[:1, :1024], rho[:1, :1024], T, None, True)  # warm
    t0 = time.perf_counter()
    O.frac_scan_slabs(u, c, kappa, rho, T, None, True, exact=False, slab=1)
    dt = time.perf_counter() - t0
    tokens = slabs * L / H
    return tokens / dt, dt


def run_reference(args, rank):
    """The reference arm: the oracle port on the host cores, one bounded sample per step."""
    if rank != 0:
        return
    from oracle import frac_oracle as O

    H, L, R, M, T = CFG["H"], CFG["L"], CFG["R"], CFG["M"], CFG["T"]
    slabs = 2
    cores = host_threads()
    u, c, kappa, rho, _ = O.scan_inputs(slabs, L, R, M, dtype=torch.bfloat16, gen="model_like", seed=0)
    for _ in range(args.warmup):
        O.frac_scan_slabs(u[:1], c[:1], kappa[:1], rho[:1], T, None, True, exact=False, slab=1)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.frac_scan_slabs(u, c, kappa, rho, T, None, True, exact=False, slab=1)
    dt = (time.perf_counter() - t0) / args.steps
    value = slabs * L / H / dt
    sample = (f"{slabs} of the {CFG['batch'] * H} (batch, head) rows per step, L {L}, "
              f"working precision (bf16 inputs), torch {torch.__version__}, "
              f"{os.cpu_count()} logical cpus, {cores} torch threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def _timed(step, steps, warmup, dev, dist):
    """W untimed + K timed calls of `step` between two events, barrier + synchronise on both sides,
    max over ranks; returns ms per step."""
    for _ in range(warmup):
        step()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    return ms


def _all_ok(ok, dev, dist):
    """True when `ok` holds on every rank."""
    flag = torch.tensor([1 if ok else 0], device=dev)
    if dist is not None:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(flag.item())


def scan_inputs_device(B, L, R, M, dev, seed):
    """Seeded scan-level inputs made on the device (the same on every rank that uses the same seed):
    u, c, kappa ~ 0.25 N(0,1) bf16, model-like decay in [1e-6, 1 - 1e-6], initial state 0.25 N(0,1)."""
    g = torch.Generator(device=dev).manual_seed(seed)
    rn = lambda *sh: torch.randn(*sh, device=dev, generator=g)
    u, c, kappa = (0.25 * rn(B, L, R)).bfloat16(), (0.25 * rn(B, L, M)).bfloat16(), (0.25 * rn(B, L, M)).bfloat16()
    tau = torch.linspace(0.0, math.log(65536.0), M, device=dev).exp()
    dt = torch.nn.functional.softplus(rn(B, L, 1) - 2.0)
    rho = torch.exp(-dt * 2.0 / tau).clamp(1e-6, 1 - 1e-6)
    return u, c, kappa, rho, 0.25 * rn(B, R, M)


def seq_parity(rank, world, dev, dist):
    """Small case of the sequence-sharded scan against the single-GPU scan of the whole sequence
    (every rank builds the same inputs from one seed): h within 2e-2, final state within 1e-3."""
    from frac_ssm_b200 import parallel
    B, R, M, T = 6, CFG["R"], CFG["M"], CFG["T"]
    L = 4096 * max(world, 2)
    u, c, kappa, rho, init = scan_inputs_device(B, L, R, M, dev, seed=5)
    h_ref, f_ref = parallel.CudaStageOps.scan(u, c, kappa, rho, T, init)
    if world == 1:      # one rank: the same composition with the segment cut into two sub-segments
        h, fin = parallel.seq_parallel_scan(u, c, kappa, rho, T, init, True, local_splits=2)
        tok = slice(0, L)
    else:
        tok = parallel.shard_tokens(L, T, rank, world)
        h, fin = parallel.seq_parallel_scan(u[:, tok].contiguous(), c[:, tok].contiguous(),
                                            kappa[:, tok].contiguous(), rho[:, tok].contiguous(), T, init, True)
    ok = torch.allclose(h.float(), h_ref[:, tok].float(), rtol=2e-2, atol=2e-2) and \
        torch.allclose(fin, f_ref, rtol=1e-3, atol=1e-3)
    return _all_ok(ok, dev, dist)


def measure_seq(args, rank, world, dev, dist, steps, warmup):
    """Config 3: batch 1, L 1,048,576, 24 heads, sequence split evenly over the ranks; per step one
    segment-summary pass, one all-gather of (state, decay) per rank (none on one rank), one scan of the
    sub-segments with their true incoming states."""
    from frac_ssm_b200 import parallel
    Ltot, H, R, M, T = 1048576, CFG["H"], CFG["R"], CFG["M"], CFG["T"]
    tok = parallel.shard_tokens(Ltot, T, rank, world)
    Ll = tok.stop - tok.start
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    u = (0.25 * torch.randn(H, Ll, R, device=dev, generator=g)).bfloat16()
    c = torch.softmax(torch.randn(H, Ll, M, device=dev, generator=g), -1).bfloat16()
    tau = torch.linspace(0.0, math.log(65536.0), M, device=dev).exp()
    dt = torch.nn.functional.softplus(torch.randn(H, Ll, 1, device=dev, generator=g) - 4.0)
    rho = torch.exp(-dt * 4.0 / tau).clamp(1e-6, 1 - 1e-6)
    kappa = ((1 - rho) * torch.softmax(torch.randn(H, Ll, M, device=dev, generator=g), -1)).bfloat16()
    del dt
    # the sub-segment count is fixed here (the same on every rank), so no step synchronises the host
    # (one rank splits too: 24 rows are 24 state chains for 148 SMs, and the extra read of u, kappa and
    # rho for the sub-segment summaries costs less than the idle SMs do)
    S = 1
    while H * S < 148 and Ll % (2 * S * T) == 0 and Ll // (2 * S) >= 1024:
        S *= 2

    def step():
        return parallel.seq_parallel_scan(u, c, kappa, rho, T, None, False, local_splits=S)

    ms = _timed(step, steps, warmup, dev, dist)
    del u, c, kappa, rho
    torch.cuda.empty_cache()
    parity_ok = seq_parity(rank, world, dev, dist)
    peak, peak_kind = measured_peak_gbs()
    alg = algorithmic_bytes(H, Ltot, R, M)
    gathered = 0 if world == 1 else H * S * (R * M + M) * 4
    return {"workload": "config 3: batch 1, L 1048576, 24 heads, R 64, M 128, chunk 256, bf16",
            "sharding": f"sequence over {world} GPU(s), {S} sub-segment(s) per rank", "ms_per_step": ms, "steps": steps, "warmup": warmup,
            "tokens_per_s": Ltot / (ms * 1e-3), "algorithmic_GBps_all_gpus": alg / (ms * 1e-3) / 1e9,
            "frac_of_hbm_peak_per_gpu": alg / (ms * 1e-3) / 1e9 / world / peak, "peak_kind": f"of {peak_kind}",
            "collective": ("none" if world == 1 else
                           f"one all_gather_into_tensor per step, {gathered} bytes sent per rank "
                           f"({S} sub-segment(s) per rank), NCCL"),
            "collective_bytes_per_rank": gathered, "parity_ok": parity_ok,
            "parity_case": f"6 rows, L {4096 * max(world, 2)}, sharded scan vs the single-GPU scan, "
                           "h within 2e-2, final state within 1e-3"}


def run_seq_workload(args, rank, world, dev, dist):
    res = measure_seq(args, rank, world, dev, dist, args.steps, max(args.warmup, 3))
    if rank == 0:
        print(json.dumps({"metric": "frac_scan fwd tokens/s, one 1,048,576-token sequence split by sequence",
                          "value": res["tokens_per_s"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                          "warmup": max(args.warmup, 3), "ms_per_step": res["ms_per_step"],
                          "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
                          "data": "synthetic", "config": {"workload": res["workload"], "sharding": res["sharding"]},
                          "config3": res}), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def measure_heads(args, rank, world, dev, dist, steps, warmup):
    """Config 4: batch 4, L 16384, 64 heads in 8 groups, R 64, M 128, chunk 256, with the skip-mix and
    gated-RMSNorm epilogue; the heads are spread over the ranks.  Per step and rank: one scan of its
    own heads, one [batch, L] float32 all-reduce for the norm, the two epilogue passes."""
    from frac_ssm_b200 import parallel
    from frac_ssm_b200.layers import scan_epilogue
    from frac_ssm_b200.ops.b200.frac_scan import frac_scan
    batch, L, H, G, R, M, T = 4, 16384, 64, 8, CFG["R"], CFG["M"], CFG["T"]
    if H % world:
        raise SystemExit(f"--workload heads: {H} heads do not divide over {world} ranks")
    hs = parallel.shard_heads(H, rank, world)
    n = hs.stop - hs.start
    # layer-level distributions mapped through the reference's prep math (seeded per head, so the
    # data of a head does not depend on how many ranks there are)
    log_tau = torch.linspace(0.0, math.log(65536.0), M, device=dev)
    gg = torch.Generator(device=dev).manual_seed(7)
    Bt = torch.randn(batch, L, G, M, device=dev, generator=gg)
    Ct = torch.randn(batch, L, G, M, device=dev, generator=gg)
    u = torch.empty(batch, n, L, R, device=dev, dtype=torch.bfloat16)
    c = torch.empty(batch, n, L, M, device=dev, dtype=torch.bfloat16)
    kappa = torch.empty_like(c)
    rho = torch.empty(batch, n, L, M, device=dev, dtype=torch.float32)
    D = torch.empty(n, R, device=dev)
    for i, head in enumerate(range(hs.start, hs.stop)):
        gh = torch.Generator(device=dev).manual_seed(1000 + head)
        u[:, i] = torch.randn(batch, L, R, device=dev, generator=gh).bfloat16()
        dt = torch.nn.functional.softplus(torch.randn(batch, L, 1, device=dev, generator=gh) - 4.0)
        lam = torch.exp(torch.rand(1, device=dev, generator=gh) * math.log(16.0))
        alpha = 0.3 + 0.6 * torch.rand(1, device=dev, generator=gh)
        D[i] = torch.randn(1, device=dev, generator=gh)
        grp = head // (H // G)
        prior = -alpha * log_tau
        r = torch.exp(-dt * lam ** (1.0 / alpha) / log_tau.exp()).clamp(1e-6, 1 - 1e-6)
        rho[:, i] = r
        c[:, i] = torch.softmax(prior + Ct[:, :, grp], -1).bfloat16()
        kappa[:, i] = ((1 - r) * torch.softmax(prior + Bt[:, :, grp], -1)).bfloat16()
    del Bt, Ct
    u, c, kappa, rho = (t.view(batch * n, L, -1) for t in (u, c, kappa, rho))
    x_conv = u.view(batch, n, L, R).permute(0, 2, 1, 3).reshape(batch, L, n * R).contiguous()
    z = torch.randn(batch, L, n * R, device=dev, generator=gg).bfloat16()
    w = torch.ones(n * R, device=dev, dtype=torch.bfloat16)

    def step():
        if args.fused_layer:
            return parallel.head_parallel_layer(u, c, kappa, rho, z, D, w, n, H, 1e-6)
        h = frac_scan(u, c, kappa, rho, T, None, False)
        if world == 1:
            return scan_epilogue(h, x_conv, z, D, w, n, R, 1e-6)
        return parallel.head_parallel_epilogue(h, x_conv, z, D, w, n, R, H, 1e-6)

    ms = _timed(step, steps, warmup, dev, dist)
    del u, c, kappa, rho, x_conv, z
    torch.cuda.empty_cache()
    parity_ok = heads_parity(rank, world, dev, dist)
    peak, peak_kind = measured_peak_gbs()
    alg = algorithmic_bytes(batch * H, L, R, M) + 4 * batch * L * H * R * 2     # scan + epilogue (h, x, z in, y out)
    return {"workload": "config 4: batch 4, L 16384, 64 heads in 8 groups, R 64, M 128, chunk 256, bf16, "
                        "with skip-mix and gated RMSNorm",
            "sharding": f"heads over {world} GPU(s)", "ms_per_step": ms, "steps": steps, "warmup": warmup,
            "tokens_per_s": batch * L / (ms * 1e-3), "algorithmic_GBps_all_gpus": alg / (ms * 1e-3) / 1e9,
            "frac_of_hbm_peak_per_gpu": alg / (ms * 1e-3) / 1e9 / world / peak, "peak_kind": f"of {peak_kind}",
            "collective": ("none" if world == 1 else
                           f"one all_reduce (sum) of a [batch, L] float32 vector per step, {batch * L * 4} bytes, NCCL"),
            "collective_bytes_per_rank": 0 if world == 1 else batch * L * 4, "parity_ok": parity_ok,
            "parity_case": "batch 2, L 512, 64 heads: the layer with its heads spread over the ranks vs the same "
                           "layer unsharded; bf16 outputs within rtol 1e-2 (two bf16 steps: the sums of squares "
                           "are added in another order) and atol 1e-3"}


def heads_parity(rank, world, dev, dist):
    """Small case at config 4's head count (same seed on every rank): the layer with its 64 heads spread
    over the ranks against the same layer unsharded, in both forms the library has: scan + two-pass
    epilogue with one all-reduce of the rows' sums of squares, and the scan with the gate fused into its
    output stage + norm pass.  One rank: two shards in turn, their sums added by hand."""
    from frac_ssm_b200 import parallel
    from frac_ssm_b200.layers import (scan_epilogue, scan_epilogue_apply, scan_epilogue_sumsq, scan_layer,
                                      scan_layer_gated, scan_layer_norm, scan_layer_sumsq)
    from frac_ssm_b200.ops.b200 import frac_scan
    batch, L, H, R, M, T = 2, 512, 64, CFG["R"], CFG["M"], CFG["T"]
    u, c, kappa, rho, _ = scan_inputs_device(batch * H, L, R, M, dev, seed=77)
    g = torch.Generator(device=dev).manual_seed(78)
    z = torch.randn(batch, L, H * R, device=dev, generator=g).bfloat16()
    D = torch.randn(H, R, device=dev, generator=g)
    w = (torch.rand(H * R, device=dev, generator=g) + 0.5).bfloat16()
    x_conv = u.view(batch, H, L, R).permute(0, 2, 1, 3).reshape(batch, L, H * R).contiguous()
    y_ref = scan_epilogue(frac_scan(u, c, kappa, rho, T, None, False), x_conv, z, D, w, H, R, 1e-6)
    y_ref_fused = scan_layer(u, c, kappa, rho, z, D, w, H, 1e-6)
    rows = lambda t, hs: t.view(batch, H, L, -1)[:, hs].reshape(-1, L, t.shape[-1]).contiguous()
    near = lambda a, b: torch.allclose(a.float(), b.float(), rtol=1e-2, atol=1e-3)
    ok = True
    shards = [parallel.shard_heads(H, r, 2) for r in range(2)] if world == 1 else [parallel.shard_heads(H, rank, world)]
    loc = []
    for hs in shards:
        cols = slice(hs.start * R, hs.stop * R)
        loc.append((hs, cols, rows(u, hs), rows(c, hs), rows(kappa, hs), rows(rho, hs), z[..., cols].contiguous(),
                    x_conv[..., cols].contiguous(), D[hs].contiguous(), w[cols].contiguous()))
    if world == 1:
        hl = [frac_scan(ul, cl, kl, rl, T, None, False) for _, _, ul, cl, kl, rl, _, _, _, _ in loc]
        tot = sum(scan_epilogue_sumsq(h, xl, zl, Dl, hs.stop - hs.start, R, 0.0)
                  for h, (hs, _, _, _, _, _, zl, xl, Dl, _) in zip(hl, loc))
        fused = [scan_layer_gated(ul, cl, kl, rl, zl, Dl, hs.stop - hs.start)[:2]
                 for hs, _, ul, cl, kl, rl, zl, _, Dl, _ in loc]
        tot_f = sum(scan_layer_sumsq(ss) for _, ss in fused)
        for h, (gated, ss), (hs, cols, _, _, _, _, zl, xl, Dl, wl) in zip(hl, fused, loc):
            y = scan_epilogue_apply(h, xl, zl, Dl, wl, hs.stop - hs.start, R, tot, H * R, 1e-6, 0.0)
            yf = scan_layer_norm(gated, ss, wl, R, 1e-6, sumsq=tot_f, norm_width=H * R)
            ok = ok and near(y, y_ref[..., cols]) and near(yf, y_ref_fused[..., cols])
    else:
        hs, cols, ul, cl, kl, rl, zl, xl, Dl, wl = loc[0]
        nl = hs.stop - hs.start
        y = parallel.head_parallel_epilogue(frac_scan(ul, cl, kl, rl, T, None, False), xl, zl, Dl, wl, nl, R, H, 1e-6)
        yf = parallel.head_parallel_layer(ul, cl, kl, rl, zl, Dl, wl, nl, H, 1e-6)
        ok = near(y, y_ref[..., cols]) and near(yf, y_ref_fused[..., cols])
    return _all_ok(ok, dev, dist)


def run_heads_workload(args, rank, world, dev, dist):
    res = measure_heads(args, rank, world, dev, dist, args.steps, max(args.warmup, 3))
    if rank == 0:
        print(json.dumps({"metric": "layer forward tokens/s (scan + skip-mix + gated RMSNorm), heads sharded",
                          "value": res["tokens_per_s"], "unit": "tokens/s", "n_gpus": world,
                          "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": res["ms_per_step"],
                          "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
                          "data": "synthetic", "config": {"workload": res["workload"], "sharding": res["sharding"]},
                          "config4": res}), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_model_workload(args, rank, world, dev, dist):
    """Config 2: prefill of the whole model (24 layers, hidden 768, 24 heads of 64, 128 modes, chunk 256,
    vocabulary 50280, bf16, random weights), batch 16 x 4096 uniform token ids split over the ranks by
    batch; independent replicas, no communication."""
    from frac_ssm_b200.models import FracConfig, FracForCausalLM
    batch, L = 16, args.seq_len or 4096
    if batch % world:
        raise SystemExit(f"--workload model: batch {batch} does not divide over {world} ranks")
    cfg = FracConfig(vocab_size=50280, hidden_size=768, num_hidden_layers=24, num_attention_heads=24,
                     frac_expand=2.0, frac_num_modes=128, frac_chunk_size=256)
    torch.manual_seed(0)
    model = FracForCausalLM(cfg).to(device=dev, dtype=torch.bfloat16).eval()
    g = torch.Generator(device=dev).manual_seed(50 + rank)
    ids = torch.randint(0, cfg.vocab_size, (batch // world, L), device=dev, generator=g)

    def step():
        with torch.no_grad():
            return model(ids, use_cache=False)[0]

    launch = {"kind": "plain launches"}

    def timed():
        for _ in range(max(args.warmup, 3)):
            step()
        # one prefill captured as a CUDA graph and replayed K times, as for config 1: a step is about 700
        # launches from Python, and a busy host (other jobs on the box) then starves the GPU between them
        # (single process only: under torchrun the captured step did not get through its first barrier
        # in one 2-GPU run, so ranks of a multi-process run launch the step plainly)
        graph = None
        if not args.no_graph and dist is None:
            try:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    step()
                torch.cuda.current_stream().wait_stream(side)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    step()
                graph.replay()
                torch.cuda.synchronize()
                launch["kind"] = "CUDA graph of one prefill, replayed once per step"
            except Exception as exc:      # noqa: BLE001 - any capture problem falls back to plain launches
                print(f"bench: CUDA graph capture of the model step failed ({exc}); timing plain launches",
                      file=sys.stderr)
                graph = None
                launch["kind"] = "plain launches"
                torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            if graph is not None:
                graph.replay()
            else:
                step()
        e1.record()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        t_ms = e0.elapsed_time(e1) / args.steps
        if dist is not None:
            t = torch.tensor([t_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_ms = t.item()
        return t_ms

    ms_f32 = timed()              # float32 scan coefficients, as the reference's prep emits them
    for layer in model.model.layers:
        layer.mixer.coeff_dtype = torch.bfloat16
    ms = timed()                  # bfloat16 coefficients: the benchmark's headline configuration
    # decode: one prefill with the cache kept, then single-token steps through the state-update kernel
    _, past = model(ids, use_cache=True)
    nxt = torch.randint(0, cfg.vocab_size, (batch // world, 1), device=dev, generator=g)
    for _ in range(3):
        _, past = model(nxt, past_key_values=past, use_cache=True)
    torch.cuda.synchronize()
    d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n_dec = 16
    d0.record()
    for _ in range(n_dec):
        _, past = model(nxt, past_key_values=past, use_cache=True)
    d1.record()
    torch.cuda.synchronize()
    dec_ms = d0.elapsed_time(d1) / n_dec
    del past
    if rank == 0:
        nparam = sum(p.numel() for p in model.parameters())
        print(json.dumps({"metric": "model prefill tokens/s (all GPUs)", "value": batch * L / (ms * 1e-3),
                          "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
                          "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                          "dtype": "bf16", "data": "synthetic",
                          "config": {"workload": f"config 2: 24-layer model prefill, batch {batch} x L {L}, hidden 768, "
                                                 "24 heads x 64, 128 modes, chunk 256, vocabulary 50280",
                                     "parameters": nparam, "scan_coefficients": "bf16",
                                     "timed_launch": launch["kind"],
                                     "ms_per_step_with_f32_scan_coefficients": ms_f32,
                                     "decode_ms_per_token_step_rank0": dec_ms,
                                     "decode_batch_per_gpu": batch // world,
                                     "sharding": f"batch over {world} GPU(s), replicas, no collective"}}), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_stages_workload(args, rank, world, dev, dist):
    """Each of the reference's five stage kernels (and the fused W+readout) timed alone on the
    config-1 scan shape, with the bytes it must move and the fraction of the HBM peak it reaches.
    The stages are the fallback route of frac_scan; the single-pass kernel replaces them on the hot
    path, so this line explains the fallback, it is not the benchmark."""
    from frac_ssm_b200.ops.b200 import stages
    B, L, R, M, T = CFG["batch"] * CFG["H"], (args.seq_len or CFG["L"]), CFG["R"], CFG["M"], CFG["T"]
    N = (L + T - 1) // T
    u, c, kappa, rho, init = scan_inputs_device(B, L, R, M, dev, seed=11 + rank)
    log_rho = torch.log(rho)
    lcr, cd = stages.chunk_cumsum(log_rho, T)
    states = stages.chunk_state(u, kappa, lcr, T)
    acc, fin = stages.state_passing(states, cd, init)
    peak, peak_kind = measured_peak_gbs()
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    f4, b2 = 4, 2
    cases = [
        ("chunk_cumsum", lambda: stages.chunk_cumsum(log_rho, T), B * L * M * f4 * 2 + B * N * M * f4),
        ("chunk_state", lambda: stages.chunk_state(u, kappa, lcr, T),
         B * L * (R * b2 + M * b2 + M * f4) + B * N * R * M * f4),
        ("state_passing", lambda: stages.state_passing(states, cd, init),
         2 * B * N * R * M * f4 + B * N * M * f4 + 2 * B * R * M * f4),
        ("chunk_w", lambda: stages.chunk_w(c, kappa, lcr, T), B * L * (2 * M * b2 + M * f4) + B * N * T * T * f4),
        ("chunk_fused_readout", lambda: stages.chunk_fused_readout(u, c, kappa, acc, lcr, T),
         B * L * (2 * R * b2 + 2 * M * b2 + M * f4) + B * N * R * M * f4),
    ]
    W = stages.chunk_w(c, kappa, lcr, T) if B * N * T * T * 4 <= 16 << 30 else None
    if W is not None:
        cases.append(("chunk_readout", lambda: stages.chunk_readout(u, c, acc, W, lcr, T),
                      B * L * (2 * R * b2 + M * b2 + M * f4) + B * N * (R * M + T * T) * f4))
    out = {}
    total_ms = 0.0
    for name, fn, nbytes in cases:
        ms = _timed(fn, steps, warmup, dev, dist)
        out[name] = {"ms": round(ms, 4), "bytes": nbytes, "gbs": round(nbytes / ms / 1e6, 1),
                     "frac_of_hbm_peak": round(nbytes / ms / 1e6 / peak, 3)}
        if name in ("chunk_cumsum", "chunk_state", "state_passing", "chunk_fused_readout"):
            total_ms += ms
    if rank == 0:
        print(json.dumps({"metric": "stage kernels, each timed alone", "workload": "stages",
                          "value": world * B * L / (total_ms * 1e-3), "unit": "tokens/s",
                          "note": "value = (batch x head) tokens over the sum of the four stages of the staged route "
                                  "(cumsum, state, passing, fused readout)",
                          "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(total_ms, 4),
                          "higher_is_better": True, "scaling": "weak", "dtype": "bf16", "data": "synthetic",
                          "peak_gbs": peak, "peak_kind": peak_kind, "stages": out,
                          "config": {"workload": f"stage kernels on the config-1 scan shape: {B} (batch, head) rows "
                                                 f"x L {L}, R {R}, M {M}, chunk {T}"}}))
    if dist is not None:
        dist.destroy_process_group()


def workload_config(n):
    return {"workload": "config 1: single-layer frac_scan forward + skip-mix/gated-RMSNorm epilogue, "
                        "batch 8 x 24 heads, L 8192, R 64, M 128, chunk 256, per GPU",
            "batch_per_gpu": CFG["batch"], "seq_len": CFG["L"], "nheads": CFG["H"], "headdim": CFG["R"],
            "d_state": CFG["M"], "chunk_size": CFG["T"], "sharding": f"batch x head over {n} GPU(s), no collective",
            "l2": "inputs (2.2 GB per step) exceed the 126 MB L2; no flush needed"}


def profiled_traffic(head_tokens):
    """DRAM bytes per launch of the single-pass kernel, from profiles/scan_fused_kernel_small_case.md.
    That file records `traffic_bytes_per_head_token` and the hash of the kernel source it was captured
    from (`kernel_source_sha256`); a capture of another build does not describe this one."""
    import hashlib
    import re
    here = os.path.dirname(os.path.abspath(__file__))
    try:
        text = open(os.path.join(here, "profiles", "scan_fused_kernel_small_case.md")).read()
        src = open(os.path.join(here, "frac-ssm-kernels_b200", "csrc", "scan_fused.cu"), "rb").read()
    except OSError:
        return None
    per = re.search(r"traffic_bytes_per_head_token:\s*([0-9.]+)", text)
    sha = re.search(r"kernel_source_sha256:\s*([0-9a-f]{64})", text)
    if not per or not sha or sha.group(1) != hashlib.sha256(src).hexdigest():
        return None
    return int(float(per.group(1)) * head_tokens)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--path", default="auto", choices=["auto", "staged", "fused"])
    ap.add_argument("--seq-len", type=int, default=None,
                    help="override L (smaller cases for profiler captures; not the benchmark workload)")
    ap.add_argument("--workload", default="layer", choices=["layer", "seq", "heads", "model", "stages"],
                    help="layer: config 1 per GPU (the benchmark); seq: config 3, one sequence of 1,048,576 "
                         "tokens x 24 heads split over the ranks; heads: config 4, one layer's 64 heads spread over the "
                         "ranks; model: config 2, prefill of the 24-layer model, batch 16 x 4096 "
                         "split over the ranks (secondary lines, not the driver's metric)")
    ap.add_argument("--step-times", action="store_true",
                    help="also print every timed step's scan-kernel time to stderr (diagnostic)")
    ap.add_argument("--watchdog", type=int, default=1500,
                    help="seconds after which a stalled run dumps its Python stacks and exits (0 = off)")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch the timed steps one by one instead of replaying a captured CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--fused-layer", action="store_true",
                    help="time the layer path with the skip-mix and the gate inside the scan kernel's output stage "
                         "(two kernels, h never written) instead of scan + one-pass epilogue; measured slower: the "
                         "scan kernel's worker warps are its bottleneck")
    ap.add_argument("--no-sharded", action="store_true",
                    help="skip the config 3 (sequence-sharded) and config 4 (head-sharded) sections of the line")
    args = ap.parse_args()
    if args.watchdog > 0:      # a stalled run must end with a traceback, not run until someone kills it
        import faulthandler
        faulthandler.dump_traceback_later(args.watchdog, exit=True)

    if args.seq_len:
        CFG["L"] = args.seq_len
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    args.warmup = max(args.warmup, 3)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    from frac_ssm_b200 import _cabi
    from frac_ssm_b200.layers import scan_epilogue, scan_layer
    from frac_ssm_b200.ops.b200 import frac_scan

    _cabi.lib()
    if args.workload == "heads":
        run_heads_workload(args, rank, world, dev, dist)
        return
    if args.workload == "model":
        run_model_workload(args, rank, world, dev, dist)
        return
    if args.workload == "stages":
        run_stages_workload(args, rank, world, dev, dist)
        return
    if args.workload == "seq":
        run_seq_workload(args, rank, world, dev, dist)
        return
    d = device_inputs(dev, seed=rank)
    H, R, T = CFG["H"], CFG["R"], CFG["T"]
    BH, L, M = d["u"].shape[0], CFG["L"], CFG["M"]
    fused = bool(_cabi.lib().fracssm_scan_fused_supported(BH, L, R, M, T, _cabi.BF16, _cabi.BF16))
    use_fused = fused and args.path != "staged"
    launches_per_step = (1 if use_fused else 4) + 1
    layer_fused = use_fused and args.fused_layer

    def step():
        if layer_fused:    # skip-mix and gate inside the scan kernel's output stage, then the norm pass
            return scan_layer(d["u"], d["c"], d["kappa"], d["rho"], d["z"], d["D"], d["w"], H, 1e-6)
        h = frac_scan(d["u"], d["c"], d["kappa"], d["rho"], T, None, False, path=args.path)
        return scan_epilogue(h, d["x_conv"], d["z"], d["D"], d["w"], H, R, 1e-6)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # preheat: a fresh GPU needs a few hundred ms of work before its clocks settle (the reference's
    # timer does the same with a 200 ms GEMM, frac_ssm/benchmark.py:274-293); untimed, like the warm-up
    t_pre = time.perf_counter()
    while time.perf_counter() - t_pre < 0.5:
        for _ in range(10):
            step()
        torch.cuda.synchronize()
    # the sampler starts before the warm-up: its thread's first queries stall kernel launches for
    # several ms; what it collected so far is dropped when the timed region begins
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        t_s = time.perf_counter()
        while len(sampler.sm) + len(sampler.rows) < 2 and time.perf_counter() - t_s < 0.5:
            step()
            torch.cuda.synchronize()
    for _ in range(args.warmup):
        step()
    barrier()
    # One step captured as a CUDA graph (workspace clear + scan kernel + epilogue kernel), replayed
    # K times in the timed region: host-side jitter (other processes on the box, the sampler thread)
    # then cannot starve the GPU between launches.  If capture is not possible the K steps are
    # launched one by one, as in the per-kernel pass below.
    graph = None
    if not args.no_graph:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step()
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                y = step()
            graph.replay()
            torch.cuda.synchronize()
        except Exception as exc:      # noqa: BLE001 - any capture problem falls back to plain launches
            print(f"bench: CUDA graph capture failed ({exc}); timing plain launches", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()
    barrier()
    timed_launch = "CUDA graph of one step, replayed once per step" if graph is not None else "plain launches"
    sampler.reset()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        if graph is not None:
            graph.replay()
        else:
            y = step()
    e1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = e0.elapsed_time(e1) / args.steps
    # per-kernel pass (plain launches, CUDA events around the scan kernel of every step)
    scan_evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                for _ in range(args.steps)]
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    for a, b in scan_evs:
        a.record()
        h = frac_scan(d["u"], d["c"], d["kappa"], d["rho"], T, None, False, path=args.path)
        b.record()
        y = scan_epilogue(h, d["x_conv"], d["z"], d["D"], d["w"], H, R, 1e-6)
    p1.record()
    barrier()
    ms_plain = p0.elapsed_time(p1) / args.steps
    scan_times = [a.elapsed_time(b) for a, b in scan_evs]
    # the scan alone, again as K replays of a captured graph between two events: its average launch
    # duration without the gaps a busy host leaves between an event and the launch that follows it
    scan_ms_graph = None
    if graph is not None:
        try:
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2):
                h = frac_scan(d["u"], d["c"], d["kappa"], d["rho"], T, None, False, path=args.path)
            g2.replay()
            torch.cuda.synchronize()
            q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            q0.record()
            for _ in range(args.steps):
                g2.replay()
            q1.record()
            torch.cuda.synchronize()
            scan_ms_graph = q0.elapsed_time(q1) / args.steps
        except Exception as exc:      # noqa: BLE001
            print(f"bench: scan-only graph failed ({exc}); using the per-step events", file=sys.stderr)
            torch.cuda.synchronize()
    scan_ms = scan_ms_graph if scan_ms_graph is not None else statistics.mean(scan_times)
    scan_ms_median = statistics.median(scan_times)
    if args.step_times and rank == 0:
        print("scan ms per step:", " ".join(f"{t:.3f}" for t in scan_times), file=sys.stderr)
    if dist is not None:
        t = torch.tensor([ms, scan_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, scan_ms = t.tolist()
    tokens = CFG["batch"] * L * world
    value = tokens / (ms * 1e-3)

    # end to end: pinned host buffers in, result out, copies inside the timed region
    e2e = None
    if not args.no_e2e:
        names = ("u", "c", "kappa", "rho", "z") if layer_fused else ("u", "c", "kappa", "rho", "x_conv", "z")
        host = {k: torch.empty(d[k].shape, dtype=d[k].dtype, pin_memory=True).copy_(d[k]) for k in names}
        y_host = torch.empty(y.shape, dtype=y.dtype, pin_memory=True)
        h2d = sum(host[k].numel() * host[k].element_size() for k in names)
        d2h = y_host.numel() * y_host.element_size()

        def e2e_step():
            t = {k: host[k].to(dev, non_blocking=True) for k in names}
            if layer_fused:
                yy = scan_layer(t["u"], t["c"], t["kappa"], t["rho"], t["z"], d["D"], d["w"], H, 1e-6)
            else:
                hh = frac_scan(t["u"], t["c"], t["kappa"], t["rho"], T, None, False, path=args.path)
                yy = scan_epilogue(hh, t["x_conv"], t["z"], d["D"], d["w"], H, R, 1e-6)
            y_host.copy_(yy, non_blocking=True)

        e2e_step()
        barrier()
        k2 = max(2, min(args.steps, 5))
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(k2):
            e2e_step()
        s1.record()
        barrier()
        ems = s0.elapsed_time(s1) / k2
        if dist is not None:
            t = torch.tensor([ems], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ems = t.item()
        e2e = {"value": tokens / (ems * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": ems, "steps": k2}
        del host, y_host

    # The two sharding modes that communicate, measured in the same process on the same ranks (at one
    # rank: the same workloads unsharded), each with a parity flag from a small case.
    config3 = config4 = None
    if not args.no_sharded and not args.seq_len:
        d.clear()                  # the config-1 tensors (2.4 GB) are no longer needed
        y = h = graph = None
        torch.cuda.empty_cache()
        k3 = max(3, min(args.steps, 10))
        config3 = measure_seq(args, rank, world, dev, dist, k3, 3)
        torch.cuda.empty_cache()
        config4 = measure_heads(args, rank, world, dev, dist, k3, 3) if 64 % world == 0 else None
        torch.cuda.empty_cache()

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        alg = algorithmic_bytes(BH, L, R, M)
        achieved = alg / (scan_ms * 1e-3) / 1e9
        # DRAM bytes per launch come from the committed ncu summary of the kernel (a small case,
        # scaled by head-tokens: traffic grows in proportion to the tiles processed); null when that
        # summary was taken from another build of the kernel than the one loaded here.
        traffic = profiled_traffic(BH * L) if use_fused else None
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                    "frac": achieved / peak, "traffic": traffic, "peak_kind": f"of {peak_kind}",
                    "kernel": "scan_fused_kernel" if use_fused else
                              "staged scan (chunk_cumsum + chunk_state + state_passing + chunk_readout<fused>)",
                    "kernel_ms": scan_ms, "kernel_ms_median": scan_ms_median,
                    "kernel_ms_timing": ("K replays of a scan-only CUDA graph between two events"
                                         if scan_ms_graph is not None else "mean of per-step event pairs"),
                    "kernel_ms_plain_mean": statistics.mean(scan_times), "algorithmic_bytes": alg}
        cpu = None
        if not args.no_cpu_baseline:
            slabs = 32
            cpu_threads = host_threads()
            v, secs = cpu_baseline_sample(slabs)
            cpu = {"value": v, "unit": "tokens/s", "cores": cpu_threads, "kind": "port",
                   "sample": f"{slabs} of {BH} (batch, head) rows of the workload, one row per call (slab = 1), "
                             f"{secs:.1f} s, working precision, {cpu_threads} torch threads on "
                             f"{os.cpu_count()} logical cpus"}
        line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(world),
                "tokens_per_s_per_gpu": value / world, "roofline": roofline, "cpu_baseline": cpu,
                "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
                "config3": config3, "config4": config4,
                "scan_path": "fused" if use_fused else "staged",
                "timed_launch": timed_launch,
                "ms_per_step_plain_launches": ms_plain}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
