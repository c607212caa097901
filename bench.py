"""
Benchmark of the SVDQuant W4A4 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the path over one batch of synthetic input: activation quantizer with fused
LoRA-down, then the fused QKV projection (W4A4 GEMM + rank-32 branch + bias + per-head RMSNorm + RoPE) at
M=4608 tokens, K=3072, N=9216 -- the FLUX.1 joint-attention QKV shape.  The metric is the GEMM's
integer throughput, 2*M*N*K operations per step divided by the step time, summed over GPUs (each rank
runs an independent replica on its own batch: weak scaling, no collective in the data path).

Rank 0 prints ONE JSON line.  ``value`` is measured with inputs resident in HBM; ``e2e`` is the same
metric through the public operator API starting from pinned host memory and ending with the result back
on the host.  ``roofline`` describes the GEMM kernel alone (CUDA events around each launch inside the
timed region); ``cpu_baseline`` is the CPU restatement of the reference's PyTorch path timed on the
host cores on a bounded sample of the same workload.  ``--impl reference`` times only that CPU path.

The same line carries ``flux``: the FLUX.1-schnell-architecture transformer (19 double + 38 single blocks, 57 distinct
random-init int4 weight sets, 4096 image + 512 text tokens) run for 4 denoising steps per image from a CUDA graph, as
images per second over all ranks, with an end-to-end figure whose timed region copies the latents from and to pinned host
memory every image.  ``--no-flux`` skips it.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M_TOK, K_IN, N_OUT, RANK = 4608, 3072, 9216, 32
TXT, GRID = 512, 64
N_SETS = 4  # rotating buffer sets: 4 x ~106 MB > 126 MB of L2


def make_cfg_inputs(M: int, K: int, N: int, R: int, device, seed: int = 0) -> dict:
    """
    Seeded synthetic tensors with the shapes and value distributions of the benchmark configuration:
    int4 weights uniform in [-8, 7] with per-64 bf16 scales U(0.005, 0.02); activations N(0, 1) with 8 outlier
    channels x20; rank-R branch N(0, 0.02); bf16 bias; smooth U(0.5, 1.5); RMSNorm weights 1 + N(0, 0.05);
    FLUX rotary table for 512 text rows + a 64 x 64 grid (when M matches).
    """
    from nunchaku_rocm_b200.models.embeddings import flux_image_ids, flux_pos_embed

    g = torch.Generator(device=device).manual_seed(seed)
    T = torch.bfloat16

    def rnd(*s):
        return torch.rand(*s, generator=g, device=device)

    def nrm(*s):
        return torch.randn(*s, generator=g, device=device)

    x = nrm(M, K)
    outliers = torch.randperm(K, generator=g, device=device)[:8]
    x[:, outliers] *= 20
    p = {
        "x": x.to(T),
        "qweight": torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g, device=device),
        "wscales": (rnd(K // 64, N) * 0.015 + 0.005).to(T),
        "bias": (nrm(N) * 0.1).to(T),
        "proj_down": (nrm(K, R) * 0.02).to(T),
        "proj_up": (nrm(N, R) * 0.02).to(T),
        "smooth": (rnd(K) + 0.5).to(T),
        "norm_q": (1 + nrm(128) * 0.05).to(T),
        "norm_k": (1 + nrm(128) * 0.05).to(T),
    }
    if M == TXT + GRID * GRID:
        p["rotary_emb"] = flux_pos_embed(flux_image_ids(TXT, GRID, GRID, device=device))
    else:
        th = rnd(M, 64) * 6.28
        p["rotary_emb"] = torch.stack([torch.sin(th), torch.cos(th)], -1).reshape(M, 64, 1, 2).float().contiguous()
    return p


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_evt = threading.Event()

    def run(self):
        try:
            import pynvml as nv

            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {
                "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
                "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                "hw_power_brake": getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80),
            }
            while not self._stop_evt.is_set():
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
                time.sleep(0.002)
        except Exception as e:  # NVML missing: report that instead of clocks
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def stop(self) -> dict:
        self._stop_evt.set()
        self.join(timeout=2)
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def measured_peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return json.load(open(path)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# --------------------------------------------------------------------------------------------------
# CPU baseline: the oracle (a port of the reference's PyTorch path) on the host cores
# --------------------------------------------------------------------------------------------------
def load_reference_cpu():
    """
    The reference's own CPU-runnable form of the path: ``reference()`` / ``reference_qk()`` of
    nunchaku/ops/triton/native/w4a4.py (pure PyTorch), loaded by file path from the unmodified copy under
    ``baseline/_ref`` the way the reference's tests load it (tests/triton/conftest.py:22-35).  ``None`` when that copy
    is not there; the CPU arm then runs the oracle's restatement of the same functions.
    """
    import importlib.util

    d = os.path.join(ROOT, "baseline", "_ref", "nunchaku", "ops", "triton", "native")
    if not os.path.exists(os.path.join(d, "w4a4.py")):
        return None
    try:
        pkg = "_nunchaku_native_ref"
        if pkg not in sys.modules:
            m = importlib.util.module_from_spec(importlib.util.spec_from_loader(pkg, loader=None, is_package=True))
            m.__path__ = [d]
            sys.modules[pkg] = m
        for name in ("build", "w4a4"):
            full = f"{pkg}.{name}"
            if full not in sys.modules:
                spec = importlib.util.spec_from_file_location(full, os.path.join(d, f"{name}.py"))
                mod = importlib.util.module_from_spec(spec)
                sys.modules[full] = mod
                spec.loader.exec_module(mod)
        return sys.modules[f"{pkg}.w4a4"]
    except Exception:
        return None


def cpu_step(p_cpu: dict, rows: int, ref=None) -> None:
    from oracle import w4a4

    x = p_cpu["x"][:rows]
    # the reference has the quantizer only as a Triton kernel: the restatement does it on the CPU in both arms
    q, s, l, _ = w4a4.quantize_act(x, p_cpu["proj_down"], p_cpu["smooth"])
    rot = p_cpu["rotary_emb"][:rows].reshape(rows, 128)
    if ref is not None:
        lin = ref.reference(q, p_cpu["qweight"], s, p_cpu["wscales"], p_cpu["bias"], l, p_cpu["proj_up"], False)
        out = ref.reference_qk(lin, p_cpu["norm_q"], p_cpu["norm_k"], rot)
    else:
        lin = w4a4.gemm_w4a4(q, p_cpu["qweight"], s, p_cpu["wscales"], p_cpu["bias"], l, p_cpu["proj_up"])
        out = w4a4.qk_norm_rope(lin, p_cpu["norm_q"], p_cpu["norm_k"], rot)
    out.to(torch.bfloat16)


def cpu_baseline(budget_s: float, steps: int, warmup: int) -> dict:
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ref = load_reference_cpu()
    p = {k: v for k, v in make_cfg_inputs(M_TOK, K_IN, N_OUT, RANK, "cpu").items()}
    # calibrate on 64 rows, then size the sample so that warmup + steps fit the budget
    t0 = time.perf_counter()
    cpu_step(p, 64, ref)
    t64 = time.perf_counter() - t0
    rows = int(64 * budget_s / max(t64 * (steps + warmup), 1e-9))
    rows = max(8, min(M_TOK, rows // 8 * 8))
    for _ in range(warmup):
        cpu_step(p, rows, ref)
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_step(p, rows, ref)
        ts.append(time.perf_counter() - t0)
    t = statistics.median(ts)
    return {
        "value": 2.0 * rows * N_OUT * K_IN / t / 1e12,
        "unit": "TOPS",
        "cores": cores,
        "kind": "reference" if ref is not None else "port",
        "sample": f"first {rows} of {M_TOK} rows of the same workload, {steps} steps, median; "
        + ("GEMM + RMSNorm/RoPE by the reference's own reference() / reference_qk() (PyTorch, all host threads), "
           "quantizer by the CPU restatement (the reference has it as a Triton kernel only)" if ref is not None
           else "CPU restatement of the reference's PyTorch path"),
        "ms_per_step": t * 1e3,
        "rows": rows,
    }


def config_dict(n_gpus: int) -> dict:
    return {
        "workload": "fused_qkv_w4a4: quantize(4608x3072, rank-32 LoRA-down) + W4A4 GEMM 4608x9216x3072 "
        "(group 64, rank 32, bias) + per-head RMSNorm + RoPE (24 heads x 128, 512 text + 64x64 image tokens)",
        "M": M_TOK,
        "K": K_IN,
        "N": N_OUT,
        "rank": RANK,
        "parallelism": f"dp{n_gpus} (independent replica per GPU, no collective)",
        "l2": f"{N_SETS} rotating buffer sets (~{N_SETS * 106} MB > 126 MB L2)",
        "weights": "int4 weights widened to the kernel's operand form once per weight tensor (load-time step), activations every step",
    }


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cb = cpu_baseline(budget_s=90.0, steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference",
        "metric": "w4a4_gemm_tops",
        "value": cb["value"],
        "unit": "TOPS",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": cb["ms_per_step"],
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "int4xint4->int32, fp32 scaling",
        "data": "synthetic",
        "config": config_dict(args.gpus),
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def max_over_ranks(ms: float, device) -> float:
    """The slowest rank's time: every multi-GPU number is the maximum over ranks (no-op for one process)."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(ms)
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def whole_job_tops(world: int, ops_per_rank: float, ms_step: float) -> float:
    """Weak scaling: every rank runs the full workload on its own replica; the job's throughput is their sum."""
    return world * ops_per_rank / (ms_step * 1e-3) / 1e12


def bind_to_gpu_cpus(local: int) -> str:
    """
    Run this process on the host cores that sit next to its GPU (the PCI device's ``local_cpulist``), so that the pinned
    host buffers it allocates afterwards land on that NUMA node.  With one process per GPU and eight GPUs on two sockets,
    copies from the far socket's memory otherwise share the inter-socket link.  Changes only this process's affinity.
    """
    try:
        pr = torch.cuda.get_device_properties(local)
        path = f"/sys/bus/pci/devices/{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0/local_cpulist"
        cpus: set[int] = set()
        for part in open(path).read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)  # stay inside what the container allows
        if not cpus:
            return "unchanged (no local cpu allowed)"
        os.sched_setaffinity(0, cpus)
        return f"{len(cpus)} cpus local to the GPU"
    except (OSError, ValueError, AttributeError) as e:
        return f"unchanged ({type(e).__name__})"


def run_ours(args) -> None:
    import torch.distributed as dist

    from nunchaku_rocm_b200.ops.quantize import svdq_quantize_w4a4_act_fuse_lora_cuda as quantize
    from nunchaku_rocm_b200.ops.triton.gemm_w4a4 import gemm_w4a4

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path for the product kernels)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    all_cpus = os.sched_getaffinity(0)
    affinity = bind_to_gpu_cpus(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    sets = []
    for i in range(N_SETS):
        p = make_cfg_inputs(M_TOK, K_IN, N_OUT, RANK, dev, seed=rank * 100 + i)
        p["out"] = torch.empty(M_TOK, N_OUT, dtype=torch.bfloat16, device=dev)
        m_pad = (M_TOK + 255) // 256 * 256
        p["q"] = torch.empty(m_pad, K_IN // 2, dtype=torch.uint8, device=dev)
        p["s"] = torch.empty(K_IN // 64, m_pad, dtype=torch.bfloat16, device=dev)
        p["l"] = torch.zeros(m_pad, RANK, dtype=torch.float32, device=dev)
        sets.append(p)

    def step(p, ev=None):
        quantize(p["x"], p["q"], p["s"], p["proj_down"], p["l"], p["smooth"])
        if ev is not None:
            ev[0].record()
        gemm_w4a4(p["q"], p["qweight"], p["out"], p["s"], p["wscales"], p["bias"], p["l"], p["proj_up"],
                  norm_q=p["norm_q"], norm_k=p["norm_k"], rotary_emb=p["rotary_emb"])
        if ev is not None:
            ev[1].record()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(sets[i % N_SETS])
    barrier()

    # ---- device-resident throughput ------------------------------------------------------------------
    # The K timed steps of the contract are repeated (each repeat bracketed by the barrier) until about a second of GPU
    # time has been measured, so that the clock sampler sees the load whatever --steps is; `ms_per_step` is the median
    # repeat, the best one is reported beside it.
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    sampler.start()
    rep_ms, gemm_samples, spent = [], [], 0.0
    while spent < 1000.0 and len(rep_ms) < 200:
        barrier()
        e0.record()
        for i in range(args.steps):
            step(sets[i % N_SETS], evs[i])
        e1.record()
        barrier()
        rep_ms.append(max_over_ranks(e0.elapsed_time(e1), dev))
        gemm_samples.append(statistics.mean(a.elapsed_time(b) for a, b in evs))
        spent += rep_ms[-1]
    clocks = sampler.stop()
    gemm_ms = statistics.median(gemm_samples)
    ms_step = statistics.median(rep_ms) / args.steps
    ms_step_best = min(rep_ms) / args.steps
    ops = 2.0 * M_TOK * N_OUT * K_IN

    # ---- end to end through the operator API, host buffers in and out --------------------------------
    # Every step copies its input from pinned host memory and its result back to pinned host memory.  The three phases
    # run on three streams (upload, compute, download) chained by events, so the copies of neighbouring steps overlap
    # the kernels as a serving loop would arrange it; all of it is inside the timed region.
    NB = 3  # steps in flight
    hx = [sets[i % N_SETS]["x"].cpu().pin_memory() for i in range(NB)]
    hout = [torch.empty(M_TOK, N_OUT, dtype=torch.bfloat16).pin_memory() for _ in range(NB)]
    dx = [torch.empty_like(sets[0]["x"]) for _ in range(NB)]
    dout = [torch.empty(M_TOK, N_OUT, dtype=torch.bfloat16, device=dev) for _ in range(NB)]
    main = torch.cuda.current_stream()
    s_up, s_down = torch.cuda.Stream(), torch.cuda.Stream()
    ev_up = [torch.cuda.Event() for _ in range(NB)]      # upload of slot b finished
    ev_done = [torch.cuda.Event() for _ in range(NB)]    # kernels of slot b finished
    ev_free = [torch.cuda.Event() for _ in range(NB)]    # download of slot b finished: its buffers are free again

    def e2e_step(i):
        b = i % NB
        p = sets[i % N_SETS]
        with torch.cuda.stream(s_up):
            s_up.wait_event(ev_done[b])   # the kernels that read dx[b] three steps ago
            dx[b].copy_(hx[b], non_blocking=True)
            ev_up[b].record(s_up)
        main.wait_event(ev_up[b])
        main.wait_event(ev_free[b])       # the download that read dout[b] three steps ago
        quantize(dx[b], p["q"], p["s"], p["proj_down"], p["l"], p["smooth"])
        gemm_w4a4(p["q"], p["qweight"], dout[b], p["s"], p["wscales"], p["bias"], p["l"], p["proj_up"],
                  norm_q=p["norm_q"], norm_k=p["norm_k"], rotary_emb=p["rotary_emb"])
        ev_done[b].record(main)
        with torch.cuda.stream(s_down):
            s_down.wait_event(ev_done[b])
            hout[b].copy_(dout[b], non_blocking=True)
            ev_free[b].record(s_down)

    def e2e_drain():
        main.wait_stream(s_up)
        main.wait_stream(s_down)

    e2e_steps = max(3, min(args.steps, 50))
    for i in range(NB):
        e2e_step(i)
    e2e_drain()
    barrier()
    e0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    e2e_drain()
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1), dev) / e2e_steps

    from nunchaku_rocm_b200 import _lib

    status = _lib.device_status(dev)
    if status:
        raise SystemExit(f"a kernel gave up on a bounded wait (status {status:#x}); numbers are void")
    del sets, dx, dout
    torch.cuda.empty_cache()
    flux = None if args.no_flux else run_flux(args, dev, world, barrier)
    qwen = None if args.no_qwen else run_qwen(args, dev, world, barrier)

    if rank == 0:
        peaks, src = measured_peaks()
        # the int8 tensor pipe runs at twice the bf16 rate; the measured bf16 burst figure x 2 is the denominator
        peak = 2.0 * float(peaks["bf16_tflops"])
        achieved = ops / (gemm_ms * 1e-3) / 1e12
        line = {
            "metric": "w4a4_gemm_tops",
            "value": whole_job_tops(world, ops, ms_step),
            "unit": "TOPS",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step,
            "ms_per_step_best": ms_step_best,
            "timed_repeats": len(rep_ms),
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "int4 x int4 -> exact integer sums (tcgen05 kind::f8f6f4, e4m3 operands, fp32 accumulators), fp32 scaling, bf16 out",
            "data": "synthetic",
            "config": config_dict(world),
            "clocks": clocks,
            "e2e": {
                "value": whole_job_tops(world, ops, e2e_ms),
                "unit": "TOPS",
                "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": hx[0].numel() * hx[0].element_size(),
                "pipelining": "3 steps in flight on upload / compute / download streams",
                "host_affinity": affinity,
                "d2h_bytes_per_step": hout[0].numel() * hout[0].element_size(),
            },
            # kernels of this library launched in the timed region: per step the quantizer, the activation pre-pass and
            # the GEMM (counted from the calls made, three launches each: see `step`)
            "gpu_launches": 3 * args.steps * len(rep_ms),
            "roofline": {
                "kernel": "gemm_tc_pair_kernel<QK_NORM_ROPE, bf16> (+ its activation pre-pass prepack_pair_kernel, timed together)",
                "bound": "tensor",
                "achieved": achieved,
                "peak": peak,
                "unit": "TFLOP/s",
                "frac": achieved / peak,
                "traffic": profiled_traffic_bytes(),
                "peak_source": f"2 x bf16_tflops of MEASURED_PEAKS.json ({src}); int8 pipe = 2 x bf16 rate",
                "gemm_ms": gemm_ms,
                "algorithmic_ops_per_launch": ops,
            },
        }
        if flux is not None:
            line["flux"] = flux
        if qwen is not None:
            line["qwen_image"] = qwen
        if world == 1 and not args.no_cpu_baseline:
            os.sched_setaffinity(0, all_cpus)  # the CPU baseline may use every core again
            cb = cpu_baseline(budget_s=20.0, steps=3, warmup=1)
            line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def profiled_traffic_bytes():
    """
    DRAM bytes (read + write) of one launch of the GEMM kernel of this workload, from the one profiler capture whose
    figures are kept beside its summary (``profiles/gemm_traffic.json``: kernel name and bytes).  ``None`` when the file
    is missing or names another kernel than the one the library now runs.
    """
    try:
        rec = json.load(open(os.path.join(ROOT, "profiles", "gemm_traffic.json")))
        return float(rec["dram_bytes_per_launch"]) if rec.get("kernel") == "gemm_tc_pair_kernel" else None
    except (OSError, ValueError, KeyError):
        return None


# --------------------------------------------------------------------------------------------------
# FLUX.1-schnell-architecture transformer: images per second
# --------------------------------------------------------------------------------------------------
def run_flux(args, dev, world: int, barrier) -> dict:
    """
    19 double + 38 single blocks with 57 distinct random-init int4 weight sets, 1024 x 1024 latents (4096 image tokens
    of 64 channels) + 512 text tokens, 4 Euler steps per image, one transformer forward per CUDA-graph replay
    (the reference times the transformer forward the same way in its "step" mode, app/flux.1/t2i/latency.py:71-92).
    Text encoders, VAE and scheduler are outside the path.  `images_per_s` sums the ranks (each rank denoises its own
    batch; the slowest rank's time is used); `e2e` includes the upload of the noise latents from pinned host memory and
    the download of the denoised latents every image batch.
    """
    from nunchaku_rocm_b200.models.flux_dit import FluxDiT, FluxDiTConfig, GraphedStep, denoise

    torch.manual_seed(0)
    cfg = FluxDiTConfig()
    with torch.no_grad():
        model = FluxDiT(cfg, device=dev).random_init(seed=int(os.environ.get("RANK", "0")))
    steps_per_image = 4
    out = {
        "model": "FLUX.1-schnell architecture: 19 double + 38 single blocks, hidden 3072, 24 x 128 heads, MLP x4, rank 32, "
                 "57 distinct random-init int4 weight sets",
        "tokens": "4096 image (1024 x 1024 latents, 64 channels packed) + 512 text",
        "steps_per_image": steps_per_image,
        "weights_gb": round(model.quantized_bytes() / 2**30, 2),
        "excluded": "text encoders, VAE, scheduler arithmetic beyond the Euler update",
        "batches": {},
    }
    for batch in [int(b) for b in args.flux_batches.split(",")]:
        with torch.no_grad():
            step = GraphedStep(model, batch=batch, txt_tokens=TXT, grid=GRID, seed=batch)
            noise = torch.randn(batch, GRID * GRID, cfg.in_channels).to(cfg.dtype).pin_memory()
            result = torch.empty_like(noise).pin_memory()
            x0 = noise.to(dev)
            for _ in range(2):
                denoise(step, x0, steps_per_image)
            n_img = max(2, min(args.flux_images, 8))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            # device-resident: latents stay on the GPU
            barrier()
            e0.record()
            for _ in range(n_img):
                x = denoise(step, x0, steps_per_image)
            e1.record()
            barrier()
            ms_dev = max_over_ranks(e0.elapsed_time(e1), dev) / n_img
            # end to end: noise from pinned host memory, denoised latents back to pinned host memory, every image batch
            barrier()
            e0.record()
            for _ in range(n_img):
                x = denoise(step, noise.to(dev, non_blocking=True), steps_per_image)
                result.copy_(x, non_blocking=True)
            e1.record()
            barrier()
            ms_e2e = max_over_ranks(e0.elapsed_time(e1), dev) / n_img
            assert torch.isfinite(result.float()).all(), "the denoised latents are not finite"
        out["batches"][str(batch)] = {
            "ms_per_transformer_step": ms_dev / steps_per_image,
            "images_per_s": world * batch / (ms_dev * 1e-3),
            "e2e_images_per_s": world * batch / (ms_e2e * 1e-3),
            "h2d_bytes_per_image_batch": noise.numel() * noise.element_size(),
            "d2h_bytes_per_image_batch": result.numel() * result.element_size(),
        }
        del step
        torch.cuda.empty_cache()
    del model
    torch.cuda.empty_cache()
    best = max(out["batches"].values(), key=lambda r: r["images_per_s"])
    out["images_per_s"] = best["images_per_s"]
    out["e2e_images_per_s"] = best["e2e_images_per_s"]
    out["n_gpus"] = world
    return out


def flux_profile_step() -> None:
    """One eager forward of the FLUX-architecture transformer (batch 1) inside a cudaProfilerStart/Stop range."""
    from nunchaku_rocm_b200.models.flux_dit import FluxDiT, FluxDiTConfig, GraphedStep

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    with torch.no_grad():
        model = FluxDiT(FluxDiTConfig(), device=dev).random_init(seed=0)
        step = GraphedStep(model, batch=1, txt_tokens=TXT, grid=GRID, seed=1)  # (runs the forward eagerly twice first)
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.cudart().cudaProfilerStart()
        e0.record()
        out = step._forward()
        e1.record()
        torch.cuda.synchronize(dev)
        torch.cuda.cudart().cudaProfilerStop()
    print(json.dumps({"flux_profile_step": {"eager_forward_ms": e0.elapsed_time(e1), "finite": bool(torch.isfinite(out.float()).all())}}),
          flush=True)


def qwen_profile_step() -> None:
    """One eager forward of the Qwen-Image-architecture transformer (batch 1) inside a cudaProfilerStart/Stop range."""
    from nunchaku_rocm_b200.models.qwen_dit import GraphedQwenStep, QwenDiT, QwenDiTConfig

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    with torch.no_grad():
        model = QwenDiT(QwenDiTConfig(), device=dev).random_init(seed=100)
        step = GraphedQwenStep(model, batch=1)  # (runs the forward eagerly twice first)
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.cudart().cudaProfilerStart()
        e0.record()
        out = step._forward()
        e1.record()
        torch.cuda.synchronize(dev)
        torch.cuda.cudart().cudaProfilerStop()
    print(json.dumps({"qwen_profile_step": {"eager_forward_ms": e0.elapsed_time(e1), "finite": bool(torch.isfinite(out.float()).all())}}),
          flush=True)


def run_qwen(args, dev, world: int, barrier) -> dict:
    """
    Qwen-Image-architecture MMDiT with NVFP4 W4A4 layers: 60 blocks, hidden 3072, 24 x 128 heads, MLP 12288, 6889 image +
    256 text tokens (1328 x 1328 latents), batch 1 per GPU, one forward per CUDA-graph replay.  Reported per transformer
    forward (the configuration names no step count); `forwards_per_s` sums the ranks over the slowest rank's time.
    """
    from nunchaku_rocm_b200.models.qwen_dit import GraphedQwenStep, QwenDiT, QwenDiTConfig

    cfg = QwenDiTConfig()
    with torch.no_grad():
        model = QwenDiT(cfg, device=dev).random_init(seed=100 + int(os.environ.get("RANK", "0")))
        step = GraphedQwenStep(model, batch=1)
        n = 3
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        step.step()
        barrier()
        e0.record()
        for _ in range(n):
            out = step.step()
        e1.record()
        barrier()
        ms = max_over_ranks(e0.elapsed_time(e1), dev) / n
        assert torch.isfinite(out.float()).all(), "the Qwen-Image forward is not finite"
    tokens = 6889 + 256
    ops = 60 * (2.0 * tokens * 3072 * (3 * 3072 + 3072 + 8 * 3072)) + 60 * 4.0 * 24 * tokens * tokens * 128
    res = {
        "model": "Qwen-Image architecture: 60 MMDiT blocks, hidden 3072, 24 x 128 heads, MLP 12288, rank 32, NVFP4 (e2m1 codes, "
                 "e4m3 scale per 16, per-channel and per-tensor scales), distinct random-init weights",
        "tokens": "6889 image + 256 text",
        "weights_gb": round(model.quantized_bytes() / 2**30, 2),
        "ms_per_forward": ms,
        "forwards_per_s": world / (ms * 1e-3),
        "tops_per_gpu": ops / (ms * 1e-3) / 1e12,
        "n_gpus": world,
    }
    del step, model
    torch.cuda.empty_cache()
    return res


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-flux", action="store_true", help="skip the FLUX-architecture images/s measurement")
    ap.add_argument("--no-qwen", action="store_true", help="skip the Qwen-Image-architecture (NVFP4) forward measurement")
    ap.add_argument("--flux-batches", default="1,4", help="per-GPU image batches to measure")
    ap.add_argument("--flux-images", type=int, default=4, help="image batches per timed region")
    ap.add_argument("--qwen-profile-step", action="store_true",
                    help="the same for the Qwen-Image-architecture (NVFP4) transformer")
    ap.add_argument("--flux-profile-step", action="store_true",
                    help="run ONE eager FLUX-architecture transformer forward between cudaProfilerStart/Stop and exit "
                         "(for a profiler's launch list; prints the forward's wall time, which is not a bench value)")
    args = ap.parse_args()
    if args.qwen_profile_step:
        qwen_profile_step()
        return
    if args.flux_profile_step:
        flux_profile_step()
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
