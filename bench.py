#!/usr/bin/env python
"""Benchmark of the Connect6 policy/value CNN hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl engine|reference]

One "step" is one self-play inference step over one batch of synthetic boards: the bf16 CNN
forward, masked policy log-softmax, one categorical draw per board from the engine's Philox
stream, and the value head (connect6/train.py:792-795 in the reference).  Per GPU the batch is
8192 boards; with N GPUs every rank owns its own 8192 boards of the global index range (weak
scaling), weights are replicated and the only collective is the sum of a 9 x int64 statistics
vector per step.  Rank 0 prints ONE JSON line.

`--impl reference` times the CPU restatement of the reference's own PyTorch path (oracle/
torch_port.py: the same torch CPU operators the reference calls) on the host cores, one bounded
sample of the workload per step.
"""
from __future__ import annotations

import argparse
import datetime as dt
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "board-evals/sec (CNN fwd, bf16, B=8192)"
UNIT = "boards/s"
BATCH = 8192
FLOP_PER_BOARD = 269_692_992            # dense conv count of the default v4 net incl. heads
CONV_LAYER_MACS = [18_333_024, 3_326_976, 6_653_952, 13_307_904, 13_307_904, 19_961_856, 29_942_784, 29_942_784]
HEAD_MACS = 69_312
INPUT_BUFFERS = 5                       # 5 x 35.5 MB of inputs rotate: larger than the 126 MB L2
# DRAM traffic of conv_tc_kernel per launch, from the ncu capture summarised under profiles/
# (dram__bytes_read.sum + dram__bytes_write.sum per layer at B = 2048, scaled by boards to 8192).
CONV_TRAFFIC_MB_B2048 = [59.4, 95.0, 154.8, 155.2, 202.4, 261.8, 166.6]   # backbone layers 1..7, one launch each
WEIGHT_SEED = 42
CPU_SAMPLE_BOARDS = 256


def load_peaks() -> tuple[dict, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return json.loads(p.read_text()), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# ------------------------------------------------------------------------------------------------
# clock sampling during the timed region
# ------------------------------------------------------------------------------------------------
# A child process polls NVML (read-only queries) every few milliseconds and writes one line per sample:
# unix time, SM MHz, max SM MHz, power in W, clock-event-reason bit mask.  nvidia-smi's own loop mode is
# the fallback when the NVML binding is missing; it is too slow to land inside a 35 ms region.
_NVML_POLLER = r"""
import sys, time
import pynvml as N
N.nvmlInit()
h = N.nvmlDeviceGetHandleByUUID(sys.argv[1]) if sys.argv[1].startswith("GPU-") else N.nvmlDeviceGetHandleByIndex(int(sys.argv[1]))
period = float(sys.argv[2])
mx = N.nvmlDeviceGetMaxClockInfo(h, N.NVML_CLOCK_SM)
out = sys.stdout
while True:
    t = time.time()
    try:
        reasons = N.nvmlDeviceGetCurrentClocksEventReasons(h)
    except Exception:
        reasons = N.nvmlDeviceGetCurrentClocksThrottleReasons(h)
    out.write("%.6f,%d,%d,%.1f,%d\n" % (t, N.nvmlDeviceGetClockInfo(h, N.NVML_CLOCK_SM), mx,
                                        N.nvmlDeviceGetPowerUsage(h) / 1000.0, reasons))
    out.flush()
    time.sleep(period)
"""
# NVML clock-event-reason bits (nvml.h): software power cap 0x4, hardware slowdown 0x8, software thermal
# slowdown 0x20, hardware thermal slowdown 0x40
_REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}
_SMI_FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
               "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
               "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def report_dir() -> Path:
    """Where side files of a run go (clock samples): $C6_REPORT_DIR, else the temp directory."""
    import tempfile
    d = Path(os.environ.get("C6_REPORT_DIR", tempfile.gettempdir()))
    d.mkdir(parents=True, exist_ok=True)
    return d


class ClockSampler:
    def __init__(self, gpu_index: int, period_s: float = 0.004):
        self.proc, self.kind = None, None
        self.path = report_dir() / f"c6_bench_clocks_gpu{gpu_index}.csv"
        who = str(gpu_index)
        try:   # NVML numbers devices by PCI order, CUDA may not: address the device by its UUID when torch knows it
            import torch
            who = "GPU-" + str(torch.cuda.get_device_properties(gpu_index).uuid)
        except Exception:
            pass
        try:
            self.fh = open(self.path, "w")
            try:
                import pynvml  # noqa: F401
                self.proc = subprocess.Popen([sys.executable, "-c", _NVML_POLLER, who, str(period_s)],
                                             stdout=self.fh, stderr=subprocess.DEVNULL)
                self.kind = "nvml"
            except ImportError:
                self.proc = subprocess.Popen(
                    ["nvidia-smi", f"--query-gpu={_SMI_FIELDS}", "--format=csv,noheader,nounits", "-lms", "10",
                     "-i", str(gpu_index)], stdout=self.fh, stderr=subprocess.DEVNULL)
                self.kind = "nvidia-smi"
            time.sleep(0.5)      # the child is polling before the warm-up ends
        except Exception:
            self.proc = None

    def _rows(self):
        for line in self.path.read_text().splitlines():
            parts = [s.strip() for s in line.split(",")]
            try:
                if self.kind == "nvml":
                    mask = int(parts[4])
                    yield (float(parts[0]), float(parts[1]), float(parts[2]), float(parts[3]),
                           [name for name, bit in _REASON_BITS.items() if mask & bit])
                else:
                    ts = dt.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
                    yield (ts, float(parts[2]), float(parts[3]), float(parts[4]),
                           [n for n, v in zip(names, parts[6:10]) if v.lower().startswith("active")])
            except Exception:
                continue

    def stop(self, t_begin: float, t_end: float) -> dict:
        """Summary of the samples taken between the two unix times; samples from outside the timed
        region are never substituted for missing ones."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock sampler unavailable"], "samples_in_timed_region": 0}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.fh.close()
        rows_all = list(self._rows())
        rows = [r for r in rows_all if t_begin <= r[0] <= t_end]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": rows_all[0][2] if rows_all else None, "reasons": [],
                    "samples_in_timed_region": 0, "sampler": self.kind,
                    "note": "no clock evidence: no sample fell inside the timed region"}
        reasons = sorted({name for r in rows for name in r[4]})
        return {"sm_mhz": statistics.median(r[1] for r in rows), "sm_min_mhz": min(r[1] for r in rows),
                "sm_max_mhz": rows[0][2], "power_w_max": max(r[3] for r in rows), "reasons": reasons,
                "samples_in_timed_region": len(rows), "sampler": self.kind}


def pick_tensor_peak(peaks: dict, peak_kind: str, clocks: dict | None, region_s: float) -> tuple[float, str]:
    """Denominator of a tensor-bound roofline fraction, chosen from what was sampled: the burst cuBLAS
    figure when the timed region ran at (nearly) the maximum SM clock or was too short for the power
    cap to bite (< 1 s), else the sustained one (a seconds-long cuBLAS loop under the same cap)."""
    burst = float(peaks["bf16_tflops"])
    sustained = float(peaks.get("bf16_tflops_sustained", burst))
    mhz, mx = (clocks or {}).get("sm_mhz"), (clocks or {}).get("sm_max_mhz")
    if region_s < 1.0:
        return burst, f"MEASURED_PEAKS.json bf16_tflops (burst: timed region {region_s:.2f} s < 1 s), of {peak_kind}"
    if mhz is not None and mx and mhz >= 0.95 * mx:
        return burst, f"MEASURED_PEAKS.json bf16_tflops (burst: median SM clock {mhz:.0f} of {mx:.0f} MHz), of {peak_kind}"
    why = f"median SM clock {mhz:.0f} of {mx:.0f} MHz" if mhz is not None and mx else "no clock sample, region >= 1 s"
    return sustained, f"MEASURED_PEAKS.json bf16_tflops_sustained ({why} over {region_s:.1f} s), of {peak_kind}"


# ------------------------------------------------------------------------------------------------
# CPU legs (the only places that touch oracle/)
# ------------------------------------------------------------------------------------------------
def _cpu_step_fn():
    """One bounded sample of the workload on the host: fp32 forward + masked categorical draw for
    CPU_SAMPLE_BOARDS boards, through the torch-CPU restatement of the reference."""
    import torch
    sys.path.insert(0, str(ROOT / "oracle"))
    import torch_port as TP
    from connect6_b200.boards import generate_planes
    from connect6_b200.model import PolicyValueNet
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    torch.manual_seed(WEIGHT_SEED)
    params = {k: v.detach() for k, v in PolicyValueNet(19).state_dict().items()}
    x = torch.from_numpy(generate_planes(0, CPU_SAMPLE_BOARDS))
    legal = ((x[:, 0] == 0) & (x[:, 1] == 0)).reshape(CPU_SAMPLE_BOARDS, -1)

    def step():
        logits, value = TP.policy_value_forward(x, params)
        logp = TP.masked_log_softmax(logits, legal, 1.0)
        actions = torch.multinomial(logp.exp(), 1)
        return actions, value

    return step, torch.get_num_threads()


def cpu_baseline(budget_s: float = 12.0) -> dict:
    step, threads = _cpu_step_fn()
    for _ in range(2):
        step()
    times = []
    t_all = time.perf_counter()
    while (time.perf_counter() - t_all < budget_s and len(times) < 40) or len(times) < 3:
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return {"value": CPU_SAMPLE_BOARDS / med, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{len(times)} x {CPU_SAMPLE_BOARDS} boards, fp32 torch-CPU restatement of the reference "
                      f"forward + masked categorical draw, median step {med * 1e3:.1f} ms"}


def library_gpu_bar(model, batches, steps: int = 10) -> dict:
    """The same self-play step through stock PyTorch/cuDNN on this GPU: the module stack of
    connect6/model.py:52-75 under bf16 autocast and inference_mode as in connect6/train.py:791-795,
    then the masked temperature-1 draw of connect6/train.py:195-205.  Reported beside the engine's
    number as the library bar on the same box; never part of the timed engine region."""
    import torch

    def lib_step(x, channels_last):
        if channels_last:
            x = x.contiguous(memory_format=torch.channels_last)
        with torch.inference_mode(), torch.autocast("cuda", dtype=torch.bfloat16):
            logits, value = model.forward_autograd(x)
        legal = ((x[:, 0] == 0) & (x[:, 1] == 0)).flatten(1)
        z = logits.float().masked_fill(~legal, torch.finfo(torch.float32).min)
        logp = torch.log_softmax(z, dim=-1)
        # rows with no legal cell would make multinomial raise; the synthetic boards have <= 200 stones
        action = torch.multinomial(logp.exp(), 1).squeeze(1)
        return action, logp.gather(1, action[:, None]).squeeze(1), value.float()

    out = {}
    for name, cl in (("nchw", False), ("channels_last", True)):
        if cl:
            model.to(memory_format=torch.channels_last)
        try:
            for i in range(3):
                lib_step(batches[i % len(batches)], cl)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(steps):
                lib_step(batches[i % len(batches)], cl)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / steps
            out[name] = {"value": batches[0].shape[0] / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms}
        except Exception as exc:  # noqa: BLE001 - a library failure must not take the engine's line down
            out[name] = {"error": f"{type(exc).__name__}: {exc}"[:200]}
        finally:
            if cl:
                model.to(memory_format=torch.contiguous_format)
    out["what"] = ("stock torch " + torch.__version__ + " / cuDNN modules, bf16 autocast, inference_mode, "
                   "mask + log_softmax + torch.multinomial; inputs resident on the device")
    out["steps"] = steps
    return out


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    step, threads = _cpu_step_fn()
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    el = time.perf_counter() - t0
    value = CPU_SAMPLE_BOARDS * args.steps / el
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": el / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "self-play inference step: default v4 CNN forward + masked log-softmax + 1 draw/board",
                   "sample_boards_per_step": CPU_SAMPLE_BOARDS, "note": "host CPU, all threads"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{args.steps} x {CPU_SAMPLE_BOARDS} boards per step"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# engine arm
# ------------------------------------------------------------------------------------------------
def run_engine(args) -> None:
    import torch
    import torch.distributed as dist
    from connect6_b200 import shard
    from connect6_b200.boards import generate_planes
    from connect6_b200.model import PolicyValueNet

    rank, world, local_rank = shard.init_from_env()
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    peaks, peak_kind = load_peaks()

    precision = args.precision
    torch.manual_seed(WEIGHT_SEED)
    model = PolicyValueNet(19, engine_precision=precision).to(dev).eval()
    eng = model.engine_for(dev)
    eng.reserve(BATCH)

    # this rank's boards: global indices [rank*BATCH*INPUT_BUFFERS, ...), INPUT_BUFFERS batches
    first = rank * BATCH * INPUT_BUFFERS
    host_batches = [torch.from_numpy(generate_planes(first + i * BATCH, BATCH)).pin_memory()
                    for i in range(INPUT_BUFFERS)]
    dev_batches = [h.to(dev) for h in host_batches]
    reducer = shard.RolloutStatsReducer(dev)

    def step(i: int):
        x = dev_batches[i % INPUT_BUFFERS]
        action, logprob, value, _ = eng.forward_step(x, temperature=1.0, seed=0xC6, offset=i,
                                                     board_index0=first + (i % INPUT_BUFFERS) * BATCH)
        # stand-in for the collector's per-step statistics vector: summed over the ranks every step, on NCCL's
        # own stream, off the compute stream's critical path
        reducer.buffer()[0] = BATCH
        reducer.submit()
        return action, logprob, value

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize(dev)
    shard.barrier()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = eng.launch_count
    eng.profile_read()
    # Per-kernel CUDA events are recorded on one step in `profile_every` of the timed region: an
    # event pair around each of the ten launches of a step costs about 3 % of the step, so sampling
    # keeps the kernel breakdown live without taxing the number it explains.
    every = max(1, args.profile_every)
    sampled_steps = 0
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    shard.barrier()
    t_begin = time.time()
    ev0.record()
    for i in range(args.steps):
        sample = i % every == 0
        eng.profile(sample)
        sampled_steps += sample
        step(args.warmup + i)
    total_stats = reducer.drain()           # the last step's reduction is inside the timed region
    ev1.record()
    torch.cuda.synchronize(dev)
    t_end = time.time()
    shard.barrier()
    if int(total_stats[0]) != BATCH * world:
        raise SystemExit(f"statistics all-reduce returned {int(total_stats[0])}, expected {BATCH * world}")
    elapsed_ms = ev0.elapsed_time(ev1)
    prof = eng.profile_read()
    eng.profile(False)
    launches = eng.launch_count - launches0
    clocks = sampler.stop(t_begin, t_end) if sampler else None
    elapsed_ms = shard.max_over_ranks(elapsed_ms, dev)
    status = eng.status()

    # ---- end to end: host buffers in, host results out, through the public host-buffer API ---------
    # HostStepPipeline uploads step i+1's planes on a side stream while step i computes; every step
    # still does its own pinned-host -> device upload and its own device -> pinned-host download.
    from connect6_b200.hostpipe import HostStepPipeline
    pipe = HostStepPipeline(model, BATCH, dev)

    def e2e_run(n_steps: int, start: int) -> None:
        pipe.submit(host_batches[start % INPUT_BUFFERS])
        for i in range(start, start + n_steps):
            if i + 1 < start + n_steps:
                pipe.submit(host_batches[(i + 1) % INPUT_BUFFERS])
            pipe.step(temperature=1.0, seed=0xC6, offset=i, board_index0=first + (i % INPUT_BUFFERS) * BATCH)

    e2e_steps = max(3, min(args.steps, 100))
    e2e_run(3, 0)
    torch.cuda.synchronize(dev)
    shard.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_run(e2e_steps, 3)
    e1.record()
    torch.cuda.synchronize(dev)
    e2e_ms = shard.max_over_ranks(e0.elapsed_time(e1), dev)
    # the same step fed with the environment's raw int8 state (363 B/board instead of 4332 B)
    hb = host_batches[0]
    boards_h = (hb[:, 0] - hb[:, 1]).to(torch.int8).pin_memory()
    player_h = torch.ones(BATCH, dtype=torch.int8).pin_memory()
    stones_h = torch.where(hb[:, 2, 0, 0] > 0, 1, 2).to(torch.int8).pin_memory()
    boards_d, player_d, stones_d = (torch.empty_like(t, device=dev) for t in (boards_h, player_h, stones_h))

    def e2e_boards_step(i: int):
        boards_d.copy_(boards_h, non_blocking=True)
        player_d.copy_(player_h, non_blocking=True)
        stones_d.copy_(stones_h, non_blocking=True)
        a, lp, v, _ = model.selfplay_step_from_boards(boards_d, player_d, stones_d, temperature=1.0, seed=0xC6, offset=i,
                                                      board_index0=first)
        pipe.actions.copy_(a, non_blocking=True)
        pipe.logprob.copy_(lp, non_blocking=True)
        pipe.value.copy_(v, non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()

    for i in range(3):
        e2e_boards_step(i)
    b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    b0.record()
    for i in range(e2e_steps):
        e2e_boards_step(i)
    b1.record()
    torch.cuda.synchronize(dev)
    e2e_boards_ms = shard.max_over_ranks(b0.elapsed_time(b1), dev)
    h2d = host_batches[0].numel() * 4
    d2h = BATCH * (8 + 4 + 4)

    if rank != 0:
        if dist.is_initialized():
            dist.destroy_process_group()
        return

    total_boards = BATCH * world * args.steps
    value = total_boards / (elapsed_ms * 1e-3)
    ms_per_step = elapsed_ms / args.steps
    # dominant kernel: the backbone layers after the stem (7 launches per step): conv_tc_kernel on the
    # tensor cores, conv_fp32_kernel on the CUDA cores in fp32 mode
    # Layers l and l + 1 that run as one launch of conv2_fused_kernel are recorded as "conv<l>" with no "conv<l+1>"
    # entry.  The roofline covers the conv_tc_kernel launches that follow the fused pairs (layers 5-7 of the default
    # network); the fused launches are reported under "kernels".
    fused_first = [l for l in (1, 3, 5) if precision != "fp32" and f"conv{l}" in prof and f"conv{l + 1}" not in prof]
    first_tc = max(fused_first) + 2 if fused_first else 1
    tc_keys = [k for k in prof if k.startswith("conv") and int(k[4:]) >= first_tc]
    conv_ms = sum(prof[k][0] for k in tc_keys)
    conv_launches = sum(prof[k][1] for k in tc_keys)
    conv_flop_per_step = 2 * (sum(CONV_LAYER_MACS[first_tc:]) + (HEAD_MACS if precision != "fp32" else 0)) * BATCH
    conv_traffic = int(sum(CONV_TRAFFIC_MB_B2048[first_tc - 1:]) / (8 - first_tc) * 1e6 * BATCH / 2048)
    burst = float(peaks["bf16_tflops"])
    if precision == "fp32":
        # no measured fp32 figure exists for this pool: nominal FMA rate, 148 SMs x 128 lanes x 2 x max SM clock
        peak = 148 * 128 * 2 * float(peaks.get("sm_max_mhz", 1965.0)) * 1e6 / 1e12
        peak_source = "nominal fp32 FMA rate (148 SMs x 128 lanes x 2 x max SM clock): no measured fp32 peak on this pool"
    else:
        peak, peak_source = pick_tensor_peak(peaks, peak_kind, clocks, elapsed_ms * 1e-3)
    roof = None
    if conv_launches:
        avg_ms = conv_ms / conv_launches
        flop_per_launch = conv_flop_per_step * sampled_steps / conv_launches
        achieved = flop_per_launch / (avg_ms * 1e-3) / 1e12
        roof = {"bound": "tensor" if precision != "fp32" else "fp32 FMA (CUDA cores)",
                "kernel": (f"conv_tc_kernel (backbone layers {first_tc}-7 + fused heads)" if precision != "fp32"
                           else "conv_fp32_kernel (backbone layers 1-7)"),
                "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "peak_source": peak_source,
                "traffic": conv_traffic if precision != "fp32" else None,
                "launches": conv_launches, "avg_launch_ms": avg_ms,
                "timed_with": f"CUDA events around every launch of {sampled_steps} of the {args.steps} timed steps",
                "flop_per_launch": flop_per_launch}
        if precision != "fp32":
            roof.update({"burst_peak": burst, "frac_of_burst": achieved / burst,
                         "sustained_peak": float(peaks.get("bf16_tflops_sustained", burst)),
                         "frac_of_sustained": achieved / float(peaks.get("bf16_tflops_sustained", burst))})
    kernels = {}
    for k, (ms, n) in sorted(prof.items()):
        entry = {"ms_per_step": ms / sampled_steps, "launches_per_step": n / sampled_steps}
        if k == "stem":
            entry["tflops_nominal"] = 2 * CONV_LAYER_MACS[0] * BATCH / (ms / sampled_steps * 1e-3) / 1e12
        elif k.startswith("conv"):
            li = int(k[4:])
            macs = CONV_LAYER_MACS[li] + (HEAD_MACS if li == 7 else 0)
            if li in fused_first:
                macs += CONV_LAYER_MACS[li + 1]
                entry["kernel"] = f"conv2_fused_kernel (layers {li} + {li + 1}, intermediate in shared memory)"
            entry["tflops_nominal"] = 2 * macs * BATCH / (ms / sampled_steps * 1e-3) / 1e12
        kernels[k] = entry
    whole_tflops = value / world * FLOP_PER_BOARD / 1e12

    line = {
        "metric": METRIC if precision == "bf16" else METRIC.replace("bf16", precision), "value": value, "unit": UNIT,
        "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": {"bf16": "bf16", "f16": "f16", "fp32": "f32"}[precision], "data": "synthetic",
        "config": {"workload": "self-play inference step: default v4 CNN (kernels [23,3x7], channels "
                               f"[32,32,64,64,64,96,96,96]) {precision} forward + masked log-softmax + 1 Philox draw/board "
                               "+ value",
                   "global_batch": BATCH * world, "per_gpu_batch": BATCH, "parallelism": f"boards sharded x{world}",
                   "l2": f"inputs rotate over {INPUT_BUFFERS} resident batches ({INPUT_BUFFERS * h2d / 1e6:.0f} MB "
                         "> 126 MB L2); inter-layer activations are 0.2-0.6 GB each",
                   "weights": f"PolicyValueNet default init, torch seed {WEIGHT_SEED}"},
        "clocks": clocks,
        "e2e": {"value": BATCH * world * e2e_steps / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                "api": "HostStepPipeline(PolicyValueNet.selfplay_step): pinned host fp32 planes in, pinned host results out, upload of step i+1 overlaps step i"},
        "e2e_int8_boards": {"value": BATCH * world * e2e_steps / (e2e_boards_ms * 1e-3), "unit": UNIT,
                            "h2d_bytes_per_step": int(boards_h.numel() + 2 * BATCH), "d2h_bytes_per_step": d2h,
                            "api": "PolicyValueNet.selfplay_step_from_boards: pinned host int8 boards + player + stones_left in, host results out"},
        "gpu_launches": launches,
        "roofline": roof,
        "whole_step": {"tflops_per_gpu": whole_tflops, "frac_of_peak": whole_tflops / peak, "frac_of_burst": whole_tflops / burst,
                       "flop_per_board": FLOP_PER_BOARD,
                       # runs at different clocks compare through time x clock: SM megacycles per step
                       "sm_mcycles_per_step": (ms_per_step * 1e-3 * clocks["sm_mhz"]) if clocks and clocks.get("sm_mhz") else None},
        "kernels": kernels,
        "device_status": status,
    }
    if world == 1 and not args.no_library_bar and precision != "fp32":
        line["library_gpu_bar"] = library_gpu_bar(model, dev_batches)
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline()
    print(json.dumps(line), flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# the other BASELINE configurations (parity-test cases; timed here for the record)
# ------------------------------------------------------------------------------------------------
WIDE_CHANNELS = (64, 64, 128, 128, 128, 192, 192, 192)
FLOP_PER_BOARD_WIDE = 1_005_162_624


def run_workload(args) -> None:
    """--workload cfg3 | cfg4 | cfg5: grouped ensemble 16 x 512, D4 inference on 65536 boards, the
    widened network on 32768 boards.  cfg4/cfg5 split their fixed board count over the ranks
    (strong scaling); cfg3 runs per rank (weak scaling)."""
    import torch
    import torch.distributed as dist
    from connect6_b200 import shard
    from connect6_b200.boards import generate_planes, shard_range
    from connect6_b200.engine import Engine
    from connect6_b200.model import DEFAULT_CHANNELS, DEFAULT_KERNELS, PolicyValueNet

    rank, world, local_rank = shard.init_from_env()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    peaks, peak_kind = load_peaks()
    wl = args.workload

    def state_for(seed, channels=None):
        torch.manual_seed(seed)
        return {k: v.detach() for k, v in PolicyValueNet(19, DEFAULT_KERNELS, channels).state_dict().items()}

    if wl == "cfg3":
        G, T = 16, 512
        eng = Engine(dev, 19, DEFAULT_KERNELS, DEFAULT_CHANNELS, G, "bf16")
        for g in range(G):
            eng.load_state_dict(state_for(1000 + g), group=g)
        x = torch.from_numpy(generate_planes(rank * G * T, G * T)).reshape(G, T, 3, 19, 19).to(dev)
        boards, flop, scaling = G * T, FLOP_PER_BOARD, "weak"
        step = lambda i: eng.forward_grouped(x, want_value=True)
        desc = "16 stacked default-architecture checkpoints x 512 boards, bf16, per-group logits and values"
    elif wl == "ensemble":
        # the ensemble shape the reference trains against (configs/train.yaml: 128 stacked opponents, 4 tables each)
        from pathlib import Path as _P
        from connect6_b200.history import HistoricalCheckpoint, HistoricalPolicyEnsemble
        G, T = 128, 4
        cfg = {"architecture_version": 4, "kernels": list(DEFAULT_KERNELS), "channels": list(DEFAULT_CHANNELS)}
        cps = [HistoricalCheckpoint(_P(f"model_update_{g + 1:08d}.pt"), g + 1, state_for(2000 + g), cfg,
                                    {"board_size": 19, "win_length": 6}) for g in range(G)]
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        ens = HistoricalPolicyEnsemble(cps, dev, dtype=torch.bfloat16)     # connect6/history.py:195-232: stack + cast + upload
        torch.cuda.synchronize(dev)
        build_s = time.perf_counter() - t0
        eng = ens._engine
        x = torch.from_numpy(generate_planes(rank * G * T, G * T)).reshape(G, T, 3, 19, 19).to(dev)
        boards, flop, scaling = G * T, FLOP_PER_BOARD, "weak"
        step = lambda i: ens.forward_grouped(x)
        desc = (f"128 stacked default-architecture checkpoints x 4 boards, bf16, policy logits; ensemble built from 128 "
                f"host state_dicts in {build_s:.3f} s, {eng.device_bytes / 1e6:.0f} MB on the device")
    elif wl == "cfg4":
        total = 65536
        lo, hi = shard_range(total, rank, world)
        eng = Engine(dev, 19, DEFAULT_KERNELS, DEFAULT_CHANNELS, 1, "bf16")
        eng.load_state_dict(state_for(WEIGHT_SEED))
        x = torch.from_numpy(generate_planes(lo, hi - lo)).to(dev)
        orient = torch.from_numpy(((torch.arange(lo, hi) % 8).numpy()).astype("uint8")).to(dev)
        boards, flop, scaling = hi - lo, FLOP_PER_BOARD, "strong"
        step = lambda i: eng.forward(x, orient, mask=True, inverse_map=True)
        desc = "65536 boards, orientation i mod 8 applied to the planes, bf16 CNN, masked logits mapped back to canonical indices"
    else:
        total = 32768
        lo, hi = shard_range(total, rank, world)
        eng = Engine(dev, 19, DEFAULT_KERNELS, WIDE_CHANNELS, 1, "bf16")
        eng.load_state_dict(state_for(WEIGHT_SEED, WIDE_CHANNELS))
        x = torch.from_numpy(generate_planes(lo, hi - lo, max_stones=200)).to(dev)
        boards, flop, scaling = hi - lo, FLOP_PER_BOARD_WIDE, "strong"
        step = lambda i: eng.forward_step(x, seed=0xC6, offset=i, board_index0=lo)
        desc = "channels [64,64,128,128,128,192,192,192], 32768 boards with up to 200 stones, bf16 self-play step"

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize(dev)
    shard.barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = eng.launch_count
    eng.profile(True)
    eng.profile_read()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = time.time()
    ev0.record()
    for i in range(args.steps):
        step(args.warmup + i)
    ev1.record()
    torch.cuda.synchronize(dev)
    t_end = time.time()
    shard.barrier()
    prof = eng.profile_read()
    ms = shard.max_over_ranks(ev0.elapsed_time(ev1), dev)
    clocks = sampler.stop(t_begin, t_end) if sampler else None
    status = eng.status()
    if rank == 0:
        total_boards = (boards * world if scaling == "weak" else (65536 if wl == "cfg4" else 32768)) * args.steps
        value = total_boards / (ms * 1e-3)
        burst = float(peaks["bf16_tflops"])
        peak, peak_source = pick_tensor_peak(peaks, peak_kind, clocks, ms * 1e-3)
        line = {"metric": METRIC.replace("B=8192", wl), "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": scaling,
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": {"workload": desc},
                "clocks": clocks, "gpu_launches": eng.launch_count - launches0,
                "whole_step": {"tflops_per_gpu": value / world * flop / 1e12, "frac_of_peak": value / world * flop / 1e12 / peak,
                               "frac_of_burst": value / world * flop / 1e12 / burst,
                               "flop_per_board": flop, "peak_source": peak_source},
                "kernels": {k: {"ms_per_step": v[0] / args.steps, "launches_per_step": v[1] / args.steps}
                            for k, v in sorted(prof.items())},
                "device_status": status}
        print(json.dumps(line), flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()


def run_backward(args) -> None:
    """--workload backward: the backward of one backbone layer (64 -> 96 channels, 3x3, the default net's layer 5)
    on 8192 boards through conv_layer_backward: dX, dW and db from x, W, b and dL/dy.  Also times PyTorch
    autograd (cuDNN, bf16 autocast) on the same layer and tensors as the library bar."""
    import torch
    from connect6_b200.train_ops import backward_status, conv_layer_backward
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, cin, cout, n = (args.boards or BATCH), 64, 96, 19
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.nn.functional.silu(torch.randn(B, cin, n, n, device=dev, generator=g))
    w = torch.randn(cout, cin, 3, 3, device=dev, generator=g) * (2.0 / (9 * cin)) ** 0.5
    b = 0.1 * torch.randn(cout, device=dev, generator=g)
    dy = torch.randn(B, cout, n, n, device=dev, generator=g) * 1e-3
    for _ in range(args.warmup):
        conv_layer_backward(x, w, b, dy)
    torch.cuda.synchronize(dev)
    sampler = ClockSampler(0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = time.time()
    e0.record()
    for _ in range(args.steps):
        dx, dw, db = conv_layer_backward(x, w, b, dy)
    e1.record()
    torch.cuda.synchronize(dev)
    t_end = time.time()
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop(t_begin, t_end)
    status = backward_status(x)
    # library bar: autograd through cuDNN under bf16 autocast, the reference's own way (connect6/train.py:1047-1119)
    xl = x.clone().requires_grad_(True)
    conv = torch.nn.Conv2d(cin, cout, 3, padding=1).to(dev)
    with torch.no_grad():
        conv.weight.copy_(w)
        conv.bias.copy_(b)

    def lib_step():
        conv.zero_grad(set_to_none=True)
        xl.grad = None
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = torch.nn.functional.silu(conv(xl))
        y.backward(dy.to(y.dtype))

    lib_ms = None
    try:
        if args.no_library_bar:
            raise RuntimeError("skipped (--no-library-bar)")
        for _ in range(3):
            lib_step()
        torch.cuda.synchronize(dev)
        l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0.record()
        for _ in range(10):
            lib_step()
        l1.record()
        torch.cuda.synchronize(dev)
        lib_ms = l0.elapsed_time(l1) / 10
    except Exception as exc:  # noqa: BLE001
        lib_ms = f"{type(exc).__name__}: {exc}"[:160]
    # per-kernel device times of three more calls (CUPTI through torch.profiler; outside the timed region)
    kernels = {}
    try:
        if args.no_library_bar:
            raise RuntimeError("skipped (--no-library-bar)")
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(3):
                conv_layer_backward(x, w, b, dy)
            torch.cuda.synchronize(dev)
        for ev in prof.key_averages():
            t_us = getattr(ev, "device_time_total", None) or getattr(ev, "cuda_time_total", 0.0)
            if t_us and ("c6::" in ev.key or "Memset" in ev.key or "Memcpy" in ev.key):
                kernels[ev.key[:70]] = {"ms_per_call": t_us / 3e3, "launches_per_call": ev.count / 3}
    except Exception as exc:  # noqa: BLE001
        kernels = {"error": f"{type(exc).__name__}: {exc}"[:160]}
    peaks, peak_kind = load_peaks()
    peak, peak_source = pick_tensor_peak(peaks, peak_kind, clocks, ms * args.steps * 1e-3)
    macs = 361 * 9 * cin * cout                     # per board and GEMM
    algorithmic = 2 * 2 * macs * B                  # data gradient + weight gradient
    executed = 2 * 3 * macs * B                     # + the forward recomputed for silu'
    achieved = algorithmic / (ms * 1e-3) / 1e12
    print(json.dumps({
        "metric": "backward of one 64->96 3x3 layer, boards/s (dX, dW, db; bf16 operands, fp32 accumulate)",
        "value": B / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": {"workload": f"conv_layer_backward, B = {B} boards, cin 64, cout 96, 19x19; fp32 NCHW "
                                                    "tensors in and out (packing and unpacking inside the timed call)"},
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "whole operator (2 conv_tc_kernel launches + wgrad_tc_kernel + packing)",
                     "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": peak_source,
                     "flop_algorithmic": algorithmic, "flop_executed": executed, "traffic": None},
        "kernels": kernels,
        "library_gpu_bar": {"ms_per_step": lib_ms, "what": "torch autograd of silu(conv2d) under bf16 autocast (cuDNN), forward + backward"},
        "device_status": status}), flush=True)


def run_train_step(args) -> None:
    """--workload train: forward + PPO loss + backward of the whole default network on `--boards` boards (default 8192;
    the reference's PPO minibatch is 256, configs/train.yaml:42) the way the reference's PPO update runs it
    (connect6/train.py:1047-1119: forward under bf16 autocast, the clipped-ratio / value / entropy loss,
    loss.backward()), with PolicyValueNet(engine_backward=True) and train_ops.ppo_loss: stem, 3x3 layers, heads and the
    loss run forward and backward on the library's kernels.  No gradient clipping, no optimizer step.  Library bar: the
    same step through the PyTorch modules, the reference's loss statements and autograd (cuDNN) on the same GPU."""
    import torch
    from connect6_b200.boards import generate_planes
    from connect6_b200.model import PolicyValueNet
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B = args.boards or BATCH
    torch.manual_seed(WEIGHT_SEED)
    ours = PolicyValueNet(19, engine_backward=True).to(dev).train()
    plain = PolicyValueNet(19).to(dev).train()
    plain.load_state_dict(ours.state_dict())
    x = torch.from_numpy(generate_planes(0, B)).to(dev)
    from torch.distributions import Categorical
    from connect6_b200.train_ops import ppo_loss
    gen = torch.Generator(device=dev).manual_seed(7)
    legal = (x[:, 0] + x[:, 1]).reshape(B, -1).eq(0)                 # empty cells (connect6/train.py:1046)
    actions = torch.multinomial(legal.float(), 1, generator=gen).squeeze(1)
    old_logprob = -torch.log(legal.sum(1).float()) + 0.2 * torch.randn(B, device=dev, generator=gen)
    advantages = torch.randn(B, device=dev, generator=gen)
    returns = torch.tanh(torch.randn(B, device=dev, generator=gen))
    clip_coef, value_coef, entropy_coef, temperature = 0.2, 0.5, 0.01, 1.0

    def step(m):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits, value = m(x)
            if m is ours:
                loss, _stats = ppo_loss(logits, value, legal, actions, old_logprob, advantages, returns, temperature, clip_coef,
                                        value_coef, entropy_coef)
            else:
                # the reference's statements (connect6/train.py:1049-1074) on PyTorch
                z = logits.masked_fill(~legal, torch.finfo(logits.dtype).min) / max(temperature, 1e-4)
                dist = Categorical(logits=z.float())
                logratio = dist.log_prob(actions) - old_logprob
                ratio = logratio.exp()
                pg = torch.maximum(-advantages * ratio, -advantages * torch.clamp(ratio, 1.0 - clip_coef, 1.0 + clip_coef)).mean()
                loss = pg + value_coef * 0.5 * (value.float() - returns).pow(2).mean() - entropy_coef * dist.entropy().mean()
        m.zero_grad(set_to_none=True)
        loss.backward()
        return loss

    loss = None
    for _ in range(max(args.warmup, 2)):
        loss = step(ours)     # kept while the next step runs, like in the timed loop: both workspaces of the pool get allocated here
    torch.cuda.synchronize(dev)
    sampler = ClockSampler(0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = time.time()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    e0.record()
    marks[0].record()
    for i in range(args.steps):
        loss = step(ours)
        marks[i + 1].record()
    e1.record()
    torch.cuda.synchronize(dev)
    t_end = time.time()
    ms = e0.elapsed_time(e1) / args.steps
    per_step = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(args.steps))
    clocks = sampler.stop(t_begin, t_end)
    lib_ms, lib_loss = None, None
    try:
        if args.no_library_bar:
            raise RuntimeError("skipped (--no-library-bar)")
        for _ in range(3):
            step(plain)
        torch.cuda.synchronize(dev)
        l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0.record()
        for _ in range(5):
            lib_loss = step(plain)
        l1.record()
        torch.cuda.synchronize(dev)
        lib_ms = l0.elapsed_time(l1) / 5
        lib_loss = float(lib_loss)
    except Exception as exc:  # noqa: BLE001
        lib_ms = f"{type(exc).__name__}: {exc}"[:160]
    # the whole minibatch update: + gradient clipping and AdamW (connect6/train.py:1121-1145), ClipAdamW against
    # clip_grad_norm_ + torch.optim.AdamW, hyper-parameters of configs/train.yaml
    update_ms = {}
    try:
        if args.no_library_bar:
            raise RuntimeError("skipped (--no-library-bar)")
        from connect6_b200.train_ops import ClipAdamW
        kw = dict(lr=2.5e-4, weight_decay=1e-4, eps=1e-5)
        opts = {"library": (ours, ClipAdamW(ours.parameters(), max_grad_norm=2.0, **kw)),
                "pytorch": (plain, torch.optim.AdamW(plain.parameters(), **kw))}
        for name, (m, opt) in opts.items():
            def update():
                step(m)
                if name == "pytorch":
                    torch.nn.utils.clip_grad_norm_(m.parameters(), 2.0)
                opt.step()
            for _ in range(3):
                update()
            torch.cuda.synchronize(dev)
            u0, u1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            u0.record()
            for _ in range(10):
                update()
            u1.record()
            torch.cuda.synchronize(dev)
            update_ms[name] = u0.elapsed_time(u1) / 10
    except Exception as exc:  # noqa: BLE001
        update_ms = {"error": f"{type(exc).__name__}: {exc}"[:160]}
    kernels = {}
    try:
        if args.no_library_bar:
            raise RuntimeError("skipped (--no-library-bar)")
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(3):
                step(ours)
            torch.cuda.synchronize(dev)
        other = 0.0
        for ev in prof.key_averages():
            t_us = getattr(ev, "device_time_total", None) or getattr(ev, "cuda_time_total", 0.0)
            if not t_us:
                continue
            if "c6::" in ev.key:
                kernels[ev.key[:70]] = {"ms_per_call": t_us / 3e3, "launches_per_call": ev.count / 3}
            else:
                other += t_us / 3e3
        kernels["(PyTorch kernels: casts, gradient copies)"] = {"ms_per_call": other}
    except Exception as exc:  # noqa: BLE001
        kernels = {"error": f"{type(exc).__name__}: {exc}"[:160]}
    peaks, peak_kind = load_peaks()
    peak, peak_source = pick_tensor_peak(peaks, peak_kind, clocks, ms * args.steps * 1e-3)
    macs = sum(CONV_LAYER_MACS) + HEAD_MACS         # per board, one pass
    algorithmic = 2 * (3 * macs - CONV_LAYER_MACS[0]) * B    # forward + data gradient (none for the stem) + weight gradient
    achieved = algorithmic / (ms * 1e-3) / 1e12
    print(json.dumps({
        "metric": "PPO minibatch forward + loss + backward of the default network, boards/s",
        "value": B / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "step_ms": {"min": per_step[0], "median": per_step[len(per_step) // 2], "max": per_step[-1]},
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"PolicyValueNet(engine_backward=True) + ppo_loss, B = {B} boards: stem + seven 3x3 layers + heads + PPO loss "
                               "forward and backward on the library's kernels (bf16 operands, fp32 accumulation), no optimizer step",
                   "loss": float(loss), "library_loss": lib_loss},
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "whole step (per 3x3 layer: 3 conv_tc_kernel launches + wgrad_tc_kernel; the stem 2 + 1)",
                     "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": peak_source,
                     "flop_algorithmic": algorithmic, "traffic": None},
        "kernels": kernels,
        "update_ms": {**update_ms, "what": "the step plus gradient clipping and AdamW: train_ops.ClipAdamW / clip_grad_norm_ + torch.optim.AdamW"},
        "library_gpu_bar": {"ms_per_step": lib_ms, "what": "the same step through the PyTorch modules, the reference's loss statements and autograd under bf16 autocast (cuDNN)"},
        "device_status": 0}), flush=True)


def run_small_case(args) -> None:
    """--workload small: a short, self-ending run for profilers -- `--steps` self-play inference steps of the
    default network on `--boards` generated boards (default 2048: the widest activations exceed L2 while
    the process holds well under 1 GB on the device), nothing else.  Prints one JSON line with a checksum,
    the device status word and the mean step time between CUDA events."""
    import torch
    from connect6_b200.boards import generate_planes
    from connect6_b200.model import PolicyValueNet
    dev = torch.device("cuda", 0)
    torch.manual_seed(WEIGHT_SEED)
    model = PolicyValueNet(19, engine_precision=args.precision).to(dev).eval()
    args.boards = args.boards or 2048
    x = torch.from_numpy(generate_planes(0, args.boards)).to(dev)
    for i in range(args.warmup):
        model.selfplay_step(x, seed=1, offset=i)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        actions, logprob, value, _ = model.selfplay_step(x, seed=1, offset=args.warmup + i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / max(1, args.steps)
    print(json.dumps({"workload": "small", "precision": args.precision, "boards": args.boards, "steps": args.steps,
                      "warmup": args.warmup, "ms_per_step": ms, "boards_per_s": args.boards / (ms * 1e-3),
                      "checksum": [int(actions.sum()), float(value.sum())],
                      "device_status": model.engine_for(dev).status()}), flush=True)


_LINE_DIRECTIONS = ((1, 0), (0, 1), (1, 1), (1, -1))


def stock_torch_env_step(state, actions, win_length: int = 6):
    """The environment step (connect6/vector_env.py:106-193) written with stock torch ops, for the
    library timing bar of --workload selfplay: zero-padded board, one gather of the 8 x (win-1)
    probe cells, cumulative product along each ray.  state = [boards, current_player, stones_left,
    empty_count, move_count], stepped in place.  tests/test_env_oracle.py checks it against games
    played by the reference."""
    import torch
    boards, current_player, stones_left, empty_count, move_count = state
    E, n, _ = boards.shape
    reach = win_length - 1
    pitch = n + 2 * reach
    dev = boards.device
    rays = torch.tensor([[sgn * s * (dr * pitch + dc) for s in range(1, reach + 1)]
                         for dr, dc in _LINE_DIRECTIONS for sgn in (1, -1)], dtype=torch.long, device=dev).reshape(8, reach)
    env_ids = torch.arange(E, device=dev)
    r, c = actions // n, actions % n
    actor = current_player.clone()
    boards[env_ids, r, c] = actor
    empty_count -= 1
    move_count += 1
    padded = torch.nn.functional.pad(boards, (reach, reach, reach, reach)).reshape(E, -1)
    probes = ((r + reach) * pitch + (c + reach)).view(E, 1, 1) + rays
    same = padded.gather(1, probes.reshape(E, -1)).reshape(E, 8, reach) == actor.view(E, 1, 1)
    runs = same.to(torch.int16).cumprod(-1).sum(-1)
    won = ((1 + runs[:, 0::2] + runs[:, 1::2]) >= win_length).any(1)
    done = won | (empty_count == 0)
    winner = torch.where(won, actor, torch.zeros_like(actor))
    remaining = stones_left - 1
    stay = ~done & (remaining > 0)
    switch = ~done & ~(remaining > 0)
    stones_left.copy_(torch.where(stay, remaining, torch.where(switch, torch.full_like(remaining, 2), stones_left)))
    current_player.copy_(torch.where(switch, -current_player, current_player))
    return won.to(torch.float32), done, winner, stay.to(torch.int8) - switch.to(torch.int8), move_count.clone()


def run_selfplay_loop(args) -> None:
    """--workload selfplay: the device-resident self-play loop around the network -- board-input
    inference step (D4 view p = step mod 8), environment step with the action mapped back from the
    view, finished-game bookkeeping -- on 8192 environments per rank, with no host synchronisation
    inside the loop.  Also times the environment part alone and the same integer work done with
    stock PyTorch ops on this GPU."""
    import torch
    import torch.distributed as dist
    from connect6_b200 import shard
    from connect6_b200.model import PolicyValueNet
    from connect6_b200.vector_env import RolloutBookkeeper, VectorConnect6

    rank, world, local_rank = shard.init_from_env()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    E = BATCH
    torch.manual_seed(WEIGHT_SEED)
    model = PolicyValueNet(19).to(dev).eval()
    eng = model.engine_for(dev)
    eng.reserve(E)
    env = VectorConnect6(E, 19, 6, device=dev)
    total_steps = args.warmup + args.steps
    book = RolloutBookkeeper(env, E + E * max(8, total_steps // 10))
    orients = [torch.full((E,), p, dtype=torch.uint8, device=dev) for p in range(8)]
    ev_env = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
              for _ in range(args.steps)]
    finished = torch.zeros((), dtype=torch.int64, device=dev)

    def loop_step(i: int, events=None):
        p = i % 8
        action, logprob, value, _ = model.selfplay_step_from_boards(
            env.boards, env.current_player, env.stones_left, temperature=1.0, seed=0xC6, offset=i,
            board_index0=rank * E, orient=orients[p])
        if events:
            events[0].record()
        step = env.step(action, view_phase=p)
        if events:
            events[1].record()
        book.current_segment_lengths += 1
        _, stats = book.collect(step)
        if events:
            events[2].record()
        finished.add_(stats[9])

    for i in range(args.warmup):
        loop_step(i)
    torch.cuda.synchronize(dev)
    shard.barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = eng.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = time.time()
    e0.record()
    for i in range(args.steps):
        loop_step(args.warmup + i, ev_env[i])
    e1.record()
    torch.cuda.synchronize(dev)
    t_end = time.time()
    shard.barrier()
    ms = shard.max_over_ranks(e0.elapsed_time(e1), dev)
    clocks = sampler.stop(t_begin, t_end) if sampler else None
    env_ms = sorted(a.elapsed_time(b) for a, b, _ in ev_env)
    col_ms = sorted(b.elapsed_time(c) for _, b, c in ev_env)
    faults = env.faults.tolist()
    n_finished = int(finished)

    # the same integer work with stock torch ops on this GPU (environment step + nonzero/reset)
    lib_ms = None
    if rank == 0:
        state = [env.boards.clone(), env.current_player.clone(), env.stones_left.clone(), env.empty_count.clone(),
                 env.move_count.clone()]
        gen = torch.Generator(device=dev).manual_seed(1)

        def lib_step():
            legal = (state[0].reshape(E, -1) == 0).float()
            legal[legal.sum(1) == 0] = 1.0
            a = torch.multinomial(legal, 1, generator=gen).squeeze(1)
            l0.record()
            out = stock_torch_env_step(state, a, 6)
            idx = torch.nonzero(out[1]).flatten()
            if idx.numel():
                state[0][idx] = 0; state[1][idx] = 1; state[2][idx] = 1; state[3][idx] = 361; state[4][idx] = 0
            l1.record()

        l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        times = []
        for i in range(25):
            lib_step()
            torch.cuda.synchronize(dev)
            if i >= 5:
                times.append(l0.elapsed_time(l1))
        lib_ms = sorted(times)[len(times) // 2]

    if rank == 0:
        value = E * world * args.steps / (ms * 1e-3)
        med = lambda v: v[len(v) // 2]
        # bytes one environment step must move per environment: the action (8), five state scalars
        # read and written (2 * 8), up to 4 * 10 probe cells in mostly distinct 32-byte sectors
        # (about 26 sectors for an interior stone: 1-2 for the row, 10 for the column, 2 x ~7 for the
        # diagonals ... counted as sectors because that is the DRAM granularity), 9 bytes of results
        env_bytes = E * (8 + 16 + 26 * 32 + 9)
        peaks, peak_kind = load_peaks()
        hbm = float(peaks["hbm_gbs"])
        line = {"metric": "self-play loop boards/s (board-input bf16 inference step + env step + finished-game bookkeeping), 8192 envs per GPU",
                "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16 network, int8/int16 environment", "data": "synthetic",
                "config": {"workload": "8192 environments per rank stepped by the default v4 CNN's own draws from the "
                                       "empty board on, D4 view = step mod 8, no host synchronisation in the loop",
                           "l2": "activations of each layer (0.2-0.6 GB) pass through HBM between kernels"},
                "clocks": clocks, "gpu_launches": (eng.launch_count - launches0) + 3 * args.steps,
                "env_step": {"median_ms": med(env_ms), "launches_per_step": 1},
                "collect_done": {"median_ms": med(col_ms), "launches_per_step": 2,
                                 "note": "includes one torch elementwise add (segment lengths)"},
                "roofline": {"bound": "hbm", "kernel": "env_step_kernel", "achieved": env_bytes / (med(env_ms) * 1e-3) / 1e9,
                             "peak": hbm, "unit": "GB/s", "frac": env_bytes / (med(env_ms) * 1e-3) / 1e9 / hbm,
                             "peak_source": f"MEASURED_PEAKS.json hbm_gbs, of {peak_kind}", "traffic": None,
                             "note": "6.9 MB of algorithmic traffic per launch: the kernel is launch- and latency-bound, "
                                     "its duration here includes the event records around one launch"},
                "library_gpu_bar": {"env_step_plus_reset_median_ms": lib_ms,
                                    "what": "stock torch ops (pad + gather + cumprod step, nonzero + indexed reset) on the same state"},
                "finished_games": n_finished, "env_faults": faults, "device_status": eng.status()}
        print(json.dumps(line), flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="engine", choices=["engine", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-every", type=int, default=8,
                    help="record per-kernel CUDA events on one timed step in this many (1 = every step)")
    ap.add_argument("--no-library-bar", action="store_true",
                    help="skip the stock PyTorch/cuDNN timing of the same step on this GPU")
    ap.add_argument("--precision", default="bf16", choices=["bf16", "f16", "fp32"],
                    help="arithmetic mode of the engine for --workload cfg2: bf16 is the contract's benchmark; f16 the "
                         "fp16 tensor-core mode; fp32 the CUDA-core exact mode")
    ap.add_argument("--workload", default="cfg2", choices=["cfg2", "cfg3", "cfg4", "cfg5", "ensemble", "selfplay", "small", "backward", "train"],
                    help="cfg2 (default) is the contract's benchmark; cfg3-5 are BASELINE's other configurations; "
                         "ensemble is the reference's training shape of the historical opponents (128 models x 4 boards); "
                         "selfplay adds the environment step and bookkeeping around the network; small is a short "
                         "self-ending run of --boards boards for profilers; backward is one layer's backward, train the PPO-style forward + loss + "
                         "backward of the whole network")
    ap.add_argument("--boards", type=int, default=None, help="boards of --workload small (default 2048) and backward (default 8192)")
    args = ap.parse_args()
    if args.impl == "reference":
        args.steps = 20 if args.steps is None else args.steps
        args.warmup = 3 if args.warmup is None else args.warmup
        run_reference(args)
    elif args.workload == "backward":
        args.steps = 50 if args.steps is None else args.steps
        args.warmup = 3 if args.warmup is None else args.warmup
        run_backward(args)
    elif args.workload == "train":
        args.steps = 20 if args.steps is None else args.steps
        args.warmup = 3 if args.warmup is None else args.warmup
        run_train_step(args)
    elif args.workload == "small":
        args.steps = 2 if args.steps is None else args.steps
        args.warmup = 1 if args.warmup is None else args.warmup
        run_small_case(args)
    elif args.workload == "selfplay":
        args.steps = 200 if args.steps is None else args.steps
        args.warmup = 10 if args.warmup is None else max(args.warmup, 3)
        run_selfplay_loop(args)
    elif args.workload != "cfg2":
        args.steps = 50 if args.steps is None else args.steps
        args.warmup = 5 if args.warmup is None else max(args.warmup, 3)
        run_workload(args)
    else:
        # default: a timed region of a few seconds, so that the power cap and the sampled clocks apply to it
        args.steps = (1500 if args.precision != "fp32" else 12) if args.steps is None else args.steps
        args.warmup = (10 if args.precision != "fp32" else 3) if args.warmup is None else max(args.warmup, 3)
        run_engine(args)


if __name__ == "__main__":
    main()
