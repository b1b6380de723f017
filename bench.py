"""Benchmark of the fused MoE layer (one "step" = one layer call over one batch of tokens).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--workload mixtral|qwen3|gptoss|dsv3|toy] [--tokens T]

Default workload: the Mixtral-8x7B-shaped layer (H 4096, I 14336, 8 experts, top-2) at 4096
tokens per GPU, synthetic seeded inputs, weights quantised to NVFP4 (FF1) / int4-g128 (FF2).
With N > 1 (launched by torch.distributed.run, one rank per GPU) experts are sharded
expert-parallel and every rank brings its own 4096 tokens (weak scaling).

Prints ONE JSON line on rank 0: tokens/s with inputs resident in HBM (`value`), the same
through the host-buffer API with copies inside the timed region (`e2e`), a roofline object
for the dominant kernel (per-stage CUDA-event times recorded on the launching stream during
the timed steps), clocks sampled during the timed region, and - at N = 1 - the CPU oracle
timed on the host cores on a bounded sample (`cpu_baseline`). `--impl reference` times only
that CPU path (the reference project has no CPU or B200 implementation of its own).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from xcaliber_b200 import synth  # noqa: E402

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
NVFP4_NOMINAL_TFLOPS = 9000.0  # dense NVFP4 spec figure; there is no measured FP4 peak on this pool

def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """SM clock and clock-event reasons of one GPU, read through NVML every 10 ms by a thread while
    the timed region runs (read-only queries; nothing is set). The samples are also written to a CSV
    file (one per rank) beside the other run outputs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.path = ROOT / "gpurun_out" / f"clocks_rank{gpu_index}.csv"
        self.samples, self.thread, self.handle, self.nv = [], None, None, None
        self.stop_flag = threading.Event()
        try:
            import pynvml as nv

            nv.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(gpu_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            try:
                self.handle = nv.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.handle = nv.nvmlDeviceGetHandleByIndex(gpu_index)
            self.nv = nv
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(self.handle, nv.NVML_CLOCK_SM)
        except Exception as exc:  # NVML missing: report that instead of guessing
            self.error = f"NVML unavailable: {exc}"

    def _sample(self):
        nv = self.nv
        sm = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
        try:
            reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
        except Exception:
            reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
        power = float("nan")
        if len(self.samples) % 8 == 0:  # the power query is slow; the clock is what the timed region needs
            try:
                power = nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
            except Exception:
                pass
        self.samples.append((time.perf_counter(), sm, int(reasons), power))

    def _run(self):
        while not self.stop_flag.is_set():
            try:
                self._sample()
            except Exception:
                break
            self.stop_flag.wait(0.005)

    def start(self):
        if self.nv is None:
            return
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [self.error], "samples": 0}
        try:
            self._sample()  # at least one sample taken while the last kernels are still in flight
        except Exception:
            pass
        self.stop_flag.set()
        self.thread.join(timeout=2)
        sm = [s[1] for s in self.samples]
        bits = 0
        for s in self.samples:
            bits |= s[2]
        try:
            self.path.parent.mkdir(exist_ok=True)
            with open(self.path, "w") as fh:
                fh.write("t_s,sm_mhz,reason_bits,power_w\n")
                for t, mhz, r, pw in self.samples:
                    fh.write(f"{t:.4f},{mhz},{r:#x},{pw:.1f}\n")
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(name for bit, name in self.REASONS.items() if bits & bit), "samples": len(sm)}


def cpu_oracle_tokens_per_s(shape, weights_cpu, sample_tokens: int, steps: int, warmup: int):
    """The dequantise-then-bf16-matmul CPU path on a bounded sample of the workload."""
    from oracle import moe_oracle as O  # the checker, used here only as the timed CPU baseline

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x, logits = synth.make_inputs(shape, weights_cpu, sample_tokens, seed=0)
    for _ in range(warmup):
        O.layer_forward(x, logits, weights_cpu, shape, precision="bf16")
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        O.layer_forward(x, logits, weights_cpu, shape, precision="bf16")
        times.append(time.perf_counter() - t0)
    return sample_tokens / statistics.median(times), cores, statistics.median(times)


def to_cpu_weights(w):
    return synth.LayerWeights(*[None if t is None else t.cpu() for t in (
        w.w13_packed, w.w13_scale, w.w13_gs, w.w2_qweight, w.w2_scales, w.router_weight, w.router_bias, w.logit_bias)])


def router_on_cpu(w):
    """Only the router parts (what make_inputs needs), on the CPU."""
    return synth.LayerWeights(None, None, None, None, None, w.router_weight.cpu(), None,
                              None if w.logit_bias is None else w.logit_bias.cpu())


_REAL_STDOUT = None


def claim_stdout() -> None:
    """stdout carries exactly one JSON line. Libraries print there too (NCCL's version banner, for one):
    keep the real stdout for the result and point file descriptor 1 at stderr for everything else."""
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(line: dict) -> None:
    out = _REAL_STDOUT or sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main() -> int:
    claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="mixtral", choices=sorted(synth.SHAPES))
    ap.add_argument("--tokens", type=int, default=4096, help="tokens per GPU per step")
    ap.add_argument("--cpu-sample-tokens", type=int, default=128)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (for short profiler captures)")
    ap.add_argument("--no-decode", action="store_true", help="skip the supplementary decode point")
    ap.add_argument("--decode-tokens", type=int, default=16)
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    shape = synth.SHAPES[args.workload]
    n = args.tokens
    workload = f"{shape.name}-shaped MoE layer H{shape.hidden} I{shape.inter} E{shape.num_experts} top{shape.top_k}"
    config = {"workload": workload, "tokens_per_gpu": n, "global_tokens": n * max(world, 1),
              "parallelism": f"ep{world}" if world > 1 else "single",
              "l2": "inputs larger than L2 (expert weights re-streamed from HBM every step)"}

    # ------------------------------------------------------------------ reference arm
    if args.impl == "reference":
        if rank != 0:
            return 0
        # same weights as the native arm; synthesised on the GPU when there is one (minutes faster), timed on the CPU
        if torch.cuda.is_available():
            w_cpu = to_cpu_weights(synth.make_weights(shape, seed=0, device=torch.device("cuda", local_rank)))
        else:
            w_cpu = synth.make_weights(shape, seed=0, device="cpu")
        sample = min(args.cpu_sample_tokens, n)
        tps, cores, med = cpu_oracle_tokens_per_s(shape, w_cpu, sample, max(1, min(args.steps, 3)), 1)
        line = {"metric": METRIC, "value": tps, "unit": UNIT, "impl": "reference", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": med * 1e3, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4 x nvfp4 (FF1), int4 x bf16 (FF2), fp32 accumulate",
                "data": "synthetic", "config": config,
                "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": "port",
                                 "sample": f"{sample} tokens of the same workload, dequantise-then-bf16-matmul, "
                                           f"median of {max(1, min(args.steps, 3))} runs after 1 warm-up"},
                "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "note": "the reference project has no CPU path and its GPU kernels do not assemble for sm_100a; "
                        "this arm times the CPU restatement of its algorithm (oracle/) on the host cores"}
        emit(line)
        return 0

    # ------------------------------------------------------------------ native arm
    if not torch.cuda.is_available():
        emit({"error": "no CUDA device: the native arm has no CPU fallback"})
        return 1
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    from xcaliber_b200 import ops

    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    ckpt = synth.make_weights(shape, seed=0, device=dev)
    x_cpu, logits_cpu = synth.make_inputs(shape, router_on_cpu(ckpt), n, seed=rank)
    x, logits = x_cpu.to(dev), logits_cpu.to(dev)

    if world > 1:
        from xcaliber_b200.ep import ExpertParallelMoE

        layer = ExpertParallelMoE(shape, ckpt, device=dev, max_tokens=n)
        fwd = lambda: layer.forward(x, logits)  # noqa: E731
        # home side: router, amax, route pack (2), post counts, dispatch, scale, wait data, return, wait
        # returns, combine; owner side: route pack (2), quantise, FF1, FF2 (+ activation top-k)
        launches_per_step = 11 + layer.local.kernel_launches_per_forward - 3
    else:
        pw = ops.PreparedWeights.from_checkpoint(shape, ckpt.w13_packed, ckpt.w13_scale, ckpt.w13_gs,
                                                 ckpt.w2_qweight, ckpt.w2_scales, router_bias=ckpt.router_bias,
                                                 device=dev)
        layer = ops.FusedMoE(shape, pw)
        y_buf = torch.empty_like(x)
        fwd = lambda: layer.forward(x, logits, out=y_buf)  # noqa: E731
        launches_per_step = layer.kernel_launches_per_forward

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        fwd()
    sync_all()

    ops.profile_begin(args.steps)
    sampler = ClockSampler(local_rank)
    sampler.start()
    sync_all()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        fwd()
    ev1.record()
    sync_all()
    clocks = sampler.stop()
    ms_total = ev0.elapsed_time(ev1)
    stage_ms, prof_steps = ops.profile_read()
    ops.profile_begin(0)
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = n * world / (ms_step * 1e-3)

    # ---- end to end: host buffers in, host buffer out, copies inside the timed region
    xh, lh = x_cpu.pin_memory(), logits_cpu.pin_memory()
    yh = torch.empty_like(x_cpu).pin_memory()
    if world > 1:
        def e2e_step():
            x.copy_(xh, non_blocking=True)
            logits.copy_(lh, non_blocking=True)
            yh.copy_(layer.forward(x, logits), non_blocking=True)
            torch.cuda.current_stream().synchronize()
    else:
        def e2e_step():
            layer.forward_host(xh, lh, yh)
    e2e_steps = 0 if args.no_e2e else args.steps
    for _ in range(3 if e2e_steps else 0):
        e2e_step()
    sync_all()
    ev0.record()
    for _ in range(e2e_steps):
        e2e_step()
    ev1.record()
    sync_all()
    e2e_ms = ev0.elapsed_time(ev1) if e2e_steps else float("nan")
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = n * world / (e2e_ms / args.steps * 1e-3) if e2e_steps else None
    h2d = x_cpu.numel() * 2 + logits_cpu.numel() * 2
    d2h = x_cpu.numel() * 2

    # ---- roofline of the dominant kernel (local pipeline stages, this rank)
    peaks = measured_peaks()
    per_stage = {k: v / max(prof_steps, 1) for k, v in stage_ms.items()}
    dominant = max(("ff1", "ff2"), key=lambda k: per_stage.get(k, 0.0))
    rows_local = n * shape.k_eff  # assignments processed per rank per step (uniform in expectation under EP)
    e_local = shape.e_tot if world == 1 else shape.num_experts // world + shape.num_shared_experts
    flops_ff1 = 4.0 * rows_local * shape.hidden * shape.inter
    flops_ff2 = 2.0 * rows_local * shape.hidden * shape.inter
    w_bytes_ff1 = e_local * (2 * shape.inter * shape.hidden // 2 + 2 * shape.inter * shape.hidden // 16 + 8)
    w_bytes_ff2 = e_local * (shape.hidden * shape.inter // 2 + 2 * shape.hidden * ((shape.inter + 127) // 128))
    avg_rows_per_expert = rows_local / max(e_local, 1)
    tensor_bound = avg_rows_per_expert >= 256
    dom_ms = per_stage.get(dominant, 0.0)
    if tensor_bound:
        fl = flops_ff1 if dominant == "ff1" else flops_ff2
        achieved = fl / (dom_ms * 1e-3) / 1e12 if dom_ms else 0.0
        peak = NVFP4_NOMINAL_TFLOPS if dominant == "ff1" else peaks["bf16_tflops_sustained"]
        roofline = {"kernel": dominant, "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                    "frac": achieved / peak if peak else None, "traffic": None,
                    "peak_source": ("nominal dense NVFP4 (no measured FP4 figure)" if dominant == "ff1"
                                    else f"{peaks['source']} bf16 sustained")}
    else:
        by = (w_bytes_ff1 + rows_local * (shape.hidden // 2 + shape.hidden // 16 + 2 * shape.inter)) if dominant == "ff1" \
            else (w_bytes_ff2 + rows_local * 2 * (shape.inter + shape.hidden))
        achieved = by / (dom_ms * 1e-3) / 1e9 if dom_ms else 0.0
        roofline = {"kernel": dominant, "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_source": f"{peaks['source']} copy"}
    traffic_file = ROOT / "profiles" / "traffic.json"
    if traffic_file.exists():
        tr = json.loads(traffic_file.read_text()).get(f"{args.workload}:{n}:{dominant}")
        if tr is not None:
            roofline["traffic"] = tr
    ff1_ms, ff2_ms = per_stage.get("ff1", 0.0), per_stage.get("ff2", 0.0)
    # the tensor-pipe ceiling for NVFP4 as this GPU delivers it (resident operands, no data movement):
    # there is no library GEMM to take an NVFP4 peak from
    mma_probe = {}
    if world == 1 and rank == 0:
        try:
            mma_probe = {"nvfp4_mma_tflops_measured": ops.probe_mma_rate("nvfp4", 262144),
                         "bf16_mma_tflops_measured": ops.probe_mma_rate("bf16", 262144)}
        except Exception as exc:  # the probe is an aid; the bench line stands without it
            mma_probe = {"mma_probe_error": str(exc)}
    extra = {
        "stage_ms": {k: round(v, 5) for k, v in per_stage.items()},
        "ff1_tflops": flops_ff1 / (ff1_ms * 1e-3) / 1e12 if ff1_ms else None,
        "ff1_frac_of_nominal_nvfp4": flops_ff1 / (ff1_ms * 1e-3) / 1e12 / NVFP4_NOMINAL_TFLOPS if ff1_ms else None,
        "ff2_tflops": flops_ff2 / (ff2_ms * 1e-3) / 1e12 if ff2_ms else None,
        "ff2_frac_of_bf16_sustained": flops_ff2 / (ff2_ms * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"] if ff2_ms else None,
        "layer_useful_tflops": synth.algorithmic_flops(shape, n) / (ms_step * 1e-3) / 1e12,
        **mma_probe,
    }
    if ff1_ms and mma_probe.get("nvfp4_mma_tflops_measured"):
        extra["ff1_frac_of_measured_nvfp4_mma_rate"] = extra["ff1_tflops"] / mma_probe["nvfp4_mma_tflops_measured"]

    # ---- decode point of the same layer (N = 16 per GPU), CUDA-graph replay, HBM roofline
    decode = None
    if world == 1 and not args.no_decode:
        nd = args.decode_tokens
        xd, ld = x[:nd].contiguous(), logits[:nd].contiguous()
        yd = torch.empty_like(xd)
        for _ in range(3):
            layer.forward(xd, ld, out=yd)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            layer.forward(xd, ld, out=yd)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        ev0.record()
        reps = 50
        for _ in range(reps):
            g.replay()
        ev1.record()
        torch.cuda.synchronize()
        dms = ev0.elapsed_time(ev1) / reps
        ops.profile_begin(10)
        for _ in range(10):
            layer.forward(xd, ld, out=yd)
        dstage, dsteps = ops.profile_read()
        ops.profile_begin(0)
        live = int((layer.view(nd)["counts"] > 0).sum().item())
        by = synth.algorithmic_bytes(shape, nd, live)
        decode = {"tokens": nd, "ms_per_step": dms, "tokens_per_s": nd / (dms * 1e-3), "live_experts": live,
                  "algorithmic_gb": by / 1e9, "hbm_gbs": by / (dms * 1e-3) / 1e9,
                  "hbm_frac_of_measured": by / (dms * 1e-3) / 1e9 / peaks["hbm_gbs"], "launch": "cuda graph replay",
                  "stage_ms_stream_launch": {k: round(v / max(dsteps, 1), 5) for k, v in dstage.items()}}

    cpu_baseline = None
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        sample = min(args.cpu_sample_tokens, n)
        tps, cores, med = cpu_oracle_tokens_per_s(shape, to_cpu_weights(ckpt), sample, 1, 0)
        cpu_baseline = {"value": tps, "unit": UNIT, "cores": cores, "kind": "port",
                        "sample": f"{sample} tokens of the same workload (all experts dequantised once), "
                                  f"dequantise-then-bf16-matmul oracle, 1 run, {med:.1f} s"}

    if world > 1:
        statuses = [loc.status(m) for loc in layer._local_by_tile.values() for (m, _h) in list(loc._ws)[:1]]
        if layer.peer is not None:
            statuses.append(layer.peer.status())
    else:
        statuses = [layer.status(n)]
    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "nvfp4 x nvfp4 (FF1), int4 x bf16 (FF2), fp32 accumulate",
                "data": "synthetic", "config": config, "clocks": clocks,
                "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
                "gpu_launches": launches_per_step * args.steps, "roofline": roofline, "cpu_baseline": cpu_baseline,
                "device_status": statuses, **extra}
        if decode is not None:
            line["decode"] = decode
        emit(line)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
