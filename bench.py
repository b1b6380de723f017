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
the timed steps), clocks sampled during the timed region, whether the first warm-up step
passed the stage-wise parity spot check against the CPU oracle (`parity_checked`), and - at
N = 1 - the CPU oracle timed on the host cores (`cpu_baseline`). `--impl reference` times only
that CPU path (the reference project has no CPU or B200 implementation of its own): the
dequantise-then-bf16-matmul layer on the FULL batch, weights dequantised once at set-up as a CPU
deployment would, as many steps as fit a fixed time budget (the number really run is printed).
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
    the timed region runs (read-only queries; nothing is set). With --clock-csv PREFIX the samples are also
    written to PREFIX<rank>.csv."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, gpu_index: int, csv_prefix: str | None = None):
        self.gpu_index = gpu_index
        self.path = Path(f"{csv_prefix}{gpu_index}.csv") if csv_prefix else None
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
        if self.path is not None:
            try:
                self.path.parent.mkdir(parents=True, exist_ok=True)
                with open(self.path, "w") as fh:
                    fh.write("t_s,sm_mhz,reason_bits,power_w\n")
                    for t, mhz, r, pw in self.samples:
                        fh.write(f"{t:.4f},{mhz},{r:#x},{pw:.1f}\n")
            except OSError:
                pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(name for bit, name in self.REASONS.items() if bits & bit), "samples": len(sm)}


DENSE_LIMIT_BYTES = 12 << 30  # bf16 copies of all experts beyond this stay quantised (dequantised per call, sampled batch)


def cpu_oracle_run(shape, weights, n_tokens: int, steps: int, warmup: int, budget_s: float, dense_device=None,
                   sample_tokens: int = 128):
    """Times the CPU restatement of the layer (oracle/, dequantise-then-bf16-matmul) on the host cores.

    Normal case: every expert is dequantised to bf16 ONCE at set-up (untimed, like loading a checkpoint) and
    each step runs the full batch of n_tokens. `steps` is an upper bound: after the warm-up, as many steps as
    fit `budget_s` are run (at least one) and that number is returned. Shapes whose dense bf16 weights exceed
    DENSE_LIMIT_BYTES keep the 4-bit weights and dequantise inside every call, on `sample_tokens` tokens.
    Returns dict(tokens, tokens_per_s, step_s, steps_run, warmup_run, cores, how)."""
    from oracle import moe_oracle as O  # the checker, used here only as the timed CPU baseline

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    dense_bytes = 2 * 3 * shape.e_tot * shape.hidden * shape.inter
    dense = None
    if dense_bytes <= DENSE_LIMIT_BYTES:
        dense = O.dense_expert_weights(weights, shape, device=dense_device)
        tokens = n_tokens
        how = f"full batch of {tokens} tokens; experts dequantised to bf16 once at set-up (untimed), bf16 matmuls"
    else:
        tokens = min(sample_tokens, n_tokens)
        how = (f"SAMPLE of {tokens} tokens (dense bf16 weights would take {dense_bytes >> 30} GiB): experts "
               "dequantised inside every call, bf16 matmuls")
    w_cpu = to_cpu_weights(weights) if dense is None else router_on_cpu(weights, keep_router_bias=True)
    x, logits = synth.make_inputs(shape, w_cpu, tokens, seed=0)
    t_warm = []
    for _ in range(warmup):
        t0 = time.perf_counter()
        O.layer_forward(x, logits, w_cpu, shape, precision="bf16", dense=dense)
        t_warm.append(time.perf_counter() - t0)
    est = min(t_warm) if t_warm else None
    steps_run = max(1, min(steps, int(budget_s / est))) if est else max(1, steps)
    times = []
    for _ in range(steps_run):
        t0 = time.perf_counter()
        O.layer_forward(x, logits, w_cpu, shape, precision="bf16", dense=dense)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return dict(tokens=tokens, tokens_per_s=tokens / med, step_s=med, steps_run=steps_run, warmup_run=warmup,
                cores=cores, how=how)


def to_cpu_weights(w):
    return synth.LayerWeights(*[None if t is None else t.cpu() for t in (
        w.w13_packed, w.w13_scale, w.w13_gs, w.w2_qweight, w.w2_scales, w.router_weight, w.router_bias, w.logit_bias)])


def router_on_cpu(w, keep_router_bias: bool = False):
    """Only the router parts (what make_inputs and the routing oracle need), on the CPU."""
    rb = w.router_bias.cpu() if (keep_router_bias and w.router_bias is not None) else None
    return synth.LayerWeights(None, None, None, None, None, w.router_weight.cpu(), rb,
                              None if w.logit_bias is None else w.logit_bias.cpu())


def parity_spot_check(shape, ckpt, layer, x_cpu, logits_cpu, y, n, world) -> dict:
    """The first warm-up step against the CPU oracle (oracle/stagewise.py: routing, permutation and NVFP4 packets
    bit-exact on every token, the combine bit-exact, FF1 and FF2 within max rel 2e-2 / mean 5e-3 on sampled
    experts, rows and output columns). Single-GPU arm only: the expert-parallel arm is compared with the
    single-GPU path by the test suite instead."""
    if world > 1:
        return {"parity_checked": False, "parity_note": "expert-parallel arm: compared with the 1-GPU path in tests/"}
    if 0 < shape.act_topk_keep < shape.inter:
        return {"parity_checked": False, "parity_note": "activation top-k shapes are checked in tests/ (need a dense twin)"}
    from oracle import stagewise  # the checker; never on the timed path

    torch.cuda.synchronize()
    if layer.status(n):
        return {"parity_checked": False, "parity_note": f"device status {layer.status(n):#x}"}
    try:
        res = stagewise.check_layer_stages(shape, ckpt, router_on_cpu(ckpt, keep_router_bias=True), x_cpu, logits_cpu,
                                           y, layer.view(n), experts_cap=3, rows_cap=24, ff1_cols=160, ff2_cols=96)
    except AssertionError as exc:
        return {"parity_checked": True, "parity_ok": False, "parity_note": str(exc)[:300]}
    w = res["worst"]
    return {"parity_checked": True, "parity_ok": True,
            "parity_note": f"routing/permutation/packets/combine exact on all {n} tokens; FF1 max rel {w['ff1'][0]:.2g} "
                           f"mean {w['ff1'][1]:.2g}, FF2 max rel {w['ff2'][0]:.2g} mean {w['ff2'][1]:.2g} on experts "
                           f"{res['experts']} (sampled rows and columns)"}


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
    ap.add_argument("--cpu-sample-tokens", type=int, default=128,
                    help="CPU legs: batch used only when the dense bf16 weights do not fit the host (see cpu_oracle_run)")
    ap.add_argument("--cpu-budget-s", type=float, default=150.0, help="--impl reference: seconds of timed CPU steps")
    ap.add_argument("--clock-csv", default=None, help="write the clock samples to <this prefix><rank>.csv")
    ap.add_argument("--no-parity-check", action="store_true", help="skip the oracle spot check of the first warm-up step")
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
            w_dev = synth.make_weights(shape, seed=0, device=torch.device("cuda", local_rank))
        else:
            w_dev = synth.make_weights(shape, seed=0, device="cpu")
        r = cpu_oracle_run(shape, w_dev, n, max(1, args.steps), 1, args.cpu_budget_s, dense_device=w_dev.w13_packed.device,
                           sample_tokens=args.cpu_sample_tokens)
        config = dict(config, tokens_per_gpu=r["tokens"], global_tokens=r["tokens"],
                      workload=workload + ("" if r["tokens"] == n else f" (CPU SAMPLE of {r['tokens']} tokens)"))
        line = {"metric": METRIC, "value": r["tokens_per_s"], "unit": UNIT, "impl": "reference", "n_gpus": args.gpus,
                "steps": r["steps_run"], "warmup": r["warmup_run"], "steps_requested": args.steps,
                "ms_per_step": r["step_s"] * 1e3, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4 x nvfp4 (FF1), int4 x bf16 (FF2), fp32 accumulate",
                "data": "synthetic", "config": config,
                "cpu_baseline": {"value": r["tokens_per_s"], "unit": UNIT, "cores": r["cores"], "kind": "port",
                                 "sample": f"{r['how']}; median of {r['steps_run']} steps after {r['warmup_run']} warm-up"},
                "e2e": {"value": r["tokens_per_s"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
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

    parity = {"parity_checked": False, "parity_note": "skipped"}
    for step in range(max(args.warmup, 3)):
        y_step = fwd()
        if step == 0 and not args.no_parity_check:
            parity = parity_spot_check(shape, ckpt, layer, x_cpu, logits_cpu, y_step, n, world)
    sync_all()

    ep_phases = None
    if world > 1 and layer.peer is not None:
        # where an expert-parallel step spends its time on this rank (a second short run, so that the event records do
        # not sit inside the timed region)
        layer.profile_phases(True)
        for _ in range(5):
            fwd()
        ep_phases = {k: round(v, 5) for k, v in layer.phase_ms().items()}
        layer.profile_phases(False)
        sync_all()
    # per-stage CUDA events (the roofline's kernel durations) on the first steps of the timed region only: every event
    # record costs the stream about 2.6 us, nine of them per layer call
    ops.profile_begin(min(args.steps, 10))
    sampler = ClockSampler(local_rank, args.clock_csv)
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

    # ---- end to end: host buffers in, host buffer out, copies inside the timed region. Every step copies its
    # inputs from pinned host memory and its result back. `serial`: one synchronous call after the other
    # (xmoe_forward_host). `value`: the serving loop, E2E_DEPTH calls in flight, each on its own stream with its
    # own workspace and host buffers (xmoe_forward_host_async), so that one call's PCIe copies overlap another's
    # kernels; a slot is reused only after its previous call has been synchronised.
    E2E_DEPTH = 3
    xh, lh = x_cpu.pin_memory(), logits_cpu.pin_memory()
    yh = torch.empty_like(x_cpu).pin_memory()
    e2e_steps = 0 if args.no_e2e else args.steps

    def timed(run_steps):
        if not e2e_steps:
            return float("nan")
        sync_all()
        ev0.record()
        run_steps(e2e_steps)
        ev1.record()
        sync_all()
        ms = ev0.elapsed_time(ev1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    if world > 1:
        def serial_steps(k):
            for _ in range(k):
                x.copy_(xh, non_blocking=True)
                logits.copy_(lh, non_blocking=True)
                yh.copy_(layer.forward(x, logits), non_blocking=True)
                torch.cuda.current_stream().synchronize()
        pipelined_steps = None
    else:
        def serial_steps(k):
            for _ in range(k):
                layer.forward_host(xh, lh, yh)

        slots = [(torch.cuda.Stream(device=dev), x_cpu.pin_memory(), logits_cpu.pin_memory(),
                  torch.empty_like(x_cpu).pin_memory()) for _ in range(E2E_DEPTH)]

        def pipelined_steps(k):
            cur = torch.cuda.current_stream()
            for st, *_ in slots:
                st.wait_stream(cur)
            for i in range(k):
                st, xs, ls, ys = slots[i % E2E_DEPTH]
                st.synchronize()  # the slot's previous call is complete: its result may be read, its buffers reused
                layer.forward_host_async(xs, ls, ys, slot=i % E2E_DEPTH, stream=st)
            for st, *_ in slots:
                cur.wait_stream(st)

    if e2e_steps:
        serial_steps(3)
        if pipelined_steps:
            pipelined_steps(2 * E2E_DEPTH)
    e2e_serial_ms = timed(serial_steps)
    e2e_ms = timed(pipelined_steps) if pipelined_steps else e2e_serial_ms
    e2e_value = n * world / (e2e_ms / args.steps * 1e-3) if e2e_steps else None
    e2e_serial_value = n * world / (e2e_serial_ms / args.steps * 1e-3) if e2e_steps else None
    if e2e_steps and pipelined_steps and not torch.equal(slots[0][3], yh):
        raise RuntimeError("pipelined host-buffer calls returned a different result than the synchronous call")
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
    dom_ms = per_stage.get(dominant, 0.0)
    # the bound of the dominant kernel is the slower of its two floors: algorithmic bytes at the measured copy
    # bandwidth, flops at the tensor peak (NVFP4: nominal dense; bf16: measured burst)
    fl = flops_ff1 if dominant == "ff1" else flops_ff2
    by = (w_bytes_ff1 + rows_local * (shape.hidden // 2 + shape.hidden // 16 + 2 * shape.inter)) if dominant == "ff1" \
        else (w_bytes_ff2 + rows_local * 2 * (shape.inter + shape.hidden))
    tensor_peak = NVFP4_NOMINAL_TFLOPS if dominant == "ff1" else peaks["bf16_tflops"]
    floor_tensor_ms = fl / (tensor_peak * 1e12) * 1e3
    floor_hbm_ms = by / (peaks["hbm_gbs"] * 1e9) * 1e3
    tensor_bound = floor_tensor_ms >= floor_hbm_ms
    if tensor_bound:
        achieved = fl / (dom_ms * 1e-3) / 1e12 if dom_ms else 0.0
        # the timed region is tens of milliseconds, not a seconds-long step: the burst figure is the denominator
        roofline = {"kernel": dominant, "bound": "tensor", "achieved": achieved, "peak": tensor_peak, "unit": "TFLOP/s",
                    "frac": achieved / tensor_peak if tensor_peak else None, "traffic": None,
                    "peak_source": ("nominal dense NVFP4 (no measured FP4 figure)" if dominant == "ff1"
                                    else f"{peaks['source']} bf16 burst"),
                    "frac_of_sustained": None if dominant == "ff1" else achieved / peaks["bf16_tflops_sustained"]}
    else:
        achieved = by / (dom_ms * 1e-3) / 1e9 if dom_ms else 0.0
        roofline = {"kernel": dominant, "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_source": f"{peaks['source']} copy"}
    roofline["floor_ms"] = {"tensor": round(floor_tensor_ms, 5), "hbm": round(floor_hbm_ms, 5)}
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
        r = cpu_oracle_run(shape, ckpt, n, 1, 1, 1.0, dense_device=dev, sample_tokens=args.cpu_sample_tokens)
        cpu_baseline = {"value": r["tokens_per_s"], "unit": UNIT, "cores": r["cores"], "kind": "port",
                        "tokens": r["tokens"],
                        "sample": f"{r['how']}; 1 timed step of {r['step_s']:.2f} s after 1 warm-up"}

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
                "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "calls_in_flight": E2E_DEPTH if world == 1 else 1, "serial_value": e2e_serial_value},
                "gpu_launches": launches_per_step * args.steps, "roofline": roofline, "cpu_baseline": cpu_baseline,
                "device_status": statuses, **parity, **extra}
        if ep_phases is not None:
            line["ep_phase_ms_rank0"] = ep_phases
        if decode is not None:
            line["decode"] = decode
        emit(line)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
