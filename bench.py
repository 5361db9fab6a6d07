#!/usr/bin/env python
"""Benchmark of the power-retention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload train|decode]

Workload `train` (default): forward + backward of one power-retention layer at
b=1, t=65536, h=8, d=64, deg=2, bf16, chunk 1024, gated (synthetic N(0,1) inputs,
log_G = logsigmoid(N(0,1))).  A step is one forward+backward pass.  With N > 1 GPUs the
kv heads are split across ranks (no collective on the data path); the reported value is
batch*tokens per second of the whole job, timed on the device, max over ranks.

One JSON line is printed by rank 0.  `--impl reference` times the CPU restatement of the
reference's algorithm (oracle/) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(b=1, t=65536, h=8, d=64, deg=2, chunk=1024, dtype="bf16", gated=True)
D_EXACT = 64 * 65 // 2  # C(d+1, 2) = 2080: the algorithmic expanded dimension


def algorithmic_flops(b, t, hq, h, d, c, D=D_EXACT):
    """Per-kernel algorithmic FLOPs (exact D, causal half counted once)."""
    att = b * hq * t * c * d  # one causal c x c x d product summed over chunks
    exp_q = 2 * b * hq * t * D * d
    exp_k = 2 * b * h * t * D * d
    return {
        "pr_chunk_state": None,  # filled per call site below
        "fwd": 2 * att + exp_q + exp_k,
        "bwd": 5 * att + 2 * exp_q + 2 * exp_k,
        "att": att, "exp_q": exp_q, "exp_k": exp_k,
    }


def make_inputs(b, t, h, d, device, seed0=0, heads=None):
    """Seeded synthetic inputs; `heads` selects a slice of the h heads (for sharding)."""
    hs = heads if heads is not None else range(h)
    out = []
    for i, shape in enumerate([(b, t, h, d)] * 3 + [(b, t, h)] + [(b, t, h, d)]):
        g = torch.Generator().manual_seed(seed0 + i)
        x = torch.randn(*shape, generator=g)
        x = x[:, :, list(hs)].contiguous()
        out.append(x)
    Q, K, V, G, dO = out
    return (Q.bfloat16(), K.bfloat16(), V.bfloat16(), F.logsigmoid(G).float(), dO.bfloat16())


# DRAM bytes (read + write) per launch of each tensor-core kernel, from the ncu capture of the t = 8192, h = 8 case
# summarised in profiles/train_kernels_ncu_full_b1_t8192_h8_d64.md; traffic grows in proportion to tokens x heads
NCU_DRAM_BYTES_T8192_H8 = {"pr_expand_grad": 34.6e6, "pr_chunk_dkv": 73.1e6, "pr_chunk_out": 50.5e6,
                           "pr_chunk_state": 21.0e6, "pr_chunk_dq": 51.9e6}

# the reference's only published figure for this exact metric and shape: 16.8 ms per fwd+bwd step on one H100
PUBLISHED_TOKENS_PER_S = 65536 / 16.8e-3


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            if len(s) < 6:
                continue
            try:
                sm.append(float(s[0]))
                mx = float(s[1])
            except ValueError:
                continue
            for nme, val in zip(names, s[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nme)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_reference_run(steps, warmup, sample_t=16384, sample_h=2):
    """Times the CPU restatement of the reference (oracle/) on a bounded sample of the
    workload: t=sample_t tokens of sample_h heads, forward+backward, all host threads."""
    from oracle import power_retention_oracle as oracle

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    Q, K, V, G, dO = make_inputs(CFG["b"], sample_t, CFG["h"], CFG["d"], "cpu", heads=range(sample_h))

    def step():
        q, k, v = (x.clone().requires_grad_(True) for x in (Q, K, V))
        g = G.clone().requires_grad_(True)
        O = oracle.power_retention(q, k, v, g, deg=2, chunk_size=CFG["chunk"])
        O.backward(dO)
        return O

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    # tokens/s of the full-width (h heads) layer: cost is linear in heads and in tokens
    value = CFG["b"] * sample_t / dt * (sample_h / CFG["h"])
    return value, dt, cores, (f"oracle port of retention/reference.py, fwd+bwd, bf16, t={sample_t} tokens x "
                              f"{sample_h} of {CFG['h']} heads, chunk {CFG['chunk']}; throughput scaled by heads")


def run_reference(args, rank):
    if rank != 0:
        return
    steps = max(1, min(args.steps, 3))
    value, dt, cores, sample = cpu_reference_run(steps, min(args.warmup, 1))
    line = {
        "impl": "reference", "metric": "fwd_bwd_tokens_per_sec", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "power_retention fwd+bwd b1 t65536 h8 d64 deg2 chunk1024 gated bf16"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_decode(args):
    """Inference workload: b=16, h=32, d=64 bf16 gated; a 2048-token prefill compressed into the
    state (switch_over 1024), then 512 single-token steps whose cache grows from 1 to 512 tokens.
    Reports decode tokens/s and the achieved HBM bandwidth of the state read."""
    import retention_integration_b200 as prb
    from retention_integration_b200 import _lib, ops

    dev = torch.device("cuda", 0)
    b, h, d, t0, steps = 16, 32, 64, 2048, args.decode_steps
    g = torch.Generator().manual_seed(0)
    mk = lambda *s: torch.randn(*s, generator=g).bfloat16().to(dev)
    Kp, Vp, qp = mk(b, t0, h, d), mk(b, t0, h, d), mk(b, 1, h, d)
    lgp = F.logsigmoid(torch.randn(b, t0, h, generator=g)).to(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    prb.power_retention_inference(qp, Kp, Vp, lgp, switch_over_seq_len=1024)  # warm-up
    torch.cuda.synchronize()
    e0.record()
    _, state, sk = prb.power_retention_inference(qp, Kp, Vp, lgp, switch_over_seq_len=1024)
    e1.record()
    torch.cuda.synchronize()
    prefill_ms = e0.elapsed_time(e1)
    Kc, Vc, Qs = mk(b, steps, h, d), mk(b, steps, h, d), mk(b, steps, h, d)
    lgc = F.logsigmoid(torch.randn(b, steps, h, generator=g)).to(dev)

    def decode_all():
        for i in range(steps):
            prb.power_retention_inference(Qs[:, i:i + 1], Kc[:, :i + 1], Vc[:, :i + 1], lgc[:, :i + 1], state, sk,
                                          switch_over_seq_len=1024)

    decode_all()
    torch.cuda.synchronize()
    ops.launch_log.reset(timing=True)
    e0.record()
    decode_all()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    kern = ops.launch_log.summary()
    launches = ops.launch_log.count
    ops.launch_log.reset()
    # the state read timed alone, launches queued back to back (inside a decode step the GPU
    # waits for the host between launches, so per-launch events there include that wait)
    qd = Qs[:, :1].contiguous()
    ops.decode_state(qd, state, sk, None, 0.125)
    torch.cuda.synchronize()
    n_state = 50
    e0.record()
    for _ in range(n_state):
        ops.decode_state(qd, state, sk, None, 0.125)
    e1.record()
    torch.cuda.synchronize()
    ms_state = e0.elapsed_time(e1)
    state_bytes = state.numel() * 2 + sk.numel() * 4
    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except OSError:
        pass
    peak = peaks.get("hbm_gbs") or 6650.0
    achieved = state_bytes / (ms_state / n_state * 1e-3) / 1e9
    print(json.dumps({
        "metric": "decode_tokens_per_sec", "value": b * steps / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "ms_per_step": ms / steps, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"power_retention_inference decode b16 h32 d64 gated, state [16,32,2080,64], cache 1..{steps}"},
        "prefill_to_state_ms": prefill_ms, "gpu_launches": launches,
        "roofline": {"bound": "hbm", "kernel": "pr_decode_state", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_source": "measured" if "hbm_gbs" in peaks else "fallback",
                     "traffic": 140.67e6,  # ncu dram__bytes_read of one launch (profiles/decode_state_ncu_b16_h32_d64.md)
                     "algorithmic_bytes": state_bytes},
        "kernels": {k: {"launches": n, "ms_total": t} for k, (n, t) in kern.items()},
        "device_status": _lib.device_status(0)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--t", type=int, default=CFG["t"], help="sequence length override (profiling small cases)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch the timed steps eagerly instead of replaying a graph")
    ap.add_argument("--workload", default="train", choices=["train", "decode"])
    ap.add_argument("--decode-steps", type=int, default=512, help="single-token steps of the decode workload")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.workload == "decode":
        run_decode(args)
        return

    import torch.distributed as dist
    import retention_integration_b200 as prb
    from retention_integration_b200 import _lib, ops

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    b, t, h, d, c = CFG["b"], args.t, CFG["h"], CFG["d"], CFG["chunk"]
    assert h % world == 0, "kv heads must divide evenly over the ranks"
    hl = h // world
    heads = range(rank * hl, (rank + 1) * hl)
    Qh, Kh, Vh, Gh, dOh = (x.pin_memory() for x in make_inputs(b, t, h, d, "cpu", heads=heads))
    Q, K, V, G, dO = (x.to(dev) for x in (Qh, Kh, Vh, Gh, dOh))

    def step(Q, K, V, G, dO):
        q, k, v = Q.detach().requires_grad_(True), K.detach().requires_grad_(True), V.detach().requires_grad_(True)
        g = G.detach().requires_grad_(True)
        O = prb.power_retention(q, k, v, g, deg=2, chunk_size=c)
        O.backward(dO)
        return O, q.grad, k.grad, v.grad, g.grad

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # clocks are sampled from before the warm-up to the end of the timed regions (nvidia-smi
    # needs a few hundred ms to start, longer than a short timed region)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step(Q, K, V, G, dO)
    barrier()
    if _lib.device_status(local_rank) != 0:
        raise SystemExit("a kernel reported a timed-out wait during warm-up")
    if rank == 0:
        # keep the GPU busy until the sampler has delivered its first readings
        t_wait = time.time()
        while len(sampler.samples) < 3 and time.time() - t_wait < 5.0:
            step(Q, K, V, G, dO)
            torch.cuda.synchronize()
    barrier()

    # ---- per-kernel breakdown: a separate pass with CUDA events around every launch (the event
    # records cost host time, so this pass is not the one the headline is taken from)
    ops.launch_log.reset(timing=True)
    for _ in range(min(args.steps, 3)):
        step(Q, K, V, G, dO)
    barrier()
    kernels = ops.launch_log.summary()
    breakdown_steps = min(args.steps, 3)
    launches_per_step = ops.launch_log.count // breakdown_steps
    ops.launch_log.reset(timing=False)

    # ---- device-resident timed region.  One step is captured into a CUDA graph (the library's kernels are
    # plain stream launches, so torch.cuda.graph records forward and backward as they are) and replayed K
    # times: with one head per GPU a step is ~0.6 ms of GPU work against ~0.5 ms of Python launch code, and
    # eight ranks share the host's cores.  If the capture is refused the same K steps are launched eagerly.
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    graph, launch_mode = None, "eager launches"
    if not args.no_graph:
        try:
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                step(Q, K, V, G, dO)
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                graph_out = step(Q, K, V, G, dO)
            graph.replay()
            torch.cuda.synchronize()
            ref_out = step(Q, K, V, G, dO)
            torch.cuda.synchronize()
            if not all(torch.equal(a_, b_) for a_, b_ in zip(graph_out, ref_out)):
                raise RuntimeError("graph replay and eager step disagree")
            launch_mode = "cuda graph replay of one captured step"
        except Exception as exc:  # noqa: BLE001 - any refusal falls back to eager launches
            graph = None
            launch_mode = f"eager launches (graph capture refused: {type(exc).__name__})"
            torch.cuda.synchronize()
    barrier()
    e0.record()
    for _ in range(args.steps):
        if graph is not None:
            graph.replay()
        else:
            step(Q, K, V, G, dO)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = launches_per_step * args.steps
    status = _lib.device_status(local_rank)
    tms = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms_per_step = float(tms.item()) / args.steps

    # ---- end to end: pinned host inputs in, results out, every step (the library's host-tensor
    # call: head slices pipelined over copy-in / compute / copy-out streams)
    from retention_integration_b200.host import HostPipeline

    # equal two-head slices: slices of one head copy their 128-byte rows at 46 instead of 55 GB/s and launch less
    # efficiently; measured per step: 2,2,2,2 heads 7.1 ms, 1,1,2,2,2 8.0 ms, eight one-head slices 10.8 ms
    n_slices = 4 if hl % 4 == 0 else (2 if hl % 2 == 0 else 1)
    pipe = HostPipeline(b, t, hl, d, torch.bfloat16, dev, c, n_slices=n_slices)
    outs_h = {k: torch.empty(b, t, hl, d, dtype=torch.bfloat16).pin_memory() for k in ("O", "dQ", "dK", "dV")}
    outs_h["dlog_G"] = torch.empty(b, t, hl).pin_memory()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pipe.fwd_bwd(Qh, Kh, Vh, Gh, dOh, outs_h)
    barrier()
    e2.record()
    for _ in range(args.steps):
        pipe.fwd_bwd(Qh, Kh, Vh, Gh, dOh, outs_h)
    e3.record()
    barrier()
    tms2 = torch.tensor([e2.elapsed_time(e3)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tms2, op=dist.ReduceOp.MAX)
    e2e_ms = float(tms2.item()) / args.steps
    outs_h = list(outs_h.values())
    clocks = sampler.stop() if rank == 0 else None
    h2d = sum(x.numel() * x.element_size() for x in (Qh, Kh, Vh, Gh, dOh))
    d2h = sum(x.numel() * x.element_size() for x in outs_h)

    if rank == 0:
        tokens = b * t
        fl = algorithmic_flops(b, t, hl, hl, d, c)
        # algorithmic FLOPs per launch of each tensor-core kernel on this rank
        per_launch = {
            "pr_chunk_out": 2 * fl["att"] + fl["exp_q"],
            "pr_chunk_state": fl["exp_k"],          # forward (keys) and backward (queries): same count at hq = h
            "pr_expand_grad": fl["exp_q"],
            "pr_chunk_dq": 2 * fl["att"],           # dP and dQ (S is recomputed, not counted)
            "pr_chunk_dkv": 3 * fl["att"] + fl["exp_k"],  # dV, dK, one shared S/dP; plus the state path of dV
        }
        peaks = {}
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peaks = json.load(f)
        except OSError:
            pass
        peak_tf = peaks.get("bf16_tflops_sustained") or 1400.0
        peak_src = "measured (sustained)" if "bf16_tflops_sustained" in peaks else "fallback"
        breakdown = {k: {"launches": n, "ms_per_step": tot / breakdown_steps} for k, (n, tot) in kernels.items()}
        tensor_kernels = {k: v for k, v in kernels.items() if k in per_launch}
        top = max(tensor_kernels, key=lambda k: tensor_kernels[k][1])
        n_top, ms_top = tensor_kernels[top]
        achieved = per_launch[top] / (ms_top / n_top * 1e-3) / 1e12
        total_achieved = (fl["fwd"] + fl["bwd"]) / (ms_per_step * 1e-3) / 1e12
        line = {
            "metric": "fwd_bwd_tokens_per_sec", "value": tokens / (ms_per_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": (tokens / (ms_per_step * 1e-3) / PUBLISHED_TOKENS_PER_S) if t == CFG["t"] else None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"power_retention fwd+bwd b{b} t{t} h{h} d{d} deg2 chunk{c} gated bf16",
                       "baseline": "reference's published 16.8 ms/step (3.9 M tokens/s) for this shape, Triton path on one "
                                   "H100 (docs/benchmarking.md:33); other hardware, single GPU",
                       "sharding": f"kv heads split over {world} rank(s), no collective",
                       "launch": launch_mode,
                       "l2": "working set (inputs 0.34 GB + states) exceeds the 126 MB L2; no explicit flush"},
            "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d * world,
                    "d2h_bytes_per_step": d2h * world, "ms_per_step": e2e_ms},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": top, "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": achieved / peak_tf, "peak_source": peak_src,
                         "traffic": NCU_DRAM_BYTES_T8192_H8[top] * (t * hl) / (8192 * 8),
                         "traffic_source": "ncu dram bytes read+write of the t=8192 h=8 capture, scaled by tokens x heads",
                         "whole_step_achieved": total_achieved, "whole_step_frac": total_achieved / peak_tf},
            "kernels": breakdown,
            "device_status": status,
        }
        if not args.no_cpu_baseline and world == 1:
            v, dt, cores, sample = cpu_reference_run(1, 1, sample_t=8192, sample_h=1)
            line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
