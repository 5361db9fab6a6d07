#!/usr/bin/env python
"""Benchmark of the power-retention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload train|decode|seqpar|caller]

Workload `train` (default): forward + backward of one power-retention layer at
b=1, t=65536, h=8, d=64, deg=2, bf16, chunk 1024, gated (synthetic N(0,1) inputs,
log_G = logsigmoid(N(0,1))).  A step is one forward+backward pass.  With N > 1 GPUs the
kv heads are split across ranks (no collective on the data path); the reported value is
batch*tokens per second of the whole job, timed on the device, max over ranks.

The default line also carries the other parts of the metric: at N = 1 a `decode` object
(b=16, h=32, d=64: 2048-token prefill into the state, then 512 single-token steps replayed from a
CUDA graph) and a `caller_prep` object (the callers' split + gate + rotary glue at the training
shape), at N > 1 a `seq_parallel` object (b=1, t=1048576, h=8 split by sequence over the ranks,
boundary states exchanged over NCCL).  `--workload decode|seqpar|caller` prints those as lines of
their own.  A timed region that takes several times the sum of its own kernels (a stall from
outside the job) is timed once more; the line then carries both figures under `retimed`.

One JSON line is printed by rank 0.  `--impl reference` times the CPU restatement of the
reference's algorithm (oracle/) on the host cores instead.
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

import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(b=1, t=65536, h=8, d=64, deg=2, chunk=1024, dtype="bf16", gated=True)
D_EXACT = 64 * 65 // 2  # C(d+1, 2) = 2080: the algorithmic expanded dimension
WORKLOAD = "power_retention fwd+bwd b1 t65536 h8 d64 deg2 chunk1024 gated bf16"
# the CPU sample both arms time: a bounded slice of the workload above
CPU_SAMPLE = dict(t=16384, heads=2, repeats=3)


def algorithmic_flops(b, t, hq, h, d, c, D=D_EXACT):
    """Per-kernel algorithmic FLOPs (exact D, causal half counted once)."""
    att = b * hq * t * c * d  # one causal c x c x d product summed over chunks
    exp_q = 2 * b * hq * t * D * d
    exp_k = 2 * b * h * t * D * d
    return {"fwd": 2 * att + exp_q + exp_k, "bwd": 5 * att + 2 * exp_q + 2 * exp_k, "att": att, "exp_q": exp_q,
            "exp_k": exp_k}


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


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch of each tensor-core kernel, from an ncu
# capture of this benchmark at t = 65536 with two heads per launch (0.25 GB of operands per launch, twice the L2);
# traffic grows in proportion to the heads processed.  None: not captured.
NCU_DRAM_BYTES_DECODE_STATE = 147.0e6  # decode_tc_kernel, b16 h32: dram__bytes_read + write per launch
NCU_DRAM_BYTES_T65536_H2 = {"pr_expand_grad": 86.2e6, "pr_chunk_dkv": 187.2e6, "pr_chunk_out": 105.4e6,
                            "pr_chunk_state": 55.8e6, "pr_chunk_dq": 110.1e6}

# the reference's only published figure for this exact metric and shape: 16.8 ms per fwd+bwd step on one H100
PUBLISHED_TOKENS_PER_S = 65536 / 16.8e-3


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f)
    except OSError:
        return {}


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


# --------------------------------------------------------------------------- CPU legs
def cpu_sample_run(repeats=CPU_SAMPLE["repeats"], sample_t=CPU_SAMPLE["t"], sample_h=CPU_SAMPLE["heads"]):
    """Times the CPU restatement of the reference (oracle/) on a bounded sample of the workload:
    sample_t tokens of sample_h heads, forward+backward in bf16, all host threads; one untimed
    warm-up, then the median of `repeats` runs.  Both arms of the benchmark call this with the
    same arguments, so their figures are directly comparable."""
    from oracle import power_retention_oracle as oracle

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    Q, K, V, G, dO = make_inputs(CFG["b"], sample_t, CFG["h"], CFG["d"], "cpu", heads=range(sample_h))

    def step():
        q, k, v = (x.clone().requires_grad_(True) for x in (Q, K, V))
        g = G.clone().requires_grad_(True)
        O = oracle.power_retention(q, k, v, g, deg=2, chunk_size=CFG["chunk"])
        O.backward(dO)

    step()
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    dt = statistics.median(times)
    # tokens/s of the full-width (h heads) layer: the sample's token rate scaled by the share of heads it holds
    value = CFG["b"] * sample_t / dt * (sample_h / CFG["h"])
    sample = (f"oracle port of retention/reference.py, fwd+bwd, bf16, t={sample_t} tokens x {sample_h} of "
              f"{CFG['h']} heads, chunk {CFG['chunk']}; median of {repeats} after one warm-up; token rate scaled by "
              f"the share of heads")
    return {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample,
            "seconds_per_sample": dt, "spread": [min(times), max(times)]}


def cpu_config1_run():
    """The reference's own CPU-runnable case exactly: forward only, fp32, b1 t1024 h4 d64 deg2 chunk 128,
    gated; median of 5 after one warm-up."""
    from oracle import power_retention_oracle as oracle

    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(0)
    Q, K, V = (torch.randn(1, 1024, 4, 64, generator=g) for _ in range(3))
    G = F.logsigmoid(torch.randn(1, 1024, 4, generator=g))
    with torch.no_grad():
        oracle.power_retention(Q, K, V, G, deg=2, chunk_size=128)
        times = []
        for _ in range(5):
            t0 = time.perf_counter()
            oracle.power_retention(Q, K, V, G, deg=2, chunk_size=128)
            times.append(time.perf_counter() - t0)
    dt = statistics.median(times)
    return {"workload": "forward fp32 b1 t1024 h4 d64 deg2 chunk128 gated", "seconds": dt, "tokens_per_s": 1024 / dt,
            "repeats": 5}


def run_reference(args, rank):
    if rank != 0:
        return
    base = cpu_sample_run()
    base["config1"] = cpu_config1_run()
    line = {
        "impl": "reference", "metric": "fwd_bwd_tokens_per_sec", "value": base["value"], "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": CPU_SAMPLE["repeats"], "warmup": 1, "ms_per_step": base["seconds_per_sample"] * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- decode
def decode_measure(dev, steps=512, with_extras=True, use_graph=True):
    """Inference workload: b=16, h=32, d=64 bf16 gated; a 2048-token prefill compressed into the
    state (switch_over 1024), then `steps` single-token steps whose cache grows from 1 to `steps`
    tokens (the reference's semantics: the caller's cache grows until the next switch-over).
    Returns the `decode` object of the benchmark line."""
    import retention_integration_b200 as prb
    from retention_integration_b200 import _lib, ops
    from retention_integration_b200.cache import RetentionCache

    b, h, d, t0 = 16, 32, 64, 2048
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
        y = None
        for i in range(steps):
            y = prb.power_retention_inference(Qs[:, i:i + 1], Kc[:, :i + 1], Vc[:, :i + 1], lgc[:, :i + 1], state, sk,
                                              switch_over_seq_len=1024)[0]
        return y

    def timed_ms(fn, reps=1):
        """Device time of `fn()`, replayed from a CUDA graph when `use_graph` (a serving loop replays its token
        loop the same way: the Python launch code costs about as much as the 30 us kernel), else launched eagerly."""
        y_ref = fn()
        torch.cuda.synchronize()
        graph = None
        if use_graph:
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    y_g = fn()
                graph.replay()
                torch.cuda.synchronize()
                if y_ref is not None and not torch.equal(y_g, y_ref):
                    raise RuntimeError("graph replay and eager launches disagree")
            except Exception:  # noqa: BLE001 - any refusal falls back to eager launches
                graph = None
                torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            graph.replay() if graph is not None else fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps, graph is not None

    ops.launch_log.reset(timing=False)
    decode_all()
    torch.cuda.synchronize()
    launches = ops.launch_log.count
    ms, replayed = timed_ms(decode_all)
    peaks = load_peaks()
    peak = peaks.get("hbm_gbs") or 6650.0
    state_bytes = state.numel() * 2 + sk.numel() * 4
    # algorithmic bytes of the average step: the state and its normaliser once, plus the cached keys and values
    avg_tk = (steps + 1) / 2
    step_bytes = state_bytes + 2 * b * avg_tk * h * d * 2
    step_gbs = step_bytes / (ms / steps * 1e-3) / 1e9
    out = {
        "metric": "decode_tokens_per_sec", "value": b * steps / (ms * 1e-3), "unit": "tokens/s", "steps": steps,
        "ms_per_step": ms / steps,
        "workload": f"power_retention_inference decode b16 h32 d64 bf16 gated, state [16,32,2080,64], cache 1..{steps}",
        "prefill_to_state_ms": prefill_ms, "gpu_launches": launches,
        "launch": f"cuda graph replay of the {steps} captured steps" if replayed else "eager launches",
        "roofline": {"bound": "hbm", "kernel": "decode step (one kernel)", "achieved": step_gbs, "peak": peak,
                     "unit": "GB/s", "frac": step_gbs / peak,
                     "peak_source": "measured" if "hbm_gbs" in peaks else "fallback",
                     "algorithmic_bytes_per_step": step_bytes, "state_bytes": state_bytes,
                     "traffic": NCU_DRAM_BYTES_DECODE_STATE + (step_bytes - state_bytes),
                     "traffic_source": "ncu dram bytes read+write of one launch with 5-8 cached tokens (147 MB for "
                                       "141 MB of state), plus the algorithmic bytes of the average step's cache"},
    }
    if with_extras:
        # the same step with an empty cache: the state read alone, launches queued back to back
        qd = Qs[:, :1].contiguous()
        n_state = 100

        def state_only():
            y = None
            for _ in range(n_state):
                y = prb.power_retention_inference(qd, None, None, None, state, sk)[0]
            return y

        ms_state = timed_ms(state_only)[0] / n_state
        out["state_read"] = {"ms": ms_state, "achieved_gbs": state_bytes / (ms_state * 1e-3) / 1e9,
                             "frac": state_bytes / (ms_state * 1e-3) / 1e9 / peak}
        # pure-recurrent mode: the state is advanced and read once per token (read + write of the state)
        cache = RetentionCache(b, h, d, torch.bfloat16, dev, recurrent=True)
        cache.update_state(state.clone(), sk.clone())
        def recurrent_all():
            for i in range(steps):
                cache.decode(Qs[:, i:i + 1], Kc[:, i:i + 1], Vc[:, i:i + 1], lgc[:, i:i + 1])

        ms_rec = timed_ms(recurrent_all)[0] / steps
        out["recurrent"] = {"tokens_per_s": b / (ms_rec * 1e-3), "ms_per_step": ms_rec,
                            "achieved_gbs": 2 * state_bytes / (ms_rec * 1e-3) / 1e9,
                            "frac": 2 * state_bytes / (ms_rec * 1e-3) / 1e9 / peak}
        # end to end through the cache object: each step's q, k, v, gate come from pinned host memory and its
        # output goes back to the host (the token loop of a server: one synchronisation per generated token)
        cache = RetentionCache(b, h, d, torch.bfloat16, dev, capacity=steps, switch_over_seq_len=1024)
        cache.update_state(state, sk)
        hq_, hk_, hv_ = (x.cpu().pin_memory() for x in (Qs, Kc, Vc))
        hg_ = lgc.cpu().pin_memory()
        yh = torch.empty(b, 1, h, d, dtype=torch.bfloat16).pin_memory()
        n_e2e = min(steps, 128)
        t_start = time.perf_counter()
        for i in range(n_e2e):
            q, k, v, lg = (x[:, i:i + 1].to(dev, non_blocking=True) for x in (hq_, hk_, hv_, hg_))
            y = cache.decode(q, k, v, lg)
            yh.copy_(y, non_blocking=True)
            torch.cuda.synchronize()
        dt = (time.perf_counter() - t_start) / n_e2e
        out["e2e"] = {"value": b / dt, "unit": "tokens/s", "ms_per_step": dt * 1e3,
                      "h2d_bytes_per_step": 3 * b * h * d * 2 + b * h * 4, "d2h_bytes_per_step": b * h * d * 2,
                      "steps": n_e2e}
    out["device_status"] = _lib.device_status(dev.index or 0)
    return out


# --------------------------------------------------------------------------- caller glue
def caller_prep_measure(dev, t=65536, h=8, d=64):
    """The fused split + gate + rotary + layout write between the projection and the operator
    (retention_integration_b200/caller.py) at the benchmark's shape, forward and gradient, against the
    same glue written as the reference's callers write it (torch elementwise ops, deploy/nanoGPT/model.py:66-84)
    on the same GPU.  HBM bound: bytes = projection output read + Q, K, V, log_g written (and the reverse)."""
    import retention_integration_b200 as prb
    from retention_integration_b200 import ops

    b, W = 1, 3 * h * d + h
    gen = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn(b, t, W, generator=gen, device=dev).bfloat16()
    sin, cos = prb.rotary_tables(t, d, dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn, reps=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    Q, K, V, lg = ops.caller_prep_fwd(x, cos, sin, h, h, d, True, prb.caller.GATE_BIAS, False)
    dlg = torch.randn_like(lg)
    ms_f = timed(lambda: ops.caller_prep_fwd(x, cos, sin, h, h, d, True, prb.caller.GATE_BIAS, False))
    ms_b = timed(lambda: ops.caller_prep_bwd(x, cos, sin, h, h, d, True, prb.caller.GATE_BIAS, False, Q, K, V, dlg))

    def unfused():
        q, k, v = x[..., : 3 * h * d].split([h * d, h * d, h * d], dim=2)
        q, k, v = q.view(b, t, h, d), k.view(b, t, h, d), v.view(b, t, h, d)
        g = F.logsigmoid(prb.caller.GATE_BIAS + x[..., 3 * h * d:].float()).contiguous()
        s2, c2 = sin.repeat_interleave(2, dim=1)[None, :, None], cos.repeat_interleave(2, dim=1)[None, :, None]
        rot = lambda z: torch.stack((-z[..., 1::2], z[..., ::2]), -1).reshape(z.shape)
        q = ((q * c2) + (rot(q) * s2)).to(x.dtype)
        k = ((k * c2) + (rot(k) * s2)).to(x.dtype)
        return q.contiguous(), k.contiguous(), v.contiguous(), g

    ms_u = timed(unfused, reps=5)
    peak = load_peaks().get("hbm_gbs") or 6650.0
    bytes_f = b * t * (W * 2 + 3 * h * d * 2 + h * 4)
    bytes_b = b * t * (3 * h * d * 2 + h * 4 + h * 2 + W * 2)  # gradients in, the gate column re-read, dqkvg out
    return {"workload": f"split + logsigmoid gate + rotary + layout write, b{b} t{t} h{h} d{d} bf16 gated",
            "fwd_ms": ms_f, "fwd_gbs": bytes_f / (ms_f * 1e-3) / 1e9, "fwd_frac_of_hbm_peak": bytes_f / (ms_f * 1e-3) / 1e9 / peak,
            "bwd_ms": ms_b, "bwd_gbs": bytes_b / (ms_b * 1e-3) / 1e9, "bwd_frac_of_hbm_peak": bytes_b / (ms_b * 1e-3) / 1e9 / peak,
            "unfused_torch_fwd_ms": ms_u, "algorithmic_bytes_fwd": bytes_f}


# --------------------------------------------------------------------------- sequence parallel
def seqpar_measure(dev, rank, world, t_total, steps=3, warmup=1):
    """b=1, t=t_total, h=8, d=64 bf16, chunk 1024, slow-decay gates, the sequence split evenly over the ranks
    (rank order = sequence order); forward+backward with the boundary states exchanged over NCCL.
    Returns the `seq_parallel` object (identical on every rank; rank 0 prints it)."""
    import torch.distributed as dist

    from retention_integration_b200 import parallel

    b, h, d, c = 1, CFG["h"], CFG["d"], CFG["chunk"]
    tl = t_total // world
    gen = torch.Generator(device=dev).manual_seed(1000 + rank)
    mk = lambda *s: torch.randn(*s, generator=gen, device=dev)
    Q, K, V, dO = (mk(b, tl, h, d).bfloat16() for _ in range(4))
    G = F.logsigmoid(mk(b, tl, h) + 2.0)
    comm = parallel.DistComm()

    def step():
        q, k, v = (x.detach().requires_grad_(True) for x in (Q, K, V))
        g = G.detach().requires_grad_(True)
        O = parallel.power_retention_sequence_parallel(q, k, v, g, deg=2, chunk_size=c, comm=comm)
        O.backward(dO)

    for _ in range(warmup):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    tms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms = float(tms.item()) / steps
    fl = algorithmic_flops(b, t_total, h, h, d, c)
    peaks = load_peaks()
    peak_tf = peaks.get("bf16_tflops") or 1590.0
    tf = (fl["fwd"] + fl["bwd"]) / (ms * 1e-3) / 1e12
    return {"metric": "fwd_bwd_tokens_per_sec", "value": b * t_total / (ms * 1e-3), "unit": "tokens/s",
            "ms_per_step": ms, "steps": steps, "n_gpus": world,
            "workload": f"power_retention fwd+bwd b1 t{t_total} h8 d64 deg2 chunk1024 bf16, "
                        f"log_G = logsigmoid(N(0,1)+2), sequence split over {world} ranks",
            "exchange": "one all-gather of per-rank boundary summaries (fp32 state + Gram + gate sums) per direction",
            "whole_job_tflops": tf, "frac_of_all_gpus_peak": tf / (peak_tf * world)}


# --------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--t", type=int, default=CFG["t"], help="sequence length override (profiling small cases)")
    ap.add_argument("--heads", type=int, default=CFG["h"], help="kv heads override (profiling small cases)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the decode / seq_parallel objects and e2e")
    ap.add_argument("--no-graph", action="store_true", help="launch the timed steps eagerly instead of replaying a graph")
    ap.add_argument("--workload", default="train", choices=["train", "decode", "seqpar", "caller"])
    ap.add_argument("--decode-steps", type=int, default=512, help="single-token steps of the decode workload")
    ap.add_argument("--seq-t", type=int, default=1048576, help="total tokens of the sequence-parallel workload")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
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

    if args.workload == "decode":
        if rank == 0:
            obj = decode_measure(dev, args.decode_steps, use_graph=not args.no_graph)
            obj.update({"n_gpus": 1, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                        "config": {"workload": obj["workload"]}})
            print(json.dumps(obj), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    if args.workload == "caller":
        if rank == 0:
            obj = caller_prep_measure(dev)
            obj.update({"metric": "caller_prep_gbs", "value": obj["fwd_gbs"], "unit": "GB/s", "n_gpus": 1,
                        "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                        "config": {"workload": obj["workload"]}})
            print(json.dumps(obj), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    if args.workload == "seqpar":
        if world < 2:
            raise SystemExit("the sequence-parallel workload needs at least 2 ranks")
        obj = seqpar_measure(dev, rank, world, args.seq_t, steps=max(1, min(args.steps, 5)))
        if rank == 0:
            obj.update({"higher_is_better": True, "dtype": "bf16", "data": "synthetic", "scaling": "strong",
                        "config": {"workload": obj["workload"]}})
            print(json.dumps(obj), flush=True)
        dist.destroy_process_group()
        return

    b, t, h, d, c = CFG["b"], args.t, args.heads, CFG["d"], CFG["chunk"]
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
    from retention_integration_b200 import retention as _ret

    ops.launch_log.reset(timing=True)
    _ret.NATIVE_SEQUENCER = False  # kernel by kernel from Python for this pass: one event pair per launch
    for _ in range(min(args.steps, 3)):
        step(Q, K, V, G, dO)
    barrier()
    _ret.NATIVE_SEQUENCER = True
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
    def timed_region():
        barrier()
        e0.record()
        for _ in range(args.steps):
            if graph is not None:
                graph.replay()
            else:
                step(Q, K, V, G, dO)
        e1.record()
        barrier()
        tms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        return float(tms.item())

    timed_region_ms = timed_region()
    # A stall from outside the job (a neighbour on the shared host, children of an earlier command still
    # exiting) shows as a region several times longer than the sum of its own kernels, which the breakdown
    # pass has just measured.  Such a region is timed once more and both figures are reported.
    retimed_from = None
    ksum = torch.tensor([sum(tot for _, tot in kernels.values()) / breakdown_steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ksum, op=dist.ReduceOp.MAX)  # every rank takes the same decision
    kernel_sum_ms = float(ksum.item())
    if timed_region_ms / args.steps > 3.0 * kernel_sum_ms:
        retimed_from = timed_region_ms / args.steps
        timed_region_ms = timed_region()
    launches = launches_per_step * args.steps
    status = _lib.device_status(local_rank)
    ms_per_step = timed_region_ms / args.steps

    # ---- end to end: pinned host inputs in, results out, every step (the library's host-tensor
    # call: head slices pipelined over copy-in / compute / copy-out streams)
    e2e = None
    if not args.no_extras:
        from retention_integration_b200.host import HostPipeline

        # equal two-head slices measured fastest at eight heads per GPU (one-head slices copy their 128-byte rows
        # less efficiently and launch more kernels)
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
        h2d = sum(x.numel() * x.element_size() for x in (Qh, Kh, Vh, Gh, dOh))
        d2h = sum(x.numel() * x.element_size() for x in outs_h.values())
        e2e = {"value": b * t / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d * world,
               "d2h_bytes_per_step": d2h * world, "ms_per_step": e2e_ms}
        del pipe, outs_h
    clocks = sampler.stop() if rank == 0 else None

    # ---- the other parts of the metric ride on the default line
    extra = {}
    if not args.no_extras and t == CFG["t"] and h == CFG["h"]:
        del Q, K, V, G, dO, graph
        torch.cuda.empty_cache()
        if world == 1:
            extra["decode"] = decode_measure(dev, args.decode_steps, use_graph=not args.no_graph)
            extra["caller_prep"] = caller_prep_measure(dev)
        else:
            extra["seq_parallel"] = seqpar_measure(dev, rank, world, args.seq_t)

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
        # algorithmic bytes per launch of the bandwidth-bound scans: the exact state (2080 rows) and its normaliser
        n = t // c
        scan_unit = b * n * hl * (D_EXACT * d * 2 + D_EXACT * 4)
        per_launch_bytes = {"pr_discumsum_fwd": 2 * scan_unit, "pr_discumsum_bwd": 3 * scan_unit}
        peaks = load_peaks()
        burst = peaks.get("bf16_tflops") or 1590.0
        sustained = peaks.get("bf16_tflops_sustained") or 1400.0
        hbm = peaks.get("hbm_gbs") or 6650.0
        src = "measured" if "bf16_tflops" in peaks else "fallback"
        breakdown = {}
        for k, (nl, tot) in kernels.items():
            per = tot / nl
            entry = {"launches": nl // breakdown_steps, "ms_per_launch": per, "ms_per_step": tot / breakdown_steps}
            if k in per_launch:
                entry["tflops"] = per_launch[k] / (per * 1e-3) / 1e12
                entry["frac_of_burst_peak"] = entry["tflops"] / burst
            if k in per_launch_bytes:
                entry["gbs"] = per_launch_bytes[k] / (per * 1e-3) / 1e9
                entry["frac_of_hbm_peak"] = entry["gbs"] / hbm
            breakdown[k] = entry
        tensor_kernels = {k: v for k, v in kernels.items() if k in per_launch}
        top = max(tensor_kernels, key=lambda k: tensor_kernels[k][1])
        achieved = breakdown[top]["tflops"]
        total_achieved = (fl["fwd"] + fl["bwd"]) / (ms_per_step * 1e-3) / 1e12
        traffic = NCU_DRAM_BYTES_T65536_H2.get(top)
        roofline = {"bound": "tensor", "kernel": top, "achieved": achieved, "peak": burst, "unit": "TFLOP/s",
                    "frac": achieved / burst,
                    "peak_source": f"{src}: burst figure, the per-kernel pass is a few ms at full clock",
                    "traffic": traffic * hl / 2 if (traffic and t == CFG["t"]) else None,
                    "traffic_source": "ncu dram bytes read+write of one launch at t=65536 with 2 heads, scaled by heads"
                                      if traffic else "not captured",
                    "whole_step_achieved": total_achieved, "whole_step_frac_of_burst": total_achieved / burst}
        if timed_region_ms >= 1000.0:
            roofline["whole_step_frac_of_sustained"] = total_achieved / sustained
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
            "e2e": e2e,
            "gpu_launches": launches,
            **({"retimed": {"first_region_ms_per_step": retimed_from,
                            "why": "first timed region took over 3x the sum of its kernels; timed once more"}}
               if retimed_from is not None else {}),
            "clocks": clocks,
            "roofline": roofline,
            "kernels": breakdown,
            "device_status": status,
        }
        line.update(extra)
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_sample_run()
            line["cpu_baseline"]["config1"] = cpu_config1_run()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
