#!/usr/bin/env python
"""Benchmark of the litnicelm token loop on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload c2]

Metric: generated tokens/s (greedy decode). One "step" is one complete
generation of the workload: for the default workload `c2` a 256-token Zipf
prompt followed by 768 greedy tokens at batch 1 on the 6-layer / 512-wide /
vocab-96 model, every token recomputing its whole context as the reference
does (no KV cache). With N GPUs each rank decodes its own independent stream
(weak scaling, no collective on the data path); rank 0 prints one JSON line.

`--impl reference` times the reference's own CPU backend (oracle/_ref, built
from the reference sources) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from litnicelm_b200 import formats  # noqa: E402

WORKLOADS = {
    # name: (dims key, streams per GPU, prompt_len, max_new, temp, top_k, top_p, config index)
    "c1": ("c1", 1, 6, 58, 0.0, 0, 1.0, 1),
    "c2": ("c2", 1, 256, 768, 0.0, 0, 1.0, 2),
    "c3": ("c3", 64, 128, 512, 0.8, 40, 0.95, 3),
    "c5": ("c5", 512, 256, 256, 0.0, 0, 1.0, 5),
}


def algorithmic_flops(d: formats.ModelDims, streams: int, s: int) -> float:
    """Flops of one forward step at context s: projections on every row,
    causal-useful attention, output head on the last row only."""
    D, F, L, V = d.d_model, d.d_ff, d.n_layers, d.vocab
    return streams * (2.0 * s * L * (4 * D * D + 2 * D * F) + 2.0 * L * s * (s + 1) * D + 2.0 * D * V)


def reference_flops(d: formats.ModelDims, s: int) -> float:
    """Flops the reference CPU backend executes for one forward at context s:
    full (not causal) s x s score and context products per head and the output
    head on all rows (device_backend.cpp:1112-1235, output_head.cpp:70)."""
    D, F, L, V = d.d_model, d.d_ff, d.n_layers, d.vocab
    return 2.0 * s * L * (4 * D * D + 2 * D * F) + 4.0 * L * s * s * D + 2.0 * s * D * V


# dram__bytes_read.sum + dram__bytes_write.sum per projection launch from the ncu
# capture summarised under profiles/ (mean over the four projections of a layer).
NCU_DRAM_BYTES_PER_GEMM_LAUNCH = {"c2": 6.4e6}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def make_inputs(workload: str, rank: int):
    key, streams, plen, max_new, temp, top_k, top_p, cidx = WORKLOADS[workload]
    d = formats.CONFIG_DIMS[key]
    arena = formats.make_param_arena(d, 1000 + cidx)
    prompts = np.stack([formats.zipf_prompt(d.vocab, plen, 2000 * cidx + rank * streams + i)
                        for i in range(streams)])
    seeds = np.array([3000 + rank * streams + i for i in range(streams)], dtype=np.uint32)
    return d, arena, prompts, seeds, (streams, plen, max_new, temp, top_k, top_p)


def time_reference_sample(d, arena, prompt, seq_lens, concurrent=1):
    """Times the reference CPU backend (oracle/_ref/ref_driver, unmodified
    reference model code) on single forwards at the given context lengths.
    `concurrent` copies run side by side (independent streams on separate host
    cores; the reference itself is single-threaded) and the slowest one counts.
    Returns [(s, seconds)]."""
    from oracle import binding as ob
    if not ob.have_ref():
        raise RuntimeError("oracle/_ref is missing (build it where the reference sources are)")
    out = []
    with tempfile.TemporaryDirectory() as tmp:
        ckpt = os.path.join(tmp, "m.ckpt")
        formats.write_checkpoint(ckpt, d, arena)
        yaml = os.path.join(tmp, "c.yaml")
        formats.write_yaml(yaml, d, backend_library=ob.REF_CPU_PLUGIN, checkpoint=ckpt,
                           attention="fused_inplace", ffn="inplace_fused_bias_relu")
        for s in seq_lens:
            idp = os.path.join(tmp, f"ids{s}.i32")
            np.ascontiguousarray(prompt[:s], np.int32).tofile(idp)
            procs = [subprocess.Popen([ob.REF_DRIVER, "--config", yaml, "--vocab", str(d.vocab), "--ids", idp,
                                       "--mode", "forward", "--out", os.path.join(tmp, f"o{c}.f32")],
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
                     for c in range(concurrent)]
            worst = 0.0
            for p in procs:
                so, se = p.communicate()
                if p.returncode != 0:
                    raise RuntimeError("ref_driver failed: " + se[-500:])
                info = json.loads([ln for ln in so.splitlines() if ln.startswith("{")][-1])
                worst = max(worst, float(info["seconds"]))
            out.append((s, worst))
    return out


def extrapolate_reference_tokens_per_s(d, samples, plen, max_new):
    """The reference executes reference_flops(s) per generated token; its cost
    per flop is taken from the timed forwards and applied to the whole schedule
    s = plen .. plen+max_new-1."""
    flops = sum(reference_flops(d, s) for s, _ in samples)
    secs = sum(t for _, t in samples)
    per_flop = secs / flops
    total = sum(reference_flops(d, s) for s in range(plen, plen + max_new)) * per_flop
    return max_new / total, per_flop


def run_reference_arm(args, rank, world):
    """Reference arm: the reference's own single-threaded CPU backend, each step
    a bounded sample (two forwards) of the same workload."""
    if rank != 0:
        return
    d, arena, prompts, seeds, (streams, plen, max_new, temp, top_k, top_p) = make_inputs(args.workload, 0)
    full = np.concatenate([prompts[0], formats.zipf_prompt(d.vocab, d.max_seq, 999)])[:d.max_seq]
    sample_lens = [16, 48] if d.d_model >= 512 else [min(d.max_seq, 24), min(d.max_seq, 56)]
    # With N GPUs the workload is N independent replicas; the CPU arm runs as
    # many of them side by side as it has cores for.
    conc = max(1, min(world, os.cpu_count() or 1))
    for _ in range(args.warmup):
        time_reference_sample(d, arena, full, sample_lens[:1], conc)
    t0 = time.time()
    rates = []
    for _ in range(args.steps):
        samples = time_reference_sample(d, arena, full, sample_lens, conc)
        r, _ = extrapolate_reference_tokens_per_s(d, samples, plen, max_new)
        rates.append(r * streams * conc)
    wall = time.time() - t0
    value = statistics.mean(rates)
    sample = (f"per step: single reference forwards at context {sample_lens} of the workload's model, "
              f"cost per executed flop applied to the schedule s={plen}..{plen + max_new - 1} "
              "(extrapolated from subsample)")
    line = {
        "impl": "reference", "metric": "generated tokens/s (greedy decode)", "value": value,
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * wall / max(1, args.steps), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args.workload, streams, plen, max_new), "l2": "not applicable (CPU)"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": conc, "kind": "reference", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_name(workload, streams, plen, max_new):
    d = formats.CONFIG_DIMS[WORKLOADS[workload][0]]
    return (f"{workload}: L{d.n_layers} H{d.n_heads} D{d.d_model} F{d.d_ff} V{d.vocab} S{d.max_seq}, "
            f"{streams} stream(s)/GPU, {plen}-token Zipf(1.1) prompt, {max_new} new tokens, "
            "whole-context recomputation per token")


def run_b200_arm(args, rank, local_rank, world):
    import torch
    from litnicelm_b200.plugin import Session

    os.environ["LITNICE_B200_DEVICE"] = str(local_rank)
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    d, arena, prompts, seeds, (streams, plen, max_new, temp, top_k, top_p) = make_inputs(args.workload, rank)
    peaks = load_peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # larger than the 126 MB L2

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sess = Session(d, streams)
    sess.load_params(arena)
    pinned_prompts = torch.from_numpy(prompts.copy()).pin_memory()
    pinned_out = torch.zeros((streams, max_new), dtype=torch.int32).pin_memory()

    # ---- device-resident pass: prompts already in HBM when the clock starts ----
    for _ in range(args.warmup):
        sess.upload_prompts(prompts, seeds)
        sess.run(max_new, temp, top_k, top_p)
    clocks = ClockSampler(local_rank)
    barrier()
    if rank == 0:
        clocks.start()
    dev_ms, launches, tokens = 0.0, 0, 0
    t0 = time.perf_counter()
    for _ in range(args.steps):
        flush.fill_(1)
        torch.cuda.synchronize()
        sess.upload_prompts(prompts, seeds)          # untimed: not inside the event bracket
        produced = sess.run(max_new, temp, top_k, top_p)
        st = sess.stats()
        dev_ms += st.device_ms
        launches += st.kernel_launches
        tokens += st.tokens
    barrier()
    wall_s = time.perf_counter() - t0
    clock_info = clocks.stop() if rank == 0 else None
    dev_ms = max_over_ranks(dev_ms)
    value = world * tokens / (dev_ms * 1e-3)

    # ---- end-to-end pass: host buffers in, host buffers out, copies inside the clock ----
    import ctypes as C
    from litnicelm_b200.plugin import B200Sampling
    sp = B200Sampling(temp, top_k, top_p)
    count = C.c_int32(0)
    i32p = C.POINTER(C.c_int32)
    seeds_p = seeds.ctypes.data_as(C.POINTER(C.c_uint32))

    def e2e_once():
        rc = sess.lib.litnice_b200_generate(sess.h, C.cast(pinned_prompts.data_ptr(), i32p), streams, plen,
                                            max_new, C.byref(sp), seeds_p,
                                            C.cast(pinned_out.data_ptr(), i32p), C.byref(count))
        if rc != 0:
            raise RuntimeError(sess.lib.litnice_b200_last_error(sess.h).decode())

    e2e_once()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        flush.fill_(1)
        torch.cuda.synchronize()
        e2e_once()
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    st = sess.stats()
    e2e_value = world * args.steps * streams * count.value / e2e_s
    first_tokens = pinned_out[0, :8].tolist()

    line = None
    if rank == 0:
        # ---- roofline of the dominant kernel (the projection GEMM), events per launch ----
        s_mid = plen + max_new // 2
        prof = sess.profile_step(streams, s_mid, 3)
        gemm_tflops = prof.gemm_flops / (prof.gemm_ms * 1e-3) / 1e12 if prof.gemm_ms > 0 else 0.0
        roofline = {
            "bound": "tensor", "kernel": "projection GEMM (gemm_tc_kernel: tcgen05 + TMEM, three products of fp16 pairs)",
            "achieved": gemm_tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
            "frac": gemm_tflops / peaks["bf16_tflops"], "peak_source": f"bf16 burst, {peaks['source']}",
            # fp32-grade products execute three fp16 MMAs (22-bit operand pairs) per algorithmic
            # flop, so algorithmic flops cannot exceed 1/3 of the dense 16-bit peak
            "ceiling_frac_3_products": 1.0 / 3.0,
            "traffic": NCU_DRAM_BYTES_PER_GEMM_LAUNCH.get(args.workload),
            "note": (f"algorithmic 2*M*N*K flops of {prof.gemm_launches} launches at context {s_mid} / "
                     f"{prof.gemm_ms:.3f} ms (CUDA events around each launch on the session stream); "
                     f"attention: {prof.attn_launches} launches, {prof.attn_ms:.3f} ms"),
        }
        # The same kernel where the path's definition puts it on the tensor roofline (many rows): the
        # QKV projection of the config-4/5 model on 16 384 rows, warm, back to back.
        try:
            from litnicelm_b200.plugin import projection_time
            m_big, k_big, n_big = 16384, 1024, 3072
            us = projection_time(m_big, k_big, n_big, repeats=20, engine=2)
            big = 2.0 * m_big * k_big * n_big / (us * 1e-6) / 1e12
            roofline["at_scale"] = {"shape_mkn": [m_big, k_big, n_big], "us_per_launch": us, "achieved": big,
                                    "frac": big / peaks["bf16_tflops"],
                                    "frac_of_3_product_ceiling": 3.0 * big / peaks["bf16_tflops"]}
        except Exception as e:
            roofline["at_scale"] = {"unavailable": str(e)}
        # ---- CPU baseline: the reference itself on a bounded sample ----
        cpu = None
        if not args.no_cpu_baseline:
            try:
                full = np.concatenate([prompts[0], formats.zipf_prompt(d.vocab, d.max_seq, 999)])[:d.max_seq]
                lens = [32, 96] if d.d_model >= 512 else [min(d.max_seq, 24), min(d.max_seq, 56)]
                samples = time_reference_sample(d, arena, full, lens)
                rate, per_flop = extrapolate_reference_tokens_per_s(d, samples, plen, max_new)
                cpu = {"value": rate * streams, "unit": "tokens/s", "cores": 1, "kind": "reference",
                       "host_cores_present": os.cpu_count(),
                       "sample": (f"reference CPU backend, single forwards at context {lens} "
                                  f"({', '.join(f'{t:.2f}s' for _, t in samples)}); {per_flop * 1e9:.3f} ns per "
                                  "executed flop applied to the full schedule (extrapolated from subsample)")}
            except Exception as e:  # the bench line must still be printed
                cpu = {"value": None, "unit": "tokens/s", "cores": 1, "kind": "reference",
                       "sample": f"unavailable: {e}"}
        line = {
            "metric": "generated tokens/s (greedy decode)", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(args.workload, streams, plen, max_new),
                       "l2": "256 MB buffer written between timed steps (L2 flush)",
                       "sampling": {"temp": temp, "top_k": top_k, "top_p": top_p}},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": int(st.h2d_bytes),
                    "d2h_bytes_per_step": int(st.d2h_bytes)},
            "gpu_launches": int(launches),
            "roofline": roofline, "cpu_baseline": cpu, "clocks": clock_info,
            "wall_s_timed_region": wall_s, "first_tokens": first_tokens,
        }
    sess.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)


def run_prefill_arm(args, rank, local_rank, world):
    """Config 4: 32 sequences of 2048 tokens per GPU, one whole-context forward
    each, output = the full next-token distribution per sequence
    (inspect_distribution of the reference, inference.cpp:298-359). A step is one
    such batch; the value is sequences per second."""
    import torch
    from litnicelm_b200.plugin import Session

    os.environ["LITNICE_B200_DEVICE"] = str(local_rank)
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    d = formats.CONFIG_DIMS["c5"]
    streams, s_len = 32, d.max_seq
    arena = formats.make_param_arena(d, 1004)
    ids = np.stack([formats.zipf_prompt(d.vocab, s_len, 2000 * 4 + rank * streams + i) for i in range(streams)])
    peaks = load_peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sess = Session(d, streams)
    sess.load_params(arena)
    for _ in range(args.warmup):
        sess.inspect(ids)
    clocks = ClockSampler(local_rank)
    barrier()
    if rank == 0:
        clocks.start()
    dev_ms, launches, e2e_s = 0.0, 0, 0.0
    for _ in range(args.steps):
        flush.fill_(1)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        probs = sess.inspect(ids)               # host ids in, host probabilities out
        e2e_s += time.perf_counter() - t0
        st = sess.stats()
        dev_ms += st.device_ms                  # CUDA events around the forward, ids already on the device
        launches += st.kernel_launches
    barrier()
    clock_info = clocks.stop() if rank == 0 else None
    dev_ms = max_over_ranks(dev_ms)
    e2e_s = max_over_ranks(e2e_s)
    if rank == 0:
        flops = algorithmic_flops(d, streams, s_len) * args.steps
        tflops = flops / (dev_ms * 1e-3) / 1e12
        line = {
            "metric": "prefill sequences/s (whole-context forward, full next-token distribution)",
            "value": world * streams * args.steps / (dev_ms * 1e-3), "unit": "sequences/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": (f"c4: L{d.n_layers} H{d.n_heads} D{d.d_model} F{d.d_ff} V{d.vocab} S{d.max_seq}, "
                                    f"{streams} sequences of {s_len} tokens per GPU"),
                       "l2": "256 MB buffer written between timed steps (L2 flush)"},
            "e2e": {"value": world * streams * args.steps / e2e_s, "unit": "sequences/s",
                    "h2d_bytes_per_step": int(ids.nbytes), "d2h_bytes_per_step": int(probs.nbytes)},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "kernel": "whole forward (projections + attention)", "achieved": tflops,
                         "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": tflops / peaks["bf16_tflops"],
                         "peak_source": f"bf16 burst, {peaks['source']}", "ceiling_frac_3_products": 1.0 / 3.0,
                         "traffic": None,
                         "note": "algorithmic flops of the step (projections on all rows, causal-useful attention, "
                                 "head on the last rows) / device time of the step"},
            "cpu_baseline": None, "clocks": clock_info,
            "probability_row_sums": [float(probs[0].sum()), float(probs[-1].sum())],
        }
        print(json.dumps(line), flush=True)
    sess.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + ["c4"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        if args.workload == "c4":
            ap.error("the prefill workload c4 has no reference arm; use c1, c2, c3 or c5")
        run_reference_arm(args, rank, world)
        return
    if args.warmup < 3:
        args.warmup = 3
    if args.workload == "c4":
        run_prefill_arm(args, rank, local_rank, world)
        return
    run_b200_arm(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
