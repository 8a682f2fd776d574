#!/usr/bin/env python
"""Benchmark of the litnicelm token loop on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload c2]

Metric: generated tokens/s (greedy decode). One "step" is one complete
generation of the workload: for the default workload `c2` a 256-token Zipf
prompt followed by 768 greedy tokens at batch 1 on the 6-layer / 512-wide /
vocab-96 model, every token recomputing its whole context as the reference
does (no KV cache). With N GPUs each rank decodes its own independent stream
(weak scaling, no collective on the data path); `--workload c5` is one job of
512 streams cut into contiguous blocks over the GPUs (strong scaling). Rank 0
prints one JSON line. Beside the headline the default line carries: `parity`
(the run's tokens against the committed oracle fixture of the same inputs),
`hbm` (the output-head product of configs 4/5 against the HBM roofline), and
`extra` (config 3: 64 lockstep streams with the fused sampler; config 5 cut
over the GPUs; config 2 in the opt-in cached mode).

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
# capture summarised under profiles/ (mean over the four projections of a layer at
# context 640). A figure of that capture, not of the run that prints it; other
# workloads have none and report null.
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
    # The job is `job_streams` independent streams (N replicas of the per-GPU count, or the 512
    # streams of config 5 whatever N is). The reference decodes one stream per process on one
    # thread, so the CPU arm runs as many streams side by side as it has cores for (bounded by
    # host memory at the large model) and its throughput is that many times one stream's.
    _, per_gpu, scaling = rank_streams(args.workload, world, 0)
    job_streams = streams if scaling == "strong" else streams * world
    conc = max(1, min(job_streams, os.cpu_count() or 1, 8 if d.d_model <= 512 else 2))
    for _ in range(args.warmup):
        time_reference_sample(d, arena, full, sample_lens[:1], conc)
    t0 = time.time()
    rates = []
    for _ in range(args.steps):
        samples = time_reference_sample(d, arena, full, sample_lens, conc)
        r, _ = extrapolate_reference_tokens_per_s(d, samples, plen, max_new)
        rates.append(r * conc)
    wall = time.time() - t0
    value = statistics.mean(rates)
    sample = (f"per step: single reference forwards at context {sample_lens} of the workload's model, "
              f"cost per executed flop applied to the schedule s={plen}..{plen + max_new - 1} "
              f"(extrapolated from subsample); {conc} stream(s) side by side, one core each")
    line = {
        "impl": "reference", "metric": "generated tokens/s (greedy decode)", "value": value,
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * wall / max(1, args.steps), "higher_is_better": True, "scaling": scaling,
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args.workload, per_gpu, plen, max_new), "l2": "not applicable (CPU)",
                   "sampling": {"temp": temp, "top_k": top_k, "top_p": top_p},
                   "mode": "whole-context recomputation, as the reference"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": conc, "kind": "reference", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_name(workload, streams, plen, max_new):
    d = formats.CONFIG_DIMS[WORKLOADS[workload][0]]
    prompt = 'the prompt "a b c " of the reference\'s smoke script' if workload == "c1" else f"{plen}-token Zipf(1.1) prompt"
    return (f"{workload}: L{d.n_layers} H{d.n_heads} D{d.d_model} F{d.d_ff} V{d.vocab} S{d.max_seq}, "
            f"{streams} stream(s)/GPU, {prompt}, {max_new} new tokens, "
            "whole-context recomputation per token")


DTYPE = "f32 storage; projections and attention as three 16-bit tensor-core products per fp32 product (fp16 / tf32 pairs, 22-bit operands), fp32 accumulate"


def rank_streams(workload: str, world: int, rank: int):
    """(first stream, count, scaling) of this rank. Config 5 is one job of 512
    streams cut into contiguous blocks over the GPUs (strong scaling); the other
    workloads give every GPU its own copy of the per-GPU stream count (weak)."""
    from litnicelm_b200.streams import partition_streams
    streams = WORKLOADS[workload][1]
    if workload == "c5":
        first, count = partition_streams(streams, world, rank)
        return first, count, "strong"
    return rank * streams, streams, "weak"


def make_rank_inputs(workload: str, first: int, count: int):
    key, _, plen, max_new, temp, top_k, top_p, cidx = WORKLOADS[workload]
    d = formats.CONFIG_DIMS[key]
    if workload == "c1":
        # the reference's own smoke case: the inputs of tests/golden/small_c1.npz (prompt "a b c ", biases drawn)
        arena = formats.make_param_arena(d, 1001, bias_std=0.02)
        prompts = np.stack([np.array([0, 1, 2, 1, 3, 1], dtype=np.int32) for _ in range(count)])
    else:
        arena = formats.make_param_arena(d, 1000 + cidx)
        prompts = np.stack([formats.zipf_prompt(d.vocab, plen, 2000 * cidx + first + i) for i in range(count)])
    seeds = np.array([3000 + first + i for i in range(count)], dtype=np.uint32)
    return d, arena, prompts, seeds, (plen, max_new, temp, top_k, top_p)


def check_against_fixture(workload: str, first: int, tokens: np.ndarray):
    """Tokens of the timed run against the committed fixture of the same inputs
    (tests/golden/, made by the oracle). Greedy: identical up to a first
    mismatch, whose top-2 gap in the oracle is reported. Returns None when this
    rank holds none of the fixture's streams."""
    gold = os.path.join(ROOT, "tests", "golden")
    try:
        if workload == "c2" and first == 0:
            z = np.load(os.path.join(gold, "c2_full.npz"))
            ref, got, gaps = z["greedy_tokens"], tokens[0], z["top2_gap"]
            name = "tests/golden/c2_full.npz"
        elif workload == "c1" and first == 0:
            z = np.load(os.path.join(gold, "small_c1.npz"))
            step = z["greedy_step_logits"].astype(np.float64)
            srt = np.sort(step, axis=1)
            ref, got, gaps = z["greedy_tokens"], tokens[0], (srt[:, -1] - srt[:, -2])
            name = "tests/golden/small_c1.npz (written by the reference itself)"
        elif workload == "c5" and first == 0:
            z = np.load(os.path.join(gold, "c5_dims.npz"))
            ref, gaps = z["greedy_tokens"], z["top2_gap"]
            got = tokens[0][:len(ref)]
            name = "tests/golden/c5_dims.npz (stream 0, first 8 tokens)"
        elif workload == "c3" and first == 0:
            z = np.load(os.path.join(gold, "c3_streams.npz"))
            which = [int(i) for i in z["streams"]]
            n = z["sampled_tokens"].shape[1]
            agree = [int(np.argmin(np.append(tokens[i][:n] == z["sampled_tokens"][j], False)))
                     for j, i in enumerate(which)]
            return {"fixture": "tests/golden/c3_streams.npz", "streams": which, "tokens_compared": n,
                    "tokens_equal_per_stream": agree}
        else:
            return None
    except (OSError, KeyError) as e:
        return {"unavailable": str(e)}
    n = min(len(ref), len(got))
    neq = np.nonzero(got[:n] != ref[:n])[0]
    first_bad = int(neq[0]) if len(neq) else None
    return {"fixture": name, "tokens_compared": int(n), "tokens_equal": int(n if first_bad is None else first_bad),
            "first_mismatch_step": first_bad,
            "first_mismatch_gap": None if first_bad is None else float(gaps[first_bad])}


class Box:
    """torch / torch.distributed plumbing shared by the measurements of one process."""

    def __init__(self, rank, local_rank, world):
        import torch
        self.torch = torch
        self.rank, self.local_rank, self.world = rank, local_rank, world
        os.environ["LITNICE_B200_DEVICE"] = str(local_rank)
        torch.cuda.set_device(local_rank)
        self.dist = None
        if world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            self.dist = dist
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # larger than the 126 MB L2

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.dist:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def reduce(self, x: float, op: str = "max") -> float:
        if not self.dist:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX if op == "max" else self.dist.ReduceOp.SUM)
        return float(t.item())

    def close(self):
        if self.dist:
            self.dist.barrier()
            self.dist.destroy_process_group()


def measure_generation(box: Box, workload: str, steps: int, warmup: int, sample_clocks: bool, kv_cache: bool = False):
    """W warm-up and K timed generations of this rank's streams, device-timed with
    the prompts resident, then K more through litnice_b200_generate with pinned
    host buffers. Returns the figures of the job over all ranks and the session."""
    import ctypes as C
    from litnicelm_b200.plugin import B200Sampling, Session
    torch = box.torch
    first, count, scaling = rank_streams(workload, box.world, box.rank)
    d, arena, prompts, seeds, (plen, max_new, temp, top_k, top_p) = make_rank_inputs(workload, first, count)
    # kv_cache: the opt-in cached mode (an extension; the reference recomputes the context)
    old_kv = os.environ.get("LITNICE_B200_KV_CACHE")
    os.environ["LITNICE_B200_KV_CACHE"] = "1" if kv_cache else "0"
    try:
        sess = Session(d, count)
    finally:
        if old_kv is None:
            del os.environ["LITNICE_B200_KV_CACHE"]
        else:
            os.environ["LITNICE_B200_KV_CACHE"] = old_kv
    sess.load_params(arena)
    pinned_prompts = torch.from_numpy(prompts.copy()).pin_memory()
    pinned_out = torch.zeros((count, max_new), dtype=torch.int32).pin_memory()

    # ---- device-resident pass: prompts already in HBM when the clock starts ----
    for _ in range(warmup):
        sess.upload_prompts(prompts, seeds)
        sess.run(max_new, temp, top_k, top_p)
    clocks = ClockSampler(box.local_rank) if sample_clocks and box.rank == 0 else None
    box.barrier()
    if clocks:
        clocks.start()
    dev_ms, launches, tokens = 0.0, 0, 0
    t0 = time.perf_counter()
    for _ in range(steps):
        box.flush.fill_(1)
        torch.cuda.synchronize()
        sess.upload_prompts(prompts, seeds)          # untimed: not inside the event bracket
        sess.run(max_new, temp, top_k, top_p)
        st = sess.stats()
        dev_ms += st.device_ms
        launches += st.kernel_launches
        tokens += st.tokens
    box.barrier()
    wall_s = time.perf_counter() - t0
    clock_info = clocks.stop() if clocks else None
    dev_ms = box.reduce(dev_ms, "max")
    total_tokens = box.reduce(float(tokens), "sum")
    value = total_tokens / (dev_ms * 1e-3)

    # ---- end-to-end pass: host buffers in, host buffers out, copies inside the clock ----
    sp = B200Sampling(temp, top_k, top_p)
    produced = C.c_int32(0)
    i32p = C.POINTER(C.c_int32)
    seeds_p = seeds.ctypes.data_as(C.POINTER(C.c_uint32))

    def e2e_once():
        rc = sess.lib.litnice_b200_generate(sess.h, C.cast(pinned_prompts.data_ptr(), i32p), count, plen,
                                            max_new, C.byref(sp), seeds_p,
                                            C.cast(pinned_out.data_ptr(), i32p), C.byref(produced))
        if rc != 0:
            raise RuntimeError(sess.lib.litnice_b200_last_error(sess.h).decode())

    if warmup > 1:
        e2e_once()
    box.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        box.flush.fill_(1)
        torch.cuda.synchronize()
        e2e_once()
    box.barrier()
    e2e_s = box.reduce(time.perf_counter() - t0, "max")
    st = sess.stats()
    e2e_tokens = box.reduce(float(steps * count * produced.value), "sum")
    out = pinned_out.numpy()[:, :produced.value].copy()
    parity = check_against_fixture(workload, first, out)
    return {
        "dims": d, "arena": arena, "prompts": prompts, "sess": sess, "scaling": scaling,
        "streams_this_rank": count, "plen": plen, "max_new": max_new,
        "sampling": {"temp": temp, "top_k": top_k, "top_p": top_p},
        "value": value, "dev_ms_per_step": dev_ms / steps, "launches": int(launches),
        "e2e": {"value": e2e_tokens / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": int(st.h2d_bytes),
                "d2h_bytes_per_step": int(st.d2h_bytes)},
        "clocks": clock_info, "wall_s": wall_s, "first_tokens": out[0, :8].tolist(), "parity": parity,
    }


def whole_loop_flops(d, streams_total: int, plen: int, max_new: int) -> float:
    return sum(algorithmic_flops(d, streams_total, s) for s in range(plen, plen + max_new))


def hbm_block(peaks):
    """The few-row product of the output head at the config-4/5 shape (1024 x 32000 fp32
    weights, 131 MB): the kernel of the path that HBM bandwidth bounds. 50 launches back to
    back between one pair of CUDA events, each on the next of a ring of weight copies that
    exceeds three times the L2, so every launch reads its matrix from HBM."""
    from litnicelm_b200.plugin import gemv_time
    k, n = 1024, 32000
    out = {"kernel": "gemv_tma_kernel: out[m, 32000] = x[m, 1024] . W (output head of configs 4/5)",
           "algorithmic_bytes_per_launch": 4 * k * n + 4 * (k + n), "peak": peaks["hbm_gbs"], "unit": "GB/s",
           "peak_source": f"copy bandwidth, {peaks['source']}", "launches_timed": 50,
           "l2": "ring of weight copies larger than three times the L2: every launch reads HBM"}
    for m in (1, 8):
        try:
            us, nl = gemv_time(m, k, n, 50, 2)
            gbs = (4.0 * k * n + 4.0 * m * (k + n)) / (us * 1e-6) / 1e9
            out[f"m{m}"] = {"us_per_launch": us, "achieved": gbs, "frac": gbs / peaks["hbm_gbs"], "kernels_per_call": nl}
        except Exception as e:
            out[f"m{m}"] = {"unavailable": str(e)}
    return out


def run_b200_arm(args, rank, local_rank, world):
    box = Box(rank, local_rank, world)
    peaks = load_peaks()
    main = measure_generation(box, args.workload, args.steps, args.warmup, sample_clocks=True,
                              kv_cache=args.kv_cache)
    sess, d = main["sess"], main["dims"]
    plen, max_new = main["plen"], main["max_new"]
    streams_total = WORKLOADS[args.workload][1] * (1 if main["scaling"] == "strong" else world)
    line = None
    if rank == 0:
        # ---- roofline of the dominant kernel (the projection GEMM) ----
        s_mid = plen + max_new // 2
        prof = sess.profile_step(main["streams_this_rank"], s_mid, 3)
        isolated = prof.gemm_flops / (prof.gemm_ms * 1e-3) / 1e12 if prof.gemm_ms > 0 else 0.0
        in_loop = prof.gemm_span_flops / (prof.gemm_span_ms * 1e-3) / 1e12 if prof.gemm_span_ms > 0 else None
        # per GPU: this rank's streams over this rank's time (every rank does the same amount of work)
        whole = whole_loop_flops(d, main["streams_this_rank"], plen, max_new) / (main["dev_ms_per_step"] * 1e-3) / 1e12
        achieved = in_loop if in_loop is not None else isolated
        roofline = {
            "bound": "tensor",
            "kernel": "projection GEMM (gemm_tc_kernel: tcgen05 + TMEM, three products of fp16 pairs)",
            "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
            "frac": achieved / peaks["bf16_tflops"], "peak_source": f"bf16 burst, {peaks['source']}",
            # fp32-grade products execute three 16-bit MMAs per algorithmic flop, so algorithmic
            # flops cannot exceed 1/3 of the dense 16-bit peak
            "ceiling_frac_3_products": 1.0 / 3.0,
            "executed_mma_frac": 3.0 * achieved / peaks["bf16_tflops"],
            "how": (f"in the loop: algorithmic 2*M*N*K flops of the {prof.gemm_span_launches} projection launches of "
                    f"one step at context {s_mid} / the sum of their device-clock spans (from the completion of a "
                    f"launch's predecessor to the end of its last CTA, {prof.gemm_span_ms:.3f} ms; no event between "
                    f"the launches, which overlap as in the token loop; "
                    f"attention {prof.attn_span_launches} launches {prof.attn_span_ms:.3f} ms; whole step "
                    f"{prof.step_span_ms:.3f} ms)") if in_loop is not None else
                   "CUDA events around each launch (the device-clock spans need the tensor-core path)",
            "isolated": {"achieved": isolated, "frac": isolated / peaks["bf16_tflops"],
                         "how": f"{prof.gemm_launches} launches, CUDA events around each, {prof.gemm_ms:.3f} ms"},
            "whole_loop": {"achieved": whole, "frac": whole / peaks["bf16_tflops"],
                           "frac_of_sustained": whole / peaks["bf16_tflops_sustained"],
                           "how": "all algorithmic flops of one GPU's generation (projections on every row, "
                                  "causal-useful attention, head on the last rows) / ms_per_step"},
            "traffic": NCU_DRAM_BYTES_PER_GEMM_LAUNCH.get(args.workload),
            "traffic_source": ("profiles/gemm_tc_c2_context640_and_c5shape.md (ncu dram__bytes_read + write, mean "
                               "per projection launch at context 640)")
            if args.workload in NCU_DRAM_BYTES_PER_GEMM_LAUNCH else None,
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
    sess.close()
    hbm = None
    if rank == 0 and not args.no_extras:
        hbm = hbm_block(peaks)
    # ---- CPU baseline: the reference itself on a bounded sample ----
    cpu = None
    if rank == 0 and not args.no_cpu_baseline:
        try:
            prompts = main["prompts"]
            full = np.concatenate([prompts[0], formats.zipf_prompt(d.vocab, d.max_seq, 999)])[:d.max_seq]
            lens = [32, 96, 256] if d.d_model == 512 else ([32, 96] if d.d_model > 512 else
                                                           [min(d.max_seq, 24), min(d.max_seq, 56)])
            samples = time_reference_sample(d, main["arena"], full, lens)
            rate, per_flop = extrapolate_reference_tokens_per_s(d, samples, plen, max_new)
            cpu = {"value": rate, "unit": "tokens/s", "cores": 1, "kind": "reference",
                   "host_cores_present": os.cpu_count(),
                   "sample": (f"reference CPU backend, single forwards at context {lens} "
                              f"({', '.join(f'{t:.2f}s' for _, t in samples)}); {per_flop * 1e9:.3f} ns per "
                              "executed flop applied to the full schedule (extrapolated from subsample)")}
        except Exception as e:  # the bench line must still be printed
            cpu = {"value": None, "unit": "tokens/s", "cores": 1, "kind": "reference",
                   "sample": f"unavailable: {e}"}
    # ---- the other halves of the metric: 64 lockstep streams (config 3) and the 512-stream job of
    # config 5 cut over the GPUs; one warm-up and one timed generation each ----
    extra = {}
    if args.workload == "c2" and not args.no_extras:
        for name in ("c3", "c5"):
            r = measure_generation(box, name, 1, 1, sample_clocks=True)
            r["sess"].close()
            total = WORKLOADS[name][1] * (1 if r["scaling"] == "strong" else world)
            wl = whole_loop_flops(r["dims"], r["streams_this_rank"], r["plen"], r["max_new"]) / \
                (r["dev_ms_per_step"] * 1e-3) / 1e12   # per GPU
            extra["c5_split" if name == "c5" else name] = {
                "workload": workload_name(name, r["streams_this_rank"], r["plen"], r["max_new"]),
                "value": r["value"], "unit": "tokens/s", "scaling": r["scaling"],
                "streams_total": total, "streams_per_gpu": r["streams_this_rank"],
                "ms_per_step": r["dev_ms_per_step"], "steps": 1, "warmup": 1, "e2e": r["e2e"],
                "gpu_launches": r["launches"], "sampling": r["sampling"],
                "whole_loop_tflops": wl, "whole_loop_frac": wl / peaks["bf16_tflops"], "clocks": r["clocks"],
                "parity": r["parity"],
            }
    if args.workload == "c2" and not args.no_extras:
        # the same workload in the opt-in cached mode: keys and values of earlier positions kept in
        # HBM, one new row per step (the regime the few-row products are for); reported beside the
        # headline, never instead of it, because the reference itself keeps no cache
        r = measure_generation(box, "c2", 3, 3, sample_clocks=False, kv_cache=True)
        r["sess"].close()
        extra["c2_kv_cache"] = {
            "workload": workload_name("c2", r["streams_this_rank"], r["plen"], r["max_new"]).replace(
                "whole-context recomputation per token", "keys and values cached (LITNICE_B200_KV_CACHE=1)"),
            "value": r["value"], "unit": "tokens/s", "ms_per_step": r["dev_ms_per_step"], "steps": 3, "warmup": 3,
            "e2e": r["e2e"], "gpu_launches": r["launches"], "parity": r["parity"],
        }
    if rank == 0:
        line = {
            "metric": "generated tokens/s (greedy decode)", "value": main["value"], "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": main["dev_ms_per_step"], "higher_is_better": True, "scaling": main["scaling"],
            "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
            "config": {"workload": workload_name(args.workload, main["streams_this_rank"], plen, max_new),
                       "l2": "256 MB buffer written between timed steps (L2 flush)",
                       "sampling": main["sampling"],
                       "mode": "keys and values cached (extension)" if args.kv_cache else
                               "whole-context recomputation, as the reference"},
            "e2e": main["e2e"], "gpu_launches": main["launches"],
            "roofline": roofline, "hbm": hbm, "cpu_baseline": cpu, "clocks": main["clocks"],
            "parity": main["parity"], "extra": extra,
            "wall_s_timed_region": main["wall_s"], "first_tokens": main["first_tokens"],
        }
    box.close()
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
            "parity": check_prefill_against_fixture(probs),
        }
        print(json.dumps(line), flush=True)
    sess.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def check_prefill_against_fixture(probs: np.ndarray) -> dict:
    """Rank 0's sequences 0 and 31 of the prefill batch against the oracle's last-row logits of the
    same inputs (tests/golden/c4_prefill.npz): most likely token and largest probability error."""
    path = os.path.join(ROOT, "tests", "golden", "c4_prefill.npz")
    if not os.path.exists(path):
        return {"fixture": None}
    z = np.load(path)
    out = {"fixture": "tests/golden/c4_prefill.npz", "sequences": z["sequences"].tolist(), "argmax_equal": 0,
           "max_abs_probability_error": 0.0}
    for i, seq in enumerate(z["sequences"].tolist()):
        row = z["last_logits"][i].astype(np.float64)
        want = np.exp(row - row.max())
        want /= want.sum()
        out["argmax_equal"] += int(int(np.argmax(probs[seq])) == int(np.argmax(want)))
        out["max_abs_probability_error"] = max(out["max_abs_probability_error"],
                                               float(np.abs(probs[seq] - want).max()))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + ["c4"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kv-cache", action="store_true",
                    help="run the workload in the opt-in cached mode (an extension; not the headline)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the output-head bandwidth block and the config-3 / config-5 side measurements")
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
