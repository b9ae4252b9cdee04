#!/usr/bin/env python
"""Benchmark of the llama / qwen2 GGUF decoder path on B200: batch-1 decode tok/s and prefill tok/s on a Q4_0 model, the decode GEMV's achieved HBM
bandwidth, and the CPU restatement of the same decoder timed beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config I]

--config 0..3 are the batch-1 configurations (default 2, the one the metric is quoted on); --config 4 is the many-sequence serving load on the config-0
model (256 seeded sequences, batched decode steps per GPU, sequences dealt over the N GPUs with no collective: "scaling": "weak" is not claimed, the
total work is fixed).

One step = the reference's own measurement (bench/bench_llm.cpp:97-119): reset, the whole prompt in one eval_tokens call, then `gen` greedy tokens with
generate(gen + 1, depth); end of generation is ignored. The model is synthetic: the configuration's architecture with seeded N(0, 0.02) weights quantized
like `llama-quantize --pure`, written as a GGUF file and loaded through the loader, prompt = seeded uniform token ids.
With N > 1 (launched by torch.distributed.run) the same model runs tensor-parallel over the N GPUs: total work fixed, "scaling": "strong".
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# (prompt tokens, generated tokens, n_batch) per configuration; n_batch = min(prompt, 2048) as bench/bench_llm.cpp:82-85
WORKLOADS = {0: (512, 128, 512), 1: (512, 128, 512), 2: (2048, 256, 2048), 3: (8192, 256, 2048)}
WORKLOAD_NAMES = {0: "qwen2.5-0.5b-arch q4_0, 512-token prompt + 128 greedy tokens, batch 1",
                  1: "qwen2.5-0.5b-arch q4_k_m-style mix, 512-token prompt + 128 greedy tokens, batch 1",
                  2: "llama-3-8b-arch q4_0, 2048-token prompt + 256 greedy tokens, batch 1",
                  3: "qwen2.5-32b-arch q4_k_m-style mix, 8192-token prompt + 256 greedy tokens, batch 1",
                  4: "qwen2.5-0.5b-arch q4_0, 256 sequences, prompts U[32,4096] + U[16,512] greedy tokens, batched per GPU, data parallel"}


def config_dict(config: int, world: int, depth: int, matrix_bytes: int) -> dict:
    """The workload description both arms print, key for key."""
    return {"workload": WORKLOAD_NAMES[config] + (" [all matrices f16]" if WEIGHTS == "f16" else "") + (f" [cut to {LAYERS} layers]" if LAYERS else ""), "parallelism": f"dp{world}" if config == 4 else f"tp{world}", "l2": "inputs larger than L2: a decode step streams "
            f"{matrix_bytes / 1e9:.2f} GB of weights, {matrix_bytes / 126e6:.0f}x the 126 MB L2", "queue_depth": depth}


def host_threads() -> int:
    """Cores this process may run on (a launcher can pin its workers; os.cpu_count() would overstate)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.index = device_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "samples": len(sm), "reasons": sorted(reasons)}


LAYERS = 0            # --layers N: the configuration's shape cut to its first N layers (a check of a large shape on few GPUs, not a benchmark line)
WEIGHTS = "plan"      # --weights f16: the configuration's architecture with every matrix as f16 (the reference's default published form of its models)


def model_file(config: int, rank: int, world: int, dist) -> tuple[str, object]:
    """The configuration's synthetic GGUF file, generated once per box (rank 0) and shared by path."""
    import dataclasses
    from dooms_b200 import synth
    from dooms_b200 import _lib as L
    import torch
    spec = synth.config_spec(config)
    tag = ""
    if WEIGHTS == "f16":
        spec = dataclasses.replace(spec, plan=synth.pure(L.F16), name=spec.name + "-f16")
        tag = "_f16"
    if LAYERS:
        spec = dataclasses.replace(spec, n_layer=LAYERS, name=f"{spec.name}-{LAYERS}-layers")
        tag += f"_{LAYERS}layers"
    path = os.path.join(os.environ.get("DOOMS_BENCH_DIR", tempfile.gettempdir()), f"dooms_bench_config{config}{tag}_seed{1000 + config}.gguf")
    if rank == 0 and not os.path.exists(path):
        device = "cuda" if torch.cuda.is_available() else "cpu"
        tmp = path + ".part"
        synth.write_model(spec, tmp, 1000 + config, device=device)
        os.replace(tmp, path)
    if world > 1:
        dist.barrier()
    return path, spec


def time_cpu_port(path: str, spec, n_prompt: int, n_decode: int, repeats: int) -> tuple[float, int, str]:
    """Decode tok/s of the CPU restatement (f32, all host cores) on the same file: a bounded sample of the workload."""
    from oracle import binding as ob
    from dooms_b200 import synth
    cores = ob.set_threads(host_threads())      # torch.distributed.run exports OMP_NUM_THREADS=1 to its workers
    o = ob.OracleDecoder(path, n_prompt + n_decode * (repeats + 1) + 4, fast=True)
    prompt = synth.prompt_tokens(n_prompt, spec.n_vocab, 2000)
    logits = o.eval_tokens(prompt)
    tok = ob.argmax(logits)
    logits = o.eval_tokens([tok])      # one untimed step
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        for _ in range(n_decode):
            tok = ob.argmax(logits)
            logits = o.eval_tokens([tok])
        times.append((time.perf_counter() - t0) / n_decode)
    sample = f"{n_decode} greedy decode steps x {repeats} after a {n_prompt}-token prompt on the same GGUF file, p50 per token"
    return 1.0 / statistics.median(times), cores, sample


def run_reference_arm(args, rank, world, dist):
    """--impl reference: the reference's llama.cpp-linked CPU path cannot be built here (its sources are fetched at configure time and are not on disk), so
    the arm times the CPU restatement of the reference decoder's math (oracle/, kind "port": f32 quantized dot products with the offsets folded out, all
    host threads) on the same file: per step a bounded sample of the workload's decode phase. Under torch.distributed.run rank 0 alone does the work."""
    if rank != 0:
        return
    config = args.config
    path, spec = model_file(0 if config == 4 else config, 0, 1, None)
    n_decode = 4 if config in (2, 3) else 16
    steps, warmup = args.steps, args.warmup
    from oracle import binding as ob
    from dooms_b200 import synth
    cores = ob.set_threads(host_threads())      # the launcher exports OMP_NUM_THREADS=1 to its workers; the baseline is meant to use the whole host
    o = ob.OracleDecoder(path, 8 + (steps + warmup + 1) * n_decode, fast=True)
    logits = o.eval_tokens(synth.prompt_tokens(8, spec.n_vocab, 2000 + config))
    per_step = []
    for s in range(warmup + steps):
        t0 = time.perf_counter()
        for _ in range(n_decode):
            logits = o.eval_tokens([ob.argmax(logits)])
        if s >= warmup:
            per_step.append(time.perf_counter() - t0)
    total = sum(per_step)
    value = n_decode * steps / total
    matrix_bytes = spec.matrix_bytes()
    sample = f"{n_decode} greedy decode steps per step after an 8-token prompt on the same GGUF file"
    line = {"impl": "reference", "metric": "decode_tok_s", "value": value, "unit": "tok/s", "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
            "ms_per_step": 1e3 * total / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_dict(config, args.gpus, args.depth, matrix_bytes),
            "cpu_baseline": {"value": value, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample,
                             "weight_gbs": matrix_bytes * value / 1e9},
            "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "the reference's own CPU path links llama.cpp, which is not vendored and cannot be built offline; this is the CPU restatement of its decoder"}
    print(json.dumps(line), flush=True)


def gemv_roofline(spec, torch, lib, L, hbm_gbs: float, source: str, world: int = 1) -> dict:
    """The dominant decode kernel (the fused gate/up GEMV, ~58% of the bytes a token reads) on the shape a rank runs (the model's, or its 1 / world row
    share under tensor parallelism), timed with CUDA events over launches that walk distinct matrices (so nothing is served from L2).
    achieved = matrix bytes per launch / average launch time."""
    from dooms_b200.quantize import quantize
    F, E = spec.n_ff // world, spec.n_embd
    dt = spec.plan("ffn_gate", 0)
    row_bytes = E // L.BLOCK_ELEMS[dt] * L.BLOCK_BYTES[dt]
    per_launch = 2 * F * row_bytes
    n_mats = max(4, int(600e6 // per_launch) + 1)          # more than the 126 MB L2 several times over
    gen = torch.Generator(device="cuda").manual_seed(7)
    mats = []
    for _ in range(n_mats):
        g = quantize(dt, torch.randn(F, E, device="cuda", generator=gen) * 0.02)
        u = quantize(dt, torch.randn(F, E, device="cuda", generator=gen) * 0.02)
        mats.append((g, u))
    x = torch.randn(E, device="cuda", generator=gen)
    h = torch.empty(F, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    # Inside a decode step the kernel finds its input already split into int8 digits by the kernel before it; that is the form timed here (the split is
    # made once, outside the timed region). The same launches on the f32 input, which every block splits for itself first, are reported beside it.
    split = None
    if dt in (L.Q4_0, L.Q4_K):
        split = torch.empty(lib.dooms_cuda_split_input_bytes(E), dtype=torch.uint8, device="cuda")
        L.check(lib.dooms_cuda_split_input(x.data_ptr(), E, split.data_ptr(), stream))
        if lib.dooms_cuda_matvec_split(dt, mats[0][0].data_ptr(), mats[0][1].data_ptr(), split.data_ptr(), h.data_ptr(), None, F, E, 0, stream) != 0:
            split = None

    def sweep(given):
        for g, u in mats:
            if given:
                L.check(lib.dooms_cuda_matvec_split(dt, g.data_ptr(), u.data_ptr(), split.data_ptr(), h.data_ptr(), None, F, E, 0, stream))
            else:
                L.check(lib.dooms_cuda_gate_up(dt, g.data_ptr(), u.data_ptr(), x.data_ptr(), h.data_ptr(), F, E, stream))

    def timed(given):
        for _ in range(3):
            sweep(given)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            sweep(given)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e3 / (reps * n_mats)
    reps = 5
    us_f32 = timed(False)
    us = timed(True) if split is not None else us_f32
    achieved = per_launch / (us * 1e-6) / 1e9
    return {"bound": "hbm", "kernel": "gate_up GEMV " + L.DTYPE_NAMES[dt] + f" {F}x{E} x2" + (", input already split as in the decode step" if split is not None else ""),
            "us_per_launch_f32_input": us_f32, "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s",
            "frac": achieved / hbm_gbs, "peak_source": source, "frac_of_nominal_8000": achieved / 8000.0,
            # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this shape (ncu capture summarised under profiles/): 66 129 920 + 897 792
            "traffic": 67027712 if (F, E, dt) == (14336, 4096, L.Q4_0) else None, "rows_per_rank": F,
            "bytes_per_launch": per_launch, "us_per_launch": us, "launches_timed": reps * n_mats}


def gemm_roofline(spec, torch, lib, L, pk: dict, n_tokens: int, world: int = 1) -> dict:
    """The dominant prefill kernel (the fused gate/up GEMM on the tcgen05 tensor cores) on the shape a rank runs, timed with CUDA events.
    achieved = 2 * tokens * rows * cols * 2 matrices / average launch time."""
    from dooms_b200.quantize import quantize
    F, E = spec.n_ff // world, spec.n_embd
    dt = spec.plan("ffn_gate", 0)
    gen = torch.Generator(device="cuda").manual_seed(11)
    g = quantize(dt, torch.randn(F, E, device="cuda", generator=gen) * 0.02)
    u = quantize(dt, torch.randn(F, E, device="cuda", generator=gen) * 0.02)
    x = torch.randn(n_tokens, E, device="cuda", generator=gen).half()
    y = torch.empty(n_tokens, F, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def launch():
        L.check(lib.dooms_cuda_matmul(dt, g.data_ptr(), u.data_ptr(), x.data_ptr(), y.data_ptr(), None, n_tokens, F, E, 0, stream))
    for _ in range(3):
        launch()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 10
    a.record()
    for _ in range(reps):
        launch()
    b.record()
    torch.cuda.synchronize()
    us = a.elapsed_time(b) * 1e3 / reps
    flops = 2.0 * n_tokens * F * E * 2
    achieved = flops / (us * 1e-6) / 1e12
    return {"bound": "tensor", "kernel": "gate_up GEMM " + L.DTYPE_NAMES[dt] + f" {n_tokens}x{F}x{E} x2 (tcgen05, weights dequantized in the kernel)",
            "achieved": achieved, "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": achieved / pk["bf16_tflops"], "peak_source": pk["source"] + " burst",
            "frac_of_sustained": achieved / pk["bf16_tflops_sustained"], "frac_of_nominal_2250": achieved / 2250.0, "traffic": None,
            "flops_per_launch": flops, "us_per_launch": us, "launches_timed": reps, "rows_per_rank": F}


def tp_check(path: str, prompt, n_gen: int, n_batch: int, tokens_tp: list[int], logits_tp, local: int) -> dict:
    """With N > 1, outside the timed region: rank 0 runs the same file on one GPU and compares the prompt's last-row logits and every greedy token of the
    tensor-parallel run with it."""
    from dooms_b200 import CudaLlamaDecoder
    one = CudaLlamaDecoder.load(path, len(prompt) + n_gen + 16, n_batch, device=local)
    one.eval_tokens(prompt)
    want = one.logits().astype(np.float64)
    got = np.asarray(logits_tp, dtype=np.float64)
    toks: list[int] = []
    one.generate(n_gen + 1, 4, lambda t: toks.append(t) or True)
    one.close()
    n_equal = 0
    for a, b in zip(toks, tokens_tp):
        if a != b:
            break
        n_equal += 1
    return {"logits_rel_l2": float(np.sqrt(((got - want) ** 2).sum() / (want ** 2).sum())), "logits_max_abs": float(np.abs(got - want).max()),
            "greedy_tokens_equal": toks == list(tokens_tp), "n_tokens": len(toks), "first_difference": None if toks == list(tokens_tp) else n_equal}


def run_serving_config(args, rank, world, local):
    """--config 4: the many-sequence load on the config-0 model. The 256 seeded sequences are dealt over the ranks (longest first, round-robin; no
    collective on the data path), each rank evaluates its prompts into KV-cache slots and then decodes all of its sequences together, one pass over the
    weights per step. One bench step = the whole job. value = generated tokens of all ranks / the slowest rank's device time in the decode steps."""
    import torch
    import torch.distributed as dist
    from dooms_b200 import CudaLlamaDecoder, serving
    from dooms_b200 import _lib as L
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decoder has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))      # barriers and the max over ranks of the timings only
    path, spec = model_file(0, rank, world, dist)
    seqs = serving.workload(256, spec.n_vocab, 3000)
    order = sorted(range(len(seqs)), key=lambda i: -(seqs[i][1] * 8 + len(seqs[i][0])))
    mine = order[rank::world]
    n_ctx = max(len(p) + d for p, d in seqs) + 8
    dec = CudaLlamaDecoder.load(path, n_ctx, 2048, device=local, max_sequences=len(mine))
    share = [seqs[i] for i in mine]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    tokens = None
    for _ in range(max(args.warmup, 3)):
        tokens, _ = serving.run_batched(dec, share)
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    t_begin = time.perf_counter()
    tot = {"prefill_ms": 0.0, "decode_ms": 0.0, "prefill_wall_s": 0.0, "decode_wall_s": 0.0}
    steps_run = 0
    for _ in range(args.steps):
        tokens, st = serving.run_batched(dec, share)
        for k in tot:
            tot[k] += st[k]
        steps_run = st["steps"]
    launches = dec.timings()["last_batch_launches"]
    barrier()
    t_total = time.perf_counter() - t_begin
    clocks = sampler.stop() if rank == 0 else None
    stats = torch.tensor([tot["prefill_ms"], tot["decode_ms"], tot["prefill_wall_s"], tot["decode_wall_s"]], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    prefill_ms, decode_ms, prefill_wall, decode_wall = [float(v) for v in stats.cpu()]
    check = None
    if rank == 0:
        # outside the timed region: a sample of this rank's sequences run alone (one position per call), compared token by token
        dec.close()
        one = CudaLlamaDecoder.load(path, n_ctx, 2048, device=local)
        sample = list(range(0, len(share), max(1, len(share) // 8)))[:8]
        agree = total = identical = 0
        for j in sample:
            alone = serving.run_sequence(one, share[j][0], share[j][1])[0]
            prefix = next((i for i, (a, b) in enumerate(zip(alone, tokens[j])) if a != b), len(alone))
            agree += prefix
            total += len(alone)
            identical += prefix == len(alone)
        one.close()
        check = {"sequences_checked": len(sample), "identical_sequences": identical, "tokens": total, "tokens_before_first_difference": agree,
                 "note": "a batched step rounds operands to f16 in its tensor-core tiles, a single run does not: a sequence may part from its single run at a near tie"}
    else:
        dec.close()
    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    pk = peaks()
    K = args.steps
    n_gen = sum(d for _, d in seqs)
    n_prompt = sum(len(p) for p, _ in seqs)
    decode_tokens = n_gen - len(seqs)                  # a sequence's first token comes out of its prompt
    matrix_bytes = spec.matrix_bytes()
    step_us = decode_ms / K / max(steps_run, 1) * 1e3
    # what a step reads: every matrix once, and of every live sequence the keys and values of all its positions so far, in every layer
    per_position = 2 * spec.n_layer * spec.n_head_kv * spec.head_dim * 2
    kv_bytes = sum(per_position * (len(p) + t) for p, d in share for t in range(1, d)) / max(steps_run, 1)
    step_bytes = matrix_bytes + kv_bytes
    line = {
        "metric": "decode_tok_s", "value": decode_tokens * K / (decode_ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": max(args.warmup, 3),
        "ms_per_step": 1e3 * t_total / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "impl": "ours",
        "config": config_dict(4, world, args.depth, matrix_bytes), "sequences_per_gpu": len(mine),
        "prefill_tok_s": n_prompt * K / (prefill_ms * 1e-3), "prefill_ms": prefill_ms / K, "decode_ms": decode_ms / K, "decode_steps": steps_run,
        "decode_step_us": step_us,
        "e2e": {"value": decode_tokens * K / decode_wall, "unit": "tok/s", "h2d_bytes_per_step": int(n_prompt * 4 + steps_run * 0 + 3 * 4 * len(mine)),
                "d2h_bytes_per_step": int(n_gen * 4), "wall_ms_per_step": 1e3 * (prefill_wall + decode_wall) / K,
                "total_tok_s_wall": (n_prompt + n_gen) * K / (prefill_wall + decode_wall)},
        "gpu_launches": int(launches * steps_run * K),
        "roofline": {"bound": "hbm", "kernel": f"one batched decode step (up to {len(mine)} rows; all its kernels): every weight matrix once plus the live "
                     "sequences' keys and values, averaged over the run's steps", "achieved": step_bytes / (step_us * 1e-6) / 1e9,
                     "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": step_bytes / (step_us * 1e-6) / 1e9 / pk["hbm_gbs"], "peak_source": pk["source"],
                     "traffic": None, "bytes_per_launch": step_bytes, "weight_bytes": matrix_bytes, "kv_bytes": kv_bytes, "us_per_launch": step_us},
        "clocks": clocks, "dp_check": check, "cpu_baseline": None,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=[0, 1, 2, 3, 4])
    ap.add_argument("--depth", type=int, default=4)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layers", type=int, default=0, help="cut the configuration's model to its first N layers (0: all)")
    ap.add_argument("--weights", default="plan", choices=["plan", "f16"], help="f16: every matrix of the configuration as f16 instead of its quantization plan")
    args = ap.parse_args()
    global WEIGHTS, LAYERS
    WEIGHTS = args.weights
    LAYERS = max(0, args.layers)
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    if os.environ.get("DOOMS_BENCH_WATCHDOG"):      # dump every thread's stack and exit if the run is still going after this many seconds
        import faulthandler
        faulthandler.dump_traceback_later(int(os.environ["DOOMS_BENCH_WATCHDOG"]), exit=True)

    if args.impl == "reference":
        run_reference_arm(args, rank, world, None)
        return
    if args.config == 4:
        run_serving_config(args, rank, world, local)
        return

    import torch
    import torch.distributed as dist
    from dooms_b200 import CudaLlamaDecoder, synth
    from dooms_b200 import _lib as L
    from dooms_b200.decoder import nccl_unique_id
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decoder has no CPU fallback")
    lib = L.lib()
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    config = args.config
    n_prompt, n_gen, n_batch = WORKLOADS[config]
    path, spec = model_file(config, rank, world, dist)
    uid = None
    if world > 1:
        box = [nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        uid = box[0]
    dec = CudaLlamaDecoder.load(path, n_prompt + n_gen + 16, n_batch, device=local, tp_rank=rank, tp_size=world, nccl_unique_id=uid,
                                use_graphs=os.environ.get("DOOMS_BENCH_NO_GRAPHS") is None)
    prompt = synth.prompt_tokens(n_prompt, spec.n_vocab, 2000 + config)
    tokens: list[int] = []

    def step():
        """One pass through the public calls with host buffers: the prompt ids go host -> device inside eval_tokens, every token comes back to the host."""
        tokens.clear()
        dec.reset()
        t0 = time.perf_counter()
        dec.eval_tokens(prompt)
        dec.generate(n_gen + 1, args.depth, lambda t: tokens.append(t) or True)
        wall = time.perf_counter() - t0
        tm = dec.timings()
        return wall, tm["last_eval_ms"], tm["last_generate_ms"], tm["last_eval_launches"] + tm["last_generate_launches"]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    t_begin = time.perf_counter()
    walls, prefill_ms, decode_ms, launches = [], [], [], 0
    for _ in range(args.steps):
        w, p, d, n = step()
        walls.append(w)
        prefill_ms.append(p)
        decode_ms.append(d)
        launches += n
    barrier()
    t_total = time.perf_counter() - t_begin
    clocks = sampler.stop() if rank == 0 else None
    # max over ranks of the device-timed parts
    stats = torch.tensor([sum(prefill_ms), sum(decode_ms), sum(walls)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    sum_prefill_ms, sum_decode_ms, sum_wall = [float(v) for v in stats.cpu()]
    logits_tp = None
    if world > 1:      # one more pass outside the timed region, for the comparison with one GPU below
        dec.reset()
        dec.eval_tokens(prompt)
        logits_tp = dec.logits()
        tokens.clear()
        dec.generate(n_gen + 1, args.depth, lambda t: tokens.append(t) or True)
    tp_flags = dec.timings()
    dec.close()      # every rank at the same point: tearing down the tensor-parallel group is collective
    if rank != 0:
        if world > 1:
            dist.barrier()       # rank 0 compares with a one-GPU decoder meanwhile
            dist.destroy_process_group()
        return

    pk = peaks()
    K = args.steps
    decode_tok_s = n_gen * K / (sum_decode_ms * 1e-3)
    prefill_tok_s = n_prompt * K / (sum_prefill_ms * 1e-3)
    e2e_decode_tok_s = n_gen * K / max(sum_wall - sum_prefill_ms * 1e-3, 1e-9)      # wall time of the calls minus the device-timed prefill
    matrix_bytes = spec.matrix_bytes()
    kv_bytes_per_pos = 2 * spec.n_layer * spec.n_head_kv * spec.head_dim * 2
    avg_pos = n_prompt + n_gen / 2
    step_bytes = matrix_bytes + kv_bytes_per_pos * avg_pos
    linear_flops = 2.0 * n_prompt * sum(r * c for name, kind, l, r, c in spec.matrices() if kind not in ("token_embd", "output"))
    attn_flops = 4.0 * spec.n_head * spec.head_dim * n_prompt * (n_prompt + 1) / 2 * spec.n_layer
    roof = gemv_roofline(spec, torch, lib, L, pk["hbm_gbs"], pk["source"], world)
    roof_tensor = gemm_roofline(spec, torch, lib, L, pk, min(n_prompt, n_batch), world)
    prefill_tflops = (linear_flops + attn_flops) / (sum_prefill_ms / K * 1e-3) / 1e12      # the whole group's
    line = {
        "metric": "decode_tok_s", "value": decode_tok_s, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": max(args.warmup, 3),
        "ms_per_step": 1e3 * t_total / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "impl": "ours",
        "config": config_dict(config, world, args.depth, matrix_bytes),
        "prefill_tok_s": prefill_tok_s, "prefill_ms": sum_prefill_ms / K, "decode_ms_per_token": sum_decode_ms / K / n_gen,
        "prefill_tflops": prefill_tflops, "prefill_tflops_per_gpu": prefill_tflops / world,
        "prefill_frac_of_bf16_sustained": prefill_tflops / world / pk["bf16_tflops_sustained"],
        "prefill_frac_of_bf16_burst": prefill_tflops / world / pk["bf16_tflops"],
        "decode_step_gbs": step_bytes / (sum_decode_ms / K / n_gen * 1e-3) / 1e9,
        "decode_step_frac_of_hbm": step_bytes / world / (sum_decode_ms / K / n_gen * 1e-3) / 1e9 / pk["hbm_gbs"],
        "e2e": {"value": e2e_decode_tok_s, "unit": "tok/s", "h2d_bytes_per_step": int(n_prompt * 4), "d2h_bytes_per_step": int((n_gen + 1) * 4),
                "wall_ms_per_step": 1e3 * sum_wall / K},
        "gpu_launches": int(launches),
        "roofline": roof,
        "roofline_tensor": roof_tensor,
        "clocks": clocks,
        "tokens_tail": tokens[-4:],
    }
    if not args.no_cpu_baseline and world == 1:
        n_dec = 8 if config >= 2 else 32
        v, cores, sample = time_cpu_port(path, spec, 8, n_dec, 3)
        line["cpu_baseline"] = {"value": v, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample, "weight_gbs": matrix_bytes * v / 1e9}
    else:
        line["cpu_baseline"] = None
    if world > 1:
        line["tp_allreduce"] = {"peer_memory_kernel": int(tp_flags["tp_peer_allreduce"]), "nccl_symmetric_window": int(tp_flags["tp_symmetric_window"])}
        line["tp_check"] = tp_check(path, prompt, n_gen, n_batch, list(tokens), logits_tp, local)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
