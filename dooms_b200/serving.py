"""Many independent sequences over one or more GPUs, data parallel: one worker process per GPU, each with its own decoder (weights replicated, its own KV
cache). No collective on the data path. Three ways to run a GPU's share:
  * batched (serve_batched, the default of the command below): the decoder holds one KV-cache slot per sequence, every prompt is evaluated into its slot,
    and then all sequences decode together, one pass over the weights per step for all of them (CudaLlamaDecoder.decode_batch); a sequence that has all
    its tokens leaves its row idle;
  * continuous (run_continuous): more sequences than slots; finished sequences hand their slots to waiting prompts between batched steps;
  * one at a time (serve): sequences pulled from a shared queue and run one after another, the reference's serving loop (docs/USING.md:103,
    python/dooms/server.py:262-269), optionally several decoders per GPU on their own streams.

    python -m dooms_b200.serving --model m.gguf --gpus 2 --sequences 256 [--check 4]

prints one JSON line: sequences, prompt and generated tokens, wall seconds, aggregate decode tok/s (generated tokens of all decoders / the slowest
decoder's device time in generate), tokens per wall second, and with --check the number of sequences re-run alone whose tokens were identical.
--streams K runs K decoders per GPU, each on its own CUDA stream and host thread: on the 0.5B shape one B200 finished 48 sequences in 13.7 s with one
decoder, 9.1 s with two and 7.2 s with four (a batch-1 step of a small model leaves most of the GPU idle between its kernels).
"""
import argparse
import json
import multiprocessing as mp
import time

import numpy as np


def workload(n_sequences: int, n_vocab: int, seed: int = 3000, prompt_range=(32, 4096), decode_range=(16, 512)):
    """Seeded prompt and decode lengths (uniform, inclusive) and token ids, as the serving configuration describes them."""
    g = np.random.Generator(np.random.PCG64(seed))
    out = []
    for _ in range(n_sequences):
        n_prompt = int(g.integers(prompt_range[0], prompt_range[1] + 1))
        n_decode = int(g.integers(decode_range[0], decode_range[1] + 1))
        out.append((g.integers(0, n_vocab, n_prompt, dtype=np.int32), n_decode))
    return out


def run_sequence(dec, prompt, n_decode: int, depth: int = 4):
    """One sequence on a decoder: returns (tokens, device ms of the prompt, device ms of the decode steps)."""
    dec.reset()
    dec.eval_tokens(prompt)
    prefill_ms = dec.timings()["last_eval_ms"]
    tokens: list[int] = []
    dec.generate(n_decode, depth, lambda t: tokens.append(t) or True)
    return tokens, prefill_ms, dec.timings()["last_generate_ms"]


def run_batched(dec, sequences, max_steps_per_call: int = 256):
    """Every (prompt, n_decode) of `sequences` on one decoder with at least len(sequences) slots: prompts one after another into their slots, then batched
    decode steps until the longest is done. Returns (tokens per sequence, {device ms and wall seconds of the prompts and of the decode steps, steps run})."""
    n = len(sequences)
    tokens: list[list[int]] = []
    prefill_ms = 0.0
    t_start = time.perf_counter()
    for s, (prompt, _) in enumerate(sequences):
        dec.select_sequence(s)
        dec.reset()
        dec.eval_tokens(prompt)
        prefill_ms += dec.timings()["last_eval_ms"]
        tokens.append([dec.pending_token()])          # the first token comes from the prompt
    need = [d - 1 for _, d in sequences]               # decode steps each sequence still wants
    decode_ms, steps_run = 0.0, 0
    t_decode = time.perf_counter()
    while any(k > 0 for k in need):
        k = min(min(k for k in need if k > 0), max_steps_per_call)
        slots = [s if need[s] > 0 else -1 for s in range(n)]      # always n rows: one captured graph serves every call
        out = dec.decode_batch(slots, k)
        decode_ms += dec.timings()["last_batch_ms"]
        steps_run += k
        for s in range(n):
            if need[s] > 0:
                tokens[s].extend(int(t) for t in out[:, s])
                need[s] -= k
    t_end = time.perf_counter()
    return tokens, {"prefill_ms": prefill_ms, "decode_ms": decode_ms, "steps": steps_run, "prefill_wall_s": t_decode - t_start, "decode_wall_s": t_end - t_decode}


def run_continuous(dec, sequences, max_live: int, max_steps_per_call: int = 64):
    """More sequences than slots: at most max_live of them are live at a time, each in a KV-cache slot; whenever sequences finish, the next waiting prompts
    are evaluated into the freed slots and join the following batched steps (continuous batching). A step always has max_live rows (idle ones marked -1),
    so one captured graph serves the whole run, and a row's arithmetic does not depend on which other sequences share its step: a sequence's tokens are
    those of run_batched with the same number of rows. Returns (tokens per sequence, {prefill / decode device ms, steps, largest number of live rows})."""
    n = len(sequences)
    tokens: list[list[int]] = [[] for _ in range(n)]
    slot_of = [-1] * max_live                        # the sequence in each slot, -1: free
    need = [0] * max_live
    waiting = list(range(n))
    prefill_ms = decode_ms = 0.0
    steps_run = most_live = 0
    while waiting or any(s >= 0 for s in slot_of):
        for slot in range(max_live):                 # admit
            if slot_of[slot] < 0 and waiting:
                i = waiting.pop(0)
                prompt, n_decode = sequences[i]
                dec.select_sequence(slot)
                dec.reset()
                dec.eval_tokens(prompt)
                prefill_ms += dec.timings()["last_eval_ms"]
                tokens[i].append(dec.pending_token())
                if n_decode > 1:
                    slot_of[slot], need[slot] = i, n_decode - 1
        live = [slot for slot in range(max_live) if slot_of[slot] >= 0]
        if not live:
            continue
        most_live = max(most_live, len(live))
        # as many steps as the first sequence to finish still wants: nothing is generated past a sequence's end, and its slot frees up at once
        k = min(min(need[slot] for slot in live), max_steps_per_call)
        rows = [slot if slot_of[slot] >= 0 else -1 for slot in range(max_live)]
        out = dec.decode_batch(rows, k)
        decode_ms += dec.timings()["last_batch_ms"]
        steps_run += k
        for slot in live:
            tokens[slot_of[slot]].extend(int(t) for t in out[:, slot])
            need[slot] -= k
            if need[slot] == 0:
                slot_of[slot] = -1
    return tokens, {"prefill_ms": prefill_ms, "decode_ms": decode_ms, "steps": steps_run, "most_live": most_live}


def _batched_worker(device: int, path: str, n_ctx: int, n_batch: int, sequences, mine, done):
    from . import CudaLlamaDecoder
    dec = CudaLlamaDecoder.load(path, n_ctx, n_batch, device=device, max_sequences=max(2, len(mine)))
    done.put(("ready", device))
    tokens, st = run_batched(dec, [sequences[i] for i in mine])
    done.put(("batch", device, mine, tokens, st["prefill_ms"], st["decode_ms"], st["steps"]))
    dec.close()
    done.put(("closed", device))


def serve_batched(path: str, sequences, devices, n_ctx: int, n_batch: int = 2048):
    """The sequences dealt over the devices (longest first, round-robin, so that every device's longest sequences are alike), each device's share run as
    one batch. Returns (tokens per sequence, stats); decode_tok_s = generated tokens of all devices / the slowest device's decode time."""
    ctx = mp.get_context("spawn")
    done = ctx.Queue()
    order = sorted(range(len(sequences)), key=lambda i: -(sequences[i][1] * 8 + len(sequences[i][0])))
    shares = [order[k::len(devices)] for k in range(len(devices))]
    workers = [ctx.Process(target=_batched_worker, args=(d, path, n_ctx, n_batch, sequences, mine, done), daemon=True) for d, mine in zip(devices, shares)]
    for w in workers:
        w.start()
    tokens = [None] * len(sequences)
    pre, dec_ms, steps = {}, {}, {}
    ready = closed = 0
    t0 = None
    while closed < len(workers):
        msg = done.get()
        if msg[0] == "ready":
            ready += 1
            if ready == len(workers):
                t0 = time.perf_counter()          # (the workers start on their own; this wall clock is a lower bound of the job's)
        elif msg[0] == "batch":
            _, dev, mine, toks, p_ms, d_ms, st = msg
            for i, t in zip(mine, toks):
                tokens[i] = t
            pre[dev], dec_ms[dev], steps[dev] = p_ms, d_ms, st
        elif msg[0] == "closed":
            closed += 1
    wall = time.perf_counter() - (t0 or time.perf_counter())
    for w in workers:
        w.join()
    n_gen = sum(len(t) for t in tokens)
    n_prompt = sum(len(s[0]) for s in sequences)
    slowest = max(dec_ms.values()) / 1e3
    stats = {"sequences": len(sequences), "prompt_tokens": n_prompt, "generated_tokens": n_gen, "wall_s": wall, "mode": "batched",
             "decode_tok_s": (n_gen - len(sequences)) / slowest if slowest > 0 else 0.0,
             "prefill_tok_s": n_prompt / (max(pre.values()) / 1e3) if max(pre.values()) > 0 else 0.0,
             "decode_steps": max(steps.values()), "workers": len(devices)}
    return tokens, stats


def _worker(device: int, path: str, n_ctx: int, n_batch: int, sequences, todo, done, streams: int = 1):
    """One process per device; `streams` decoders in it, each on its own CUDA stream and host thread, share the device: a batch-1 decode step of a small
    model leaves most of the GPU idle between its kernels, and a second sequence's kernels fill some of that."""
    import threading
    from . import CudaLlamaDecoder
    decoders = [CudaLlamaDecoder.load(path, n_ctx, n_batch, device=device) for _ in range(streams)]
    done.put(("ready", device))

    def loop(dec, k):
        while True:
            i = todo.get()
            if i is None:               # one end mark per decoder thread
                break
            prompt, n_decode = sequences[i]
            tokens, pre_ms, gen_ms = run_sequence(dec, prompt, n_decode)
            done.put(("seq", i, (device, k), tokens, pre_ms, gen_ms))
    threads = [threading.Thread(target=loop, args=(d, k)) for k, d in enumerate(decoders)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for d in decoders:
        d.close()
    done.put(("closed", device))


def serve(path: str, sequences, devices, n_ctx: int, n_batch: int = 2048, streams: int = 1):
    """Runs every (prompt, n_decode) of `sequences` on the devices (one worker each, repeated ids allowed); longest first, so the tail is short.
    Returns (tokens per sequence, stats)."""
    ctx = mp.get_context("spawn")
    todo, done = ctx.Queue(), ctx.Queue()
    workers = [ctx.Process(target=_worker, args=(d, path, n_ctx, n_batch, sequences, todo, done, streams), daemon=True) for d in devices]
    for w in workers:
        w.start()
    for _ in workers:
        assert done.get()[0] == "ready"
    order = sorted(range(len(sequences)), key=lambda i: -(len(sequences[i][0]) + 8 * sequences[i][1]))
    t0 = time.perf_counter()
    for i in order:
        todo.put(i)
    for _ in range(len(workers) * streams):
        todo.put(None)
    tokens = [None] * len(sequences)
    gen_ms, pre_ms = {}, {}          # device time per decoder (device, thread)
    closed = 0
    while closed < len(workers):
        msg = done.get()
        if msg[0] == "seq":
            _, i, who, toks, p_ms, g_ms = msg
            tokens[i] = toks
            gen_ms[who] = gen_ms.get(who, 0.0) + g_ms
            pre_ms[who] = pre_ms.get(who, 0.0) + p_ms
        elif msg[0] == "closed":
            closed += 1
    wall = time.perf_counter() - t0
    for w in workers:
        w.join()
    n_gen = sum(len(t) for t in tokens)
    n_prompt = sum(len(s[0]) for s in sequences)
    slowest_gen = max(gen_ms.values()) / 1e3
    stats = {"sequences": len(sequences), "prompt_tokens": n_prompt, "generated_tokens": n_gen, "wall_s": wall,
             "decode_tok_s": (n_gen - len(sequences)) / slowest_gen if slowest_gen > 0 else 0.0,      # the first token of a sequence comes from the prompt
             "prefill_tok_s": n_prompt / (max(pre_ms.values()) / 1e3) if max(pre_ms.values()) > 0 else 0.0,
             "total_tok_s_wall": (n_prompt + n_gen) / wall, "generated_tok_s_wall": n_gen / wall, "workers": len(devices), "streams_per_worker": streams}
    return tokens, stats


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--sequences", type=int, default=256)
    ap.add_argument("--check", type=int, default=0, help="re-run this many sequences alone on GPU 0 and compare their tokens")
    ap.add_argument("--seed", type=int, default=3000)
    ap.add_argument("--streams", type=int, default=0, help="0: each GPU's share as one batch; K > 0: one sequence at a time on K decoders per GPU")
    args = ap.parse_args(argv)
    from . import CudaLlamaDecoder
    from .gguf_io import GgufFile
    f = GgufFile(args.model)
    n_vocab = int(f.find_tensor("token_embd.weight")["shape"][0])
    f.close()
    seqs = workload(args.sequences, n_vocab, args.seed)
    n_ctx = max(len(p) + d for p, d in seqs) + 8
    if args.streams > 0:
        tokens, stats = serve(args.model, seqs, list(range(args.gpus)), n_ctx, streams=args.streams)
    else:
        tokens, stats = serve_batched(args.model, seqs, list(range(args.gpus)), n_ctx)
    if args.check:
        dec = CudaLlamaDecoder.load(args.model, n_ctx, 2048, device=0)
        same = 0
        for i in range(0, len(seqs), max(1, len(seqs) // args.check))[:args.check]:
            alone = run_sequence(dec, seqs[i][0], seqs[i][1])[0]
            same += alone == tokens[i]
        dec.close()
        stats["checked"] = args.check
        stats["identical"] = int(same)
    print(json.dumps(stats))


if __name__ == "__main__":
    main()
