"""Many independent sequences over one or more GPUs, data parallel: one worker process per GPU, each with its own decoder (weights replicated, its own KV
cache), pulling sequences from a shared queue and running them one after another: prompt in chunks, then greedy decode. No collective on the data path.
This is the replicas form of the reference's serving loop, which handles one request at a time (docs/USING.md:103, python/dooms/server.py:262-269);
batching several sequences into one decode step is not built.

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
    ap.add_argument("--streams", type=int, default=1, help="decoders per GPU, each on its own stream and thread")
    args = ap.parse_args(argv)
    from . import CudaLlamaDecoder
    from .gguf_io import GgufFile
    f = GgufFile(args.model)
    n_vocab = int(f.find_tensor("token_embd.weight")["shape"][0])
    f.close()
    seqs = workload(args.sequences, n_vocab, args.seed)
    n_ctx = max(len(p) + d for p, d in seqs) + 8
    tokens, stats = serve(args.model, seqs, list(range(args.gpus)), n_ctx, streams=args.streams)
    if args.check:
        dec = CudaLlamaDecoder.load(args.model, n_ctx, 2048, device=0)
        same = 0
        for i in range(0, len(seqs), max(1, len(seqs) // args.check))[:args.check]:
            same += run_sequence(dec, seqs[i][0], seqs[i][1])[0] == tokens[i]
        dec.close()
        stats["checked"] = args.check
        stats["identical"] = int(same)
    print(json.dumps(stats))


if __name__ == "__main__":
    main()
