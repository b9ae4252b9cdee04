"""Measurement harness beside bench.py: one kernel on one small case, through the C ABI: a correctness check plus CUDA-event timing, sized for a profiler capture.

    python bench_kernels.py gemv  [--rows 14336 --cols 4096 --gate --split --mats 4]   decode GEMV (dooms_cuda_matvec / _gate_up / _matvec_split)
    python bench_kernels.py gemm  [--tokens 2048 --rows 4096 --cols 4096 --gate]  tcgen05 prefill GEMM (dooms_cuda_matmul)
    python bench_kernels.py attention [--config 2 --layers 2 --prompt 2048 --steps 8]  prefill and decode attention inside a decoder cut to a few layers
    python bench_kernels.py batch [--config 0 --sequences 256 --steps 8]           a batched decode step over many sequences of mixed lengths
    python bench_kernels.py launches <ncu csv>                                     per-kernel totals and shares of an ncu launch list

The GEMV case walks over several distinct matrices so that every launch reads its weights from device memory, not from L2.
"""
import argparse
import collections
import csv
import re
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))


def _gemv(args):
    import torch
    from dooms_b200 import _lib as L
    from dooms_b200.quantize import quantize
    lib = L.lib()
    gen = torch.Generator(device='cuda').manual_seed(1)
    dt = L.DTYPE_NAMES.index(args.dtype.lower())
    mats = []
    for _ in range(args.mats):
        g = quantize(dt, torch.randn(args.rows, args.cols, device='cuda', generator=gen) * 0.02)
        u = quantize(dt, torch.randn(args.rows, args.cols, device='cuda', generator=gen) * 0.02) if args.gate else None
        mats.append((g, u))
    x = torch.randn(args.cols, device='cuda', generator=gen)
    y = torch.empty(args.rows, device='cuda')
    st = torch.cuda.current_stream().cuda_stream

    split = None
    if args.split:      # the input already split into int8 digits, as the kernels of a decode step hand it to each other
        split = torch.empty(lib.dooms_cuda_split_input_bytes(args.cols), dtype=torch.uint8, device='cuda')
        L.check(lib.dooms_cuda_split_input(x.data_ptr(), args.cols, split.data_ptr(), st))

    def launch(g, u):
        if split is not None:
            L.check(lib.dooms_cuda_matvec_split(dt, g.data_ptr(), u.data_ptr() if args.gate else None, split.data_ptr(), y.data_ptr(), None, args.rows, args.cols, 0, st))
        elif args.gate:
            L.check(lib.dooms_cuda_gate_up(dt, g.data_ptr(), u.data_ptr(), x.data_ptr(), y.data_ptr(), args.rows, args.cols, st))
        else:
            L.check(lib.dooms_cuda_matvec(dt, g.data_ptr(), x.data_ptr(), y.data_ptr(), None, args.rows, args.cols, 0, st))

    # check the last matrix against the dequantized product in f64
    g, u = mats[-1]
    launch(g, u)
    wd = torch.empty(args.rows, args.cols, device='cuda')
    L.check(lib.dooms_cuda_dequantize(dt, g.data_ptr(), args.rows, args.cols, wd.data_ptr(), st))
    ref = wd.double() @ x.double()
    if args.gate:
        L.check(lib.dooms_cuda_dequantize(dt, u.data_ptr(), args.rows, args.cols, wd.data_ptr(), st))
        ref = torch.nn.functional.silu(ref) * (wd.double() @ x.double())
    err = (y.double() - ref).abs().max().item()
    print(f'max abs error against the f64 product: {err:.3e}')
    assert err < 1e-3, err
    nbytes = (2 if args.gate else 1) * g.numel()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(args.reps):
        a.record()
        for g, u in mats:
            launch(g, u)
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / len(mats)
        print(f'{us:.1f} us per call (input split + GEMV), {nbytes / us / 1e3:.0f} GB/s of weight bytes ({nbytes / 1e6:.1f} MB per call)')


def _gemm(args):
    import torch
    from dooms_b200 import _lib as L
    from dooms_b200.quantize import quantize
    lib = L.lib()
    gen = torch.Generator(device='cuda').manual_seed(1)
    dt = L.DTYPE_NAMES.index(args.dtype.lower())
    M, N, K = args.tokens, args.rows, args.cols
    w = quantize(dt, torch.randn(N, K, device='cuda', generator=gen) * 0.02)
    w2 = quantize(dt, torch.randn(N, K, device='cuda', generator=gen) * 0.02) if args.gate else None
    x = torch.randn(M, K, device='cuda', generator=gen).half()
    y = torch.zeros(M, N, device='cuda')
    st = torch.cuda.current_stream().cuda_stream

    def launch():
        L.check(lib.dooms_cuda_matmul(dt, w.data_ptr(), w2.data_ptr() if args.gate else None, x.data_ptr(), y.data_ptr(), None, M, N, K, 0, st))

    launch()
    wd = torch.empty(N, K, device='cuda')
    L.check(lib.dooms_cuda_dequantize(dt, w.data_ptr(), N, K, wd.data_ptr(), st))
    ref = x.float() @ wd.half().float().T
    if args.gate:
        L.check(lib.dooms_cuda_dequantize(dt, w2.data_ptr(), N, K, wd.data_ptr(), st))
        ref = torch.nn.functional.silu(ref) * (x.float() @ wd.half().float().T)
    rel = ((y - ref).norm() / ref.norm()).item()
    print(f'relative error against the f16-operand product: {rel:.2e}')
    assert rel < 2e-3, rel
    flops = 2.0 * M * N * K * (2 if args.gate else 1)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(args.reps):
        a.record()
        for _ in range(4):
            launch()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / 4
        print(f'{ms * 1e3:.1f} us per call, {flops / ms / 1e9:.1f} TFLOP/s')


def _attention(args):
    """A decoder of the configuration's shape cut to a few layers and a small vocabulary: one prompt call (k_attention_flash once per layer) and a few greedy
    steps (k_attention_decode once per layer and step), checked against a second run fed token by token."""
    import dataclasses
    import os
    import tempfile
    import torch
    from dooms_b200 import CudaLlamaDecoder, synth
    spec = dataclasses.replace(synth.config_spec(args.config), n_layer=args.layers, n_vocab=4096, tied=False)
    path = os.path.join(tempfile.gettempdir(), f'dooms_attention_case_{args.config}_{args.layers}.gguf')
    synth.write_model(spec, path, 77, device='cuda')
    prompt = [int(t) for t in synth.prompt_tokens(args.prompt, spec.n_vocab, 78)]
    n_ctx = args.prompt + args.steps + 8
    dec = CudaLlamaDecoder.load(path, n_ctx, min(args.prompt, 2048))
    a, b, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    for rep in range(args.reps):
        dec.reset()
        torch.cuda.synchronize()
        a.record()
        dec.eval_tokens(prompt)
        dec.pending_token()
        b.record()
        out = []
        dec.generate(args.steps, 2, lambda tok: out.append(tok) is None)
        c.record()
        torch.cuda.synchronize()
        kv = 2 * (args.prompt + args.steps / 2) * spec.n_head_kv * spec.head_dim * 2
        print(f'prompt of {args.prompt}: {a.elapsed_time(b):.2f} ms; {args.steps} steps: {b.elapsed_time(c) / args.steps * 1e3:.1f} us each '
              f'({kv / 1e6:.2f} MB of keys and values per layer and step)')
    dec.reset()
    dec.eval_tokens(prompt[:-64])
    for t in prompt[-64:]:
        dec.eval_tokens([t])                         # the last 64 positions through the decode attention kernel
    again = []
    dec.generate(args.steps, 2, lambda tok: again.append(tok) is None)
    print('tokens', out, 'token by token', again)
    assert out == again or args.prompt < 65, (out, again)
    dec.close()
    os.remove(path)


def _batch(args):
    """The serving load's decode step: `sequences` slots filled with prompts of U[32, 4096] tokens, then a few batched greedy steps. The steps sit inside
    cudaProfilerStart / Stop, so that a profiler run with --profile-from-start off sees only them."""
    import os
    import tempfile
    import numpy as np
    import torch
    from dooms_b200 import CudaLlamaDecoder, synth
    spec = synth.config_spec(args.config)
    path = os.path.join(os.environ.get('DOOMS_BENCH_DIR', tempfile.gettempdir()), f'dooms_bench_config{args.config}_seed{1000 + args.config}.gguf')
    if not os.path.exists(path):
        synth.write_model(spec, path + '.part', 1000 + args.config, device='cuda')
        os.replace(path + '.part', path)
    g = np.random.Generator(np.random.PCG64(9))
    lengths = g.integers(32, 4097, args.sequences)
    dec = CudaLlamaDecoder.load(path, 4096 + args.steps * (args.reps + 1) + 8, 2048, max_sequences=args.sequences)
    for s, n in enumerate(lengths):
        dec.select_sequence(s)
        dec.eval_tokens([int(t) for t in synth.prompt_tokens(int(n), spec.n_vocab, 100 + s)])
    slots = list(range(args.sequences))
    dec.decode_batch(slots, args.steps)                       # captures the graph
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    for _ in range(args.reps):
        out = dec.decode_batch(slots, args.steps)
        t = dec.timings()
        kv = 2 * 2 * spec.n_layer * spec.n_head_kv * spec.head_dim * float(lengths.sum())
        print(f'{t["last_batch_ms"] / args.steps * 1e3:.0f} us per step of {args.sequences} rows, {t["last_batch_launches"] // args.steps} launches; '
              f'{kv / 1e9:.2f} GB of keys and values per step: {kv / (t["last_batch_ms"] / args.steps * 1e-3) / 1e9:.0f} GB/s')
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print('tokens of the last step', out[-1][:8])
    dec.close()


def summarize_launches(path, out=sys.stdout):
    """Totals per kernel of an `ncu --metrics gpu__time_duration.sum --csv` launch list."""
    header, agg = None, collections.OrderedDict()
    for row in csv.reader(open(path, newline='')):
        if header is None:
            if 'Kernel Name' in row:
                header = row
            continue
        if len(row) < len(header):
            continue
        d = dict(zip(header, row))
        if d.get('Metric Name') != 'gpu__time_duration.sum':
            continue
        name = re.sub(r'\(.*', '', d['Kernel Name'])
        name = re.sub(r'^void |dooms::cuda::|\(anonymous namespace\)::|<unnamed>::', '', name)
        value = float(d['Metric Value'].replace(',', ''))
        us = value / 1000 if d['Metric Unit'] in ('ns', 'nsecond') else value
        slot = agg.setdefault(name, [0, 0.0])
        slot[0] += 1
        slot[1] += us
    total = sum(v[1] for v in agg.values())
    print(f'{sum(v[0] for v in agg.values())} launches, {total:.1f} us in total', file=out)
    print(f'{"total us":>10} {"share":>6} {"launches":>8} {"us each":>9}  kernel', file=out)
    for name, (n, us) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
        print(f'{us:10.1f} {100 * us / total:5.1f}% {n:8d} {us / n:9.2f}  {name[:100]}', file=out)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest='case', required=True)
    g = sub.add_parser('gemv')
    g.add_argument('--rows', type=int, default=14336)
    g.add_argument('--cols', type=int, default=4096)
    g.add_argument('--gate', action='store_true')
    g.add_argument('--split', action='store_true', help='q4_0 / q4_k: the input already split (dooms_cuda_matvec_split)')
    g.add_argument('--mats', type=int, default=4)
    g.add_argument('--reps', type=int, default=3)
    g.add_argument('--dtype', default='q4_0')
    m = sub.add_parser('gemm')
    m.add_argument('--tokens', type=int, default=2048)
    m.add_argument('--rows', type=int, default=4096)
    m.add_argument('--cols', type=int, default=4096)
    m.add_argument('--gate', action='store_true')
    m.add_argument('--reps', type=int, default=3)
    m.add_argument('--dtype', default='q4_0')
    t = sub.add_parser('attention')
    t.add_argument('--config', type=int, default=2)
    t.add_argument('--layers', type=int, default=2)
    t.add_argument('--prompt', type=int, default=2048)
    t.add_argument('--steps', type=int, default=8)
    t.add_argument('--reps', type=int, default=2)
    b = sub.add_parser('batch')
    b.add_argument('--config', type=int, default=0)
    b.add_argument('--sequences', type=int, default=256)
    b.add_argument('--steps', type=int, default=8)
    b.add_argument('--reps', type=int, default=2)
    l = sub.add_parser('launches')
    l.add_argument('csv')
    args = ap.parse_args(argv)
    if args.case == 'gemv':
        _gemv(args)
    elif args.case == 'gemm':
        _gemm(args)
    elif args.case == 'attention':
        _attention(args)
    elif args.case == 'batch':
        _batch(args)
    else:
        summarize_launches(args.csv)


if __name__ == '__main__':
    main()
