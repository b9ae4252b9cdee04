"""Tensor parallelism. On CPU (gloo, two ranks): the shares the library hands out partition every matrix exactly, and a layer computed from the shares with
one all-reduce after attn_output and one after ffn_down equals the unsharded layer. On GPUs (two or more visible): the tensor-parallel decoder's logits and
greedy tokens against the one-GPU decoder, as child processes over NCCL."""
import ctypes as C
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from dooms_b200 import _lib as L

ROOT = Path(__file__).resolve().parent.parent


def share(cfg, rank, tp, attn_block=1, ffn_block=1):
    s = L.TpShare()
    s.struct_size = C.sizeof(L.TpShare)
    L.check(L.lib().dooms_cuda_tp_share_blocks(C.byref(cfg), rank, tp, attn_block, ffn_block, C.byref(s)))
    return s


def config(n_head=8, n_head_kv=4, head_dim=16, n_ff=96, n_vocab=101):
    c = L.LlamaConfig()
    c.struct_size = C.sizeof(L.LlamaConfig)
    c.n_head, c.n_head_kv, c.head_dim, c.n_ff, c.n_vocab = n_head, n_head_kv, head_dim, n_ff, n_vocab
    c.n_embd = n_head * head_dim
    return c


def test_shares_partition_the_model():
    for tp in (1, 2, 4):
        cfg = config()
        covered = {k: [] for k in ("q", "kv", "ff", "vocab")}
        for r in range(tp):
            s = share(cfg, r, tp)
            assert s.q_rows % cfg.head_dim == 0 and s.kv_rows % cfg.head_dim == 0          # whole heads
            assert s.q_rows // s.kv_rows == cfg.n_head // cfg.n_head_kv                    # a rank's query heads use only its own key/value heads
            assert s.q_row0 // cfg.head_dim // (cfg.n_head // cfg.n_head_kv) == s.kv_row0 // cfg.head_dim
            for k, (a, n) in {"q": (s.q_row0, s.q_rows), "kv": (s.kv_row0, s.kv_rows), "ff": (s.ff_row0, s.ff_rows), "vocab": (s.vocab_row0, s.vocab_rows)}.items():
                covered[k] += list(range(a, a + n))
        assert covered["q"] == list(range(cfg.n_head * cfg.head_dim)) and covered["kv"] == list(range(cfg.n_head_kv * cfg.head_dim))
        assert covered["ff"] == list(range(cfg.n_ff)) and covered["vocab"] == list(range(cfg.n_vocab))
    lib = L.lib()
    s = L.TpShare()
    s.struct_size = C.sizeof(L.TpShare)
    assert lib.dooms_cuda_tp_share(C.byref(config()), 0, 3, C.byref(s)) == L.UNSUPPORTED          # 8 heads over 3 GPUs
    assert lib.dooms_cuda_tp_share(C.byref(config()), 2, 2, C.byref(s)) == L.INVALID_ARGUMENT


def test_column_shards_are_whole_blocks_where_the_heads_are_not():
    """The 32B shape over 8 GPUs (40 / 8 heads of 128, n_ff 27648, 256-element super-blocks): 640 attention columns per rank are two and a half
    super-blocks, 3456 feed-forward columns thirteen and a half. The feed-forward width is dealt in whole blocks (14 or 13 per rank); of attn_output every
    rank holds the three blocks that cover its heads and multiplies them with its attention row padded with zeros, and the ranks' sums add up to the
    unsharded product. Also a small shape over two ranks."""
    g = np.random.default_rng(3)
    for (nh, nkv, hd, ff, tp, blk) in ((40, 8, 128, 27648, 8, 256), (10, 2, 128, 1792, 2, 256), (8, 4, 16, 160, 4, 32), (6, 2, 16, 160, 2, 32)):
        cfg = config(n_head=nh, n_head_kv=nkv, head_dim=hd, n_ff=ff)
        qw = nh * hd
        shares = [share(cfg, r, tp, blk, blk) for r in range(tp)]
        # feed-forward: whole blocks, consecutive, complete, sizes differing by at most one block
        assert [s.ff_row0 for s in shares] == [sum(t.ff_rows for t in shares[:r]) for r in range(tp)] and sum(s.ff_rows for s in shares) == ff
        assert all(s.ff_rows % blk == 0 and s.ff_row0 % blk == 0 for s in shares)
        assert max(s.ff_rows for s in shares) - min(s.ff_rows for s in shares) <= blk
        # attention: the cover is whole blocks inside the matrix and contains the rank's heads
        att = g.standard_normal(qw)
        wo = g.standard_normal((7, qw))
        total = np.zeros(7)
        for s in shares:
            assert s.attn_col0 % blk == 0 and s.attn_cols % blk == 0 and s.attn_col0 + s.attn_cols <= qw
            assert s.attn_col0 <= s.q_row0 and s.q_row0 + s.q_rows <= s.attn_col0 + s.attn_cols
            assert s.attn_cols < s.q_rows + 2 * blk
            padded = np.zeros(s.attn_cols)
            padded[s.q_row0 - s.attn_col0:s.q_row0 - s.attn_col0 + s.q_rows] = att[s.q_row0:s.q_row0 + s.q_rows]
            total += wo[:, s.attn_col0:s.attn_col0 + s.attn_cols] @ padded
        assert np.allclose(total, wo @ att, rtol=1e-12, atol=1e-12)
    s32 = [share(config(n_head=40, n_head_kv=8, head_dim=128, n_ff=27648), r, 8, 256, 256) for r in range(8)]
    assert [s.ff_rows // 256 for s in s32] == [14, 14, 14, 14, 13, 13, 13, 13] and all(s.attn_cols == 768 for s in s32)
    lib = L.lib()
    s = L.TpShare()
    s.struct_size = C.sizeof(L.TpShare)
    assert lib.dooms_cuda_tp_share_blocks(C.byref(config(n_ff=96)), 0, 4, 32, 32, C.byref(s)) == L.UNSUPPORTED      # three blocks of 32 for four ranks
    assert lib.dooms_cuda_tp_share_blocks(C.byref(config(n_ff=100)), 0, 2, 32, 32, C.byref(s)) == L.UNSUPPORTED     # not whole blocks
    assert lib.dooms_cuda_tp_share_blocks(C.byref(config()), 0, 2, 0, 32, C.byref(s)) == L.INVALID_ARGUMENT


GLOO_CHILD = r"""
import ctypes as C, os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["DOOMS_ROOT"]); sys.path.insert(0, os.path.join(os.environ["DOOMS_ROOT"], "tests"))
from test_tp import config, share
dist.init_process_group("gloo")
rank, tp = dist.get_rank(), dist.get_world_size()
cfg = config()
E, hd, nh, nkv, F = cfg.n_embd, cfg.head_dim, cfg.n_head, cfg.n_head_kv, cfg.n_ff
g = np.random.default_rng(0)                       # every rank draws the same full model
wq, wk, wv = g.standard_normal((nh * hd, E)), g.standard_normal((nkv * hd, E)), g.standard_normal((nkv * hd, E))
wo, wg, wu, wd = g.standard_normal((E, nh * hd)), g.standard_normal((F, E)), g.standard_normal((F, E)), g.standard_normal((E, F))
x = g.standard_normal((5, E))                      # five positions, causal attention

def layer(x, wq, wk, wv, wo, wg, wu, wd, n_q_heads, n_kv_heads, reduce):
    q, k, v = x @ wq.T, x @ wk.T, x @ wv.T
    att = np.zeros((x.shape[0], n_q_heads * hd))
    for h in range(n_q_heads):
        kv = h // (n_q_heads // n_kv_heads)
        for t in range(x.shape[0]):
            s = k[: t + 1, kv * hd:(kv + 1) * hd] @ q[t, h * hd:(h + 1) * hd] / np.sqrt(hd)
            p = np.exp(s - s.max()); p /= p.sum()
            att[t, h * hd:(h + 1) * hd] = p @ v[: t + 1, kv * hd:(kv + 1) * hd]
    x = x + reduce(att @ wo.T)
    gate, up = x @ wg.T, x @ wu.T
    return x + reduce((gate / (1 + np.exp(-gate)) * up) @ wd.T)

def all_reduce(a):
    t = torch.from_numpy(np.ascontiguousarray(a)); dist.all_reduce(t); return t.numpy()

full = layer(x, wq, wk, wv, wo, wg, wu, wd, nh, nkv, lambda a: a)
s = share(cfg, rank, tp)
q, kv, ff = slice(s.q_row0, s.q_row0 + s.q_rows), slice(s.kv_row0, s.kv_row0 + s.kv_rows), slice(s.ff_row0, s.ff_row0 + s.ff_rows)
mine = layer(x, wq[q], wk[kv], wv[kv], wo[:, q], wg[ff], wu[ff], wd[:, ff], nh // tp, nkv // tp, all_reduce)
assert np.allclose(mine, full, rtol=1e-10, atol=1e-10), np.abs(mine - full).max()
# the vocabulary slices gathered in rank order give the full logits; the first maximum over the gathered vector is the global argmax
wout = g.standard_normal((cfg.n_vocab, E))
logits = full[-1] @ wout.T
part = torch.full(((cfg.n_vocab + tp - 1) // tp,), -np.inf, dtype=torch.float64)
part[: s.vocab_rows] = torch.from_numpy(logits[s.vocab_row0:s.vocab_row0 + s.vocab_rows])
parts = [torch.empty_like(part) for _ in range(tp)]
dist.all_gather(parts, part)
assert int(torch.cat(parts).argmax()) == int(np.argmax(logits))
# what the decoder does instead of gathering logits: every rank sends one (value, global index) pair of its slice; the pick among the pairs takes the
# lowest index on ties and never a NaN (llama_kernels.h:949-975, src/core/argmax.h:15-16), so it equals the first-index argmax of the whole vector
for case in (logits, np.where(np.arange(cfg.n_vocab) % 7 == 0, logits.max(), logits), np.where(np.arange(cfg.n_vocab) < 60, np.nan, logits)):
    mine = case[s.vocab_row0:s.vocab_row0 + s.vocab_rows]
    ok = ~np.isnan(mine)
    pair = torch.tensor([mine[ok].max(), float(s.vocab_row0 + int(np.flatnonzero(ok & (mine == mine[ok].max()))[0]))] if ok.any() else [0.0, -1.0], dtype=torch.float64)
    pairs = [torch.empty_like(pair) for _ in range(tp)]
    dist.all_gather(pairs, pair)
    cand = [(float(p[0]), int(p[1])) for p in pairs if int(p[1]) >= 0]
    best = min(cand, key=lambda c: (-c[0], c[1]))[1]
    want = int(np.flatnonzero(case == np.nanmax(case))[0])
    assert best == want, (best, want)
dist.destroy_process_group()
os.write(1, f"ok {rank}\n".encode())      # one write per rank: the two ranks share the pipe
"""


def test_sharded_layer_with_two_all_reduces_equals_the_full_layer_gloo(tmp_path):
    script = tmp_path / "child.py"
    script.write_text(GLOO_CHILD)
    env = dict(os.environ, DOOMS_ROOT=str(ROOT), MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port",
                        "29533", str(script)], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "ok 0" in r.stdout and "ok 1" in r.stdout


NCCL_CHILD = r"""
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["DOOMS_ROOT"])
from dooms_b200 import CudaLlamaDecoder, synth, _lib as L
from dooms_b200.decoder import nccl_unique_id
rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
if os.environ.get("DOOMS_TP_CASE") == "cover":
    # 640 attention columns and 3.5 feed-forward super-blocks per rank: column shards that do not fall on the 256-element blocks of q4_K / q6_K
    spec = synth.tiny_spec(synth.q4_k_m_large, arch="qwen2", n_embd=1280, n_head=10, n_head_kv=2, n_ff=1792, n_vocab=1001, n_layer=3)
else:
    spec = synth.tiny_spec(synth.pure(L.Q4_0), arch="qwen2", n_embd=512, n_head=8, n_head_kv=4, n_ff=2048, n_vocab=1001, n_layer=3)
path = os.environ["DOOMS_TP_MODEL"]
if rank == 0: synth.write_model(spec, path, 5)
dist.barrier()
box = [nccl_unique_id() if rank == 0 else None]
dist.broadcast_object_list(box, src=0)
prompt = [(i * 7 + 3) % 1001 for i in range(150)]
dec = CudaLlamaDecoder.load(path, 512, 128, device=local, tp_rank=rank, tp_size=world, nccl_unique_id=box[0])
dec.eval_tokens(prompt)
lg = dec.logits(); toks = []
dec.generate(12, 2, lambda t: toks.append(t) or True)
peer = dec.timings()["tp_peer_allreduce"]
assert peer == (1 if os.environ.get("DOOMS_TP_ALLREDUCE") == "peer" else 0), peer      # the variant under test is the one that ran
window = dec.timings()["tp_symmetric_window"]
if os.environ.get("DOOMS_TP_SYMMETRIC") == "0": assert window == 0, window
if rank == 0:
    ref = CudaLlamaDecoder.load(path, 512, 128, device=local)
    ref.eval_tokens(prompt)
    lr = ref.logits(); tr = []
    ref.generate(12, 2, lambda t: tr.append(t) or True)
    err = float(np.sqrt(((lg - lr) ** 2).sum() / (lr ** 2).sum()))
    # Only the summation order differs, but a key or value that lands on the other side of an f16 rounding boundary in the cache moves the logits by
    # ~1e-4 .. 1e-3, the same effect the reference's one-call bound allows for.
    assert err < 3e-3, err
    assert toks == tr, (toks, tr)
    print("tp ok", world, err, "symmetric window", window)
dist.barrier()
dist.destroy_process_group()
"""


@pytest.mark.gpu
@pytest.mark.parametrize("allreduce,case,symmetric", [("nccl", "even", "1"), ("nccl", "even", "0"), ("peer", "even", "1"), ("nccl", "cover", "1")])
def test_tensor_parallel_decoder_matches_one_gpu(tmp_path, allreduce, case, symmetric):
    """Two ranks against one GPU: last-position logits and greedy tokens; with NCCL's all-reduce and with the peer-memory all-reduce + add kernel; and
    on a model whose column shards do not fall on block boundaries (every rank holds the covering blocks of attn_output, the feed-forward width is dealt
    in whole blocks). symmetric: the reduced buffers as a registered NCCL window (where the library has them) or as plain device memory."""
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "child.py"
    script.write_text(NCCL_CHILD)
    env = dict(os.environ, DOOMS_ROOT=str(ROOT), DOOMS_TP_MODEL=str(tmp_path / "tp.gguf"), NCCL_NVLS_ENABLE="0", DOOMS_TP_ALLREDUCE=allreduce, DOOMS_TP_CASE=case, DOOMS_TP_SYMMETRIC=symmetric)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port",
                        "29534", str(script)], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "tp ok 2" in r.stdout
