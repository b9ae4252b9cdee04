"""Several sequences on one decoder: KV-cache slots, and decode steps that run all of them at once (decode_batch). Each sequence's tokens are held to the
CPU checker run on that sequence alone, with the checker rounding operands to f16 where the step's tensor-core tiles do (every projection of the step,
the output projection included); a token may differ only where the checker's two best logits are closer than the benchmark's logit bound, and the
comparison of that sequence ends there. The same sequences run singly on the decoder give the second comparison the serving configuration asks for."""
import numpy as np
import pytest

from dooms_b200 import CudaLlamaDecoder, synth
from dooms_b200 import _lib as L
from dooms_b200._lib import DoomsError
from oracle import binding as ob

from helpers import QUANT_PLANS, write

pytestmark = pytest.mark.gpu

ABS_TOL, REL_TOL = 2e-2, 1e-2
LENGTHS = [3, 11, 40, 70, 130, 257]


def prompts(n_vocab):
    return [[int(t) for t in synth.prompt_tokens(n, n_vocab, 300 + i)] for i, n in enumerate(LENGTHS)]


def near_tie(logits, a, b):
    return abs(logits[a] - logits[b]) <= ABS_TOL + REL_TOL * max(abs(logits[a]), abs(logits[b]))


@pytest.fixture(scope="module")
def model(model_dir):
    return write(model_dir, "batch_mix", synth.tiny_spec(QUANT_PLANS["q4_0"], n_vocab=200), 41)


def checker_tokens(path, prompt, steps, n_ctx=512):
    """(pending token, [(token, logits)] of `steps` steps) of one sequence alone: the prompt as one chunk, then single positions through the chunk tiles."""
    o = ob.OracleDecoder(path, n_ctx, round_operands=True)
    logits = o.eval_tokens(prompt)
    o.set_round_operands(2)
    pending = ob.argmax(logits)
    out, t = [], pending
    for _ in range(steps):
        logits = o.eval_tokens([t])
        t = ob.argmax(logits)
        out.append((t, logits))
    o.close()
    return pending, out


def compare(got_tokens, want):
    """got_tokens against [(token, logits)]: equal until the first near tie, nothing else."""
    for step, (g, (w, logits)) in enumerate(zip(got_tokens, want)):
        if int(g) != w:
            assert near_tie(logits, int(g), w), (step, int(g), w, logits[w] - logits[int(g)])
            return step
    return len(want)


def test_batched_steps_match_each_sequence_alone(model):
    dec = CudaLlamaDecoder.load(model, 512, 320, max_sequences=8)
    assert dec.max_sequences() == 8 and dec.max_batch_rows() >= 6
    ps = prompts(200)
    pend = []
    for s, p in enumerate(ps):
        dec.select_sequence(s)
        dec.eval_tokens(p)
        pend.append(dec.pending_token())
    steps = 6
    slots = [0, 1, -1, 2, 3, 4, 5]                       # one idle row in the middle
    first = dec.decode_batch(slots, steps)
    second = dec.decode_batch(slots, 3)                   # the slots carry their state from call to call
    got = np.concatenate([first, second], axis=0)
    assert got.shape == (9, 7) and np.all(got[:, 2] == -1)
    agreed = 0
    for row, s in enumerate(slots):
        if s < 0:
            continue
        pending, want = checker_tokens(model, ps[s], 9)
        assert pend[s] == pending
        agreed += compare(got[:, row], want)
        dec.select_sequence(s)
        assert dec.position() == len(ps[s]) + 9 and dec.pending_token() == int(got[-1, row])
    assert agreed >= 6 * 9 * 0.8                          # near ties are the exception, not the rule


@pytest.mark.parametrize("head_dim", [64, 128])
def test_long_rows_spread_over_several_ranges(model_dir, head_dim):
    """Rows of very different lengths in one step, the longest spread over three ranges of the cache whose results are merged by the last block to finish;
    key/value heads of 64 and of 128 elements (two tile sizes of the tensor-core attention), three query heads per key/value head."""
    spec = synth.tiny_spec(QUANT_PLANS["q4_0"], n_embd=6 * head_dim, n_head=6, n_head_kv=2, n_ff=1024, n_vocab=200, context_length=2048)
    path = write(model_dir, f"batch_long_{head_dim}", spec, 43)
    lengths = [5, 300, 515, 1100, 1290]
    ps = [[int(t) for t in synth.prompt_tokens(n, 200, 900 + i)] for i, n in enumerate(lengths)]
    dec = CudaLlamaDecoder.load(path, 1300, 512, max_sequences=5)
    pend = []
    for s, p in enumerate(ps):
        dec.select_sequence(s)
        dec.eval_tokens(p)
        pend.append(dec.pending_token())
    steps = 5
    got = dec.decode_batch([4, 3, 2, 1, 0], steps)
    agreed = 0
    for row, s in enumerate([4, 3, 2, 1, 0]):
        pending, want = checker_tokens(path, ps[s], steps, n_ctx=1300)
        if pend[s] != pending:
            continue                                      # the prompt itself ended on a near tie: nothing to follow
        agreed += compare(got[:, row], want)
    assert agreed >= 5 * steps * 0.8
    dec.close()


def test_batched_steps_match_the_same_sequences_run_singly(model):
    """What the serving configuration states: per-sequence tokens checked against single-sequence runs of the same decoder code (one position per call
    there: f32 activations, exact weights, so the two differ by the tiles' operand rounding and may part at a near tie)."""
    ps = prompts(200)
    dec = CudaLlamaDecoder.load(model, 512, 320, max_sequences=6)
    for s, p in enumerate(ps):
        dec.select_sequence(s)
        dec.eval_tokens(p)
    got = dec.decode_batch(list(range(6)), 8)
    single = CudaLlamaDecoder.load(model, 512, 320)
    same = 0
    for s, p in enumerate(ps):
        single.reset()
        single.eval_tokens(p)
        toks = []
        single.generate(9, 2, lambda t: toks.append(t) or True)      # the pending token first, then 8 more
        _, want = checker_tokens(model, p, 8)
        for step in range(8):
            if int(got[step, s]) != toks[step + 1]:
                assert near_tie(want[step][1], int(got[step, s]), toks[step + 1]), (s, step)
                break
            same += 1
    assert same >= 6 * 8 * 0.8
    dec.close()
    single.close()


def test_a_slot_continues_alone_after_batched_steps(model):
    ps = prompts(200)
    dec = CudaLlamaDecoder.load(model, 512, 320, max_sequences=3)
    for s in range(3):
        dec.select_sequence(s)
        dec.eval_tokens(ps[s + 1])
    got = dec.decode_batch([0, 1, 2], 4)
    dec.select_sequence(1)
    toks = []
    dec.generate(4, 2, lambda t: toks.append(t) or True)
    assert toks[0] == int(got[-1, 1])                                 # the pending token is the last one the batch produced
    # the same continuation from a fresh decoder that is fed the batch's tokens one by one
    ref = CudaLlamaDecoder.load(model, 512, 320)
    ref.eval_tokens(ps[2])
    fed = [ref.pending_token()] + [int(t) for t in got[:-1, 1]]
    for t in fed:
        ref.eval_tokens([t])
    want = []
    ref.generate(4, 2, lambda t: want.append(t) or True)
    assert toks[1:] == want[1:] or toks[0] != want[0]                 # same cache contents up to the tiles' rounding: the tokens follow unless a tie intervened
    dec.close()
    ref.close()


def test_decode_batch_refusals(model):
    one = CudaLlamaDecoder.load(model, 64, 32)
    with pytest.raises(DoomsError) as e:
        one.decode_batch([0], 1)
    assert e.value.code == L.UNSUPPORTED
    one.close()
    dec = CudaLlamaDecoder.load(model, 64, 32, max_sequences=4)
    dec.eval_tokens([1, 2, 3])
    for slots, steps, code in (([0, 0], 1, L.INVALID_ARGUMENT), ([4], 1, L.INVALID_ARGUMENT), ([1], 1, L.INVALID_ARGUMENT), ([0], 0, L.INVALID_ARGUMENT),
                               ([0], 257, L.INVALID_ARGUMENT), ([0], 62, L.RESOURCE_EXHAUSTED), ([0, -1, -1, -1, -1], 1, L.RESOURCE_EXHAUSTED)):
        with pytest.raises(DoomsError) as e:
            dec.decode_batch(slots, steps)
        assert e.value.code == code, (slots, steps)
    with pytest.raises(DoomsError) as e:
        dec.select_sequence(4)
    assert e.value.code == L.INVALID_ARGUMENT
    assert dec.decode_batch([0], 2).shape == (2, 1) and dec.position() == 5
    dec.close()
