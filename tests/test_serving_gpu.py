"""Data-parallel serving of many sequences: every sequence's greedy tokens equal those of the same sequence run alone; the workload generator is seeded."""
import numpy as np
import pytest

from dooms_b200 import CudaLlamaDecoder, serving, synth
from dooms_b200 import _lib as L

from helpers import write


def test_workload_is_seeded_and_within_the_ranges():
    a = serving.workload(40, 1000, 3000)
    b = serving.workload(40, 1000, 3000)
    assert all(np.array_equal(x[0], y[0]) and x[1] == y[1] for x, y in zip(a, b))
    assert all(32 <= len(p) <= 4096 and 16 <= d <= 512 and p.min() >= 0 and p.max() < 1000 for p, d in a)
    assert serving.workload(3, 1000, 1)[0][1] != a[0][1] or not np.array_equal(serving.workload(3, 1000, 1)[0][0], a[0][0])


class FakeDecoder:
    """The decoder's slot interface with arithmetic a test can predict: a sequence's next token depends only on its own history, as the real steps'
    rows depend only on their own slot."""

    def __init__(self, slots):
        self.state = [None] * slots
        self.cur = 0
        self.calls = []

    @staticmethod
    def step(history):
        return (sum(history) * 31 + len(history) * 7) % 1009

    def select_sequence(self, s):
        self.cur = s

    def reset(self):
        self.state[self.cur] = []

    def eval_tokens(self, tokens):
        self.state[self.cur] = list(self.state[self.cur] or []) + [int(t) for t in tokens]

    def pending_token(self):
        return self.step(self.state[self.cur])

    def timings(self):
        return {"last_eval_ms": 1.0, "last_batch_ms": 1.0}

    def decode_batch(self, rows, steps):
        self.calls.append((list(rows), steps))
        out = np.full((steps, len(rows)), -1, dtype=np.int32)
        for k in range(steps):
            for r, slot in enumerate(rows):
                if slot >= 0:
                    h = self.state[slot]
                    h.append(self.step(h))          # the pending token is fed back ...
                    out[k, r] = self.step(h)        # ... and the next one comes out
        return out


def alone(prompt, n_decode):
    h = [int(t) for t in prompt]
    toks = [FakeDecoder.step(h)]
    for _ in range(n_decode - 1):
        h.append(toks[-1])
        toks.append(FakeDecoder.step(h))
    return toks


def test_continuous_batching_schedule_on_a_fake_decoder():
    """The scheduler alone (no GPU): every sequence gets the tokens it gets alone, no step is run for a finished sequence, slots are reused, and every
    call has max_live rows."""
    seqs = serving.workload(23, 1000, 7, prompt_range=(1, 9), decode_range=(1, 14))
    dec = FakeDecoder(5)
    tokens, stats = serving.run_continuous(dec, seqs, max_live=5, max_steps_per_call=4)
    assert tokens == [alone(p, d) for p, d in seqs]
    assert all(len(rows) == 5 and 1 <= steps <= 4 for rows, steps in dec.calls)
    assert stats["most_live"] == 5 and stats["steps"] == sum(steps for _, steps in dec.calls)
    assert sum(steps * sum(r >= 0 for r in rows) for rows, steps in dec.calls) == sum(d - 1 for _, d in seqs)      # no step beyond a sequence's end
    # the one-batch driver on the same fake
    dec = FakeDecoder(23)
    tokens, _ = serving.run_batched(dec, seqs)
    assert tokens == [alone(p, d) for p, d in seqs]


@pytest.mark.gpu
def test_sequences_served_concurrently_equal_single_runs(model_dir):
    import torch
    path = write(model_dir, "serve_q4_0", synth.tiny_spec(synth.pure(L.Q4_0)), 5)
    seqs = serving.workload(10, 50, 3000, prompt_range=(3, 70), decode_range=(2, 12))
    devices = [0, 1] if torch.cuda.device_count() > 1 else [0]
    tokens, stats = serving.serve(path, seqs, devices, n_ctx=96, n_batch=32, streams=2)      # two decoders per GPU, on their own streams
    assert stats["sequences"] == 10 and stats["generated_tokens"] == sum(d for _, d in seqs) and stats["decode_tok_s"] > 0
    dec = CudaLlamaDecoder.load(path, 96, 32)
    for (prompt, n_decode), got in zip(seqs, tokens):
        assert serving.run_sequence(dec, prompt, n_decode)[0] == got
    dec.close()


@pytest.mark.gpu
def test_sequences_served_as_one_batch_follow_single_runs(model_dir):
    """Each GPU's share as one batch (slots + decode_batch). The batched step rounds operands to f16 in its tensor-core tiles, a single run does not, so a
    sequence may part from its single run at a near tie; most tokens (and every first token, which comes from the same prefill) are equal."""
    import torch
    path = write(model_dir, "serve_batched_q4_0", synth.tiny_spec(synth.pure(L.Q4_0), n_vocab=200), 5)
    seqs = serving.workload(12, 200, 3000, prompt_range=(3, 90), decode_range=(2, 20))
    devices = [0, 1] if torch.cuda.device_count() > 1 else [0]
    tokens, stats = serving.serve_batched(path, seqs, devices, n_ctx=128, n_batch=64)
    assert stats["sequences"] == 12 and stats["generated_tokens"] == sum(d for _, d in seqs) and stats["decode_tok_s"] > 0
    dec = CudaLlamaDecoder.load(path, 128, 64)
    agree = total = 0
    for (prompt, n_decode), got in zip(seqs, tokens):
        alone = serving.run_sequence(dec, prompt, n_decode)[0]
        assert len(got) == n_decode and got[0] == alone[0]
        prefix = next((i for i, (a, b) in enumerate(zip(alone, got)) if a != b), n_decode)
        agree += prefix
        total += n_decode
    assert agree >= 0.8 * total
    dec.close()


@pytest.mark.gpu
def test_continuous_batching_gives_each_sequence_the_tokens_of_a_full_batch(model_dir):
    """Twelve sequences through four slots: prompts join as others finish. A row's arithmetic does not depend on its neighbours, so every sequence gets
    exactly the tokens it gets when all rows of a four-row batch are its own group (run_batched over the same four rows, idle rows included)."""
    path = write(model_dir, "serve_continuous_q4_0", synth.tiny_spec(synth.pure(L.Q4_0), n_vocab=200), 5)
    seqs = serving.workload(12, 200, 3001, prompt_range=(3, 90), decode_range=(1, 20))
    dec = CudaLlamaDecoder.load(path, 128, 64, max_sequences=4)
    tokens, stats = serving.run_continuous(dec, seqs, max_live=4)
    assert [len(t) for t in tokens] == [d for _, d in seqs]
    assert 2 <= stats["most_live"] <= 4 and stats["steps"] < sum(d for _, d in seqs)      # steps were shared
    # the same sequences four at a time, each group as one batch of four rows
    for g in range(0, 12, 4):
        want, _ = serving.run_batched(dec, seqs[g:g + 4])
        for i in range(4):
            assert tokens[g + i] == want[i][:len(tokens[g + i])], (g, i)
    # and against single runs: equal up to a near tie
    one = CudaLlamaDecoder.load(path, 128, 64)
    agree = total = 0
    for (prompt, n_decode), got in zip(seqs, tokens):
        alone = serving.run_sequence(one, prompt, n_decode)[0]
        assert got[0] == alone[0]
        agree += next((i for i, (a, b) in enumerate(zip(alone, got)) if a != b), n_decode)
        total += n_decode
    assert agree >= 0.8 * total
    dec.close()
    one.close()
