"""The benchmark configurations at their real shapes (0.5B q4_0, 0.5B mixed k-quants, 8B q4_0) with seeded synthetic weights: prompt logits and
teacher-forced greedy tokens against the CPU checker's fast port, within the benchmark's own bound for logits (2e-2 absolute / 1e-2 relative). The prompts
are short because the checker runs at ~10 (0.5B) and ~0.7 (8B) tokens per second; the long-prompt cases live in test_decoder_gpu.py on small models."""
import os
import tempfile

import numpy as np
import pytest

from dooms_b200 import CudaLlamaDecoder, synth
from oracle import binding as ob

pytestmark = pytest.mark.gpu

ABS_TOL, REL_TOL = 2e-2, 1e-2


def model_path(config):
    """The same file name bench.py uses, so one box generates each model once."""
    spec = synth.config_spec(config)
    path = os.path.join(os.environ.get("DOOMS_BENCH_DIR", tempfile.gettempdir()), f"dooms_bench_config{config}_seed{1000 + config}.gguf")
    if not os.path.exists(path):
        tmp = path + f".tmp{os.getpid()}"
        synth.write_model(spec, tmp, 1000 + config, device="cuda")
        os.replace(tmp, path)
    return path, spec


def close_enough(got, want):
    return bool(np.all(np.abs(got - want) <= ABS_TOL + REL_TOL * np.abs(want)))


@pytest.mark.parametrize("config,n_prompt,n_decode", [(0, 80, 6), (1, 80, 6), (2, 5, 2)])
def test_configuration_shape_matches_the_checker(config, n_prompt, n_decode):
    path, spec = model_path(config)
    prompt = [int(t) for t in synth.prompt_tokens(n_prompt, spec.n_vocab, 2000 + config)]
    o = ob.OracleDecoder(path, n_prompt + n_decode + 2, fast=True)
    dec = CudaLlamaDecoder.load(path, 256, 128)
    want = o.eval_tokens(prompt)
    dec.eval_tokens(prompt)                          # one call: the tensor-core prefill path where the widths allow
    got = dec.logits().astype(np.float64)
    # the prefill tiles round both operands to f16 as the reference's do (llama_kernels.h:186-199): within the bound of the checker run with that
    # rounding, and within twice the bound of the exact one (on the 8B shape the rounding alone moves the exact logits by up to ~3e-2)
    o_r = ob.OracleDecoder(path, n_prompt + 2, fast=True, round_operands=True)
    rounded = o_r.eval_tokens(prompt)
    o_r.close()
    assert close_enough(got, rounded), np.abs(got - rounded).max()
    assert bool(np.all(np.abs(got - want) <= 2 * (ABS_TOL + REL_TOL * np.abs(want)))), np.abs(got - want).max()
    for _ in range(n_decode):
        tok_want, tok_got = ob.argmax(want), dec.pending_token()
        # equal unless the checker's two candidates are closer than the logit bound (a near tie)
        assert tok_got == tok_want or want[tok_want] - want[tok_got] <= 2 * (ABS_TOL + REL_TOL * abs(want[tok_want])), (tok_got, tok_want)
        want = o.eval_tokens([tok_want])            # teacher-forced: both sides continue with the checker's token
        dec.eval_tokens([tok_want])
        got = dec.logits().astype(np.float64)
        assert close_enough(got, want), np.abs(got - want).max()
    dec.close()
    o.close()
