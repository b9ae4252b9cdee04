"""The text-model surface (reference: src/pipeline/llm_pipeline.{h,cpp}; C face include/dooms/dooms_c.h:73-138): vocabulary, text assembly with UTF-8
hold-back and stop strings, sampler on the host (no GPU), and generation on the decoder (GPU)."""
import numpy as np
import pytest

from dooms_b200 import _lib as L
from dooms_b200 import synth
from dooms_b200._lib import DoomsError
from dooms_b200.llm import Llm, Vocab, sample

from helpers import QUANT_PLANS

N_VOCAB = 320
EOS = N_VOCAB - 1


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    path = str(tmp_path_factory.mktemp("llm") / "llm_tiny.gguf")
    synth.write_model(synth.tiny_spec(QUANT_PLANS["q4_0"], n_vocab=N_VOCAB), path, 77, vocab=True)
    return path


def test_vocabulary_round_trips_text_and_merges_by_rank(model):
    v = Vocab(model)
    assert len(v) == N_VOCAB and v.is_end_of_generation(EOS) and not v.is_end_of_generation(5) and v.piece(EOS) == b""
    text = "hello world, the héllo 42 \U0001F600!"
    ids = v.tokenize(text)
    assert b"".join(v.piece(t) for t in ids) == text.encode()
    assert len(ids) < len(text.encode())                       # merges happened
    assert v.tokenize("hello") == [v.tokenize("hello")[0]] and v.piece(v.tokenize("hello")[0]) == b"hello"      # h e l l o -> he ll o -> hell o -> hello
    assert v.piece(v.tokenize(" world")[0]) == b" world"
    assert all(v.piece(b) == bytes([b]) for b in range(256))   # the byte alphabet undone
    with pytest.raises(DoomsError) as e:
        v.tokenize("")
    assert e.value.code == L.INVALID_ARGUMENT


def test_sentencepiece_vocabulary_merges_by_score_and_falls_back_to_bytes(tmp_path):
    """A sentencepiece vocabulary (tokenizer.ggml.model = llama): a space in front, spaces as U+2581, pairs merged best score first, characters the
    vocabulary lacks as <0xHH> byte tokens; the pieces of the ids give the text back (with the space put in front)."""
    path = str(tmp_path / "spm_tiny.gguf")
    synth.write_model(synth.tiny_spec(QUANT_PLANS["q4_0"], n_vocab=N_VOCAB), path, 78, vocab="sentencepiece")
    v = Vocab(path)
    tok = {v.piece(i): i for i in range(3 + 256, 3 + 256 + 46) if v.piece(i)}
    assert v.tokenize("hello world", add_special=False) == [tok[b" hello"], tok[b" world"]]
    assert v.tokenize("hello world") == [1, tok[b" hello"], tok[b" world"]]                       # the file asks for its <s> in front
    assert v.tokenize("the hell", add_special=False) == [tok[b" the"], tok[b" "], tok[b"hell"]]   # no piece " hell": a space piece, then the best-scoring split
    text = "hello w\u00e9 the!"
    ids = v.tokenize(text, add_special=False)
    assert b"".join(v.piece(t) for t in ids) == (" " + text).encode()
    assert [t for t in ids if 3 <= t < 259] == [3 + b for b in "\u00e9".encode()]                  # the accented letter went out as its two bytes
    assert v.piece(1) == b"" and v.is_end_of_generation(2)


def test_sentencepiece_tokenizer_matches_the_sentencepiece_library(tmp_path):
    """The ids the sentencepiece library itself gives for a BPE model with byte fallback trained on synthetic text (tests/golden/sentencepiece_tiny.json,
    written by tests/golden/make_sentencepiece_fixture.py) are what Vocab.tokenize gives for the same pieces and scores read from a GGUF file: the
    reference gets this tokenizer from llama.cpp (src/models/vlm/text_decoder.cpp:123-145), whose "llama" tokenizer follows the same library."""
    import json
    from pathlib import Path
    from dooms_b200.gguf_io import GgufWriter
    whole = json.loads((Path(__file__).parent / "golden" / "sentencepiece_tiny.json").read_text())
    for fx, space_prefix in ((whole["no_space_prefix"], False), (whole, True)):
        path = str(tmp_path / f"spm_golden_{int(space_prefix)}.gguf")
        md = {"general.architecture": "llama", "tokenizer.ggml.model": "llama", "tokenizer.ggml.tokens": fx["pieces"], "tokenizer.ggml.scores": [float(x) for x in fx["scores"]],
              "tokenizer.ggml.token_type": fx["types"], "tokenizer.ggml.bos_token_id": fx["bos"], "tokenizer.ggml.eos_token_id": fx["eos"], "tokenizer.ggml.add_bos_token": True}
        if not space_prefix:
            md["tokenizer.ggml.add_space_prefix"] = False
        GgufWriter().write(path, md, [])
        v = Vocab(path)
        assert len(v) == len(fx["pieces"])
        for case in fx["cases"]:
            assert v.tokenize(case["text"], add_special=False) == case["ids"], (space_prefix, case["text"])
            assert b"".join(v.piece(t) for t in case["ids"]) == ((" " if space_prefix else "") + case["text"]).encode()      # the pieces give the text back
    assert v.tokenize("hello world") == [fx["bos"]] + fx["cases"][0]["ids"]


@pytest.mark.parametrize("pre", ["gpt-2", "llama-bpe", "qwen2"])
def test_byte_level_bpe_tokenizer_matches_the_tokenizers_library(tmp_path, pre):
    """The ids the `tokenizers` library gives for a byte-level BPE vocabulary trained on synthetic text (tests/golden/byte_bpe_tiny.json, written by
    tests/golden/make_byte_bpe_fixture.py) are what Vocab.tokenize gives for the same tokens and merges read from a GGUF file, for each of the three
    pre-tokenizers a file can name in tokenizer.ggml.pre: fixed texts plus seeded random mixtures of words, digits, punctuation, contractions, spaces,
    line breaks and non-ASCII characters. The reference gets its tokenizer from llama.cpp (src/models/vlm/text_decoder.cpp:123-145), which applies the
    same patterns."""
    import json
    from pathlib import Path
    from dooms_b200.gguf_io import GgufWriter
    fx = json.loads((Path(__file__).parent / "golden" / "byte_bpe_tiny.json").read_text())
    n, eot = len(fx["tokens"]), fx["end_of_text"]
    path = str(tmp_path / "bpe_golden.gguf")
    GgufWriter().write(path, {"general.architecture": "llama", "tokenizer.ggml.model": "gpt2", "tokenizer.ggml.pre": pre, "tokenizer.ggml.tokens": fx["tokens"],
                              "tokenizer.ggml.merges": fx["merges"], "tokenizer.ggml.token_type": [3 if i == eot else 1 for i in range(n)],
                              "tokenizer.ggml.eos_token_id": eot, "tokenizer.ggml.bos_token_id": eot, "tokenizer.ggml.add_bos_token": False}, [])
    v = Vocab(path)
    cases = [c for c in fx["cases"] if c["pre"] == pre]
    assert len(cases) > 100
    for case in cases:
        assert v.tokenize(case["text"], add_special=False) == case["ids"], case["text"]
        assert b"".join(v.piece(t) for t in case["ids"]) == case["text"].encode()
    assert v.tokenize("hello<|endoftext|>", add_special=False, parse_special=True) == v.tokenize("hello", add_special=False) + [eot] and v.is_end_of_generation(eot)


def test_tokenizers_agree_with_their_libraries_on_random_text(tmp_path):
    """Live differential run where the `tokenizers` and `sentencepiece` packages are installed (skipped otherwise; the committed fixtures above hold without
    them): seeded random mixtures that include unusual spaces, digits and letters of other scripts, combining marks and long digit runs."""
    import json
    import random
    import sys
    from pathlib import Path
    tk = pytest.importorskip("tokenizers")
    spm = pytest.importorskip("sentencepiece")
    golden = Path(__file__).parent / "golden"
    sys.path.insert(0, str(golden))
    try:
        import make_byte_bpe_fixture as B
        import make_sentencepiece_fixture as S
    finally:
        sys.path.pop(0)
    from dooms_b200.gguf_io import GgufWriter
    rng = random.Random(17)
    fx = json.loads((golden / "byte_bpe_tiny.json").read_text())
    tokens, merges, eot = fx["tokens"], fx["merges"], fx["end_of_text"]
    vocab, pairs = {t: i for i, t in enumerate(tokens)}, [tuple(m.split(" ")) for m in merges]
    pieces = B.PIECES + ["\u2003", "\u2028", "\u202f", "\u0085", "\v", "\f", "\r", "\u0663\u0664\u0665", "\u216b", "\u01c5", "\u02b0", "\u093c", "\u203f", "\u20ac", "\u200b",
                         "\ufeff", "a\u0301", "\ufb01", "\U0001d518", "\U0001d7d8", "Z\u00dcRICH", "'Ll", "'T", "'M", "9" * 7, "ab12cd", "x'sy", "\n\n\n ", " \t\n", "\n a",
                         "  a", "\t\ta", "end\n", "!!\n\nX", " !\r\n\r\nq"]
    for name, pattern in B.PATTERNS.items():
        enc = tk.Tokenizer(tk.models.BPE(vocab=vocab, merges=pairs, ignore_merges=(name == "llama-bpe")))
        if pattern is None:
            enc.pre_tokenizer = tk.pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
        else:
            enc.pre_tokenizer = tk.pre_tokenizers.Sequence([tk.pre_tokenizers.Split(tk.Regex(pattern), behavior="isolated", invert=False),
                                                            tk.pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
        path = str(tmp_path / f"fuzz_{name}.gguf")
        GgufWriter().write(path, {"general.architecture": "llama", "tokenizer.ggml.model": "gpt2", "tokenizer.ggml.pre": name, "tokenizer.ggml.tokens": tokens,
                                  "tokenizer.ggml.merges": merges, "tokenizer.ggml.token_type": [3 if i == eot else 1 for i in range(len(tokens))],
                                  "tokenizer.ggml.eos_token_id": eot, "tokenizer.ggml.bos_token_id": eot, "tokenizer.ggml.add_bos_token": False}, [])
        v = Vocab(path)
        for _ in range(1500):
            text = "".join(rng.choice(pieces) for _ in range(rng.randint(1, 10)))
            assert v.tokenize(text, add_special=False) == enc.encode(text).ids, (name, text)
    corpus = tmp_path / "corpus.txt"
    words = random.Random(5)
    corpus.write_text("\n".join(" ".join(words.choice(S.WORDS) for _ in range(words.randint(3, 12))) for _ in range(3000)), encoding="utf-8")
    sp = S.train(str(tmp_path), corpus, True)
    d = S.describe(sp)
    path = str(tmp_path / "fuzz_spm.gguf")
    GgufWriter().write(path, {"general.architecture": "llama", "tokenizer.ggml.model": "llama", "tokenizer.ggml.tokens": d["pieces"],
                              "tokenizer.ggml.scores": [float(x) for x in d["scores"]], "tokenizer.ggml.token_type": d["types"], "tokenizer.ggml.bos_token_id": 1,
                              "tokenizer.ggml.eos_token_id": 2}, [])
    v = Vocab(path)
    pieces = S.WORDS + [" ", " ", "  ", "\n", "\t", "x", "q", "Z", "1", "23", ".", ",", "!", "\u00e9", "\u65e5", "\u672c", "\u2603", "\U0001F600", "ll", "he", "th", "e", "o", "s"]
    for _ in range(3000):
        text = "".join(rng.choice(pieces) for _ in range(rng.randint(1, 12)))
        assert v.tokenize(text, add_special=False) == sp.encode(text, out_type=int), text


def _chat_file(tmp_path, family):
    path = str(tmp_path / f"chat_{family}.gguf")
    synth.write_model(synth.tiny_spec(QUANT_PLANS["q4_0"], n_vocab=N_VOCAB), path, 79, vocab=family)
    return path


CONVERSATION = [("system", "the world"), ("user", " hello world \n"), ("assistant", "hello"), ("user", "the")]


def test_chat_templates_are_written_by_family_and_their_control_tokens_are_parsed(tmp_path):
    """apply_chat_template (src/models/vlm/text_decoder.cpp:257-278): the family is read off the template's markers, the conversation is written in that
    family's format; tokenizing it with parse_special gives the control tokens' own ids around the plainly tokenized text."""
    v = Vocab(_chat_file(tmp_path, "chatml"))
    text = v.apply_chat_template(CONVERSATION)
    assert text == "".join(f"<|im_start|>{r}\n{c}<|im_end|>\n" for r, c in CONVERSATION) + "<|im_start|>assistant\n"
    assert v.apply_chat_template(CONVERSATION[:2], add_generation_prompt=False) == "<|im_start|>system\nthe world<|im_end|>\n<|im_start|>user\n hello world \n<|im_end|>\n"
    start, end = N_VOCAB - 3, N_VOCAB - 2
    ids = v.tokenize("<|im_start|>user\nhello world<|im_end|>\n", add_special=False, parse_special=True)
    assert ids == [start] + v.tokenize("user\nhello world", add_special=False) + [end] + v.tokenize("\n", add_special=False)
    plain = v.tokenize("<|im_start|>user", add_special=False)                       # without parse_special the marker is ordinary text
    assert start not in plain and b"".join(v.piece(t) for t in plain) == b"<|im_start|>user"
    assert v.is_end_of_generation(end) and v.is_end_of_generation(N_VOCAB - 1) and v.piece(start) == b""

    v3 = Vocab(_chat_file(tmp_path, "llama3"))
    want = "".join(f"<|start_header_id|>{r}<|end_header_id|>\n\n{c.strip()}<|eot_id|>" for r, c in CONVERSATION) + "<|start_header_id|>assistant<|end_header_id|>\n\n"
    assert v3.apply_chat_template(CONVERSATION) == want
    ids3 = v3.tokenize(want, add_special=False, parse_special=True)
    assert ids3.count(N_VOCAB - 4) == 5 and ids3.count(N_VOCAB - 3) == 5 and ids3.count(N_VOCAB - 2) == 4 and v3.is_end_of_generation(N_VOCAB - 2)

    vs = Vocab(_chat_file(tmp_path, "smolvlm"))      # the text model of the reference's vision-language pipeline: system text, then "User:" / "Assistant:" turns
    assert vs.apply_chat_template(CONVERSATION) == ("<|im_start|>the world\n\nUser:  hello world \n<end_of_utterance>\nAssistant: hello<end_of_utterance>\n"
                                                    "User: the<end_of_utterance>\nAssistant:")
    assert vs.tokenize("<|im_start|>User: the<end_of_utterance>", add_special=False, parse_special=True)[::len(vs.tokenize("User: the", add_special=False)) + 1] == \
        [N_VOCAB - 3, N_VOCAB - 2]

    # refusals: no messages, an empty role, no template in the file, a template of an unknown family (text_decoder.cpp:259-276)
    for vocab, messages, code in ((v, [], L.INVALID_ARGUMENT), (v, [("", "x")], L.INVALID_ARGUMENT), (Vocab(_chat_file(tmp_path, True)), CONVERSATION, L.UNSUPPORTED),
                                  (Vocab(_chat_file(tmp_path, "other")), CONVERSATION, L.UNSUPPORTED)):
        with pytest.raises(DoomsError) as e:
            vocab.apply_chat_template(messages)
        assert e.value.code == code


def test_pieces_are_whole_characters_and_stop_strings_end_the_text(model):
    v = Vocab(model)
    # U+00E9 and an emoji arrive byte by byte: nothing incomplete is ever handed on
    ids = v.tokenize("aé\U0001F600b")
    pieces = []
    text, consumed, reason = v.stream(ids, on_text=lambda p: pieces.append(p) or True)
    assert text == "aé\U0001F600b" and "".join(pieces) == text and consumed == len(ids) and reason == L.FINISH_LENGTH
    assert all(p.encode().decode() == p for p in pieces) and len(pieces) >= 4
    # a stop string that spans tokens: the text ends before it, and its beginning was never shown
    ids = v.tokenize("the answer STOP and more")
    pieces = []
    text, consumed, reason = v.stream(ids, stop=["STOP", "never"], on_text=lambda p: pieces.append(p) or True)
    assert text == "the answer " and "".join(pieces) == text and reason == L.FINISH_STOP and consumed < len(ids)
    # what looked like the beginning of a stop string and was not is released
    text, _, reason = v.stream(v.tokenize("a STx b"), stop=["STOP"])
    assert text == "a STx b" and reason == L.FINISH_LENGTH
    # an end-of-generation token ends it; the token is consumed, text before it is kept
    ids = v.tokenize("hello") + [EOS] + v.tokenize("ignored")
    text, consumed, reason = v.stream(ids, stop=["zzz"])
    assert text == "hello" and consumed == len(v.tokenize("hello")) + 1 and reason == L.FINISH_STOP
    # the callback declines
    seen = []
    text, consumed, reason = v.stream(v.tokenize("one two three"), on_text=lambda p: (seen.append(p), len(seen) < 2)[1])
    assert reason == L.FINISH_CANCELLED and len(seen) == 2 and consumed < len(v.tokenize("one two three"))
    with pytest.raises(DoomsError):
        v.stream([1, 2], stop=[""])


def test_sampler_rules():
    logits = np.array([0.5, 3.0, 3.0, -1.0, np.nan, 2.0], dtype=np.float32)
    assert sample(logits) == [1]                                                     # greedy: the first of the largest, NaN never wins
    assert sample(logits, 5, temperature=0.8, top_k=1, seed=3) == [1] * 5            # top_k 1 is greedy
    a = sample(logits, 64, temperature=1.0, top_k=0, top_p=1.0, seed=11)
    assert a == sample(logits, 64, temperature=1.0, top_k=0, top_p=1.0, seed=11) and a != sample(logits, 64, temperature=1.0, top_k=0, top_p=1.0, seed=12)
    assert 4 not in a
    # frequencies follow softmax(logits / T) over the kept tokens
    lg = np.array([2.0, 1.0, 0.0, -1.0], dtype=np.float32)
    draws = np.array(sample(lg, 20000, temperature=1.0, top_k=3, top_p=1.0, seed=5))
    p = np.exp(lg[:3]) / np.exp(lg[:3]).sum()
    freq = np.array([(draws == i).mean() for i in range(3)])
    assert np.abs(freq - p).max() < 0.015 and (draws == 3).sum() == 0
    # top_p keeps the smallest prefix that reaches it
    assert set(sample(lg, 2000, temperature=1.0, top_k=0, top_p=0.6, seed=1)) == {0}
    # ... measured at temperature 1, before the temperature is applied (the order of the reference's chain, src/models/vlm/text_decoder.cpp:239-242): at
    # temperature 10 the three largest are nearly equally likely, yet the prefix is still the one token that holds 0.64 of the mass at temperature 1
    assert set(sample(lg, 2000, temperature=10.0, top_k=0, top_p=0.6, seed=1)) == {0}
    hot = np.array(sample(lg, 6000, temperature=10.0, top_k=0, top_p=0.9, seed=2))      # prefix {0, 1, 2} at temperature 1 (0.64 + 0.24 + 0.09), drawn from at 10
    want = np.exp(lg[:3] / 10.0) / np.exp(lg[:3] / 10.0).sum()
    assert set(hot) == {0, 1, 2} and np.abs(np.array([(hot == i).mean() for i in range(3)]) - want).max() < 0.02
    # the repetition penalty pushes a token that was just drawn down
    flat = np.array([1.0, 0.99], dtype=np.float32)
    assert sample(flat, 3, temperature=0.0, repeat_penalty=1.5)[:2] == [0, 1]
    for bad in (dict(temperature=-1.0), dict(top_p=0.0), dict(top_p=1.5), dict(top_k=-1), dict(repeat_penalty=0.0)):
        with pytest.raises(DoomsError) as e:
            sample(lg, 1, **bad)
        assert e.value.code == L.INVALID_ARGUMENT


@pytest.mark.gpu
def test_generation_matches_the_decoder_and_reports_how_it_ended(model):
    from dooms_b200 import CudaLlamaDecoder
    llm = Llm(model, n_ctx=256, n_batch=64, queue_depth=3)
    v = Vocab(model)
    prompt = "hello world the"
    ids = v.tokenize(prompt)
    assert llm.count_tokens(prompt) == len(ids) and llm.context_size() == 256
    # greedy text = the decoder's greedy tokens through the text assembly
    dec = CudaLlamaDecoder.load(model, 256, 64)
    dec.eval_tokens(ids)
    want = []
    dec.generate(24, 2, lambda t: want.append(t) or True)
    want_text, consumed, reason = v.stream(want)
    text = llm.generate(prompt, 24)
    info = llm.last_generation()
    assert text == want_text and info["prompt_tokens"] == len(ids) and info["completion_tokens"] == consumed
    assert info["finish_reason"] == (L.FINISH_STOP if reason == L.FINISH_STOP else L.FINISH_LENGTH) and info["first_token_ms"] > 0 and info["prefill_ms"] > 0
    text2, toks = llm.generate_tokens(ids, 24)
    assert text2 == text and toks == want[:consumed]
    # streaming gives the same text in whole-character pieces; declining stops it
    pieces = []
    assert llm.generate(prompt, 24, on_text=lambda p: pieces.append(p) or True) == text and "".join(pieces) == text
    seen = []
    llm.generate(prompt, 24, on_text=lambda p: (seen.append(p), False)[1])
    assert len(seen) == 1 and llm.last_generation()["finish_reason"] == L.FINISH_CANCELLED
    # a stop string taken from the middle of the greedy answer cuts it there
    if len(text) > 6 and text[3:6].isascii():
        stop = text[3:6]
        assert llm.generate(prompt, 24, stop=[stop]) == text[:text.index(stop)] and llm.last_generation()["finish_reason"] == L.FINISH_STOP
    # sampling: reproducible per seed, and the logits path agrees with the greedy path at temperature 0 with a penalty of 1
    a = llm.generate(prompt, 16, temperature=0.9, top_k=20, seed=4)
    assert a == llm.generate(prompt, 16, temperature=0.9, top_k=20, seed=4)
    by_logits = llm.generate_tokens(ids, 16, temperature=0.0, repeat_penalty=1.0000001)[1]      # not "greedy" to the library: every token comes from logits()
    assert by_logits == want[:len(by_logits)]
    # argument checks (llm_pipeline.cpp:137-145)
    for kwargs, code in ((dict(prompt="", max_new_tokens=4), L.INVALID_ARGUMENT), (dict(prompt=prompt, max_new_tokens=0), L.INVALID_ARGUMENT),
                         (dict(prompt=prompt, max_new_tokens=256), L.INVALID_ARGUMENT), (dict(prompt=prompt, max_new_tokens=4, stop=[""]), L.INVALID_ARGUMENT),
                         (dict(prompt=prompt * 40, max_new_tokens=200), L.RESOURCE_EXHAUSTED), (dict(prompt=prompt, max_new_tokens=4, temperature=-1.0), L.INVALID_ARGUMENT)):
        with pytest.raises(DoomsError) as e:
            llm.generate(**kwargs)
        assert e.value.code == code, kwargs
    dec.close()
    llm.close()


@pytest.mark.gpu
def test_chat_answers_the_templated_conversation(tmp_path):
    """Llm::chat (src/pipeline/llm_pipeline.cpp:233-247): the conversation through the file's chat template, tokenized with its control tokens parsed and
    no BOS, then generation as from any prompt; a file without a template refuses."""
    path = _chat_file(tmp_path, "chatml")
    llm, v = Llm(path, n_ctx=256, n_batch=64), Vocab(path)
    ids = v.tokenize(v.apply_chat_template(CONVERSATION), add_special=False, parse_special=True)
    assert llm.count_chat_tokens(CONVERSATION) == len(ids)
    want_text, want_tokens = llm.generate_tokens(ids, 20)
    assert llm.chat(CONVERSATION, 20) == want_text
    info = llm.last_generation()
    assert info["prompt_tokens"] == len(ids) and info["completion_tokens"] == len(want_tokens)
    pieces = []
    assert llm.chat([{"role": r, "content": c} for r, c in CONVERSATION], 20, on_text=lambda p: pieces.append(p) or True) == want_text and "".join(pieces) == want_text
    with pytest.raises(DoomsError) as e:
        llm.chat([], 4)
    assert e.value.code == L.INVALID_ARGUMENT
    llm.close()
    plain = Llm(_chat_file(tmp_path, True), n_ctx=256, n_batch=64)
    for call in (lambda: plain.chat(CONVERSATION, 4), lambda: plain.count_chat_tokens(CONVERSATION)):
        with pytest.raises(DoomsError) as e:
            call()
        assert e.value.code == L.UNSUPPORTED
    plain.close()


@pytest.mark.gpu
def test_text_side_of_a_vision_language_prompt(model):
    """generate_native of the reference's VLM pipeline (src/pipeline/vlm_pipeline.cpp:177-212): token rows + image rows + token rows as one embedding sequence.
    With the image rows taken from the embedding table the answer has to be the one the same tokens give; the table's rows are the checker's, bit for bit."""
    from dooms_b200 import CudaLlamaDecoder
    from oracle import binding as ob
    llm = Llm(model, n_ctx=256, n_batch=32)
    v = Vocab(model)
    before, middle, after = v.tokenize("hello the"), [7, 300, 12, 250, 99], v.tokenize(" world")
    dec = CudaLlamaDecoder.load(model, 64, 32)
    rows = dec.embed_tokens(middle)
    o = ob.OracleDecoder(model, 8)
    assert all(np.array_equal(rows[i], o.embedding(t)) for i, t in enumerate(middle))
    want_text, want_tokens = llm.generate_tokens(before + middle + after, 12)
    pieces = []
    got = llm.generate_from_embeddings(before, rows, after, 12, on_text=lambda p: pieces.append(p) or True)
    assert got == want_text and "".join(pieces) == got and llm.last_generation()["prompt_tokens"] == len(before) + 5 + len(after)
    # rows that are no token's: the sequence still runs (the decoder-level parity of eval_embeddings is in test_decoder_gpu.py)
    noise = np.random.default_rng(0).standard_normal((6, rows.shape[1])).astype(np.float32)
    assert isinstance(llm.generate_from_embeddings(before, noise, [], 4), str)
    for kwargs, code in ((dict(before=[], image=None, after=[], max_new_tokens=4), L.INVALID_ARGUMENT), (dict(before=before, image=np.full((1, rows.shape[1]), np.nan), after=[], max_new_tokens=4), L.INVALID_ARGUMENT),
                         (dict(before=before, image=rows, after=after, max_new_tokens=300), L.INVALID_ARGUMENT), (dict(before=before * 60, image=rows, after=[], max_new_tokens=100), L.RESOURCE_EXHAUSTED)):
        with pytest.raises(DoomsError) as e:
            llm.generate_from_embeddings(**kwargs)
        assert e.value.code == code
    with pytest.raises(DoomsError):
        dec.embed_tokens([N_VOCAB])
    dec.close()
    llm.close()
