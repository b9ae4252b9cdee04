"""Writes tests/golden/sentencepiece_tiny.json: a small sentencepiece BPE model (the tokenizer family GGUF calls "llama": pieces with scores, byte
fallback, a space in front) trained here on seeded synthetic text, and what the sentencepiece library itself makes of a list of test texts. The test
(tests/test_llm.py) builds a GGUF vocabulary from the pieces and holds this backend's tokenizer to those ids; it does not need the library.

    python tests/golden/make_sentencepiece_fixture.py

Needs the `sentencepiece` package. Training is single-threaded on a fixed corpus, so the output is reproducible."""
import json
import random
import tempfile
from pathlib import Path

import sentencepiece as spm

WORDS = ["hello", "world", "the", "quick", "brown", "fox", "jumps", "over", "lazy", "dog", "token", "model", "decode", "prefill", "cache", "layer", "norm",
         "weight", "block", "scale", "héllo", "naïve", "日本", "语言", "data", "stream", "byte", "pair", "merge", "score"]
TEXTS = ["hello world", "the quick brown fox jumps over the lazy dog", "hello", " hello", "hello  world", "decode the token stream", "héllo naïve 日本语言",
         "snowman ☃ and tab\tand newline\nend", "prefillcache", "scalescalescale", "x", "the the the", "Weight Block", "a b c d e f g", "merge pair byte score data",
         "日本", "trailing space ", "   ", "modelmodel layer.norm"]


def train(tmp: str, corpus: Path, dummy_prefix: bool):
    prefix = str(Path(tmp) / ("tiny" if dummy_prefix else "tiny_noprefix"))
    spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=prefix, vocab_size=400, model_type="bpe", byte_fallback=True, character_coverage=0.98,
                                   bos_id=1, eos_id=2, unk_id=0, pad_id=-1, normalization_rule_name="identity", add_dummy_prefix=dummy_prefix,
                                   remove_extra_whitespaces=False, num_threads=1, minloglevel=2)
    return spm.SentencePieceProcessor(model_file=prefix + ".model")


def describe(sp) -> dict:
    n = sp.get_piece_size()
    types = [2 if sp.is_unknown(i) else 3 if sp.is_control(i) else 6 if sp.is_byte(i) else 1 for i in range(n)]      # GGUF token types
    return {"pieces": [sp.id_to_piece(i) for i in range(n)], "scores": [sp.get_score(i) for i in range(n)], "types": types, "bos": sp.bos_id(), "eos": sp.eos_id(),
            "cases": [{"text": t, "ids": sp.encode(t, out_type=int)} for t in TEXTS]}


def main():
    rng = random.Random(5)
    with tempfile.TemporaryDirectory() as tmp:
        corpus = Path(tmp) / "corpus.txt"
        corpus.write_text("\n".join(" ".join(rng.choice(WORDS) for _ in range(rng.randint(3, 12))) for _ in range(3000)), encoding="utf-8")
        out = describe(train(tmp, corpus, True))
        out["no_space_prefix"] = describe(train(tmp, corpus, False))      # the same, from a model that puts no space in front (tokenizer.ggml.add_space_prefix = false)
    out["sentencepiece_version"] = spm.__version__
    path = Path(__file__).resolve().parent / "sentencepiece_tiny.json"
    path.write_text(json.dumps(out, ensure_ascii=True, indent=0), encoding="utf-8")
    print(f"wrote {path}: {len(out['pieces'])} pieces, {len(TEXTS)} cases, with and without the space in front")


if __name__ == "__main__":
    main()
