"""Writes tests/golden/byte_bpe_tiny.json: a small byte-level BPE vocabulary (the tokenizer family GGUF calls "gpt2": the 256 bytes in the GPT-2 byte
alphabet, merges by rank) trained here with the `tokenizers` library on seeded synthetic text, and the ids that library gives for a list of test texts.
The test (tests/test_llm.py) builds a GGUF vocabulary from tokens and merges and holds this backend's tokenizer to those ids without needing the library.
The texts stay inside what this backend's word splitter and the GPT-2 pre-tokenizer split alike: letters, digits and punctuation runs with single or
double spaces; no contractions ('s, 're ...), no runs of three or more spaces, no line breaks.

    python tests/golden/make_byte_bpe_fixture.py
"""
import json
import random
from pathlib import Path

from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers

WORDS = ["hello", "world", "the", "quick", "brown", "fox", "jumps", "over", "lazy", "dog", "token", "model", "decode", "prefill", "cache", "layer", "norm",
         "weight", "block", "scale", "héllo", "naïve", "data", "stream", "byte", "pair", "merge", "score", "2048", "256", "x86", "a,b", "end."]
TEXTS = ["hello world", "the quick brown fox jumps over the lazy dog", "hello", " hello", "hello  world", "decode the token stream", "héllo naïve",
         "prefillcache", "scalescalescale", "x", "the the the", "Weight Block", "a b c d e f g", "merge pair byte score data", "x86 2048 256 a,b end.",
         "trailing space ", "modelmodel layer.norm", "snowman ☃ here", "日本 语言", "1 + 1 = 2;", "(hello) [world] {the}"]


def main():
    rng = random.Random(6)
    lines = [" ".join(rng.choice(WORDS) for _ in range(rng.randint(3, 12))) for _ in range(3000)]
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=420, initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), special_tokens=["<|endoftext|>"], show_progress=False)
    tok.train_from_iterator(lines, trainer)
    model = json.loads(tok.to_str())["model"]
    tokens = [t for t, _ in sorted(model["vocab"].items(), key=lambda kv: kv[1])]
    merges = [" ".join(m) if isinstance(m, list) else m for m in model["merges"]]
    import tokenizers
    out = {"tokens": tokens, "merges": merges, "end_of_text": tokens.index("<|endoftext|>"), "tokenizers_version": tokenizers.__version__,
           "cases": [{"text": t, "ids": tok.encode(t).ids} for t in TEXTS]}
    path = Path(__file__).resolve().parent / "byte_bpe_tiny.json"
    path.write_text(json.dumps(out, ensure_ascii=True, indent=0), encoding="utf-8")
    print(f"wrote {path}: {len(tokens)} tokens, {len(merges)} merges, {len(TEXTS)} cases")


if __name__ == "__main__":
    main()
