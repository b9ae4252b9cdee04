"""Writes tests/golden/byte_bpe_tiny.json: a small byte-level BPE vocabulary (the tokenizer family GGUF calls "gpt2": the 256 bytes in the GPT-2 byte
alphabet, merges by rank) trained here with the `tokenizers` library on seeded synthetic text, and the ids that library gives for a list of test texts.
The test (tests/test_llm.py) builds a GGUF vocabulary from tokens and merges and holds this backend's tokenizer to those ids without needing the library.
Each case names the pre-tokenizer it was encoded with ("gpt-2", "llama-bpe", "qwen2": the regular expressions those model families split text with
before merging, applied here through the library's regex engine); the fixed texts are followed by seeded random mixtures of words, digits, punctuation,
contractions, spaces, line breaks and non-ASCII letters, digits and spaces.

    python tests/golden/make_byte_bpe_fixture.py
"""
import json
import random
from pathlib import Path

from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers

WORDS = ["hello", "world", "the", "quick", "brown", "fox", "jumps", "over", "lazy", "dog", "token", "model", "decode", "prefill", "cache", "layer", "norm",
         "weight", "block", "scale", "héllo", "naïve", "data", "stream", "byte", "pair", "merge", "score", "2048", "256", "x86", "a,b", "end."]
TEXTS = ["hello world", "the quick brown fox jumps over the lazy dog", "hello", " hello", "hello  world", "decode the token stream", "héllo naïve",
         "prefillcache", "scalescalescale", "x", "the the the", "Weight Block", "a b c d e f g", "merge pair byte score data", "x86 2048 256 a,b end.",
         "trailing space ", "modelmodel layer.norm", "snowman ☃ here", "日本 语言", "1 + 1 = 2;", "(hello) [world] {the}"]


PATTERNS = {
    "gpt-2": None,      # the library's own ByteLevel pre-tokenizer (GPT-2's pattern)
    "llama-bpe": r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+",
    "qwen2": r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+",
}
PIECES = WORDS + ["1", "12", "1234567", "3.14", "!", "?", "...", ",", ";", "(", ")", "[x]", "{", "}", "<=", "->", "_", "\"", "'s", "'S", "'re", "'RE", "'ll", "n't", "'d", "'ve",
                  "'", "''", " ", " ", " ", "  ", "   ", "\n", "\n\n", "\t", " \n ", "\r\n", "\u00e9", "\u00df", "\u65e5\u672c", "\u044f\u0437\u044b\u043a", "\u0663",
                  "\u00bd", "\U0001F600", "\u00a0", "\u3000", "I", "I'm", "DON'T", "It's"]


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
    vocab = {t: i for i, t in enumerate(tokens)}
    pairs = [tuple(m.split(" ")) for m in merges]
    cases = []
    for name, pattern in PATTERNS.items():
        enc = Tokenizer(models.BPE(vocab=vocab, merges=pairs, ignore_merges=(name == "llama-bpe")))
        if pattern is None:
            enc.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
        else:
            enc.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(pattern), behavior="isolated", invert=False),
                                                         pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
        texts = list(TEXTS) + ["".join(rng.choice(PIECES) for _ in range(rng.randint(2, 14))) for _ in range(120)]
        cases += [{"pre": name, "text": t, "ids": enc.encode(t).ids} for t in texts if t]
    out = {"tokens": tokens, "merges": merges, "end_of_text": tokens.index("<|endoftext|>"), "tokenizers_version": tokenizers.__version__, "cases": cases}
    path = Path(__file__).resolve().parent / "byte_bpe_tiny.json"
    path.write_text(json.dumps(out, ensure_ascii=True, indent=0), encoding="utf-8")
    print(f"wrote {path}: {len(tokens)} tokens, {len(merges)} merges, {len(cases)} cases")


if __name__ == "__main__":
    main()
