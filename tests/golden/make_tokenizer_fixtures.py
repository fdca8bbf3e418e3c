"""Builds the tokenizer fixtures with the HF `tokenizers` package (0.22.2, the version the reference's tl_runtime links:
crates/tl_runtime/src/tokenizer.rs): two small tokenizer.json files in the two styles the reference's chatbots load -
byte-level BPE with the Llama-3 split pattern, and SentencePiece-style BPE with byte fallback (TinyLlama / Llama-2) -
trained on a seeded synthetic corpus, and the ids / strings the package itself produces for a list of probe texts.

    python tests/golden/make_tokenizer_fixtures.py      (writes tokenizer_bytelevel.json, tokenizer_sp.json, tokenizer_golden.json)
"""
import json
import os
import random

from tokenizers import Regex, Tokenizer, decoders, models, normalizers, pre_tokenizers, trainers
from tokenizers import AddedToken

HERE = os.path.dirname(os.path.abspath(__file__))
LLAMA3_PATTERN = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+")

WORDS = ("the of and to in is that it was for on are as with his they at be this from have or by one had not but what all were when we "
         "there can an your which their said if do will each about how up out them then she many some so these would other into has more "
         "her two like him see time could no make than first been its who now people my made over did down only way find use may water "
         "long little very after words called just where most know tensor logic kernel matrix quantized llama token decode stream").split()
EXTRA = ["naïve", "café", "über", "señor", "日本語", "テンソル", "论理", "Привет", "мир", "🙂", "x²", "½", "٣٤", "don't", "I'M", "we'll", "they'd"]


def corpus(seed=7, lines=3000):
    rng = random.Random(seed)
    out = []
    for _ in range(lines):
        n = rng.randint(3, 14)
        toks = []
        for _ in range(n):
            r = rng.random()
            if r < 0.72:
                w = rng.choice(WORDS)
                toks.append(w.capitalize() if rng.random() < 0.1 else w)
            elif r < 0.80:
                toks.append(str(rng.randint(0, 10 ** rng.randint(1, 6))))
            elif r < 0.88:
                toks.append(rng.choice(EXTRA))
            else:
                toks.append(rng.choice([",", ".", "!", "?", ";", ":", "(", ")", "--", "...", "\n", "\n\n", "  ", "\t", "\r\n", "#", "@", "=="]))
        out.append(" ".join(toks))
    return out


def build_bytelevel(texts):
    tok = Tokenizer(models.BPE(ignore_merges=True))
    tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(LLAMA3_PATTERN), behavior="isolated", invert=False),
                                                 pre_tokenizers.ByteLevel(add_prefix_space=False, trim_offsets=True, use_regex=False)])
    tok.decoder = decoders.ByteLevel(add_prefix_space=True, trim_offsets=True, use_regex=True)
    special = ["<|begin_of_text|>", "<|end_of_text|>", "<|start_header_id|>", "<|end_header_id|>", "<|eot_id|>"]
    trainer = trainers.BpeTrainer(vocab_size=700, special_tokens=[], initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
    tok.train_from_iterator(texts, trainer)
    tok.add_special_tokens([AddedToken(s, special=True, normalized=False) for s in special])
    return tok


def build_sp(texts):
    base = Tokenizer(models.BPE())
    base.normalizer = normalizers.Sequence([normalizers.Prepend("▁"), normalizers.Replace(" ", "▁")])
    trainer = trainers.BpeTrainer(vocab_size=500, special_tokens=[], show_progress=False)
    base.train_from_iterator([t for t in texts if not any(ord(c) > 0x2FF for c in t)], trainer)   # rarer scripts stay out: byte fallback
    js = json.loads(base.to_str())
    trained, merges = js["model"]["vocab"], js["model"]["merges"]
    vocab = {"<unk>": 0, "<s>": 1, "</s>": 2}
    for b in range(256):
        vocab["<0x%02X>" % b] = len(vocab)
    for t, _ in sorted(trained.items(), key=lambda kv: kv[1]):
        if t not in vocab:
            vocab[t] = len(vocab)
    merges = [tuple(m) if isinstance(m, list) else tuple(m.split(" ")) for m in merges]
    tok = Tokenizer(models.BPE(vocab=vocab, merges=merges, unk_token="<unk>", fuse_unk=True, byte_fallback=True))
    tok.normalizer = normalizers.Sequence([normalizers.Prepend("▁"), normalizers.Replace(" ", "▁")])
    tok.decoder = decoders.Sequence([decoders.Replace("▁", " "), decoders.ByteFallback(), decoders.Fuse(), decoders.Strip(" ", 1, 0)])
    tok.add_special_tokens([AddedToken(s, special=True, normalized=False) for s in ("<unk>", "<s>", "</s>")])
    return tok


PROBES = [
    "", " ", "  ", "hello", "Hello world", "the quick brown fox", " leading space", "trailing space ", "two  spaces", "tabs\tand\nnewlines\r\n",
    "line one\nline two\n\nline four", "don't I'M we'll they'd it's", "DON'T", "12345 6789 1 22 333 4444", "3.14159, 2.71828!", "a,b;c:d(e)f",
    "naïve café über señor", "日本語のテンソル", "Привет, мир!", "🙂 emoji 🙂🙂", "x² ½ ٣٤", "what?! ...", "== -- ## @@", "\n", "\n\n\n", " \n ",
    "tensor logic kernel matrix quantized llama token decode stream", "The time is 10:45pm on 2024-01-02.", "You are a helpful assistant.",
    "<|begin_of_text|>hello<|eot_id|>", "a<|eot_id|>b<|start_header_id|>user<|end_header_id|>\n\nhi", "</s> <s>hello</s>", "<|system|>\nYou are</s>\n<|user|>\nhi</s>\n",
    "mixed 日本 and english words 123", "    four spaces then text", "end with spaces   ", "\t\tindent", "a b", "ǅ ǈ", "don’t",
]


def main():
    texts = corpus()
    golden = {"probes": PROBES}
    for name, tok in (("bytelevel", build_bytelevel(texts)), ("sp", build_sp(texts))):
        tok.save(os.path.join(HERE, "tokenizer_%s.json" % name))
        tok = Tokenizer.from_file(os.path.join(HERE, "tokenizer_%s.json" % name))
        enc = [tok.encode(p, add_special_tokens=False).ids for p in PROBES]
        golden[name] = {"ids": enc, "decoded": [tok.decode(e, skip_special_tokens=True) for e in enc],
                        "vocab_size": tok.get_vocab_size(with_added_tokens=True),
                        "id_to_token": {str(i): tok.id_to_token(i) for i in range(0, tok.get_vocab_size(with_added_tokens=True), 7)}}
    json.dump(golden, open(os.path.join(HERE, "tokenizer_golden.json"), "w"), ensure_ascii=True, indent=0)


if __name__ == "__main__":
    main()
