"""The tokenizer against the Hugging Face `tokenizers` package (0.22.2, the crate version the reference links): the committed
fixtures (tests/golden/make_tokenizer_fixtures.py) hold two tokenizer.json files - byte-level BPE with the Llama-3 split
pattern, SentencePiece-style BPE with byte fallback - and the ids / strings the package produced for a list of probe texts;
where the package is importable the comparison is also made live on more texts.  Host code only: no GPU."""
import json
import os
import random

import pytest

import tl_b200 as tl

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
golden = json.load(open(os.path.join(GOLD, "tokenizer_golden.json")))


@pytest.fixture(scope="module", params=["bytelevel", "sp"])
def pair(request):
    return request.param, tl.Tokenizer(os.path.join(GOLD, "tokenizer_%s.json" % request.param))


def test_encode_matches_the_package(pair):
    name, tok = pair
    assert tok.vocab_size() == golden[name]["vocab_size"]
    for i, text in enumerate(golden["probes"]):
        assert tok.encode_ids(text) == golden[name]["ids"][i], (name, text)


def test_decode_matches_the_package(pair):
    name, tok = pair
    for i, text in enumerate(golden["probes"]):
        ids = golden[name]["ids"][i]
        if len(ids) != 1:       # one id takes the runtime's own path (next test)
            assert tok.decode_ids(ids) == golden[name]["decoded"][i], (name, text)
    for k, v in golden[name]["id_to_token"].items():
        assert tok.id_to_token(int(k)) == v
    assert tok.id_to_token(10 ** 6) is None


def test_single_token_decode_follows_the_runtime():
    # crates/tl_runtime/src/tokenizer.rs:89-117: id_to_token, byte tokens as their byte, <|...|> dropped, U+2581 / U+0120 -> space, U+010A -> newline
    sp = tl.Tokenizer(os.path.join(GOLD, "tokenizer_sp.json"))
    bl = tl.Tokenizer(os.path.join(GOLD, "tokenizer_bytelevel.json"))
    assert sp.decode_ids([3 + 0x41]) == "A"                      # <0x41>
    the = sp.encode_ids("the")
    assert sp.decode_ids(the[:1]).startswith(" ")                # the leading U+2581 survives as a space
    hdr = bl.encode_ids("<|eot_id|>")
    assert len(hdr) == 1 and bl.decode_ids(hdr) == ""
    sp_world = bl.encode_ids(" world")
    assert bl.decode_ids(sp_world[:1]).startswith(" ")
    assert bl.decode_ids(bl.encode_ids("\n")[:1]) == "\n"


def test_live_against_the_package(pair):
    tokenizers = pytest.importorskip("tokenizers")
    name, tok = pair
    ref = tokenizers.Tokenizer.from_file(os.path.join(GOLD, "tokenizer_%s.json" % name))
    rng = random.Random(11)
    alphabet = list("abcdefghijklmnopqrstuvwxyzABCDEFGHIJ 0123456789  .,;:!?'\"()-\n\t") + ["é", "ü", "ß", "日", "本", "語", "Ж", "🙂", "'s", "'LL", " the", " of", "\r\n", "</s>", "<|eot_id|>", "  "]
    for _ in range(300):
        text = "".join(rng.choice(alphabet) for _ in range(rng.randint(0, 40)))
        want = ref.encode(text, add_special_tokens=False).ids
        assert tok.encode_ids(text) == want, (name, text)
        if len(want) != 1:
            assert tok.decode_ids(want) == ref.decode(want, skip_special_tokens=True), (name, text)


def test_refuses_what_it_does_not_implement(tmp_path):
    js = json.load(open(os.path.join(GOLD, "tokenizer_bytelevel.json")))
    js["pre_tokenizer"]["pretokenizers"][0]["pattern"]["Regex"] = r"\w+|\s+"
    p = tmp_path / "other.json"
    p.write_text(json.dumps(js))
    with pytest.raises(tl.TlbError) as e:
        tl.Tokenizer(p)
    assert e.value.code == 7
    js = json.load(open(os.path.join(GOLD, "tokenizer_sp.json")))
    js["model"]["type"] = "Unigram"
    p.write_text(json.dumps(js))
    with pytest.raises(tl.TlbError):
        tl.Tokenizer(p)
    p.write_text("{ not json")
    with pytest.raises(tl.TlbError):
        tl.Tokenizer(p)
    with pytest.raises(tl.TlbError):
        tl.Tokenizer(tmp_path / "missing.json")


@pytest.mark.gpu
def test_tensor_forms_and_chat_templates():
    tl.init(-1)
    bl = tl.Tokenizer(os.path.join(GOLD, "tokenizer_bytelevel.json"))
    sp = tl.Tokenizer(os.path.join(GOLD, "tokenizer_sp.json"))
    ids = [int(v) for v in bl.encode("Hello world").numpy()]
    assert ids == [1] + bl.encode_ids("Hello world")                      # BOS = 1 in front
    chat = [int(v) for v in bl.encode_chat("what time is it?").numpy()]
    e = bl.encode_ids
    want = [128000, 128006] + e("system") + [128007] + e("\n\n") + e("You are a helpful assistant.") + [128009, 128006] + e("user") + [128007] + \
        e("\n\n") + e("what time is it?") + [128009, 128006] + e("assistant") + [128007] + e("\n\n")
    assert chat == want
    z = [int(v) for v in sp.encode_chat_zephyr("hi there").numpy()]
    assert z == [1] + sp.encode_ids("<|system|>\nYou are a helpful assistant.</s>\n<|user|>\nhi there</s>\n<|assistant|>\n")
    assert z.count(2) == 2                                                 # </s> found as the added token it is
    t = sp.encode("the time")
    assert sp.decode(t) == sp.decode_ids([int(v) for v in t.numpy()])
