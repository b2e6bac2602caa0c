"""The tokenizer of the library (csrc/tokenizer.cpp behind mlc_tokenizer_*) against the reference's Tokenizer
(compiler/runtime/tokenizer.cpp, its own unigram / byte-pair / longest-match code, i.e. as built without llama.cpp):
what the reference did with thirteen vocabularies and sixteen texts is recorded in tests/golden/tokenizer.json
(tests/golden/make_tokenizer_golden.py); the same comparison runs live where the reference library can be built.
Host code only: no GPU."""
import json
from pathlib import Path

import pytest

import gguf_cases
from mlcompiler_b200.host import GgufFile, Tokenizer

GOLDEN = json.loads((Path(__file__).parent / "golden" / "tokenizer.json").read_text())
MODES = [(True, False), (True, True), (False, False), (False, True)]


def _product(tmp_path, name):
    path = tmp_path / (name + ".gguf")
    vocab = gguf_cases.tokenizer_file(path, name)
    f = GgufFile(path)
    t = Tokenizer(f)
    f.close()                      # the tokenizer keeps its own copy of the vocabulary
    return path, vocab, t


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_tokenizer_matches_what_the_reference_recorded(name, tmp_path):
    _, vocab, t = _product(tmp_path, name)
    want = GOLDEN[name]
    assert (t.valid(), t.vocabSize(), t.bosId(), t.eosId(), t.unkId()) == \
        (want["valid"], want["vocab_size"], want["bos"], want["eos"], want["unk"])
    assert len(want["texts"]) == len(gguf_cases.TOKENIZER_TEXTS)
    for text, entry in zip(gguf_cases.TOKENIZER_TEXTS, want["texts"]):
        data = gguf_cases.text_bytes(text)
        assert data.hex() == entry["text_hex"]
        for add_bos, add_eos in MODES:
            assert t.encode(data, add_bos, add_eos) == entry["encode"][f"bos{int(add_bos)}_eos{int(add_eos)}"], (text, add_bos, add_eos)
        assert t.decode_bytes(entry["encode"]["bos1_eos1"]).hex() == entry["decode_hex"], text
    probe = want["probe_ids"]
    assert t.decode_bytes(probe).hex() == want["probe_decode_hex"]
    assert [t.tokenString(i).hex() for i in probe] == want["token_strings_hex"]
    assert [int(t.isControlToken(i)) | 2 * int(t.isEogToken(i)) for i in probe] == want["flags"]


def test_live_differential_against_the_reference(oracle_mod, tmp_path):
    if oracle_mod.ref() is None:
        pytest.skip("reference library not available")
    import numpy as np
    rng = np.random.default_rng(99)
    alphabet = list("helowrdtan ,.!é日本▁xs") + ["the", "ing", " world", "<0x41>", "\x00", "\xff"]
    texts = [gguf_cases.text_bytes(t) for t in gguf_cases.TOKENIZER_TEXTS]
    texts += [gguf_cases.text_bytes("".join(rng.choice(alphabet, size=int(rng.integers(1, 60))))) for _ in range(60)]
    texts += [bytes(rng.integers(0, 256, int(rng.integers(1, 40)), dtype=np.uint8)) for _ in range(20)]
    for name in sorted(gguf_cases.TOKENIZER_CASES):
        path, vocab, t = _product(tmp_path, name)
        ref = oracle_mod.ReferenceTokenizer(path)
        assert (t.valid(), t.vocabSize(), t.bosId(), t.eosId(), t.unkId()) == (ref.valid, ref.vocab_size, ref.bos, ref.eos, ref.unk)
        for data in texts:
            for add_bos, add_eos in MODES:
                ids = t.encode(data, add_bos, add_eos)
                assert ids == ref.encode(data, add_bos, add_eos), (name, data, add_bos, add_eos)
            assert t.decode_bytes(ids) == ref.decode(ids), (name, data)
        for i in list(range(vocab)) + [vocab, vocab + 9]:
            assert t.tokenString(i) == ref.token_string(i)
            assert int(t.isControlToken(i)) | 2 * int(t.isEogToken(i)) == ref.flags(i)
        everything = list(range(vocab))
        assert t.decode_bytes(everything) == ref.decode(everything)


def test_vocabulary_of_the_reference_test(tmp_path):
    """The vocabulary of tests/test_runtime.cpp:3377-3441. That test expects <s>, hello, " ", world, <eos> = [0, 14, 7, 18, 1]
    for "hello world" - what the llama.cpp path gives. The reference's own merge code, the behaviour restated here
    (and recorded in the golden file from the reference built without llama.cpp), applies the merge "  w" first, gets
    " w", which is no piece of the vocabulary, and answers [0, 14, 2, 6, 9, 5, 10, 1]; its decode does not treat "<eos>" as
    special."""
    _, _, t = _product(tmp_path, "reference_test")
    assert t.valid() and t.encode("hello world", add_bos=True, add_eos=True) == [0, 14, 2, 6, 9, 5, 10, 1]
    assert t.decode([0, 14, 7, 18, 1]) == "hello world<eos>"
    assert t.encode("hello", add_bos=False) == [14]


def test_round_trips_and_text_interface(tmp_path):
    _, _, t = _product(tmp_path, "spm")
    ids = t.encode("the hello and the world", add_bos=True)
    assert ids[0] == t.bosId() and t.decode(ids) == "the hello and the world"
    assert t.encode("") == [t.bosId()] and t.encode("", add_bos=False) == []
    _, _, b = _product(tmp_path, "bpe")
    ids = b.encode("lower newest", add_bos=False)
    assert b.decode(ids) == "lower newest" and len(ids) < len("lower newest")
    assert b.tokenString(ids[0]) == b"lower"
    assert b.isControlToken(0) and b.isEogToken(0) and not b.isControlToken(5)
