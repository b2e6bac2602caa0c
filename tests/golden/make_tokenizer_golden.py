#!/usr/bin/env python3
"""Records what the reference's Tokenizer (compiler/runtime/tokenizer.cpp, compiled unmodified and without llama.cpp
into oracle/_ref by oracle/build_ref.py) does with the vocabularies and texts of tests/gguf_cases.py: encode with and
without BOS / EOS, decode of the ids it produced and of a fixed id list, the special ids and per-token flags. Needs
the reference checkout; the result, tests/golden/tokenizer.json, is committed and checked by tests/test_tokenizer.py."""
import json
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import gguf_cases  # noqa: E402
import oracle  # noqa: E402


def record(path, vocab):
    t = oracle.ReferenceTokenizer(path)
    out = {"valid": t.valid, "vocab_size": t.vocab_size, "bos": t.bos, "eos": t.eos, "unk": t.unk, "texts": []}
    for text in gguf_cases.TOKENIZER_TEXTS:
        data = gguf_cases.text_bytes(text)
        entry = {"text_hex": data.hex(), "encode": {}}
        for add_bos in (True, False):
            for add_eos in (False, True):
                ids = t.encode(data, add_bos, add_eos)
                entry["encode"][f"bos{int(add_bos)}_eos{int(add_eos)}"] = ids
        entry["decode_hex"] = t.decode(entry["encode"]["bos1_eos1"]).hex()
        out["texts"].append(entry)
    probe = list(range(0, min(vocab + 3, 400), 7)) + [vocab - 1, vocab, vocab + 5]
    out["probe_ids"] = probe
    out["probe_decode_hex"] = t.decode(probe).hex()
    out["token_strings_hex"] = [t.token_string(i).hex() for i in probe]
    out["flags"] = [t.flags(i) for i in probe]
    return out


def main():
    assert oracle.ref() is not None, "needs oracle/_ref (the reference checkout)"
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        for name in gguf_cases.TOKENIZER_CASES:
            path = Path(tmp) / (name + ".gguf")
            vocab = gguf_cases.tokenizer_file(path, name)
            out[name] = record(path, vocab)
    target = Path(__file__).with_name("tokenizer.json")
    target.write_text(json.dumps(out, indent=None, sort_keys=True, separators=(",", ":")) + "\n")
    print(f"wrote {target} ({target.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
