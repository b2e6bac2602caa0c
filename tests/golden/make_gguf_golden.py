#!/usr/bin/env python3
"""Records what the reference's GGUFLoader (compiler/frontends/gguf_loader.cpp, compiled unmodified into
oracle/_ref by oracle/build_ref.py) reads out of the test files of tests/gguf_cases.py: its description of each
file and the SHA-256 of every tensor's bytes, with and without concatenateBlockWeights(). Needs the reference
checkout; the result, tests/golden/gguf_loader.json, is committed and checked by tests/test_gguf.py everywhere."""
import hashlib
import json
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import gguf_cases  # noqa: E402
import oracle  # noqa: E402


def record(path, concatenate):
    desc = gguf_cases.canonical(oracle.reference_gguf_describe(path, concatenate))
    sha = {}
    for name in desc["tensors"]:
        data = oracle.reference_gguf_tensor(path, name, concatenate)
        sha[name] = None if data is None else hashlib.sha256(data.tobytes()).hexdigest()
    return {"describe": desc, "sha256": sha}


def main():
    assert oracle.ref() is not None, "needs oracle/_ref (the reference checkout)"
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        for name, (version, alignment, declared, kind) in gguf_cases.ZOO_CASES.items():
            path = tmp / (name + ".gguf")
            gguf_cases.zoo(path, version, alignment, declared, kind)
            out[name] = record(path, False)
        for case in gguf_cases.V1_CASES:
            path = tmp / ("v1_" + case + ".gguf")
            gguf_cases.v1_file(path, case)
            out["v1_" + case] = record(path, False)
        for case in gguf_cases.BLOCK_CASES:
            path = tmp / (case + ".gguf")
            gguf_cases.blocks(path, case)
            out["blocks_" + case] = record(path, True)
    target = Path(__file__).with_name("gguf_loader.json")
    target.write_text(json.dumps(out, indent=1, sort_keys=True) + "\n")
    print(f"wrote {target} ({target.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
