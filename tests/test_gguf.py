"""The GGUF loader of the library (csrc/gguf_file.cpp behind mlc_gguf_*) against the reference's GGUFLoader
(compiler/frontends/gguf_loader.cpp): descriptions and tensor bytes recorded from the reference in
tests/golden/gguf_loader.json (tests/golden/make_gguf_golden.py), the same comparison live where the reference
library can be built, and the refusals. Host code only: no GPU."""
import hashlib
import json
import struct
from pathlib import Path

import numpy as np
import pytest

import gguf_cases
from mlcompiler_b200 import synth
from mlcompiler_b200.host import GgufFile

GOLDEN = json.loads((Path(__file__).parent / "golden" / "gguf_loader.json").read_text())


def _write_case(name, tmp_path):
    path = tmp_path / (name + ".gguf")
    if name in gguf_cases.ZOO_CASES:
        gguf_cases.zoo(path, *gguf_cases.ZOO_CASES[name])
        return path, False
    if name.startswith("v1_"):
        gguf_cases.v1_file(path, name[len("v1_"):])
        return path, False
    gguf_cases.blocks(path, name[len("blocks_"):])
    return path, True


def _product(path, concatenate):
    f = GgufFile(path)
    if concatenate:
        f.concatenate_block_weights()
    desc = f.describe()
    sha = {name: hashlib.sha256(f.tensor_data(name).tobytes()).hexdigest() for name in desc["tensors"]}
    return f, desc, sha


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_loader_matches_what_the_reference_recorded(name, tmp_path):
    path, concatenate = _write_case(name, tmp_path)
    f, desc, sha = _product(path, concatenate)
    want = GOLDEN[name]
    assert gguf_cases.canonical(desc) == want["describe"]
    assert sha == want["sha256"]
    if name in gguf_cases.ZOO_CASES:
        version, alignment, _, _ = gguf_cases.ZOO_CASES[name]
        assert desc["alignment"] == alignment and desc["data_start"] % alignment == 0
        offsets = [t["offset"] for t in desc["tensors"].values()]
        assert min(offsets) == desc["data_start"] and all(o % alignment == 0 for o in offsets)


def test_tensor_bytes_are_the_files(tmp_path):
    path = tmp_path / "zoo.gguf"
    _, tensors = gguf_cases.zoo(path)
    f = GgufFile(path)
    last = {name: data for name, _, _, data in tensors}          # a repeated name keeps its last entry
    for name, data in last.items():
        assert np.array_equal(f.tensor_data(name), data), name
    with pytest.raises(RuntimeError, match="no tensor named"):
        f.tensor_data("absent")


def test_concatenation_rules(tmp_path):
    path = tmp_path / "ok.gguf"
    t = {name: data for name, _, _, data in gguf_cases.blocks(path, "ok")}
    f = GgufFile(path)
    assert f.concatenate_block_weights() == 6
    assert f.concatenate_block_weights() == 0                     # already built
    d = f.describe()["tensors"]
    for blk in (0, 2, 10):
        pre = f"blk.{blk}."
        assert d[pre + "attn_qkv.weight"] == {"shape": [64, 16], "dtype": 2, "offset": -1, "n_bytes": 16 * 36}
        assert d[pre + "ffn_gate_up.weight"] == {"shape": [64, 12], "dtype": 2, "offset": -1, "n_bytes": 12 * 36}
        assert np.array_equal(f.tensor_data(pre + "attn_qkv.weight"),
                              np.concatenate([t[pre + p + ".weight"] for p in ("attn_q", "attn_k", "attn_v")]))
        assert np.array_equal(f.tensor_data(pre + "ffn_gate_up.weight"),
                              np.concatenate([t[pre + p + ".weight"] for p in ("ffn_gate", "ffn_up")]))
    for case, absent in (("f16_k", "blk.0.attn_qkv.weight"), ("cols", "blk.0.ffn_gate_up.weight"),
                         ("missing_v", "blk.0.attn_qkv.weight")):
        p = tmp_path / (case + ".gguf")
        gguf_cases.blocks(p, case)
        g = GgufFile(p)
        assert g.concatenate_block_weights() == 5
        assert absent not in g.describe()["tensors"]


def test_live_differential_against_the_reference(oracle_mod, tmp_path):
    """The same files, and a model file, through both loaders now (skipped where the reference is not built)."""
    if oracle_mod.ref() is None:
        pytest.skip("reference library not available")
    cases = [(n,) + _write_case(n, tmp_path) for n in sorted(GOLDEN)]
    model = synth.SyntheticModel(3, 2, 4, 2, 64, 512, 320)
    mpath = tmp_path / "model.gguf"
    model.write_gguf(mpath)
    cases.append(("model", mpath, True))
    for name, path, concatenate in cases:
        _, desc, sha = _product(path, concatenate)
        assert gguf_cases.canonical(desc) == gguf_cases.canonical(oracle_mod.reference_gguf_describe(path, concatenate)), name
        for tensor, digest in sha.items():
            ref = oracle_mod.reference_gguf_tensor(path, tensor, concatenate)
            assert ref is not None and hashlib.sha256(ref.tobytes()).hexdigest() == digest, (name, tensor)


def _header(version=3, n_tensors=0, n_kv=0, magic=0x46554747):
    return struct.pack("<IIQQ", magic, version, n_tensors, n_kv)


def _string(s):
    return struct.pack("<Q", len(s)) + s


@pytest.mark.parametrize("blob,message", [
    (_header(magic=0x46554746), "Invalid GGUF magic"),
    (_header(version=7), "Unsupported GGUF version: 7"),
    (_header(version=0), "Unsupported GGUF version: 0"),
    (_header(version=4), "Unsupported GGUF version: 4"),
    (_header()[:10], "unexpected end of file"),
    (_header(n_kv=1) + _string(b"k") + struct.pack("<I", 99), "Invalid value type 99"),
    (_header(n_kv=1) + _string(b"k") + struct.pack("<IIQ", 9, 99, 0), "Invalid value type 99"),
    (_header(n_kv=1) + _string(b"k") + struct.pack("<I", 4), "unexpected end of file"),
    (_header(n_kv=1) + struct.pack("<Q", 1 << 40) + b"k", "string longer than the rest of the file"),
    (_header(n_kv=1) + _string(b"k") + struct.pack("<IIQ", 9, 4, 1 << 50), "array longer than the rest of the file"),
    (_header(n_tensors=1) + _string(b"t") + struct.pack("<IQQIQ", 2, 1 << 40, 1 << 40, 0, 0), "Overflow while calculating"),
    (_header(n_tensors=1) + _string(b"t") + struct.pack("<I", 17), "dimensions"),
])
def test_refusals(tmp_path, blob, message):
    path = tmp_path / "bad.gguf"
    path.write_bytes(blob)
    with pytest.raises(RuntimeError, match=message):
        GgufFile(path)


def test_version_1_fixture_of_the_reference_tests(tmp_path):
    """tests/test_gguf_loader.cpp:108-178 on the file of :20-86: header, the one key, both tensors, their bytes."""
    path = tmp_path / "mock.gguf"
    gguf_cases.v1_file(path, "mock")
    f = GgufFile(path)
    d = f.describe()
    assert (d["version"], d["n_tensors"], d["n_kv"]) == (1, 2, 1)
    assert d["kv"] == {"test.key": {"type": "STRING", "value": "test.value"}}
    assert d["tensors"]["tensor1"] == {"shape": [3, 4], "dtype": 0, "offset": 256, "n_bytes": 48}
    assert d["tensors"]["tensor2"]["shape"] == [10] and d["tensors"]["tensor2"]["offset"] == 400
    assert np.array_equal(f.tensor_data("tensor1").view(np.float32), np.full(12, 1.5, np.float32))
    gguf_cases.v1_file(tmp_path / "over.gguf", "overflow")
    with pytest.raises(RuntimeError, match="Overflow while calculating"):
        GgufFile(tmp_path / "over.gguf")
    gguf_cases.v1_file(tmp_path / "ck.gguf", "corrupt_key")
    assert GgufFile(tmp_path / "ck.gguf").describe()["kv"] == {"valid.key": {"type": "STRING", "value": "ok"}}


def test_refusal_details(tmp_path, oracle_mod):
    with pytest.raises(RuntimeError, match="Failed to open GGUF file"):
        GgufFile(tmp_path / "absent.gguf")
    # a tensor whose bytes are not in the file: opening works (as in the reference), reading it does not
    path = tmp_path / "short.gguf"
    path.write_bytes(_header(n_tensors=1) + _string(b"t") + struct.pack("<IQIQ", 1, 1000, 0, 64))
    f = GgufFile(path)
    assert f.describe()["tensors"]["t"]["n_bytes"] == 4000
    with pytest.raises(RuntimeError, match="Failed to read complete tensor data: t"):
        f.tensor_data("t")
    if oracle_mod.ref() is not None:
        assert oracle_mod.reference_gguf_tensor(path, "t") is None
        # the messages the two loaders share
        gguf_cases.v1_file(tmp_path / "over.gguf", "overflow")
        with pytest.raises(RuntimeError, match="Overflow while calculating"):
            oracle_mod.reference_gguf_describe(tmp_path / "over.gguf")
        for blob, message in ((_header(magic=1), "Invalid GGUF magic"), (_header(version=7), "Unsupported GGUF version: 7")):
            bad = tmp_path / "bad.gguf"
            bad.write_bytes(blob)
            with pytest.raises(RuntimeError, match=message):
                oracle_mod.reference_gguf_describe(bad)
