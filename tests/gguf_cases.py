"""GGUF files for the loader tests, written with mlcompiler_b200.synth.write_gguf from seeded data. Used by
tests/test_gguf.py and by tests/golden/make_gguf_golden.py (which records what the reference's loader makes of them)."""
import numpy as np

from mlcompiler_b200 import synth

# ggml type -> (weights per block, bytes per block), for sizing the stored bytes of a test tensor
BLOCKS = {0: (1, 4), 1: (1, 2), 2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 9: (32, 36),
          10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176), 14: (256, 210), 15: (256, 292),
          24: (1, 1), 25: (1, 2), 26: (1, 4), 30: (1, 2)}


def stored_bytes(shape, dtype):
    if not shape:
        return 0
    n = int(np.prod(shape, dtype=np.int64))
    w, b = BLOCKS.get(dtype, (1, 4))        # an unknown type counts 4 bytes per element (gguf_loader.cpp:748-750)
    return -(-n // w) * b


def _tensor(rng, name, shape, dtype):
    return (name, shape, dtype, rng.integers(0, 256, stored_bytes(shape, dtype), dtype=np.uint8))


# name -> (version, alignment the file is laid out with, general.alignment as stored, its type)
ZOO_CASES = {
    "zoo_v3_a64": (3, 64, 64, "u32"),
    "zoo_v2_a32": (2, 32, 32, "u32"),
    "zoo_v3_a0": (3, 32, 0, "u32"),          # 0 means the default of 32
    "zoo_v3_i64": (3, 128, 128, "i64"),
    "zoo_v3_neg": (3, 32, -5, "i32"),        # a negative value is ignored
}
BLOCK_CASES = ("ok", "f16_k", "cols", "missing_v", "fused_present")


def zoo(path, version=3, alignment=64, declared=None, alignment_kind="u32"):
    """Every metadata type and most tensor types in one small file."""
    rng = np.random.default_rng(20240607)
    kv = [
        ("general.architecture", "string", "llama"),
        ("general.alignment", alignment_kind, alignment if declared is None else declared),
        ("general.quantization_version", "u64", 3),
        ("t.u8", "u8", 250), ("t.i8", "i8", -7), ("t.u16", "u16", 65000), ("t.i16", "i16", -1234),
        ("t.u32", "u32", 4000000000), ("t.i32", "i32", -2000000000), ("t.u64", "u64", 2 ** 63 + 5), ("t.i64", "i64", -2 ** 62),
        ("t.f32", "f32", 0.1), ("t.f64", "f64", 1.0 / 3.0), ("t.true", "bool", 1), ("t.false", "bool", 0),
        ("t.string", "string", 'quote " backslash \\ tab \t newline \n café 日本'),
        ("t.empty_string", "string", ""),
        ("t.raw", "raw", bytes(range(0, 40, 3))),
        ("t.arr_u32", ("array", "u32"), [1, 2, 3, 4000000000]),
        ("t.arr_i16", ("array", "i16"), [-3, 0, 3]),
        ("t.arr_f32", ("array", "f32"), [0.5, -1.25, 3.0e10]),
        ("t.arr_str", ("array", "string"), ["<s>", "</s>", "", "▁the"]),
        ("t.arr_bool", ("array", "bool"), [1, 0, 1]),
        ("t.arr_nested", ("array", ("array", "u8")), [[1, 2], [], [3]]),
        ("t.arr_empty", ("array", "f64"), []),
        ("t.duplicate", "u32", 1), ("t.duplicate", "u32", 2),      # the later entry wins
    ]
    tensors = [
        _tensor(rng, "f32.vec", [48], 0), _tensor(rng, "f16.mat", [16, 3], 1), _tensor(rng, "q4_0.mat", [64, 5], 2),
        _tensor(rng, "q4_1.mat", [32, 2], 3), _tensor(rng, "q5_0.mat", [32, 3], 6), _tensor(rng, "q5_1.mat", [64, 1], 7),
        _tensor(rng, "q8_0.mat", [32, 4], 8), _tensor(rng, "q8_1.mat", [32, 1], 9), _tensor(rng, "q2_k.mat", [256, 2], 10),
        _tensor(rng, "q3_k.mat", [256, 1], 11), _tensor(rng, "q4_k.mat", [512, 1], 12), _tensor(rng, "q5_k.mat", [256, 1], 13),
        _tensor(rng, "q6_k.mat", [256, 3], 14), _tensor(rng, "q8_k.mat", [256, 1], 15), _tensor(rng, "i8.vec", [7], 24),
        _tensor(rng, "i16.vec", [5], 25), _tensor(rng, "i32.vec", [3], 26), _tensor(rng, "i64.as_unknown", [3], 27),
        _tensor(rng, "f64.as_unknown", [2], 28), _tensor(rng, "bf16.vec", [9], 30), _tensor(rng, "type99", [5, 2], 99),
        _tensor(rng, "ragged.q4_0", [40, 3], 2),           # 120 weights: 4 blocks
        _tensor(rng, "rank3", [4, 3, 2], 0), _tensor(rng, "scalar.shape", [], 0),
        _tensor(rng, "twice", [8], 0), _tensor(rng, "twice", [4, 4], 1),       # the later entry wins
    ]
    synth.write_gguf(path, kv, tensors, version=version, alignment=alignment, tensor_padding=b"\xAB")
    return kv, tensors


def blocks(path, case):
    """Block weights for the concatenation rules (gguf_loader.cpp:877-943). case:
    "ok": blocks 0, 2 and 10 complete; "f16_k": blk.0.attn_k is F16; "cols": blk.0.ffn_up has other columns;
    "missing_v": blk.0 has no attn_v; "fused_present": blk.0.attn_qkv is already in the file."""
    rng = np.random.default_rng(77)
    cols = 64
    t = []
    for blk in (0, 2, 10):
        pre = f"blk.{blk}."
        for part, rows in (("attn_q", 8), ("attn_k", 4), ("attn_v", 4), ("ffn_gate", 6), ("ffn_up", 6)):
            dtype, c = 2, cols
            if blk == 0 and case == "f16_k" and part == "attn_k":
                dtype = 1
            if blk == 0 and case == "cols" and part == "ffn_up":
                c = 32
            if blk == 0 and case == "missing_v" and part == "attn_v":
                continue
            t.append(_tensor(rng, pre + part + ".weight", [c, rows], dtype))
    if case == "fused_present":
        t.append(_tensor(rng, "blk.0.attn_qkv.weight", [cols, 3], 2))
    t.append(_tensor(rng, "blk.x.attn_q.weight", [cols, 2], 2))       # not a block index: ignored
    synth.write_gguf(path, [("general.architecture", "string", "llama")], t)
    return t


def canonical(desc):
    """A loader's description reduced to what both loaders report: no alignment / data_start (the reference does not
    expose them), no element type for empty arrays (the reference keeps none)."""
    out = {k: desc[k] for k in ("version", "n_tensors", "n_kv", "quantization_version")}
    kv = {}
    for key, v in desc["kv"].items():
        v = dict(v)
        if v["type"] == "ARRAY" and not v["value"]:
            v.pop("elem_type", None)
        kv[key] = v
    out["kv"] = kv
    out["tensors"] = desc["tensors"]
    return out


# ---- vocabularies for the tokenizer tests ------------------------------------------------------------------------
def _spm_vocab():
    pieces = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)]
    words = ["▁", "▁the", "▁a", "▁an", "the", "th", "he", "e", "▁hello", "hello", "hell", "lo", "l", "o", "h", "▁w", "or",
             "ld", "▁world", "world", "▁wor", "a", "n", "an", "d", "▁and", "t", "s", "▁s", "er", "r", "▁", "▁▁", "é", "▁caf",
             "c", "f", "af", "!", ",", ".", "▁.", "日本", "日", "本", "<|sys|>", "in", "g", "ing", "▁th", "w", "x"]
    pieces += words
    rng = np.random.default_rng(5)
    scores = [-30.0, 0.0, 0.0] + [-20.0] * 256 + [float(-rng.uniform(1.0, 12.0)) - 0.5 * (8 - min(len(w), 8)) for w in words]
    return pieces, scores


def _bpe_vocab():
    singles = [chr(c) for c in range(32, 127)] + ["Ġ", "é"]
    merges = ["h e", "l l", "he ll", "hell o", "l o", "lo w", "e r", "low er", "t h", "th e", "w o", "wo r", "r l",
              "wor l", "worl d", "a n", "an d", "i n", "in g", "no_space_entry", "e s", "es t", "n e", "ne w", "new est",
              "h e"]           # a repeated merge keeps its last rank
    merged = sorted({m.replace(" ", "") for m in merges if " " in m})
    return ["<|endoftext|>"] + singles + merged, merges


TOKENIZER_CASES = {
    "spm": dict(model="llama", ids="u32"),
    "spm_u64_ids": dict(model="spm", ids="u64"),
    "spm_unk_zero": dict(model="llama", ids="u32", unk_score=0.0),          # an unknown byte costs nothing: it always wins
    "spm_no_unk": dict(model="unigram", ids="u32", drop=("unk",)),
    "spm_short_scores": dict(model="llama", ids="u32", short_scores=True),     # scores do not cover the vocabulary
    "spm_f64_scores": dict(model="llama", ids="u32", f64_scores=True),
    "bpe": dict(model="gpt2", ids="u32"),
    "bpe_no_merges": dict(model="bpe", ids="u32", no_merges=True),
    "no_model_merges": dict(model=None, ids="u32", base="bpe"),
    "no_model_scores": dict(model=None, ids="u32", base="spm"),
    "other_model": dict(model="wordpiece", ids="u32", base="spm"),
    "bare": dict(model=None, ids=None, base="spm", no_scores=True),            # tokens only: longest match
    "i32_ids": dict(model="llama", ids="i32"),                                 # ids of another integer type count as unset
    "empty": dict(model="llama", ids="u32", no_tokens=True),
    # the vocabulary of the reference's own tokenizer test (tests/test_runtime.cpp:3377-3441): version 1, no model key
    "reference_test": dict(model=None, ids="u32", fixture=True),
}

TOKENIZER_TEXTS = ["", "hello world", " hello world", "the hello and the world", "hello, world!", "café.", "日本 the",
                   "lower newest and lowest", "thethethe", "xyz\x01\xff", "  a  an   the ", "<s>hello</s>", "world" * 40,
                   "▁the▁world", "new\nline\ttab", "<|sys|> in going"]


def text_bytes(text) -> bytes:
    """The test texts as the bytes handed to the tokenizers: characters up to U+00FF written with \\x escapes are raw
    bytes (so that invalid UTF-8 is covered), everything else UTF-8."""
    return b"".join(bytes([ord(c)]) if ord(c) < 256 and not c.isalpha() and ord(c) > 127 or ord(c) < 32 else c.encode("utf-8") for c in text)


def tokenizer_kv(name):
    """(metadata triples of the vocabulary case, number of pieces)"""
    spec = TOKENIZER_CASES[name]
    if spec.get("fixture"):
        toks = ["<s>", "<eos>", "<unk>", "h", "e", "l", "o", " ", "w", "r", "d", "he", "hel", "hell", "hello", "wo", "wor",
                "worl", "world"]
        scores = [0.0, 0.0, -10.0] + [-1.0] * 8 + [1.0, 2.0, 3.0, 4.0] * 2
        merges = ["h e", "he l", "hel l", "hell o", "  w", "wo r", "wor l", "worl d", "hello  "]
        return [("tokenizer.ggml.tokens", ("array", "string"), toks), ("tokenizer.ggml.bos_token_id", "u32", 0),
                ("tokenizer.ggml.eos_token_id", "u32", 1), ("tokenizer.ggml.unk_token_id", "u32", 2),
                ("tokenizer.ggml.scores", ("array", "f32"), scores), ("tokenizer.ggml.merges", ("array", "string"), merges)], len(toks)
    base = spec.get("base", "bpe" if name.startswith("bpe") else "spm")
    kv = [("general.architecture", "string", "llama")]
    if spec["model"] is not None:
        kv.append(("tokenizer.ggml.model", "string", spec["model"]))
    if base == "spm":
        pieces, scores = _spm_vocab()
        merges = None
        ids = {"bos": 1, "eos": 2, "unk": 0}
    else:
        pieces, merges = _bpe_vocab()
        scores = None
        ids = {"bos": 0, "eos": 0}
    if not spec.get("no_tokens"):
        kv.append(("tokenizer.ggml.tokens", ("array", "string"), pieces))
    if scores is not None and not spec.get("no_scores"):
        if "unk_score" in spec:
            scores = [spec["unk_score"]] + scores[1:]
        if spec.get("short_scores"):
            scores = scores[:-3]
        kv.append(("tokenizer.ggml.scores", ("array", "f64" if spec.get("f64_scores") else "f32"), scores))
    if merges is not None and not spec.get("no_merges"):
        kv.append(("tokenizer.ggml.merges", ("array", "string"), merges))
    if spec["ids"]:
        for key, value in ids.items():
            if key not in spec.get("drop", ()):
                kv.append((f"tokenizer.ggml.{key}_token_id", spec["ids"], value))
    return kv, len(pieces)


def tokenizer_file(path, name):
    kv, n = tokenizer_kv(name)
    synth.write_gguf(path, kv, [], version=1 if TOKENIZER_CASES[name].get("fixture") else 3)
    return n


# ---- version-1 files laid out like the fixtures of the reference's own loader tests ----------------------------------
def _s(b):
    import struct
    b = b if isinstance(b, bytes) else b.encode()
    return struct.pack("<Q", len(b)) + b


def v1_file(path, case):
    """case "mock": tests/test_gguf_loader.cpp:20-86 (one string key, two tensors whose 32-bit dimensions follow a 64-bit
    repeat of the rank, absolute offsets 256 and 400); "plain_dims": the same without the repeat; "corrupt_key":
    :248-282 (a key of 1 MiB + 16 bytes is dropped, its value read, the next entry kept); "values": every value type
    as tests/test_gguf_values.cpp writes them, a raw blob (:275-285) and nested arrays (:325-358) among them;
    "overflow": :284-308 (three dimensions of 2^32 - 1)."""
    import struct
    head = lambda n_tensors, n_kv: struct.pack("<IIQQ", 0x46554747, 1, n_tensors, n_kv)
    if case in ("mock", "plain_dims"):
        rep = (lambda n: struct.pack("<Q", n)) if case == "mock" else (lambda n: b"")
        out = head(2, 1) + _s("test.key") + struct.pack("<I", 8) + _s("test.value")
        out += _s("tensor1") + struct.pack("<I", 2) + rep(2) + struct.pack("<II", 3, 4) + struct.pack("<IQ", 0, 256)
        out += _s("tensor2") + struct.pack("<I", 1) + rep(1) + struct.pack("<I", 10) + struct.pack("<IQ", 2, 400)
        out = out.ljust(256, b"\0") + np.full(12, 1.5, np.float32).tobytes()
        out = out.ljust(400, b"\0") + np.full(10, 0x3C00, np.uint16).tobytes()
    elif case == "corrupt_key":
        n = (1 << 20) + 16
        out = head(0, 2) + struct.pack("<Q", n) + b"A" * n + struct.pack("<IB", 0, 7)
        out += _s("valid.key") + struct.pack("<I", 8) + _s("ok")
    elif case == "values":
        kv = [("u8", 0, struct.pack("<B", 200)), ("i8", 1, struct.pack("<b", -5)), ("u16", 2, struct.pack("<H", 60000)),
              ("i16", 3, struct.pack("<h", -300)), ("u32", 4, struct.pack("<I", 123456789)), ("i32", 5, struct.pack("<i", -7)),
              ("f32", 6, struct.pack("<f", 3.25)), ("flag", 7, b"\x01"), ("str", 8, _s("hello")),
              ("ints", 9, struct.pack("<IQ", 5, 3) + struct.pack("<iii", 1, -2, 3)),
              ("strs", 9, struct.pack("<IQ", 8, 2) + _s("a") + _s("bc")),
              ("u64", 10, struct.pack("<Q", 2 ** 40)), ("i64", 11, struct.pack("<q", -2 ** 40)), ("f64", 12, struct.pack("<d", 0.1)),
              ("blob", 13, _s(bytes([1, 2, 3, 250]))),
              ("nested", 9, struct.pack("<IQ", 9, 2) + struct.pack("<IQ", 4, 2) + struct.pack("<II", 7, 8) +
               struct.pack("<IQ", 4, 1) + struct.pack("<I", 9))]
        out = head(1, len(kv)) + b"".join(_s(k) + struct.pack("<I", t) + v for k, t, v in kv)
        out += _s("t") + struct.pack("<I", 1) + struct.pack("<Q", 1) + struct.pack("<I", 4) + struct.pack("<IQ", 0, 1024)
        out = out.ljust(1024, b"\0") + np.arange(4, dtype=np.float32).tobytes()
    elif case == "overflow":
        out = head(1, 0) + _s("huge.tensor") + struct.pack("<I", 3) + struct.pack("<Q", 3) + struct.pack("<III", *[2 ** 32 - 1] * 3)
        out += struct.pack("<IQ", 0, 0)
    else:
        raise ValueError(case)
    with open(path, "wb") as f:
        f.write(out)


V1_CASES = ("mock", "plain_dims", "corrupt_key", "values")
