"""The whole walker step with a model attached - embedding, per layer RMSNorm / Q4_0 mat-vecs / rotary /
KV row write / paged attention / residual adds / SiLU * up, final norm and the Q6_K lm_head - against a
replay of the same step on the CPU oracle (oracle/paged_oracle.c, oracle/layer_oracle.c), op for op in the
order of the reference's walker (compiler/runtime/batched_walker.cpp:183-458).

The reference's own tests of this path (tests/test_batched_executor.cpp, tests/test_scheduler_e2e.cpp) need
a GGUF checkpoint; here the weights are seeded synthetic ones in the same tensor roles and formats
(mlcompiler_b200/synth.py: SyntheticModel).

Tolerance. Each GPU mat-vec rounds its activations to fp16 (relative error of a term <= 2^-11) and
attention computes in fp16 operands with fp32 sums; over a few layers these add up to a few 1e-4 of the
logits' scale. The logits must agree within 5e-3 of their rms (max-abs) with cosine >= 0.9999 per request,
the rows written to the KV pools within 3e-3 of their rms in layer 0 (they depend on embedding, norm, mat-vec
and rotary only) and 2e-2 in the last layer, and the greedy token must be the oracle's wherever its top two
logits are further apart than the tolerance.
"""
import numpy as np
import pytest

from mlcompiler_b200 import synth
from mlcompiler_b200.host import PagePool, PagedAttentionExecutor, PagedKVStorage, Scheduler

pytestmark = pytest.mark.gpu

P = 64


def make_stack(executor, model, capacity=16):
    pool = PagePool(capacity)
    storage = PagedKVStorage(executor, capacity, model.n_layers, P, model.kv_heads, model.head_dim, 2)
    assert storage.initialize()
    ex = PagedAttentionExecutor(executor, model.num_heads, model.kv_heads, model.head_dim, model.n_layers, 0)
    ex.attach_page_pool(pool, P)
    ex.attach_paged_storage(storage)
    assert ex.attach_model(model.to_device())
    return pool, storage, ex


class OracleModel:
    """The walker step on the CPU, keeping its own copy of every layer's pools."""

    def __init__(self, o, model, capacity):
        self.o, self.m = o, model
        shape = (capacity, P, model.kv_heads, model.head_dim)
        self.k = [np.zeros(shape, np.float16) for _ in range(model.n_layers)]
        self.v = [np.zeros(shape, np.float16) for _ in range(model.n_layers)]

    def step(self, slots, tables):
        o, m = self.o, self.m
        H, KVH, D, h, inner = m.num_heads, m.kv_heads, m.head_dim, m.hidden_size, m.ffn_inner
        t = m.host
        N = len(slots)
        x = np.stack([o.dequant_rows("q4_0", t["token_embd.weight"][tok:tok + 1], 1, h)[0] for _, tok, _ in slots])
        rot = [o.compute_rotary(pos, m.rotary_dim, m.rope_base, m.rope_scale) for _, _, pos in slots]
        cos_t, sin_t = np.stack([r[0] for r in rot]), np.stack([r[1] for r in rot])
        flat, off, lens, qpos, where = [], [0], [], [], []
        for rid, _, pos in slots:
            table, total = tables[rid]
            where.append((table[(total - 1) // P], (total - 1) % P))
            flat += table
            off.append(len(flat))
            lens.append(total)
            qpos.append(pos)
        for l in range(m.n_layers):
            pre = f"blk.{l}."
            n = o.rms_norm_batched(x, t[pre + "attn_norm.weight"], m.rms_epsilon)
            qkv = o.matmul_quant_batched("q4_0", t[pre + "attn_qkv.weight"], n, m.qkv_rows, h)
            q, _, _, k16, v16 = o.qkv_split_rope_cast(qkv, cos_t, sin_t, H, KVH, D, m.rotary_dim)
            for r, (page, slot) in enumerate(where):
                self.k[l][page, slot] = k16[r].view(np.float16).reshape(KVH, D)
                self.v[l][page, slot] = v16[r].view(np.float16).reshape(KVH, D)
            mix = o.paged_attention(q.reshape(N, H, D), self.k[l], self.v[l], flat, off, lens, qpos, H, KVH, D, P)
            attn_out = o.matmul_quant_batched("q4_0", t[pre + "attn_output.weight"], mix.reshape(N, h), h, h)
            r1 = o.add(x, attn_out)
            n2 = o.rms_norm_batched(r1, t[pre + "ffn_norm.weight"], m.rms_epsilon)
            gu = o.matmul_quant_batched("q4_0", t[pre + "ffn_gate_up.weight"], n2, 2 * inner, h)
            _, _, ffn_mix = o.gate_up_split_silu_mul(gu, inner)
            down = o.matmul_quant_batched("q4_0", t[pre + "ffn_down.weight"], ffn_mix, h, inner)
            x = o.add(r1, down)
        fn = o.rms_norm_batched(x, t["output_norm.weight"], m.rms_epsilon)
        return o.matmul_quant_batched(m.lm_head_quant, t["output.weight"], fn, m.vocab_size, h)


def assert_logits_close(got, want, what=""):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert np.isfinite(got).all(), what
    rms = np.sqrt((want ** 2).mean())
    err = np.abs(got - want).max()
    assert err <= 5e-3 * rms, f"{what}: max-abs {err:.3e} against rms {rms:.3e}"
    for r in range(got.shape[0]):
        cos = float(got[r] @ want[r] / (np.linalg.norm(got[r]) * np.linalg.norm(want[r])))
        assert cos >= 0.9999, f"{what}: request {r} cosine {cos}"
        top = np.sort(want[r])[-2:]
        if top[1] - top[0] > 1e-2 * rms:
            assert int(got[r].argmax()) == int(want[r].argmax()), f"{what}: greedy token differs for request {r}"


def _pools(executor, storage, model, layer, capacity):
    shape = (capacity, P, model.kv_heads, model.head_dim)
    k = np.zeros(shape, np.float16)
    v = np.zeros(shape, np.float16)
    executor.downloadFromBuffer(storage.k_buffer(layer), k)
    executor.downloadFromBuffer(storage.v_buffer(layer), v)
    return k, v


MODELS = [
    # layers, H, KVH, D, ffn_inner, vocab, rotary_dim, lm_head
    ("gqa_d64_q6k", (3, 4, 2, 64, 512, 1024, None, "q6_k")),
    ("mha_d128_q4_0_partial_rotary", (2, 2, 2, 128, 256, 300, 64, "q4_0")),
]


@pytest.mark.parametrize("reference_order", [False, True], ids=["fused", "reference_order"])
@pytest.mark.parametrize("name,shape", MODELS, ids=[m[0] for m in MODELS])
def test_model_decode_passes_match_the_oracle(executor, oracle_mod, name, shape, reference_order):
    layers, H, KVH, D, inner, vocab, rot, head = shape
    model = synth.SyntheticModel(0x5EED, layers, H, KVH, D, inner, vocab, rotary_dim=rot, lm_head_quant=head)
    capacity = 8
    pool, storage, ex = make_stack(executor, model, capacity)
    ex.set_call_order(reference_order)
    replay = OracleModel(oracle_mod, model, capacity)
    rng = np.random.default_rng(11)
    positions = {1: 0, 2: 0, 5: 0}
    launches = []
    for step in range(68):                       # crosses the 64-token page boundary
        active = [rid for rid in positions if rid != 5 or step >= 7]      # request 5 joins late
        slots = [(rid, int(rng.integers(0, vocab)), positions[rid]) for rid in active]
        before = executor.launchCount()
        out = ex.run_decode(slots)
        launches.append(executor.launchCount() - before)
        assert [o[0] for o in out] == active and all(o[1] for o in out), executor.last_error()
        tables = {rid: ex.page_state(rid) for rid in active}
        want = replay.step(slots, tables)
        if step % 6 == 0 or step > 62:
            assert_logits_close(np.stack([o[2] for o in out]), want, f"step {step}")
        for rid in active:
            positions[rid] += 1
    # launches of a pass: embedding + per layer 7 (fused: norm, QKV projection with rotary and page write, attention,
    # output projection, norm, gate | up with SiLU, down) or 13 (the reference's ops one for one) + norm + lm_head
    # (fused: up to four groups of vocabulary rows, multiples of 64); attention may add a merge launch per layer
    # when the planner splits sequences over CTAs
    per_layer = 13 if reference_order else 7
    group_rows = -(-(-(-vocab // 4)) // 64) * 64
    head_launches = 1 if reference_order else -(-vocab // group_rows)
    expect = 1 + layers * per_layer + 1 + head_launches
    assert expect <= launches[-1] <= expect + layers, launches[-1]
    # the pools, at every (page, slot) a token was written to: layer 0's rows depend on embedding, norm,
    # mat-vec and rotary only; the last layer's on everything before it
    rows = [(table[pos // P], pos % P) for table, total in (ex.page_state(r) for r in positions) for pos in range(total)]
    pg, sl = np.array([r[0] for r in rows]), np.array([r[1] for r in rows])
    for layer, tol in ((0, 3e-3), (layers - 1, 2e-2)):
        k, v = _pools(executor, storage, model, layer, capacity)
        for got, want in ((k, replay.k[layer]), (v, replay.v[layer])):
            g, w = got[pg, sl].astype(np.float32), want[pg, sl].astype(np.float32)
            assert np.abs(g - w).max() <= tol * max(1.0, float(np.sqrt((w ** 2).mean()))), f"layer {layer} pool rows"
    assert pool.pages_in_use() == 5
    ex.destroy()
    storage.destroy()


@pytest.mark.parametrize("reference_order", [False, True], ids=["chunked", "token_by_token"])
def test_model_prefill_matches_the_token_loop(executor, oracle_mod, reference_order):
    """run_prefill with a model: the reference feeds the prompt one token per pass (batched_executor.cpp:450-467),
    and so does the reference call order here; the default puts 32 prompt tokens into a pass. Either way the last
    token's logits and the rows left in the pools are those of the oracle's token loop. A second call continues
    the context."""
    model = synth.SyntheticModel(0xFEED, 2, 4, 2, 64, 256, 512)
    capacity = 8
    pool, storage, ex = make_stack(executor, model, capacity)
    ex.set_call_order(reference_order)
    replay = OracleModel(oracle_mod, model, capacity)
    rng = np.random.default_rng(3)
    prompt = [int(t) for t in rng.integers(0, model.vocab_size, 70)]      # 32 + 32 + 6, over the 64-token page boundary
    before = executor.launchCount()
    logits = ex.run_prefill(7, prompt)
    launches = executor.launchCount() - before
    assert logits.size == model.vocab_size and ex.known_position(7) == len(prompt)
    table, total = ex.page_state(7)
    assert total == len(prompt)
    for pos, tok in enumerate(prompt):
        want = replay.step([(7, tok, pos)], {7: (table, pos + 1)})
    assert_logits_close(logits[None], want, "prefill")
    if not reference_order:
        # three passes of embedding + 7 launches per layer, then the final norm and the lm_head's groups once
        head = -(-model.vocab_size // (-(-(-(-model.vocab_size // 4)) // 64) * 64))
        assert 3 * (1 + 2 * 7) + 1 + head <= launches <= 3 * (1 + 2 * 7 + 2) + 1 + head, launches
    more = [int(t) for t in rng.integers(0, model.vocab_size, 9)]
    logits = ex.run_prefill(7, more)
    table, total = ex.page_state(7)
    for i, tok in enumerate(more):
        want = replay.step([(7, tok, len(prompt) + i)], {7: (table, len(prompt) + i + 1)})
    assert_logits_close(logits[None], want, "second prefill call")
    rows = [(table[pos // P], pos % P) for pos in range(total)]
    pg, sl = np.array([r[0] for r in rows]), np.array([r[1] for r in rows])
    for layer, tol in ((0, 3e-3), (1, 2e-2)):
        k, v = _pools(executor, storage, model, layer, capacity)
        for got, ref in ((k, replay.k[layer]), (v, replay.v[layer])):
            g, w = got[pg, sl].astype(np.float32), ref[pg, sl].astype(np.float32)
            assert np.abs(g - w).max() <= tol * max(1.0, float(np.sqrt((w ** 2).mean()))), f"layer {layer} pool rows"
    # a decode pass continues from the prefilled context
    out = ex.run_decode([(7, 11, total)])
    want = replay.step([(7, 11, total)], {7: ex.page_state(7)})
    assert out[0][1]
    assert_logits_close(out[0][2][None], want, "decode after prefill")
    ex.release_request(7)
    assert pool.pages_in_use() == 0
    ex.destroy()
    storage.destroy()


def test_benchmark_shapes_at_32_requests(executor, oracle_mod):
    """Two layers of the benchmark's 1.1B shape (hidden 2048, H32 / KVH4 / D64, FFN 5632, vocabulary 32000, Q6_K head)
    with 32 requests: the launch shapes the model benchmark runs - 128-row paired tiles in three column slices for
    gate | up, the QKV projection's rotary epilogue over 40 row tiles, the lm_head in four groups of 8000 rows, a
    32-token prompt chunk - against the oracle's token loop."""
    model = synth.SyntheticModel(0xB16, 2, 32, 4, 64, 5632, 32000, lm_head_quant="q6_k")
    capacity = 40
    pool, storage, ex = make_stack(executor, model, capacity)
    replay = OracleModel(oracle_mod, model, capacity)
    rng = np.random.default_rng(21)
    ids = list(range(32))
    for step in range(2):
        slots = [(rid, int(rng.integers(0, model.vocab_size)), step) for rid in ids]
        out = ex.run_decode(slots)
        assert [o[0] for o in out] == ids and all(o[1] for o in out), executor.last_error()
        want = replay.step(slots, {rid: ex.page_state(rid) for rid in ids})
        assert_logits_close(np.stack([o[2] for o in out]), want, f"step {step}")
    # request 99: a prompt of 33 tokens = one full chunk and one token
    prompt = [int(t) for t in rng.integers(0, model.vocab_size, 33)]
    logits = ex.run_prefill(99, prompt)
    table, total = ex.page_state(99)
    for pos, tok in enumerate(prompt):
        want = replay.step([(99, tok, pos)], {99: (table, pos + 1)})
    assert_logits_close(logits[None], want, "prefill")
    ex.destroy()
    storage.destroy()


def test_greedy_decode_on_the_device_equals_argmax_of_the_logits(executor):
    """run_decode_greedy against run_decode + numpy argmax on two executors fed the same slots."""
    model = synth.SyntheticModel(0xA46, 2, 4, 2, 64, 256, 515)          # a vocabulary that is no multiple of 4
    _, sa, a = make_stack(executor, model, 8)
    _, sb, b = make_stack(executor, model, 8)
    rng = np.random.default_rng(1)
    pos = {3: 0, 4: 0, 9: 0}
    for step in range(6):
        slots = [(rid, int(rng.integers(0, model.vocab_size)), pos[rid]) for rid in pos]
        want = [int(np.argmax(o[2])) for o in a.run_decode(slots)]
        got = b.run_decode_greedy(slots)
        assert got == want, f"step {step}"
        for rid in pos:
            pos[rid] += 1
    b.set_call_order(True)
    assert b.run_decode_greedy([(3, 1, pos[3])]) is None          # the reference's call order returns logits only
    bare = PagedAttentionExecutor(executor, 4, 2, 64, 2, 0)
    assert bare.run_decode_greedy([(1, 1, 0)]) is None            # no model attached
    for x in (a, b, bare):
        x.destroy()
    for s_ in (sa, sb):
        s_.destroy()


def test_scheduler_generates_the_oracles_tokens(executor, oracle_mod):
    """The scheduler over the executor with a model generates greedy tokens that the oracle model reproduces."""
    model = synth.SyntheticModel(0xFEED, 2, 4, 2, 64, 256, 512)
    capacity = 8
    pool, storage, ex = make_stack(executor, model, capacity)

    sched = Scheduler(ex, max_batch_size=4)
    prompts = {0: [9, 8, 7], 1: [100, 200, 300, 400]}
    ids = {sched.add_request(p, max_new_tokens=6): k for k, p in prompts.items()}
    sched.run_until_idle()
    done = {r["id"]: r for r in sched.drain_completed()}
    assert len(done) == 2
    for rid, key in ids.items():
        toks = list(done[rid]["generated_tokens"])
        assert len(toks) == 6
        # replay request `rid` alone on the oracle: prompt, then greedy decoding
        rep = OracleModel(oracle_mod, model, 4)
        seq = list(prompts[key])
        table = [0]
        for pos, tok in enumerate(seq):
            lg = rep.step([(0, tok, pos)], {0: (table, pos + 1)})
        margin_ok = True
        for i in range(6):
            top = np.sort(lg[0])[-2:]
            if top[1] - top[0] <= 1e-2 * np.sqrt((lg[0].astype(np.float64) ** 2).mean()):
                margin_ok = False        # a near-tie: from here on the two may legitimately diverge
                break
            assert toks[i] == int(lg[0].argmax()), f"request {key}: token {i}"
            seq.append(toks[i])
            lg = rep.step([(0, toks[i], len(seq) - 1)], {0: (table, len(seq))})
        assert margin_ok or i > 0
    ex.destroy()
    storage.destroy()


def test_attach_model_rejects_a_description_that_does_not_fit(executor):
    model = synth.SyntheticModel(1, 2, 4, 2, 64, 256, 512)
    pool = PagePool(4)
    ex = PagedAttentionExecutor(executor, 8, 2, 64, 2, 0)          # 8 heads: hidden 512, the model has 256
    assert not ex.attach_model(model.to_device())
    ex2 = PagedAttentionExecutor(executor, 4, 2, 64, 3, 0)         # three layers, the model has two
    model3 = synth.SyntheticModel(1, 3, 4, 2, 64, 256, 512)
    model3.host.pop("blk.2.ffn_down.weight")
    with pytest.raises(KeyError):
        ex2.attach_model(model3.to_device())
    ex.destroy()
    ex2.destroy()
