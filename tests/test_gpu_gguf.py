"""A decoder loaded from a GGUF file (mlc_executor_attach_gguf) against the same weights handed over as device
pointers (mlc_executor_attach_model): the file stores q / k / v and gate / up apart, the loader concatenates them
as the reference's does (compiler/frontends/gguf_loader.cpp:877-943), so both executors hold the same bytes and
must produce the same logits bit for bit."""
import numpy as np
import pytest

from mlcompiler_b200 import synth
import gguf_cases
from mlcompiler_b200.host import GgufFile, PagePool, PagedAttentionExecutor, PagedKVStorage, Scheduler, Tokenizer

pytestmark = pytest.mark.gpu

P = 64


def _stack(executor, model, capacity=8):
    pool = PagePool(capacity)
    storage = PagedKVStorage(executor, capacity, model.n_layers, P, model.kv_heads, model.head_dim, 2)
    assert storage.initialize()
    ex = PagedAttentionExecutor(executor, model.num_heads, model.kv_heads, model.head_dim, model.n_layers, 0)
    ex.attach_page_pool(pool, P)
    ex.attach_paged_storage(storage)
    return pool, storage, ex


@pytest.mark.parametrize("shape,head,split,version,alignment", [
    ((2, 4, 2, 64, 512, 384), "q6_k", True, 3, 32),
    ((2, 4, 2, 64, 512, 384), "q4_0", False, 2, 64),
    ((1, 16, 4, 64, 1024, 40000), "q6_k", True, 3, 32),     # a 23 MB and a 34 MB tensor: several staging pieces each
])
def test_model_from_gguf_equals_model_from_pointers(executor, tmp_path, shape, head, split, version, alignment):
    layers, H, KVH, D, inner, vocab = shape
    model = synth.SyntheticModel(0xF11E, layers, H, KVH, D, inner, vocab, rotary_dim=32, lm_head_quant=head,
                                 rope_base=5000.0, rms_epsilon=2e-5)
    path = tmp_path / "model.gguf"
    model.write_gguf(path, split_fused=split, version=version, alignment=alignment)
    _, sa, a = _stack(executor, model)
    assert a.attach_model(model.to_device())
    _, sb, b = _stack(executor, model)
    f = GgufFile(path)
    assert b.attach_gguf(f), b.attach_error
    f.close()                                    # the weights are on the device: the file is no longer needed
    rng = np.random.default_rng(5)
    pos = {1: 0, 2: 0, 3: 0}
    for step in range(5):
        slots = [(rid, int(rng.integers(0, model.vocab_size)), pos[rid]) for rid in pos]
        out_a, out_b = a.run_decode(slots), b.run_decode(slots)
        assert all(o[1] for o in out_a) and all(o[1] for o in out_b), executor.last_error()
        la, lb = np.stack([o[2] for o in out_a]), np.stack([o[2] for o in out_b])
        assert la.shape == (3, model.vocab_size) and np.isfinite(la).all()
        assert np.array_equal(la, lb), f"step {step}: logits differ"
        for rid in pos:
            pos[rid] += 1
    for x in (a, b):
        x.destroy()
    for s in (sa, sb):
        s.destroy()


def test_tied_embeddings_and_refusals(executor, tmp_path):
    model = synth.SyntheticModel(7, 2, 4, 2, 64, 512, 384, lm_head_quant="q4_0")
    # a file without output.weight: the embedding table serves as the lm_head
    tied = synth.SyntheticModel(7, 2, 4, 2, 64, 512, 384, lm_head_quant="q4_0")
    tied.host["output.weight"] = tied.host["token_embd.weight"]
    path = tmp_path / "tied.gguf"
    head = model.host.pop("output.weight")
    model.write_gguf(path)
    model.host["output.weight"] = head
    _, sa, a = _stack(executor, tied)
    assert a.attach_model(tied.to_device())
    _, sb, b = _stack(executor, model)
    assert b.attach_gguf(GgufFile(path)), b.attach_error
    slots = [(1, 17, 0), (2, 300, 0)]
    la = np.stack([o[2] for o in a.run_decode(slots)])
    lb = np.stack([o[2] for o in b.run_decode(slots)])
    assert np.array_equal(la, lb)
    # an executor of another shape refuses the file and says why
    c = PagedAttentionExecutor(executor, 8, 2, 64, 2, 0)
    assert not c.attach_gguf(GgufFile(path)) and "heads" in c.attach_error
    d = PagedAttentionExecutor(executor, 4, 2, 64, 3, 0)
    assert not d.attach_gguf(GgufFile(path)) and "blocks" in d.attach_error
    # a missing tensor
    del model.host["blk.1.ffn_down.weight"]
    model.write_gguf(tmp_path / "short.gguf")
    e = PagedAttentionExecutor(executor, 4, 2, 64, 2, 0)
    assert not e.attach_gguf(GgufFile(tmp_path / "short.gguf")) and "blk.1.ffn_down.weight missing" in e.attach_error
    for x in (a, b, c, d, e):
        x.destroy()
    for s in (sa, sb):
        s.destroy()


def test_text_in_text_out_from_one_file(executor, tmp_path):
    """What the reference's chat loop does with a checkpoint (tests/test_scheduler_e2e.cpp needs the TinyLlama file):
    one GGUF file carries vocabulary and weights; the tokenizer turns a prompt into ids, the scheduler generates over
    the executor that loaded the weights, the tokenizer turns the ids back into text. The weights are synthetic, so the
    text means nothing - the ids must be those the same weights give when attached by pointer, run after run."""
    kv, vocab = gguf_cases.tokenizer_kv("spm")
    model = synth.SyntheticModel(0x7E47, 2, 4, 2, 64, 512, vocab, lm_head_quant="q6_k")
    path = tmp_path / "chat.gguf"
    model.write_gguf(path, extra_kv=[t for t in kv if t[0] != "general.architecture"])
    f = GgufFile(path)
    tok = Tokenizer(f)
    assert tok.valid() and tok.vocabSize() == vocab
    prompt = tok.encode("the hello and the world")
    assert prompt[0] == tok.bosId() and tok.decode(prompt) == "the hello and the world"

    def generate(attach):
        _, storage, ex = _stack(executor, model)
        attach(ex)
        sched = Scheduler(ex, max_batch_size=2)
        rids = [sched.add_request(prompt, max_new_tokens=12, eos_token_id=tok.eosId()),
                sched.add_request(tok.encode("hello"), max_new_tokens=5, eos_token_id=tok.eosId())]
        sched.run_until_idle()
        done = {r["id"]: list(r["generated_tokens"]) for r in sched.drain_completed()}
        ex.destroy()
        storage.destroy()
        return [done[r] for r in rids]

    def from_file(ex):
        assert ex.attach_gguf(f), ex.attach_error

    def from_pointers(ex):
        assert ex.attach_model(model.to_device())

    a, b, c = generate(from_file), generate(from_pointers), generate(from_file)
    assert a == b == c
    assert all(1 <= len(g) <= n for g, n in zip(a, (12, 5))) and all(0 <= t < vocab for g in a for t in g)
    assert isinstance(tok.decode(a[0]), str)
