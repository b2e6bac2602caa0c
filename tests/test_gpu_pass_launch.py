"""The whole-pass launch: every layer of a decode pass in one kernel.

mlc_encode_paged_decode_pass_planned may interleave the layers of a pass (they are independent by
contract): one launch deals the (layer, request, head) work items of all layers to the SMs. Its result
must be that of the per-layer call in a loop - the reference walker's layer loop,
compiler/runtime/batched_walker.cpp:299-331 - so every test here gives each layer its OWN queries, new
rows and pools, compares the pools bit for bit and the outputs within the parity tolerance with the
per-layer launches, and checks layers against the CPU oracle (tolerance of tests/util.py).
"""
import numpy as np
import pytest

from mlcompiler_b200 import synth
from mlcompiler_b200.capi import MLC_F16, MLC_F32
from tests.util import assert_attention_close

pytestmark = pytest.mark.gpu


class Layers:
    """`n` layers over one set of page tables, each with its own seeded tensors."""

    def __init__(self, case, n, seed, q_dtype="f16"):
        import torch
        self.case, self.n = case, n
        g = torch.Generator(device="cuda")
        g.manual_seed(seed)
        shape = (case.capacity, case.P, case.KVH, case.D)
        r16 = lambda s: torch.randn(s, generator=g, device="cuda", dtype=torch.float16)
        self.k_pool = [r16(shape) for _ in range(n)]
        self.v_pool = [r16(shape) for _ in range(n)]
        self.q = [r16((case.N, case.H, case.D)) for _ in range(n)]
        if q_dtype == "f32":
            self.q = [x.float() for x in self.q]
        self.k_new = [r16((case.N, case.KVH, case.D)) for _ in range(n)]
        self.v_new = [r16((case.N, case.KVH, case.D)) for _ in range(n)]
        torch.cuda.synchronize()

    def clone_pools(self):
        return [p.clone() for p in self.k_pool], [p.clone() for p in self.v_pool]

    def outs(self, dtype="f16"):
        import torch
        c = self.case
        dt = torch.float16 if dtype == "f16" else torch.float32
        return [torch.full((c.N, c.H, c.D), float("nan"), dtype=dt, device="cuda") for _ in range(self.n)]


def _plan(ex, case):
    return ex.createPlan(case.pt_flat, case.pt_off, case.seq_lens, case.q_pos, case.N, case.H, case.KVH, case.D,
                         case.P, True, case.capacity, page_ids=case.page_ids, slots_in_page=case.slots)


def _oracle_layer(oracle_mod, case, L, l, k_before, v_before):
    kp = k_before[l].cpu().numpy().view(np.uint16).copy().reshape(-1)
    vp = v_before[l].cpu().numpy().view(np.uint16).copy().reshape(-1)
    kn = L.k_new[l].cpu().numpy()
    vn = L.v_new[l].cpu().numpy()
    oracle_mod.scatter_kv_paged_batched_f16(kn, kp, case.page_ids, case.slots, case.P, case.KVH, case.D)
    oracle_mod.scatter_kv_paged_batched_f16(vn, vp, case.page_ids, case.slots, case.P, case.KVH, case.D)
    want = oracle_mod.paged_attention(L.q[l].float().cpu().numpy(), kp, vp, case.pt_flat, case.pt_off, case.seq_lens,
                                      case.q_pos, case.H, case.KVH, case.D, case.P, scale=case.scale)
    return kp, vp, want


CASES = [
    # (name, lens, H, KVH, D, layers, q/o dtype)
    ("two_layers", [100, 257, 33, 2000], 32, 4, 64, 2, "f16"),
    ("ragged_22", [1, 31, 32, 33, 64, 65, 700, 1500, 2048, 5, 129, 1024], 32, 4, 64, 22, "f16"),
    ("more_layers_than_fit_a_round", [300, 40, 900], 8, 2, 64, 40, "f16"),
    ("d128", [513, 64, 2100, 77, 1000], 32, 8, 128, 7, "f16"),
    ("g16_f32", [200, 1200, 64], 32, 2, 64, 5, "f32"),
    ("many_units", list(range(40, 40 + 70 * 23, 23)), 32, 4, 64, 3, "f16"),   # more units than SMs
    ("many_pieces", [40 + (i % 7) for i in range(700)], 32, 4, 64, 2, "f16"),  # ~19 pieces per CTA and warp
]


@pytest.mark.parametrize("name,lens,H,KVH,D,layers,dt", CASES, ids=[c[0] for c in CASES])
def test_pass_launch_equals_layer_by_layer(executor, oracle_mod, name, lens, H, KVH, D, layers, dt):
    import torch
    case = synth.make_case(70, lens, H, KVH, D, fill=False)
    L = Layers(case, layers, seed=71, q_dtype=dt)
    code = MLC_F16 if dt == "f16" else MLC_F32
    k_before, v_before = L.clone_pools()
    ka, va = L.clone_pools()            # pools of the per-layer run
    plan = _plan(executor, case)
    want, got = L.outs(dt), L.outs(dt)
    assert executor.beginForwardPassCB()
    for l in range(layers):
        assert executor.encodePagedDecodeStepPlanned(plan, L.q[l], L.k_new[l], L.v_new[l], ka[l], va[l], want[l],
                                                     case.scale, code, code), executor.last_error()
    before = executor.launchCount()
    ptrs = [executor.pointerArray(x) for x in (L.q, L.k_new, L.v_new, L.k_pool, L.v_pool, got)]
    assert executor.encodePagedDecodePassPlanned(plan, *ptrs, case.scale, code, code), executor.last_error()
    assert executor.launchCount() - before == 1, "the pass was not a single launch"
    assert executor.flushForwardPassCB(), executor.last_error()
    torch.cuda.synchronize()
    for l in range(layers):
        assert torch.isfinite(got[l].float()).all(), f"layer {l}: rows left unwritten"
        # the two forms cut a head's tokens into different parts, so their sums differ in the last bits
        assert_attention_close(got[l].float().cpu().numpy(), want[l].float().cpu().numpy())
        assert torch.equal(ka[l].view(torch.int16), L.k_pool[l].view(torch.int16)), f"layer {l}: K pool differs"
        assert torch.equal(va[l].view(torch.int16), L.v_pool[l].view(torch.int16)), f"layer {l}: V pool differs"
    for l in sorted({0, layers // 2, layers - 1}):
        kp, vp, ref = _oracle_layer(oracle_mod, case, L, l, k_before, v_before)
        assert np.array_equal(L.k_pool[l].cpu().numpy().view(np.uint16).reshape(-1), kp), "KV scatter is not bit-exact"
        assert np.array_equal(L.v_pool[l].cpu().numpy().view(np.uint16).reshape(-1), vp), "KV scatter is not bit-exact"
        assert_attention_close(got[l].float().cpu().numpy(), ref)
    plan.destroy()


def test_pass_launch_with_an_empty_request_and_graph_replay(executor, oracle_mod):
    """A request of length 1 (its only token is this step's row), captured in a CUDA graph and replayed
    with fresh queries: the layers' pointers are part of the captured launch."""
    import torch
    case = synth.make_case(72, [1, 500, 64, 1, 1300], 32, 4, 64, fill=False)
    layers = 6
    L = Layers(case, layers, seed=73)
    k_before, v_before = L.clone_pools()
    plan = _plan(executor, case)
    got = L.outs()
    ptrs = [executor.pointerArray(x) for x in (L.q, L.k_new, L.v_new, L.k_pool, L.v_pool, got)]
    assert executor.beginForwardPassCB()
    assert executor.encodePagedDecodePassPlanned(plan, *ptrs, case.scale, MLC_F16, MLC_F16), executor.last_error()
    assert executor.flushForwardPassCB(), executor.last_error()
    assert executor.beginForwardPassCB()
    assert executor.beginCapture(), executor.last_error()
    assert executor.encodePagedDecodePassPlanned(plan, *ptrs, case.scale, MLC_F16, MLC_F16), executor.last_error()
    graph = executor.endCapture()
    g = torch.Generator(device="cuda")
    g.manual_seed(74)
    for _ in range(3):
        for l in range(layers):
            L.q[l].copy_(torch.randn(L.q[l].shape, generator=g, device="cuda", dtype=torch.float16))
            got[l].fill_(float("nan"))
        torch.cuda.synchronize()
        graph.launch()
        assert executor.flushForwardPassCB(), executor.last_error()
        assert executor.beginForwardPassCB()
        torch.cuda.synchronize()
        for l in (0, layers - 1):
            _, _, ref = _oracle_layer(oracle_mod, case, L, l, k_before, v_before)
            assert_attention_close(got[l].float().cpu().numpy(), ref)
    assert executor.flushForwardPassCB(), executor.last_error()
    graph.destroy()
    plan.destroy()


def test_pass_falls_back_to_layer_launches_when_the_row_write_cannot_be_fused(executor):
    """A request whose query does not see its newest token (q_position < seq_len - 1): the row write cannot
    be fused into attention, so the pass call issues scatter + attention per layer, with the same result as
    the per-layer entry point."""
    import torch
    q_pos = np.array([899, 99, 62], np.uint32)          # the first request looks one token back
    case = synth.make_case(75, [901, 100, 63], 32, 4, 64, fill=False, q_pos=q_pos)
    layers = 3
    L = Layers(case, layers, seed=76)
    ka, va = L.clone_pools()
    plan = _plan(executor, case)
    want, got = L.outs(), L.outs()
    assert executor.beginForwardPassCB()
    for l in range(layers):
        assert executor.encodePagedDecodeStepPlanned(plan, L.q[l], L.k_new[l], L.v_new[l], ka[l], va[l], want[l],
                                                     case.scale, MLC_F16, MLC_F16), executor.last_error()
    before = executor.launchCount()
    ptrs = [executor.pointerArray(x) for x in (L.q, L.k_new, L.v_new, L.k_pool, L.v_pool, got)]
    assert executor.encodePagedDecodePassPlanned(plan, *ptrs, case.scale, MLC_F16, MLC_F16), executor.last_error()
    assert executor.launchCount() - before >= 2 * layers
    assert executor.flushForwardPassCB(), executor.last_error()
    for l in range(layers):
        assert torch.equal(want[l], got[l])
        assert torch.equal(ka[l].view(torch.int16), L.k_pool[l].view(torch.int16))
    plan.destroy()


def test_pass_launch_for_a_batch_the_planner_cuts_or_splits(executor, oracle_mod):
    """One request dwarfs the others: a launch per layer cuts its (request, head) units over CTAs (or splits
    the sequence), the pass launch works from its own list of whole units - still one launch, same output
    within tolerance of the oracle."""
    import torch
    case = synth.make_case(77, [9000, 100, 64], 32, 4, 64, fill=False)
    layers = 4
    L = Layers(case, layers, seed=78)
    k_before, v_before = L.clone_pools()
    plan = _plan(executor, case)
    got = L.outs()
    assert executor.beginForwardPassCB()
    before = executor.launchCount()
    ptrs = [executor.pointerArray(x) for x in (L.q, L.k_new, L.v_new, L.k_pool, L.v_pool, got)]
    assert executor.encodePagedDecodePassPlanned(plan, *ptrs, case.scale, MLC_F16, MLC_F16), executor.last_error()
    assert executor.launchCount() - before == 1
    assert executor.flushForwardPassCB(), executor.last_error()
    torch.cuda.synchronize()
    for l in range(layers):
        _, _, ref = _oracle_layer(oracle_mod, case, L, l, k_before, v_before)
        assert_attention_close(got[l].float().cpu().numpy(), ref)
    plan.destroy()
