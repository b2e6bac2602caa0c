"""GPU parity of the device-resident-plan entry points: planned attention, the
single-launch decode step (row write fused into attention, programmatic dependent
launch), CUDA-graph replay, and split-KV partials with the log-sum-exp combine.

The decode-step semantics follow the reference's walker: the new K/V row of every
request is written first, then attention runs over the pool including that row
(compiler/runtime/batched_walker.cpp:299-331).
"""
import numpy as np
import pytest

from mlcompiler_b200 import synth
from mlcompiler_b200.capi import MLC_F16, MLC_F32
from tests.util import DeviceCase, assert_attention_close

pytestmark = pytest.mark.gpu


def oracle_step(oracle_mod, case):
    """Pools after the scatter, and attention over them (CPU oracle)."""
    kp = case.k_pool.view(np.uint16).copy().reshape(-1)
    vp = case.v_pool.view(np.uint16).copy().reshape(-1)
    oracle_mod.scatter_kv_paged_batched_f16(case.k_new, kp, case.page_ids, case.slots, case.P, case.KVH, case.D)
    oracle_mod.scatter_kv_paged_batched_f16(case.v_new, vp, case.page_ids, case.slots, case.P, case.KVH, case.D)
    want = oracle_mod.paged_attention(case.q.astype(np.float32), kp, vp, case.pt_flat, case.pt_off, case.seq_lens,
                                      case.q_pos, case.H, case.KVH, case.D, case.P, scale=case.scale)
    return kp, vp, want


def make_plan(executor, case, with_rows=True, causal=True):
    return executor.createPlan(case.pt_flat, case.pt_off, case.seq_lens, case.q_pos, case.N, case.H, case.KVH,
                               case.D, case.P, causal, case.capacity,
                               page_ids=case.page_ids if with_rows else None,
                               slots_in_page=case.slots if with_rows else None)


def test_planned_attention_matches_host_array_path(executor, oracle_mod):
    import torch
    case = synth.config_case(2)
    dc = DeviceCase(case)
    o1, o2 = dc.out(), dc.out()
    assert executor.runPagedFlashAttention(dc.q, dc.k_pool, dc.v_pool, o1, case.pt_flat, case.pt_off, case.seq_lens,
                                           case.q_pos, case.N, case.H, case.KVH, case.D, case.P, True, case.scale,
                                           MLC_F16, MLC_F16, case.capacity)
    plan = make_plan(executor, case, with_rows=False)
    assert executor.beginForwardPassCB()
    assert executor.encodePagedFlashAttentionPlanned(plan, dc.q, dc.k_pool, dc.v_pool, o2, case.scale, MLC_F16, MLC_F16)
    assert executor.flushForwardPassCB(), executor.last_error()
    assert executor.lastAttentionKernel() == 2
    torch.cuda.synchronize()
    assert torch.equal(o1, o2)
    plan.destroy()


STEP_CASES = [
    ("cfg1", lambda: synth.config_case(1)),
    ("cfg2", lambda: synth.config_case(2)),
    ("edges", lambda: synth.make_case(31, [1, 2, 31, 32, 33, 63, 64, 65, 96, 97, 128, 129, 1000], 32, 4, 64)),
    ("shapeB", lambda: synth.make_case(32, [700, 64, 1, 2049, 333], 32, 8, 128)),
    ("g16", lambda: synth.make_case(33, [100, 257], 32, 2, 64)),
    ("g16_d128", lambda: synth.make_case(34, [100, 257, 33], 32, 2, 128)),
    ("kvh6", lambda: synth.make_case(35, [100, 257, 5], 12, 6, 64)),
    ("page128", lambda: synth.make_case(36, [100, 257, 129, 128], 32, 4, 64, P=128)),
    # one request dwarfs the others: the planner cuts its (request, head) units over CTAs
    ("longtail", lambda: synth.make_case(37, [16384, 256, 31, 256], 32, 4, 64)),
    ("lone_long", lambda: synth.make_case(38, [5000], 32, 4, 64)),
    ("longtail_d128", lambda: synth.make_case(39, [9000, 100, 70], 32, 8, 128)),
    ("longtail_g16", lambda: synth.make_case(40, [8001, 64], 32, 2, 64)),
]


@pytest.mark.parametrize("name,build", STEP_CASES, ids=[c[0] for c in STEP_CASES])
def test_decode_step_single_launch(executor, oracle_mod, name, build):
    import torch
    case = build()
    dc = DeviceCase(case)
    o = dc.out()
    plan = make_plan(executor, case)
    before = executor.launchCount()
    assert executor.beginForwardPassCB()
    assert executor.encodePagedDecodeStepPlanned(plan, dc.q, dc.k_new, dc.v_new, dc.k_pool, dc.v_pool, o, case.scale,
                                                 MLC_F16, MLC_F16), executor.last_error()
    assert executor.flushForwardPassCB(), executor.last_error()
    # row write fused into the attention kernel (+ the merge kernel when a request is split)
    assert executor.launchCount() - before in (1, 2)
    assert executor.lastAttentionKernel() == 2
    torch.cuda.synchronize()
    kp, vp, want = oracle_step(oracle_mod, case)
    # KV scatter: bit-exact
    assert np.array_equal(dc.k_pool.cpu().numpy().view(np.uint16).reshape(-1), kp)
    assert np.array_equal(dc.v_pool.cpu().numpy().view(np.uint16).reshape(-1), vp)
    assert_attention_close(o.float().cpu().numpy(), want)
    plan.destroy()


def test_decode_step_falls_back_to_two_launches(executor, oracle_mod):
    """A causal cut before the newest token cannot be fused; the result is the same."""
    import torch
    case = synth.make_case(41, [100, 200, 65], 32, 4, 64)
    case.q_pos = np.array([50, 199, 10], np.uint32)
    dc = DeviceCase(case)
    o = dc.out()
    plan = make_plan(executor, case)
    before = executor.launchCount()
    assert executor.beginForwardPassCB()
    assert executor.encodePagedDecodeStepPlanned(plan, dc.q, dc.k_new, dc.v_new, dc.k_pool, dc.v_pool, o, case.scale,
                                                 MLC_F16, MLC_F16), executor.last_error()
    assert executor.flushForwardPassCB(), executor.last_error()
    assert executor.launchCount() - before in (2, 3)    # scatter kernel + attention (+ merge)
    torch.cuda.synchronize()
    kp, vp, want = oracle_step(oracle_mod, case)
    assert np.array_equal(dc.k_pool.cpu().numpy().view(np.uint16).reshape(-1), kp)
    assert_attention_close(o.float().cpu().numpy(), want)
    plan.destroy()


def test_layers_back_to_back_and_graph_replay(executor, oracle_mod):
    """Six 'layers' (separate pools) of a step enqueued back to back: consecutive
    kernels overlap through programmatic dependent launch and alternate workspaces.
    The same sequence replayed from a CUDA graph gives identical bits."""
    import torch
    L = 6
    lens = synth.config_lengths(2)
    cases = [synth.make_case(100 + i, lens, 32, 4, 64) for i in range(L)]
    cap = max(c.capacity for c in cases)
    cases = [synth.make_case(100 + i, lens, 32, 4, 64, capacity=cap) for i in range(L)]
    # tables differ per seed; use layer 0's tables everywhere and fresh data per layer
    t0 = cases[0]
    for c in cases[1:]:
        c.pt_flat, c.pt_off, c.page_ids, c.slots = t0.pt_flat, t0.pt_off, t0.page_ids, t0.slots
    dcs = [DeviceCase(c) for c in cases]
    outs = [dc.out() for dc in dcs]
    plan = make_plan(executor, t0)

    def encode():
        for dc, o in zip(dcs, outs):
            assert executor.encodePagedDecodeStepPlanned(plan, dc.q, dc.k_new, dc.v_new, dc.k_pool, dc.v_pool, o,
                                                         t0.scale, MLC_F16, MLC_F16), executor.last_error()

    assert executor.beginForwardPassCB()
    encode()
    assert executor.flushForwardPassCB(), executor.last_error()
    torch.cuda.synchronize()
    eager = [o.clone() for o in outs]
    for c, dc, o in zip(cases, dcs, outs):
        kp, vp, want = oracle_step(oracle_mod, c)
        assert np.array_equal(dc.k_pool.cpu().numpy().view(np.uint16).reshape(-1), kp)
        assert_attention_close(o.float().cpu().numpy(), want)
    assert executor.beginForwardPassCB()
    assert executor.beginCapture(), executor.last_error()
    encode()
    graph = executor.endCapture()
    for _ in range(3):
        for o in outs:
            o.fill_(float("nan"))
        before = executor.launchCount()
        graph.launch()
        assert executor.launchCount() - before in (L, 2 * L)
        torch.cuda.synchronize()
        for o, e in zip(outs, eager):
            assert torch.equal(o, e)
    assert executor.flushForwardPassCB(), executor.last_error()
    graph.destroy()
    plan.destroy()


@pytest.mark.parametrize("parts", [2, 4, 8])
@pytest.mark.parametrize("shape", [synth.SHAPE_A, synth.SHAPE_B])
def test_split_kv_partials_and_combine(executor, oracle_mod, parts, shape):
    """Every 'rank' holds a slice of each request's pages; partial (o, m, l) per slice,
    gathered, combined: equals attention over the whole sequence."""
    import torch
    S = 64 * parts * 5
    lens = [S, 64 * parts * 3 - 17]  # second request: the last slice ends inside a page
    case = synth.make_case(50 + parts, lens, P=64, **shape)
    # request r's pages are dealt out in contiguous slices; a slice = that rank's local table
    N, H, KVH, D, P = case.N, case.H, case.KVH, case.D, case.P
    dc = DeviceCase(case)
    o_parts = torch.zeros((parts, N, H, D), dtype=torch.float32, device="cuda")
    ml_parts = torch.zeros((parts, N, H, 2), dtype=torch.float32, device="cuda")
    plans = []
    assert executor.beginForwardPassCB()
    per_rank_tables = []
    for k in range(parts):
        flat_k, off_k, lens_k = [], [0], []
        for r in range(N):
            pages = case.pt_flat[case.pt_off[r]:case.pt_off[r + 1]]
            n_pages = len(pages) // parts
            mine = pages[k * n_pages:(k + 1) * n_pages]
            total = int(case.seq_lens[r])
            # tokens of this slice: full pages except that the request's tail shortens the last slice's last page
            local = min(max(total - k * n_pages * P, 0), n_pages * P)
            flat_k.extend(mine.tolist())
            off_k.append(len(flat_k))
            lens_k.append(local)
        per_rank_tables.append((np.array(flat_k, np.uint32), np.array(off_k, np.uint32), np.array(lens_k, np.uint32)))
        plan = executor.createPlan(flat_k, off_k, lens_k, np.zeros(N, np.uint32), N, H, KVH, D, P, False, case.capacity)
        plans.append(plan)
        assert executor.encodePagedAttentionPartialPlanned(plan, dc.q, dc.k_pool, dc.v_pool, o_parts[k], ml_parts[k],
                                                           case.scale, MLC_F16), executor.last_error()
    out = torch.zeros((N, H, D), dtype=torch.float16, device="cuda")
    assert executor.encodeLseCombine(o_parts, ml_parts, parts, N * H, D, out, MLC_F16)
    assert executor.flushForwardPassCB(), executor.last_error()
    torch.cuda.synchronize()
    # whole-sequence oracle over the pages actually used, in slice order
    flat_all, off_all, lens_all = [], [0], []
    for r in range(N):
        tot = 0
        for k in range(parts):
            flat_k, off_k, lens_k = per_rank_tables[k]
            flat_all.extend(flat_k[off_k[r]:off_k[r + 1]].tolist())
            tot += int(lens_k[r])
        off_all.append(len(flat_all))
        lens_all.append(tot)
    assert lens_all == [int(x) for x in case.seq_lens]
    want = oracle_mod.paged_attention(case.q.astype(np.float32), case.k_pool, case.v_pool, flat_all, off_all, lens_all,
                                      np.zeros(N, np.uint32), H, KVH, D, P, causal=False, scale=case.scale)
    assert_attention_close(out.float().cpu().numpy(), want)
    # the gathered partials, combined by the oracle's rule, agree as well
    comb = oracle_mod.lse_combine(o_parts.cpu().numpy(), ml_parts.cpu().numpy())
    assert_attention_close(comb, want)
    # and each partial equals the oracle's partial over that token range
    for k in range(parts):
        flat_k, off_k, lens_k = per_rank_tables[k]
        o_ref, ml_ref = oracle_mod.paged_attention_tiled(case.q.astype(np.float32), case.k_pool, case.v_pool, flat_k,
                                                         off_k, lens_k, np.zeros(N, np.uint32), H, KVH, D, P,
                                                         causal=False, scale=case.scale, partial=True)
        got_o, got_ml = o_parts[k].cpu().numpy(), ml_parts[k].cpu().numpy()
        # compare in a max-independent form: o * exp(m) / (l * exp(m)) and log-sum-exp
        lse_got = got_ml[..., 0] + np.log(np.maximum(got_ml[..., 1], 1e-38))
        lse_ref = ml_ref[..., 0] + np.log(np.maximum(ml_ref[..., 1], 1e-38))
        live = lens_k > 0
        assert np.allclose(lse_got[live], lse_ref[live], atol=2e-3)
        norm_got = got_o / np.maximum(got_ml[..., 1:2], 1e-38)
        norm_ref = o_ref / np.maximum(ml_ref[..., 1:2], 1e-38)
        assert_attention_close(norm_got[live], norm_ref[live])
    for p in plans:
        p.destroy()


def test_plan_update_follows_growing_requests(executor, oracle_mod):
    """One plan object updated in place for consecutive decode steps (each request one token longer,
    crossing page boundaries, one request finishing): every step equals the oracle's scatter + attention."""
    import torch
    H, KVH, D, P = 32, 4, 64, 64
    lens0 = np.array([62, 127, 300, 64], np.uint32)
    case = synth.make_case(41, lens0 + 4, H, KVH, D, P=P)          # tables with room for 4 more tokens
    dev = torch.device("cuda:0")
    kp = torch.from_numpy(case.k_pool.view(np.int16)).to(dev)
    vp = torch.from_numpy(case.v_pool.view(np.int16)).to(dev)
    kp_ref = case.k_pool.view(np.uint16).reshape(-1).copy()
    vp_ref = case.v_pool.view(np.uint16).reshape(-1).copy()
    rng = np.random.default_rng(9)
    plan = None
    for step in range(4):
        alive = [0, 1, 2, 3] if step < 2 else [0, 2, 3]           # request 1 leaves after two steps
        lens = (lens0[alive] + step + 1).astype(np.uint32)          # length after this step's token
        off = np.zeros(len(alive) + 1, np.uint32)
        flat = []
        for i, r in enumerate(alive):
            n_pages = (int(lens[i]) + P - 1) // P
            flat.extend(case.pt_flat[case.pt_off[r]:case.pt_off[r] + n_pages].tolist())
            off[i + 1] = len(flat)
        flat = np.array(flat, np.uint32)
        q_pos = lens - 1
        ids = np.array([flat[off[i] + (int(lens[i]) - 1) // P] for i in range(len(alive))], np.uint32)
        slots = ((lens - 1) % P).astype(np.uint32)
        n = len(alive)
        q = rng.standard_normal((n, H, D), dtype=np.float32).astype(np.float16)
        kn = rng.standard_normal((n, KVH, D), dtype=np.float32).astype(np.float16)
        vn = rng.standard_normal((n, KVH, D), dtype=np.float32).astype(np.float16)
        if plan is None:
            plan = executor.createPlan(flat, off, lens, q_pos, n, H, KVH, D, P, True, case.capacity,
                                       page_ids=ids, slots_in_page=slots)
        else:
            assert plan.update(flat, off, lens, q_pos, ids, slots), executor.last_error()
        up = lambda a: torch.from_numpy(a.view(np.int16)).to(dev)
        o = torch.full((n, H, D), float("nan"), dtype=torch.float16, device=dev)
        assert executor.beginForwardPassCB()
        assert executor.encodePagedDecodeStepPlanned(plan, up(q), up(kn), up(vn), kp, vp, o, case.scale, MLC_F16,
                                                     MLC_F16), executor.last_error()
        assert executor.flushForwardPassCB(), executor.last_error()
        oracle_mod.scatter_kv_paged_batched_f16(kn, kp_ref, ids, slots, P, KVH, D)
        oracle_mod.scatter_kv_paged_batched_f16(vn, vp_ref, ids, slots, P, KVH, D)
        want = oracle_mod.paged_attention(q.astype(np.float32), kp_ref.view(np.float16), vp_ref.view(np.float16), flat,
                                          off, lens, q_pos, H, KVH, D, P, causal=True, scale=case.scale)
        assert np.array_equal(kp.cpu().numpy().view(np.uint16).reshape(-1), kp_ref)
        assert np.array_equal(vp.cpu().numpy().view(np.uint16).reshape(-1), vp_ref)
        assert_attention_close(o.float().cpu().numpy(), want)
    # rules: a table that does not fit its pages is rejected and the plan stays usable
    assert not plan.update(flat, off, lens + 10000, q_pos, ids, slots)
    plan.destroy()


def test_in_kernel_merge_option_matches_oracle():
    """MLC_B200_DECODE_INKERNEL_MERGE=1 (arrival counters + polling mergers inside the attention
    kernel, no merge kernel) in a child process: same results, one launch per layer."""
    import os
    import subprocess
    import sys
    code = r'''
import numpy as np, torch, oracle
from mlcompiler_b200 import Executor, synth
from mlcompiler_b200.capi import MLC_F16
from tests.util import DeviceCase, assert_attention_close
ex = Executor(0)
for seed, lens, shape in ((51, [2048, 64, 700, 1500, 33], dict(H=32, KVH=4, D=64)), (52, [3000, 129], dict(H=32, KVH=8, D=128))):
    case = synth.make_case(seed, lens, **shape)
    dc = DeviceCase(case)
    plan = ex.createPlan(case.pt_flat, case.pt_off, case.seq_lens, case.q_pos, case.N, case.H, case.KVH, case.D, case.P,
                         True, case.capacity, page_ids=case.page_ids, slots_in_page=case.slots)
    for rep in range(3):
        o = dc.out()
        l0 = ex.launchCount()
        assert ex.beginForwardPassCB()
        assert ex.encodePagedDecodeStepPlanned(plan, dc.q, dc.k_new, dc.v_new, dc.k_pool, dc.v_pool, o, case.scale, MLC_F16, MLC_F16), ex.last_error()
        assert ex.flushForwardPassCB(), ex.last_error()
        assert ex.launchCount() - l0 == 1
        kp = case.k_pool.view(np.uint16).reshape(-1).copy(); vp = case.v_pool.view(np.uint16).reshape(-1).copy()
        oracle.scatter_kv_paged_batched_f16(case.k_new, kp, case.page_ids, case.slots, case.P, case.KVH, case.D)
        oracle.scatter_kv_paged_batched_f16(case.v_new, vp, case.page_ids, case.slots, case.P, case.KVH, case.D)
        want = oracle.paged_attention(case.q.astype(np.float32), kp.view(np.float16), vp.view(np.float16), case.pt_flat, case.pt_off,
                                      case.seq_lens, case.q_pos, case.H, case.KVH, case.D, case.P, causal=True, scale=case.scale)
        assert_attention_close(o.float().cpu().numpy(), want)
    plan.destroy()
ex.close()
print("ok")
'''
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, MLC_B200_DECODE_INKERNEL_MERGE="1", PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr


def test_whole_pass_call_equals_layer_by_layer(executor, oracle_mod):
    """mlc_encode_paged_decode_pass_planned = the per-layer call in a loop: same pools, same outputs
    (within the parity tolerance: the single launch of the pass call groups the work differently)."""
    import torch
    case = synth.make_case(61, [100, 257, 33, 2000], 32, 4, 64)
    layers = 3
    dcs = [DeviceCase(case) for _ in range(2 * layers)]
    outs = [dc.out() for dc in dcs]
    plan = make_plan(executor, case)
    a, b = dcs[:layers], dcs[layers:]
    assert executor.beginForwardPassCB()
    for i, dc in enumerate(a):
        assert executor.encodePagedDecodeStepPlanned(plan, dc.q, dc.k_new, dc.v_new, dc.k_pool, dc.v_pool, outs[i],
                                                     case.scale, MLC_F16, MLC_F16), executor.last_error()
    ptrs = [executor.pointerArray(x) for x in ([dc.q for dc in b], [dc.k_new for dc in b], [dc.v_new for dc in b],
                                                [dc.k_pool for dc in b], [dc.v_pool for dc in b], outs[layers:])]
    assert executor.encodePagedDecodePassPlanned(plan, *ptrs, case.scale, MLC_F16, MLC_F16), executor.last_error()
    assert executor.flushForwardPassCB(), executor.last_error()
    kp, vp, want = oracle_step(oracle_mod, case)
    for i in range(layers):
        # the pass call may sum a head's tokens in other parts than the per-layer launch: same result within
        # the parity tolerance, pools bit for bit
        assert_attention_close(outs[layers + i].float().cpu().numpy(), outs[i].float().cpu().numpy())
        assert_attention_close(outs[layers + i].float().cpu().numpy(), want)
        assert torch.equal(a[i].k_pool, b[i].k_pool) and torch.equal(a[i].v_pool, b[i].v_pool)
    plan.destroy()


@pytest.mark.parametrize("layers,groups", [(3, 0), (12, 0), (12, 1), (5, 3)])
def test_host_buffer_pass_equals_layer_by_layer(executor, layers, groups):
    """mlc_encode_paged_decode_pass_host = copy in + the per-layer call + copy out: same pools and the same
    outputs (within the parity tolerance), for every way of cutting the layers into groups."""
    import torch
    case = synth.make_case(62, [100, 257, 33, 2000], 32, 4, 64)
    N, H, KVH, D = case.N, case.H, case.KVH, case.D
    plan = make_plan(executor, case)
    a = [DeviceCase(case) for _ in range(layers)]
    b = [DeviceCase(case) for _ in range(layers)]
    gen = torch.Generator().manual_seed(7)
    nq, nkv = N * H * D, N * KVH * D
    host_in = torch.randn((layers, nq + 2 * nkv), generator=gen).to(torch.float16).pin_memory()
    dev_in = torch.zeros_like(host_in, device="cuda")
    dev_o = torch.zeros((layers, N, H, D), dtype=torch.float16, device="cuda")
    host_o = torch.zeros((layers, N, H, D), dtype=torch.float16).pin_memory()
    want = [dc.out() for dc in a]
    assert executor.beginForwardPassCB()
    rows = host_in.cuda()
    torch.cuda.synchronize()
    for i, dc in enumerate(a):
        assert executor.encodePagedDecodeStepPlanned(plan, rows[i, :nq], rows[i, nq:nq + nkv], rows[i, nq + nkv:], dc.k_pool,
                                                     dc.v_pool, want[i], case.scale, MLC_F16, MLC_F16), executor.last_error()
    ptrs = [executor.pointerArray(x) for x in ([dc.k_pool for dc in b], [dc.v_pool for dc in b])]
    assert executor.encodePagedDecodePassHost(plan, host_in, dev_in, *ptrs, dev_o, host_o, case.scale, MLC_F16, MLC_F16,
                                              groups), executor.last_error()
    assert executor.flushForwardPassCB(), executor.last_error()      # host_o is complete here, no further sync
    for i in range(layers):
        # one launch for the pass (rows read from and written to host memory by the kernel) or copies +
        # a launch per layer: the same result within the parity tolerance, the same pools bit for bit
        assert_attention_close(host_o[i].float().numpy(), want[i].float().cpu().reshape(N, H, D).numpy())
        assert torch.equal(a[i].k_pool, b[i].k_pool) and torch.equal(a[i].v_pool, b[i].v_pool)
    plan.destroy()


def test_host_buffer_pass_is_refused_during_capture(executor):
    import torch
    case = synth.make_case(63, [70, 130], 8, 2, 64)
    plan = make_plan(executor, case)
    dc = DeviceCase(case)
    row = case.N * (case.H + 2 * case.KVH) * case.D
    host_in = torch.zeros((1, row), dtype=torch.float16).pin_memory()
    dev_in = torch.zeros((1, row), dtype=torch.float16, device="cuda")
    dev_o = torch.zeros((1, case.N, case.H, case.D), dtype=torch.float16, device="cuda")
    host_o = torch.zeros((1, case.N, case.H, case.D), dtype=torch.float16).pin_memory()
    ptrs = [executor.pointerArray([dc.k_pool]), executor.pointerArray([dc.v_pool])]
    torch.cuda.synchronize()
    assert executor.beginForwardPassCB()
    assert executor.beginCapture()
    assert not executor.encodePagedDecodePassHost(plan, host_in, dev_in, *ptrs, dev_o, host_o, case.scale, MLC_F16, MLC_F16)
    assert "captured" in executor.last_error()
    out = dc.out()
    assert executor.encodePagedDecodeStepPlanned(plan, dc.q, dc.k_new, dc.v_new, dc.k_pool, dc.v_pool, out, case.scale,
                                                 MLC_F16, MLC_F16), executor.last_error()     # the capture itself is intact
    graph = executor.endCapture()
    graph.launch()
    assert executor.flushForwardPassCB(), executor.last_error()
    graph.destroy()
    plan.destroy()
