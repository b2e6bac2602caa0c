"""Parity at the full size of the benchmark configurations 3, 4 and 5.

cfg3: 4 requests x 32768 tokens, H32 / KVH4 / D64 (long-context decode, units cut over CTAs).
cfg4: 128 requests, contexts U[512, 8192], H32 / KVH8 / D128 (2.3 GB of KV per layer).
cfg5: 8 requests, 512 new causal query tokens over 1536 cached + 512 new tokens, H32 / KVH8 / D128.

The pools are too large to fill from the host in reasonable time, so they are drawn on the GPU
(seeded torch generator, N(0,1) rounded to fp16) and the CPU oracle runs on a seeded sample: the
sampled requests' pages are gathered into a compact pool with renumbered page tables and handed to
the oracle, which reads the same fp16 bit patterns the kernel read. What does not depend on a sample
is checked in full: the KV writes bit for bit over the whole pool (every row of every page, written
or not), and every output row is finite. Each decode configuration runs twice: with the planner's
own choice of decomposition, and with (request, head) units forced to be cut over CTAs.

Tolerance: max-abs 2e-3 and per-(request, head) cosine 0.99999 on fp16 outputs (tests/util.py).
"""
import os

import numpy as np
import pytest

from mlcompiler_b200 import synth
from mlcompiler_b200.capi import MLC_F16
from tests.util import assert_attention_close

pytestmark = pytest.mark.gpu

FORMS = [
    ("planner", {}),
    ("unit_cut", {"MLC_B200_DECODE_MODE": "2", "MLC_B200_DECODE_UNIT_CUT_FORCE": "1"}),
]


class _Env:
    def __init__(self, kv):
        self.kv, self.prev = kv, {}

    def __enter__(self):
        for k, v in self.kv.items():
            self.prev[k] = os.environ.get(k)
            os.environ[k] = v

    def __exit__(self, *exc):
        for k, v in self.prev.items():
            if v is None:
                del os.environ[k]
            else:
                os.environ[k] = v


def _gpu_pools(case, seed):
    import torch
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    shape = (case.capacity, case.P, case.KVH, case.D)
    k = torch.randn(shape, generator=g, device="cuda", dtype=torch.float16)
    v = torch.randn(shape, generator=g, device="cuda", dtype=torch.float16)
    return k, v


def _compact(case, k_pool, v_pool, reqs):
    """Pages of the sampled requests gathered (on the GPU) into small pools on the host, with page tables
    that point into them."""
    import torch
    pages = np.concatenate([case.pt_flat[case.pt_off[r]:case.pt_off[r + 1]] for r in reqs]).astype(np.int64)
    idx = torch.from_numpy(pages).cuda()
    k = k_pool.index_select(0, idx).cpu().numpy()
    v = v_pool.index_select(0, idx).cpu().numpy()
    counts = np.array([case.pt_off[r + 1] - case.pt_off[r] for r in reqs], np.uint32)
    off = np.zeros(len(reqs) + 1, np.uint32)
    off[1:] = np.cumsum(counts)
    flat = np.arange(int(off[-1]), dtype=np.uint32)
    return k, v, flat, off


def _decode_config(executor, oracle_mod, config, sample, form_env):
    import torch
    lens = synth.config_lengths(config)
    shape = synth.SHAPE_B if config == 4 else synth.SHAPE_A
    case = synth.make_case(0xBEEF + config, lens, P=64, fill=False, **shape)
    rng = np.random.default_rng(0xBEEF + config)
    q = rng.standard_normal((case.N, case.H, case.D), dtype=np.float32).astype(np.float16)
    k_new = rng.standard_normal((case.N, case.KVH, case.D), dtype=np.float32).astype(np.float16)
    v_new = rng.standard_normal((case.N, case.KVH, case.D), dtype=np.float32).astype(np.float16)
    k_pool, v_pool = _gpu_pools(case, 0xBEEF + config)
    up = lambda a: torch.from_numpy(a.view(np.int16)).cuda()
    dq, dkn, dvn = up(q), up(k_new), up(v_new)
    # what the pools must look like after the step: one new row per request, every other byte as before
    ids = torch.from_numpy(case.page_ids.astype(np.int64)).cuda()
    sl = torch.from_numpy(case.slots.astype(np.int64)).cuda()
    want_k, want_v = k_pool.clone(), v_pool.clone()
    want_k.view(torch.int16)[ids, sl] = dkn
    want_v.view(torch.int16)[ids, sl] = dvn
    o = torch.full((case.N, case.H, case.D), float("nan"), dtype=torch.float16, device="cuda")
    with _Env(form_env):
        plan = executor.createPlan(case.pt_flat, case.pt_off, case.seq_lens, case.q_pos, case.N, case.H, case.KVH,
                                   case.D, case.P, True, case.capacity, page_ids=case.page_ids, slots_in_page=case.slots)
    assert executor.beginForwardPassCB()
    before = executor.launchCount()
    assert executor.encodePagedDecodeStepPlanned(plan, dq, dkn, dvn, k_pool, v_pool, o, case.scale, MLC_F16, MLC_F16), \
        executor.last_error()
    assert executor.flushForwardPassCB(), executor.last_error()
    torch.cuda.synchronize()
    assert executor.lastAttentionKernel() == 2
    assert executor.launchCount() - before <= 2, "one fused launch (units) or attention + merge (split form)"
    plan.destroy()
    assert torch.equal(k_pool.view(torch.int16), want_k.view(torch.int16)), "K pool differs from the expected scatter"
    assert torch.equal(v_pool.view(torch.int16), want_v.view(torch.int16)), "V pool differs from the expected scatter"
    del want_k, want_v
    got = o.float().cpu().numpy()
    assert np.isfinite(got).all()
    ks, vs, flat, off = _compact(case, k_pool, v_pool, sample)
    want = oracle_mod.paged_attention(q[sample].astype(np.float32), ks, vs, flat, off, case.seq_lens[sample],
                                      case.q_pos[sample], case.H, case.KVH, case.D, case.P, scale=case.scale)
    assert_attention_close(got[sample], want)


@pytest.mark.parametrize("form,env", FORMS, ids=[f[0] for f in FORMS])
def test_config3_full_size(executor, oracle_mod, form, env):
    _decode_config(executor, oracle_mod, 3, [0, 1, 2, 3], env)


@pytest.mark.parametrize("form,env", FORMS, ids=[f[0] for f in FORMS])
def test_config4_full_size(executor, oracle_mod, form, env):
    lens = synth.config_lengths(4)
    order = np.argsort(lens)
    rng = np.random.default_rng(4)
    # the shortest, the longest, the median and a few seeded picks
    sample = sorted(set([int(order[0]), int(order[-1]), int(order[len(order) // 2])] +
                        [int(r) for r in rng.choice(len(lens), 5, replace=False)]))
    _decode_config(executor, oracle_mod, 4, sample, env)


def test_config5_full_size(executor, oracle_mod):
    import torch
    N, cached, new = 8, 1536, 512
    case = synth.make_case(0xBEEF + 5, np.full(N, cached + new, np.uint32), P=64, fill=False, **synth.SHAPE_B)
    H, KVH, D, P = case.H, case.KVH, case.D, case.P
    k_pool, v_pool = _gpu_pools(case, 0xBEEF + 5)
    g = torch.Generator(device="cuda")
    g.manual_seed(55)
    q = torch.randn((N * new, H, D), generator=g, device="cuda", dtype=torch.float16)
    # new K / V rows in the reference's multi-token layout [KVH, tokens, D], scattered request by request
    k_src = torch.randn((N, KVH, new, D), generator=g, device="cuda", dtype=torch.float16)
    v_src = torch.randn((N, KVH, new, D), generator=g, device="cuda", dtype=torch.float16)
    want_k, want_v = k_pool.clone(), v_pool.clone()
    for r in range(N):
        table = case.pt_flat[case.pt_off[r]:case.pt_off[r + 1]]
        first = cached // P
        # scatterKVPaged takes the page table from the page that holds start_slot on (metal_runtime.mm:468-489)
        assert executor.scatterKVPaged(k_pool, table[first:], P, KVH, D, new, cached % P, k_src[r], 2, case.capacity), \
            executor.last_error()
        assert executor.scatterKVPaged(v_pool, table[first:], P, KVH, D, new, cached % P, v_src[r], 2, case.capacity), \
            executor.last_error()
        pos = np.arange(cached, cached + new)
        pg = torch.from_numpy(table[pos // P].astype(np.int64)).cuda()
        st = torch.from_numpy((pos % P).astype(np.int64)).cuda()
        want_k[pg, st] = k_src[r].permute(1, 0, 2)
        want_v[pg, st] = v_src[r].permute(1, 0, 2)
    torch.cuda.synchronize()
    assert torch.equal(k_pool.view(torch.int16), want_k.view(torch.int16)), "multi-token K scatter is not bit-exact"
    assert torch.equal(v_pool.view(torch.int16), want_v.view(torch.int16)), "multi-token V scatter is not bit-exact"
    del want_k, want_v

    o = torch.full((N * new, H, D), float("nan"), dtype=torch.float16, device="cuda")
    q_start, q_len = np.full(N, cached, np.uint32), np.full(N, new, np.uint32)
    assert executor.runPagedPrefillAttention(q, k_pool, v_pool, o, case.pt_flat, case.pt_off, case.seq_lens, q_start,
                                             q_len, N, H, KVH, D, P, case.scale, MLC_F16, MLC_F16, case.capacity), \
        executor.last_error()
    torch.cuda.synchronize()
    assert executor.lastAttentionKernel() == 3, "the tcgen05 prefill kernel did not run"
    assert torch.isfinite(o.float()).all()

    # oracle on a seeded sample of query rows: the corners of the 128-row query tiles and of the 64-token
    # pages, the first and the last row, and random ones; every sampled row with all 32 heads. A row is a
    # single-token causal step over its request's pages (compiler/runtime/operator_backend.cpp:930-955).
    rng = np.random.default_rng(5)
    rows = []
    for r in range(N):
        picks = {0, 1, 63, 64, 127, 128, 255, 256, 383, 384, new - 2, new - 1}
        picks.update(int(i) for i in rng.choice(new, 6, replace=False))
        rows += [(r, i) for i in sorted(picks)]
    reqs = sorted({r for r, _ in rows})
    ks, vs, flat, off = _compact(case, k_pool, v_pool, reqs)
    # one oracle "request" per sampled row, all pointing at their request's page list
    row_flat = np.concatenate([flat[off[reqs.index(r)]:off[reqs.index(r) + 1]] for r, _ in rows]).astype(np.uint32)
    row_off = np.zeros(len(rows) + 1, np.uint32)
    row_off[1:] = np.cumsum([off[reqs.index(r) + 1] - off[reqs.index(r)] for r, _ in rows])
    sel = np.array([r * new + i for r, i in rows])
    q_rows = q[torch.from_numpy(sel).cuda()].float().cpu().numpy()
    seq = np.full(len(rows), cached + new, np.uint32)
    pos = np.array([cached + i for _, i in rows], np.uint32)
    want = oracle_mod.paged_attention(q_rows, ks, vs, row_flat, row_off, seq, pos, H, KVH, D, P, scale=case.scale)
    got = o[torch.from_numpy(sel).cuda()].float().cpu().numpy()
    assert_attention_close(got, want)


def test_config5_launches_repeat_bit_for_bit(executor):
    """The prefill kernel's result must not depend on timing: the same launch repeated gives the same bits.
    (A parity wait in its epilogue could pass two barrier phases early - when a warp that had not followed the
    barrier phase by phase finished the last page's softmax while P.V of the page before was still running - and
    O was then read without the last two pages; rare, and visible only as run-to-run differences in one warp's rows.)"""
    import torch
    N, cached, new = 8, 1536, 512
    case = synth.make_case(0xBEEF + 5, np.full(N, cached + new, np.uint32), P=64, fill=False, **synth.SHAPE_B)
    H, KVH, D, P = case.H, case.KVH, case.D, case.P
    k_pool, v_pool = _gpu_pools(case, 0xBEEF + 5)
    g = torch.Generator(device="cuda")
    g.manual_seed(56)
    q = torch.randn((N * new, H, D), generator=g, device="cuda", dtype=torch.float16)
    torch.cuda.synchronize()
    q_start, q_len = np.full(N, cached, np.uint32), np.full(N, new, np.uint32)
    first = None
    for rep in range(12):
        o = torch.full((N * new, H, D), float("nan"), dtype=torch.float16, device="cuda")
        assert executor.runPagedPrefillAttention(q, k_pool, v_pool, o, case.pt_flat, case.pt_off, case.seq_lens, q_start,
                                                 q_len, N, H, KVH, D, P, case.scale, MLC_F16, MLC_F16, case.capacity), \
            executor.last_error()
        torch.cuda.synchronize()
        assert executor.lastAttentionKernel() == 3
        if first is None:
            first = o
        else:
            assert torch.equal(first.view(torch.int16), o.view(torch.int16)), f"launch {rep} differs from launch 0"
