"""The decode kernel has two decompositions (split over CTAs + merge kernel, and (request, head) units
per CTA, whole or - when one dwarfs the rest - cut into runs that are combined by the last CTA to
arrive) and the planner picks one per batch. These tests run the attention and planned-call parity
suites again with each form forced (MLC_B200_DECODE_MODE=1 / 2, units never cut / cut at half the fair
share), so that none depends on what the planner happens to choose for a test's batch shape."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


FORCED = [
    # the split form, and one TMA instruction per pool instead of one per K/V pair
    ("split", {"MLC_B200_DECODE_MODE": "1", "MLC_B200_DECODE_KV_PAIR": "0"}),
    ("unit", {"MLC_B200_DECODE_MODE": "2", "MLC_B200_DECODE_UNIT_CUT": "0"}),
    ("unit_cut", {"MLC_B200_DECODE_MODE": "2", "MLC_B200_DECODE_UNIT_CUT": "50", "MLC_B200_DECODE_UNIT_CUT_FORCE": "1"}),
    # the whole-pass launch with one, and with two, KV heads per CTA item instead of as many as fit
    ("pass_single_heads", {"MLC_B200_DECODE_PASS_HPC": "1"}),
    ("pass_head_pairs", {"MLC_B200_DECODE_PASS_HPC": "2"}),
    # the pass entry points as one launch per layer, and the host-buffer pass through its copy pipeline
    ("layer_launches", {"MLC_B200_DECODE_PASS": "0"}),
    ("copy_pipeline", {"MLC_B200_DECODE_ZERO_COPY": "0"}),
]


@pytest.mark.parametrize("name,forced", FORCED, ids=[f[0] for f in FORCED])
def test_parity_suites_with_the_decomposition_forced(name, forced):
    env = dict(os.environ, **forced)
    files = ["tests/test_gpu_attention.py", "tests/test_gpu_planned.py", "tests/test_gpu_walker.py"]
    if forced.get("MLC_B200_DECODE_PASS") != "0":      # that file asserts that a pass is ONE launch
        files.append("tests/test_gpu_pass_launch.py")
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider", *files,
                        "-k", "not in_kernel_merge"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, f"{name} mode:\n" + r.stdout[-3000:] + r.stderr[-1000:]


def test_planner_choice_follows_the_batch_shape():
    """Balanced batches run as whole units, a batch dominated by one long request has that request's units
    cut over CTAs - one launch per layer either way; the split form (attention + merge kernel) is what
    MLC_B200_DECODE_MODE=1 gives."""
    import numpy as np
    import torch
    from mlcompiler_b200 import Executor, synth
    from mlcompiler_b200.capi import MLC_F16
    ex = Executor(0)
    dev = torch.device("cuda:0")

    def launches(lens):
        case = synth.make_case(5, lens, fill=False, **synth.SHAPE_A)
        pool = torch.zeros((case.capacity, case.P, case.KVH, case.D), dtype=torch.float16, device=dev)
        q = torch.zeros((case.N, case.H, case.D), dtype=torch.float16, device=dev)
        o = torch.zeros_like(q)
        plan = ex.createPlan(case.pt_flat, case.pt_off, case.seq_lens, case.q_pos, case.N, case.H, case.KVH, case.D,
                             case.P, True, case.capacity)
        assert ex.beginForwardPassCB()
        before = ex.launchCount()
        assert ex.encodePagedFlashAttentionPlanned(plan, q, pool, pool, o, case.scale, MLC_F16, MLC_F16), ex.last_error()
        n = ex.launchCount() - before
        assert ex.flushForwardPassCB(), ex.last_error()
        plan.destroy()
        return n

    assert launches(np.random.default_rng(1).integers(64, 2049, 32)) == 1
    assert launches(np.array([16384] + [256] * 31)) == 1
    os.environ["MLC_B200_DECODE_MODE"] = "1"
    try:
        assert launches(np.array([16384] + [256] * 31)) == 2
    finally:
        del os.environ["MLC_B200_DECODE_MODE"]
    ex.close()


LONG_TAIL_SHAPES = [(32, 4, 64), (32, 8, 128), (32, 2, 64), (8, 8, 64), (16, 1, 128)]


@pytest.mark.parametrize("seed", range(10))
def test_random_long_tail_batches_match_the_oracle(executor, oracle_mod, seed):
    """Batches in which one or two requests dwarf the rest, so that the planner cuts their (request, head)
    units over CTAs (anything from 2 to dozens of parts, parts shorter than the CTA's warp count included):
    the fused decode step - row write, attention, in-CTA merge, cross-CTA combine - against the CPU oracle."""
    import numpy as np
    import torch
    from mlcompiler_b200 import synth
    from mlcompiler_b200.capi import MLC_F16
    from tests.test_gpu_planned import make_plan, oracle_step
    from tests.util import DeviceCase, assert_attention_close
    rng = np.random.default_rng(1000 + seed)
    H, KVH, D = LONG_TAIL_SHAPES[seed % len(LONG_TAIL_SHAPES)]
    n_long = int(rng.integers(1, 3))
    longs = rng.integers(3000, 30000 if D == 64 else 14000, n_long)
    shorts = rng.integers(1, 700, int(rng.integers(0, 6)))
    lens = rng.permutation(np.concatenate([longs, shorts])).astype(np.uint32)
    case = synth.make_case(2000 + seed, lens, H, KVH, D)
    dc = DeviceCase(case)
    o = dc.out()
    plan = make_plan(executor, case)
    before = executor.launchCount()
    assert executor.beginForwardPassCB()
    for _ in range(2):      # twice: the arrival counters must be back at zero after a launch
        assert executor.encodePagedDecodeStepPlanned(plan, dc.q, dc.k_new, dc.v_new, dc.k_pool, dc.v_pool, o, case.scale,
                                                     MLC_F16, MLC_F16), executor.last_error()
    assert executor.flushForwardPassCB(), executor.last_error()
    assert executor.launchCount() - before in (2, 4)     # one launch per call (two where the planner prefers the split form)
    torch.cuda.synchronize()
    kp, vp, want = oracle_step(oracle_mod, case)
    assert np.array_equal(dc.k_pool.cpu().numpy().view(np.uint16).reshape(-1), kp)
    assert np.array_equal(dc.v_pool.cpu().numpy().view(np.uint16).reshape(-1), vp)
    assert_attention_close(o.float().cpu().numpy(), want)
    plan.destroy()
