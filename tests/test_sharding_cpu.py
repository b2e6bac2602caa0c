"""Multi-rank host logic on CPU: world_size-2 (and 4) gloo process groups.

Sequence sharding: every rank computes the partial of its page slice (with the CPU oracle
standing in for the kernel), partials are all-gathered through torch.distributed and
combined; the result equals attention over the whole sequence. Request sharding: the
longest-first packing balances KV bytes and covers every request exactly once.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mlcompiler_b200 import sharding, synth

H, KVH, D, P = 8, 2, 32, 16


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make_case():
    return synth.make_case(77, [16 * 9 + 5, 16 * 4, 3, 16 * 20 + 1], H, KVH, D, P=P)


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    case = _make_case()
    flat, off, lens, first = sharding.slice_tables_for_rank(case.pt_flat, case.pt_off, case.seq_lens, P, rank, world)
    o_part, ml_part = oracle.paged_attention_tiled(case.q.astype(np.float32), case.k_pool, case.v_pool, flat, off, lens,
                                                   np.zeros(case.N, np.uint32), H, KVH, D, P, causal=False,
                                                   partial=True)
    o_all, ml_all = sharding.gather_partials(torch.from_numpy(o_part), torch.from_numpy(ml_part))
    combined = oracle.lse_combine(o_all.numpy(), ml_all.numpy())
    np.save(os.path.join(out_dir, f"rank{rank}.npy"), combined)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_sequence_sharded_attention_over_gloo(oracle_mod, tmp_path, world):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    case = _make_case()
    whole = oracle_mod.paged_attention(case.q.astype(np.float32), case.k_pool, case.v_pool, case.pt_flat, case.pt_off,
                                       case.seq_lens, np.zeros(case.N, np.uint32), H, KVH, D, P, causal=False)
    for rank in range(world):
        got = np.load(tmp_path / f"rank{rank}.npy")
        assert np.abs(got - whole).max() <= 2e-6        # every rank ends with the full result


def test_slices_cover_each_request_exactly_once():
    case = _make_case()
    for world in (1, 2, 3, 4, 8):
        total = np.zeros(case.N, np.int64)
        seen = [[] for _ in range(case.N)]
        for rank in range(world):
            flat, off, lens, first = sharding.slice_tables_for_rank(case.pt_flat, case.pt_off, case.seq_lens, P, rank, world)
            total += lens
            for r in range(case.N):
                seen[r] += flat[off[r]:off[r + 1]].tolist()
                if lens[r]:
                    assert first[r] % P == 0
        assert np.array_equal(total, case.seq_lens.astype(np.int64))
        for r in range(case.N):
            used = (int(case.seq_lens[r]) + P - 1) // P
            assert seen[r] == case.pt_flat[case.pt_off[r]:case.pt_off[r] + used].tolist()


def test_request_sharding_balances_kv_bytes():
    lens = synth.config_lengths(4)
    for world in (2, 4, 8):
        shards = synth.shard_requests_by_kv_bytes(lens, world)
        assert sorted(r for s in shards for r in s) == list(range(len(lens)))
        load = np.array([lens[s].sum() for s in shards], np.float64)
        assert load.max() / load.mean() < 1.05       # greedy longest-first: within 5 % of even
