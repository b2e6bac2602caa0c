"""Host-side sharding of the paged-attention path over the GPUs of one box.

Two ways, both without any collective on the K/V data itself:
  * by request (independent units): `shard_requests_by_kv_bytes` in synth.py assigns whole
    requests to ranks, each rank owns a private pool;
  * by KV sequence, for very long contexts: every rank holds a contiguous slice of each
    request's pages, computes the un-normalised partial (o, m, l) over its slice, the
    partials (tens of KiB) are all-gathered and combined with the log-sum-exp rule.
The reference has a single device (compiler/runtime/metal_runtime.mm:5774-5777) and no
counterpart for either.
"""
from __future__ import annotations

import numpy as np


def slice_tables_for_rank(pt_flat, pt_off, seq_lens, P: int, rank: int, world: int):
    """Rank `rank`'s view of every request: its contiguous share of the request's pages
    (as evenly as pages divide) and the number of tokens that fall into them.

    Returns (local_pt_flat, local_pt_off, local_seq_lens, first_token) where first_token[r]
    is the logical position of the slice's first token.
    """
    pt_flat = np.asarray(pt_flat, np.uint32)
    pt_off = np.asarray(pt_off, np.uint32)
    seq_lens = np.asarray(seq_lens, np.uint32)
    N = len(seq_lens)
    flat, off, lens, first = [], [0], [], []
    for r in range(N):
        pages = pt_flat[pt_off[r]:pt_off[r + 1]]
        used = (int(seq_lens[r]) + P - 1) // P           # pages that hold tokens
        lo = used * rank // world
        hi = used * (rank + 1) // world
        flat.extend(pages[lo:hi].tolist())
        off.append(len(flat))
        tok_lo, tok_hi = lo * P, min(hi * P, int(seq_lens[r]))
        lens.append(max(tok_hi - tok_lo, 0))
        first.append(tok_lo)
    return (np.array(flat, np.uint32), np.array(off, np.uint32), np.array(lens, np.uint32),
            np.array(first, np.uint32))


def gather_partials(o_part, ml_part, group=None):
    """All-gathers per-rank partials with torch.distributed (NCCL on GPUs, gloo on CPU).
    o_part [N, H, D] fp32, ml_part [N, H, 2] fp32 -> ([world, N, H, D], [world, N, H, 2])."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    # one collective: o and (m, l) travel in the same buffer
    n_o = o_part.numel()
    send = torch.cat([o_part.reshape(-1), ml_part.reshape(-1)])
    recv = torch.empty((world, send.numel()), dtype=send.dtype, device=send.device)
    dist.all_gather(list(recv.unbind(0)), send, group=group)
    o_all = recv[:, :n_o].reshape(world, *o_part.shape)
    ml_all = recv[:, n_o:].reshape(world, *ml_part.shape)
    return o_all.contiguous(), ml_all.contiguous()
