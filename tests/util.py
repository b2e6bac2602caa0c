"""Helpers shared by the GPU parity tests."""
from __future__ import annotations

import numpy as np

# Tolerances of the attention parity bar: fp16 outputs, fp32 accumulation.
MAX_ABS = 2e-3
MIN_COS = 0.99999


def cosine(a: np.ndarray, b: np.ndarray) -> float:
    a = a.astype(np.float64).ravel()
    b = b.astype(np.float64).ravel()
    na, nb = np.linalg.norm(a), np.linalg.norm(b)
    if na == 0.0 and nb == 0.0:
        return 1.0
    if na == 0.0 or nb == 0.0:
        return 0.0
    return float(a @ b / (na * nb))


def assert_attention_close(got: np.ndarray, want: np.ndarray, max_abs: float = MAX_ABS, min_cos: float = MIN_COS):
    got = got.astype(np.float32)
    want = want.astype(np.float32)
    assert got.shape == want.shape
    assert np.isfinite(got).all(), "non-finite output"
    err = float(np.abs(got - want).max()) if got.size else 0.0
    assert err <= max_abs, f"max-abs error {err:.3e} > {max_abs}"
    # per (request, head) cosine, the granularity the reference's own test uses
    # (tests/test_paged_flash.cpp:196-204)
    g = got.reshape(-1, got.shape[-1])
    w = want.reshape(-1, want.shape[-1])
    for i in range(g.shape[0]):
        c = cosine(g[i], w[i])
        assert c >= min_cos, f"row {i}: cosine {c:.7f} < {min_cos}"


class DeviceCase:
    """Uploads a synth.PagedCase to the GPU as torch tensors."""

    def __init__(self, case, q_dtype="f16"):
        import torch
        self.case = case
        dev = torch.device("cuda:0")
        self.k_pool = torch.from_numpy(case.k_pool.view(np.int16)).to(dev)
        self.v_pool = torch.from_numpy(case.v_pool.view(np.int16)).to(dev)
        if q_dtype == "f16":
            self.q = torch.from_numpy(case.q.view(np.int16)).to(dev)
        else:
            self.q = torch.from_numpy(case.q.astype(np.float32)).to(dev)
        self.k_new = torch.from_numpy(case.k_new.view(np.int16)).to(dev)
        self.v_new = torch.from_numpy(case.v_new.view(np.int16)).to(dev)
        torch.cuda.synchronize()

    def out(self, o_dtype="f16"):
        import torch
        c = self.case
        dt = torch.float16 if o_dtype == "f16" else torch.float32
        return torch.full((c.N, c.H, c.D), float("nan"), dtype=dt, device="cuda:0")
