"""Shared helpers of the test-suite: numpy <-> device tensors, tolerance checks."""
import ml_dtypes
import numpy as np
import torch

BF16 = ml_dtypes.bfloat16


def to_dev(a, device="cuda"):
    """numpy array (incl. ml_dtypes.bfloat16) -> torch tensor on `device`, same bits."""
    if a is None:
        return None
    a = np.ascontiguousarray(a)
    if a.dtype == BF16:
        return torch.from_numpy(a.view(np.uint16).copy()).view(torch.bfloat16).to(device)
    return torch.from_numpy(a.copy()).to(device)


def to_np(t):
    """torch tensor -> numpy array with the same bits (bf16 as ml_dtypes.bfloat16)."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy().view(BF16)
    return t.numpy()


def tol_for(q_dtype, quant):
    """Tolerances of the decode path: 1e-2 for bf16, 5e-3 for fp16, 2e-2 with int8 KV."""
    if quant:
        return 2e-2
    return 1e-2 if q_dtype == "bfloat16" else 5e-3


def assert_close(out, golden, tol, what=""):
    o = np.asarray(out).astype(np.float32)
    g = np.asarray(golden).astype(np.float32)
    assert o.shape == g.shape, (o.shape, g.shape)
    assert np.all(np.isfinite(o)), f"{what}: non-finite output"
    err = np.abs(o - g)
    lim = tol + tol * np.abs(g)
    bad = err > lim
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.size} outside rtol=atol={tol}; max err {err.max():.3e}"
