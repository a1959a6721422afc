"""Helpers shared by the GPU tests: oracle calls on torch tensors and input makers."""

import numpy as np
import torch

from oracle import nvfp4_oracle as o


def storage(t: torch.Tensor) -> np.ndarray:
    """``(rows, cols, l)`` view -> contiguous ``[l, rows, cols]`` numpy (bytes for FP8)."""
    t = t.permute(2, 0, 1).contiguous()
    if t.dtype == torch.float8_e4m3fn:
        t = t.view(torch.uint8)
    return t.cpu().numpy()


def blocked_storage(task_view: torch.Tensor) -> np.ndarray:
    return task_view.permute(5, 2, 4, 0, 1, 3).contiguous().view(torch.uint8).cpu().numpy()


def oracle_dense(inputs, out_dtype=np.float16) -> np.ndarray:
    """Oracle result ``[l, m, n]`` for dense inputs with 6-D blocked scales."""
    a, b, sfa, sfb, alpha = inputs
    m, half_k, _ = a.shape
    n, k = b.shape[0], 2 * half_k
    sa = o.from_blocked(blocked_storage(sfa), m, k // 16)
    sb = o.from_blocked(blocked_storage(sfb), n, k // 16)
    return o.gemm(storage(a), storage(b), sa, sb, float(alpha.item()), out_dtype)


def assert_matches_oracle(actual: torch.Tensor, expected: np.ndarray, name: str, exact: bool,
                          rtol=1e-3, atol=1e-3) -> None:
    got = actual.permute(2, 0, 1).contiguous().cpu().numpy() if actual.dim() == 3 else \
        actual.contiguous().cpu().numpy()
    assert got.shape == expected.shape and got.dtype == expected.dtype, name
    if exact:
        assert np.array_equal(got, expected), f"{name}: not bit-identical to the oracle"
    else:
        np.testing.assert_allclose(got.astype(np.float32), expected.astype(np.float32),
                                   rtol=rtol, atol=atol, err_msg=name)


def integer_scaled(case, default=None) -> bool:
    """Cases whose FP32 sums are exact in any order (integer scales, power-of-two or
    unit alpha), so the kernel must equal the oracle bit for bit. ``default`` is the
    workload's scale distribution when the case names none."""
    scales = case.params.get("scales", default)
    alpha = case.params.get("alpha", 1.0)
    return scales in ("int0_3", "int1_2") and alpha in (1.0, 0.015625)


def snapshot(inputs):
    return [t.to("cpu", copy=True) if isinstance(t, torch.Tensor) else t for t in inputs]


def unchanged(old, new) -> bool:
    if not isinstance(old, torch.Tensor):
        return True
    return torch.equal(old.view(torch.uint8) if old.dtype == torch.float8_e4m3fn else old,
                       (new.view(torch.uint8) if new.dtype == torch.float8_e4m3fn else new).cpu())
