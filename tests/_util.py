"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch


def f32(x: torch.Tensor) -> np.ndarray:
    return x.detach().to(torch.float32).cpu().numpy()


def u8(x: torch.Tensor) -> np.ndarray:
    return x.detach().contiguous().view(torch.uint8).cpu().numpy()


def fmt_of(dtype) -> str:
    return {torch.float8_e4m3fn: "e4m3", torch.float8_e5m2: "e5m2", torch.float4_e2m1fn_x2: "e2m1"}[dtype]


def make(shape, dtype, seed, kind="plain", device="cuda"):
    """Seeded inputs generated on the CPU (so the oracle and the kernels see identical bits)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(*shape, generator=g)
    if kind == "outlier":
        x = torch.where(torch.rand(*shape, generator=g) < 0.001, x * 50, x)
    elif kind == "small":
        x = x * 1e-3
    elif kind == "weight":
        x = x * 0.02
    elif kind == "zeros_mixed":
        x[: max(1, shape[0] // 3)] = 0
    return x.to(dtype).to(device)


def assert_bits_equal(got: np.ndarray, want: np.ndarray, what=""):
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    if got.dtype == np.float32:
        got, want = got.view(np.uint32), want.view(np.uint32)
    bad = np.flatnonzero(got.reshape(-1) != want.reshape(-1))
    assert bad.size == 0, f"{what}: {bad.size} of {got.size} differ, first at {bad[:5]}: {got.reshape(-1)[bad[:5]]} vs {want.reshape(-1)[bad[:5]]}"
