"""Helpers shared by the GPU parity tests: numpy <-> device tensors and the tolerance gate."""
import numpy as np
import torch

from tatara_b200 import synthetic as syn

# The acceptance gate of this repo on bf16 outputs against the fp32 oracle.
MAX_ABS, MIN_COSINE = 2e-2, 0.9999


def dev_bf16(a: np.ndarray) -> torch.Tensor:
    """uint16 bit patterns -> bf16 CUDA tensor of the same shape."""
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda().view(torch.bfloat16)


def dev_f32(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def host_u16(t: torch.Tensor) -> np.ndarray:
    return t.detach().view(torch.int16).cpu().numpy().view(np.uint16)


def host_f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


def cosine(a: np.ndarray, b: np.ndarray) -> float:
    a = a.astype(np.float64).ravel(); b = b.astype(np.float64).ravel()
    na, nb = np.linalg.norm(a), np.linalg.norm(b)
    if na == 0.0 and nb == 0.0:
        return 1.0
    return float(a @ b / (na * nb))


def assert_close_bf16(got_u16: np.ndarray, want_u16: np.ndarray, what: str = "",
                      max_abs: float = MAX_ABS, min_cos: float = MIN_COSINE):
    """max-abs-error <= 2e-2 and cosine >= 0.9999 on bf16 outputs."""
    got, want = syn.from_bf16(got_u16), syn.from_bf16(want_u16)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    err = float(np.max(np.abs(got - want))) if got.size else 0.0
    cos = cosine(got, want)
    assert err <= max_abs, f"{what}: max-abs {err:.4g} > {max_abs}"
    assert cos >= min_cos, f"{what}: cosine {cos:.6f} < {min_cos}"
    return err, cos


def bf16_ulp_distance(a_u16: np.ndarray, b_u16: np.ndarray) -> np.ndarray:
    """Distance in bf16 steps between two bf16 arrays (sign-magnitude ordered)."""
    def key(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return np.abs(key(a_u16) - key(b_u16))
