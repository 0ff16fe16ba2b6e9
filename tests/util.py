import numpy as np
import torch


def u8(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.uint8).numpy()


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def npf(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().float().numpy()


def rel_err(got_f32: np.ndarray, ref_f32: np.ndarray) -> float:
    """max |got-ref| / max(|ref|, 2^-7 * rms(ref)): the floor keeps near-zero outputs from dominating."""
    ref = ref_f32.astype(np.float64)
    if ref.size == 0:
        return 0.0
    floor = 2.0**-7 * np.sqrt((ref**2).mean())
    denom = np.maximum(np.abs(ref), max(floor, 1e-30))
    return float((np.abs(got_f32.astype(np.float64) - ref) / denom).max())


def bf16_ulp(ref_f32: np.ndarray) -> np.ndarray:
    """Spacing of bf16 values at |ref| (8 significand bits)."""
    a = np.abs(ref_f32.astype(np.float64))
    e = np.floor(np.log2(np.maximum(a, 2.0**-126)))
    return np.exp2(e - 7)


def assert_bf16_close(got_bits, ref_bits, min_exact=0.97):
    """bf16 outputs of two fp32-accurate computations can differ by one rounding step where the
    fp32 values straddle a rounding boundary: allow <= 1 bf16 ulp (taken at max(|ref|, 2^-7 rms(ref)),
    the same floor as rel_err, since sums that cancel to ~0 carry the absolute error of their
    terms), and require most outputs to be identical."""
    got = (got_bits.astype(np.uint32) << 16).view(np.float32)
    ref = (ref_bits.astype(np.uint32) << 16).view(np.float32)
    assert np.isfinite(got).all()
    if got.size == 0:
        return
    floor = 2.0**-7 * np.sqrt((ref.astype(np.float64) ** 2).mean())
    allowed = bf16_ulp(np.maximum(np.abs(ref), floor))
    assert (np.abs(got.astype(np.float64) - ref) <= allowed).all()
    if got.size:
        assert (got_bits == ref_bits).mean() >= min_exact
