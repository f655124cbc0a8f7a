"""Helpers shared by the tests: numpy (bf16 bit patterns) <-> torch conversions and error bounds."""
import numpy as np
import torch


def bits_to_torch(bits: np.ndarray, device="cuda"):
    """uint16 bf16 bit patterns -> torch.bfloat16 tensor of the same shape."""
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16).to(device)


def torch_to_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().cpu().view(torch.int16).numpy().view(np.uint16)


def u32_to_torch(a: np.ndarray, device="cuda"):
    """uint32 packed words -> torch.int32 (the dtype the reference's binding uses, ops.py:78)."""
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int32)).to(device)


def torch_to_u32(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().cpu().numpy().view(np.uint32)


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def check_bf16_output(y_bits, ref_f32, accum_slack):
    """Bound for a bf16 result against the unrounded fp32 oracle value.

    One correct rounding to bf16 costs at most half an ulp = 2^-9 * 2^(e+1) <= 2^-8 * |ref|; on top of
    that the kernel's fp32 accumulation may differ from the oracle's double accumulation by
    `accum_slack` times the largest output magnitude.  Returns (max_abs_err, max_rel_err_vs_scale).
    """
    y = bf16_bits_to_f32(y_bits).astype(np.float64)
    ref = ref_f32.astype(np.float64)
    scale = np.abs(ref).max() + 1e-30
    err = np.abs(y - ref)
    bound = np.abs(ref) * 2.0**-8 + accum_slack * scale
    worst = np.argmax(err - bound)
    assert np.all(np.isfinite(y)), "non-finite output"
    assert np.all(err <= bound), (
        f"bf16 output outside tolerance at flat index {worst}: got {y.flat[worst]}, ref {ref.flat[worst]}, "
        f"err {err.flat[worst]:.3e} > bound {bound.flat[worst]:.3e}")
    return float(err.max()), float(err.max() / scale)
