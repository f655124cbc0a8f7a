"""Calibrated int4 quantizer that writes the SAME weight format as ``ns_w4_quantize``.

The reference quantizes round-to-nearest per group (kernels/quant/w4a16.cuh:274-301) and names a calibrated method
(AWQ / GPTQ) as its next step (README.md:233-235: RTN costs +15.7 % perplexity on its 7B run).  This is that step for
the packed format of this library: GPTQ (Frantar et al., "GPTQ: Accurate Post-Training Quantization for Generative
Pre-trained Transformers", 2022 -- the published algorithm, restated here) quantizes the columns of a linear's weight
one after the other and, after each, spreads the rounding error over the columns not yet quantized, weighted by the
inverse Hessian ``H = 2 X^T X`` of the layer's calibration inputs.  Only the CHOICE of the nibbles and scales changes:
the output is ``Wq [N, K/8]`` (value k = 8j + i in bits 4i..4i+3 of word j, stored q = round(w / s) + 8 in 0..15) and
``S [N, K/G]`` bf16, exactly what ``ns_w4_linear`` / the on-disk container (weights_io.py) take, with the same scale
rule as the reference (largest magnitude of the group / 7, rounded to bf16, 1 for an all-zero group) applied to the
group's weights as they stand when the group is reached.

With uncorrelated inputs (H diagonal) nothing is spread and the result is the reference quantizer's, bit for bit
(tested).  A cold, offline path: plain PyTorch on whatever device the tensors live on.
"""
from typing import Optional, Tuple

import torch


def hessian(X: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    """H = 2 X^T X / T of calibration inputs X [T, K] (any float dtype); accumulate over batches by averaging."""
    X = X.reshape(-1, X.shape[-1]).to(dtype)
    return (2.0 / X.shape[0]) * (X.T @ X)


def _group_scale(Wg: torch.Tensor) -> torch.Tensor:
    """The reference's scale of a group [N, G] of fp32 weights: max |w| / 7 as fp32, rounded to bf16; 1 if all zero."""
    mx = Wg.abs().amax(dim=1)
    s = torch.where(mx > 0, mx / 7.0, torch.ones_like(mx))
    return s.to(torch.bfloat16)


def pack_nibbles(q: torch.Tensor) -> torch.Tensor:
    """q [N, K] integers in 0..15 -> int32 [N, K/8] (value k = 8j + i in bits 4i..4i+3 of word j)."""
    N, K = q.shape
    q = q.to(torch.int64).reshape(N, K // 8, 8)
    sh = 4 * torch.arange(8, device=q.device, dtype=torch.int64)
    w = (q << sh).sum(dim=2)                     # 0 .. 2^32 - 1
    w = torch.where(w >= 2**31, w - 2**32, w)    # the same 32 bits as a signed word
    return w.to(torch.int32)


def rtn_quantize(W: torch.Tensor, group: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """Round to nearest, the reference's arithmetic (w4a16.cuh:274-301), in PyTorch: (Wq int32 [N, K/8], S bf16)."""
    N, K = W.shape
    if K % group or group % 8:
        raise ValueError("K must be a multiple of the group size, the group size a multiple of 8")
    Wg = W.to(torch.float32).reshape(N, K // group, group)
    S = _group_scale(Wg.reshape(-1, group)).reshape(N, K // group)
    q = torch.clamp(torch.round(Wg / S.to(torch.float32)[:, :, None]) + 8, 0, 15)
    return pack_nibbles(q.reshape(N, K)), S


def gptq_quantize(W: torch.Tensor, H: torch.Tensor, group: int = 128, damp: float = 0.01, block: int = 128,
                  hessian_dtype=torch.float64) -> Tuple[torch.Tensor, torch.Tensor]:
    """W [N, K] (bf16 / fp32), H [K, K] = ``hessian(X)`` of the layer's calibration inputs.

    Returns (Wq int32 [N, K/8], S bf16 [N, K/G]) in the kernels' format.  ``damp``: fraction of the mean diagonal of H
    added to its diagonal (regularisation, as in the paper); ``block``: columns whose errors are spread lazily to the
    rest of the matrix in one matrix product (a multiple of ``group``).  The Cholesky factorisations run in
    ``hessian_dtype``; everything else in fp32.
    """
    N, K = W.shape
    if K % group or group % 8:
        raise ValueError("K must be a multiple of the group size, the group size a multiple of 8")
    if H.shape != (K, K):
        raise ValueError("H must be [K, K]")
    block = max(block, group) // group * group
    dev = W.device
    Wc = W.to(torch.float32).clone()
    Hh = H.to(hessian_dtype).clone()
    # a column that never saw a non-zero input carries no information: its weights are free, set them to zero
    dead = torch.diagonal(Hh) == 0
    Hh[dead, dead] = 1.0
    Wc[:, dead] = 0.0
    Hh += torch.eye(K, device=dev, dtype=hessian_dtype) * (damp * torch.diagonal(Hh).mean())
    # upper Cholesky factor U of H^-1 (H^-1 = U^T U): row i of U is what the error of column i spreads to the right
    L = torch.linalg.cholesky(Hh)
    Hinv = torch.cholesky_inverse(L)
    U = torch.linalg.cholesky(Hinv, upper=True).to(torch.float32)
    del Hh, L, Hinv

    Q = torch.empty((N, K), dtype=torch.float32, device=dev)
    S = torch.empty((N, K // group), dtype=torch.bfloat16, device=dev)
    for i1 in range(0, K, block):
        i2 = min(i1 + block, K)
        W1 = Wc[:, i1:i2].clone()
        E1 = torch.zeros_like(W1)
        U1 = U[i1:i2, i1:i2]
        s = None
        for i in range(i2 - i1):
            k = i1 + i
            if k % group == 0:  # the group's scale, from its weights as they stand now
                sb = _group_scale(W1[:, i:i + group])
                S[:, k // group] = sb
                s = sb.to(torch.float32)
            w = W1[:, i]
            q = torch.clamp(torch.round(w / s) + 8, 0, 15)
            Q[:, k] = q
            err = (w - (q - 8) * s) / U1[i, i]
            W1[:, i:] -= err[:, None] * U1[i, i:][None, :]
            E1[:, i] = err
        Wc[:, i2:] -= E1 @ U[i1:i2, i2:]
    return pack_nibbles(Q), S


def dequantize(Wq: torch.Tensor, S: torch.Tensor, group: int = 128) -> torch.Tensor:
    """fp32 weights (q - 8) * s of a packed matrix (for error measurements; the kernels never materialise this)."""
    N, KW = Wq.shape
    sh = 4 * torch.arange(8, device=Wq.device, dtype=torch.int32)
    q = ((Wq[:, :, None] >> sh) & 0xF).reshape(N, KW * 8).to(torch.float32) - 8.0
    return q * S.to(torch.float32).repeat_interleave(group, dim=1)


def output_error(W: torch.Tensor, Wq: torch.Tensor, S: torch.Tensor, X: torch.Tensor, group: int = 128) -> float:
    """|| X (W - dequant(Wq, S))^T ||_F / || X W^T ||_F on inputs X [T, K]: what the layer's consumers see."""
    Wf, Xf = W.to(torch.float32), X.reshape(-1, X.shape[-1]).to(torch.float32)
    ref = Xf @ Wf.T
    got = Xf @ dequantize(Wq, S, group).T
    return float((ref - got).norm() / ref.norm())


def quantize_linears(weights: dict, inputs: Optional[dict] = None, hessians: Optional[dict] = None, group: int = 128,
                     damp: float = 0.01, device: Optional[torch.device] = None) -> dict:
    """name -> W [N, K], and per linear either calibration inputs X [T, K] (``inputs``) or a ready H [K, K]
    (``hessians``, e.g. accumulated over batches); returns name -> (Wq uint32 numpy, S uint16 numpy bf16 bits), the
    tuples weights_io.save takes.  A linear with neither is quantized round-to-nearest."""
    out = {}
    for name, W in weights.items():
        W = W.to(device) if device is not None else W
        H = (hessians or {}).get(name)
        X = (inputs or {}).get(name)
        if H is None and X is not None:
            H = hessian(X.to(W.device))
        if H is None:
            Wq, S = rtn_quantize(W, group)
        else:
            Wq, S = gptq_quantize(W, H.to(W.device), group, damp)
        out[name] = (Wq.cpu().numpy().view("uint32"), S.view(torch.int16).cpu().numpy().view("uint16"))
    return out
