"""Tensor parallelism for the quantized linears: output rows sharded over ranks, outputs all-gathered.

The reference is single-GPU (python/nanoserve/qwen.py:12); this is new.  Rows of ``Wq [N, K/8]`` and
``S [N, K/G]`` are independent, so rank r of P keeps the contiguous row block [r*N/P, (r+1)*N/P) of every
matrix -- a zero-copy slice of the reference layout -- with K, and therefore every quantization group, whole.
X is replicated.  The only exchange is an all-gather of Y at a layer boundary (NCCL over NVLink on GPUs,
gloo in the CPU tests).  One process per GPU.
"""
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from . import synth


def _to_torch_bits(a: np.ndarray, dtype, device):
    view = {np.dtype(np.uint16): np.int16, np.dtype(np.uint32): np.int32}[a.dtype]
    t = torch.from_numpy(np.ascontiguousarray(a).view(view))
    if dtype is torch.bfloat16:
        t = t.view(torch.bfloat16)
    return t.to(device)


def gather_rows(parts: Sequence[torch.Tensor], world: int, group=None) -> List[torch.Tensor]:
    """All-gathers several local outputs ``[M, n_i / world]`` in ONE collective and returns the full
    ``[M, n_i]`` tensors.  The locals are packed back to back into one flat buffer, so a layer boundary
    costs one all-gather however many matrices end there."""
    if world == 1:
        return list(parts)
    flat = torch.cat([p.reshape(-1) for p in parts])
    out = torch.empty(world * flat.numel(), dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(out, flat, group=group)
    out = out.view(world, flat.numel())
    full, off = [], 0
    for p in parts:
        M, n_loc = p.shape
        blk = out[:, off:off + M * n_loc].reshape(world, M, n_loc)
        full.append(blk.permute(1, 0, 2).reshape(M, world * n_loc))
        off += M * n_loc
    return full


class ShardedLayer:
    """The seven quantized linears of one decoder layer, sharded by output rows."""

    # matrices whose outputs are consumed together share one all-gather
    BOUNDARIES = (("q", "k", "v"), ("o",), ("gate", "up"), ("down",))

    def __init__(self, linear: Callable, shards: Dict[str, Tuple[torch.Tensor, torch.Tensor]], G: int, rank: int,
                 world: int, group=None, full: Optional[Dict[str, Tuple[torch.Tensor, torch.Tensor]]] = None):
        self.linear, self.shards, self.G = linear, shards, G
        self.rank, self.world, self.group = rank, world, group
        self.full = full if full is not None else (shards if world == 1 else None)

    @classmethod
    def synthetic(cls, kernels, shapes, order, G, seed, rank, world, device, flags=0):
        """Random-init layer with the benchmark's distributions; each rank uploads only its rows."""
        shards = {}
        for name in order:
            N, K = shapes[name]
            if N % world:
                raise ValueError(f"{name}: {N} rows do not split evenly over {world} ranks")
            Wq, S = synth.synth_weight(N, K, G, seed)
            lo, hi = synth.shard_rows(N, rank, world)
            shards[name] = (_to_torch_bits(Wq[lo:hi], torch.int32, device),
                            _to_torch_bits(S[lo:hi], torch.bfloat16, device))

        def linear(x, Wq, S, G):
            return kernels.w4_linear(x, Wq, S, G, flags=flags)

        return cls(linear, shards, G, rank, world)

    def resident_bytes(self) -> int:
        return sum(w.numel() * 4 + s.numel() * 2 for w, s in self.shards.values())

    def decode_pass(self, x: torch.Tensor, act: torch.Tensor) -> List[torch.Tensor]:
        """One pass over the seven linears: q, k, v, o, gate, up take ``x [M, hidden]``; down takes
        ``act [M, intermediate]``.  Returns the seven full-width outputs in that order."""
        outs = []
        for names in self.BOUNDARIES:
            local = []
            for name in names:
                Wq, S = self.shards[name]
                inp = act if Wq.shape[1] * 8 == act.shape[1] and name == "down" else x
                local.append(self.linear(inp, Wq, S, self.G))
            outs.extend(gather_rows(local, self.world, self.group))
        return outs
