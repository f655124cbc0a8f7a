"""Tensor parallelism for the quantized linears: output rows sharded over ranks, outputs all-gathered.

The reference is single-GPU (python/nanoserve/qwen.py:12); this is new.  Rows of ``Wq [N, K/8]`` and
``S [N, K/G]`` are independent, so rank r of P keeps the contiguous row block [r*N/P, (r+1)*N/P) of every
matrix -- a zero-copy slice of the reference layout -- with K, and therefore every quantization group, whole.
X is replicated.  The only exchange is an all-gather of Y at a layer boundary.  Two ways to do it:
  * a collective (NCCL over NVLink on GPUs, gloo in the CPU tests): ``gather_rows``;
  * fused into the decode GEMV (``b2_w4_linear_tp``): the kernel stores its outputs straight into the gathered row of
    every rank through peer-mapped memory (``PeerBuffers``) and counts itself in; the consumer waits on the counter.
    At decode sizes a gathered row is a few KB and a collective costs more than the GEMV it follows.
One process per GPU.
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


class PeerBuffers:
    """Gathered-output rows and arrival counters of a tensor-parallel group, allocated as symmetric memory so that
    every rank holds a device pointer to every other rank's copy (plain peer loads/stores over NVLink; no multicast
    object is used).  ``rows``: name -> elements (bf16) of one gathered buffer; ``n_counters`` uint32 counters."""

    def __init__(self, rows: Dict[str, int], n_counters: int, device, group=None):
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.offsets, off = {}, 0
        for name, n in rows.items():
            self.offsets[name] = (off, n)
            off += (n * 2 + 255) & ~255
        self.counter_off = off
        nbytes = off + ((n_counters * 4 + 255) & ~255) + 256
        self.mem = symm.empty(nbytes, dtype=torch.uint8, device=device)
        self.mem.zero_()
        self.handle = symm.rendezvous(self.mem, self.group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.n_counters = n_counters
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.reset()

    def local(self, name: str, M: int) -> torch.Tensor:
        """This rank's gathered buffer ``[M, n / M]`` (bf16 view of the symmetric allocation)."""
        off, n = self.offsets[name]
        return self.mem[off:off + n * 2].view(torch.bfloat16).view(M, n // M)

    def peers(self, name: str) -> List[int]:
        off, _ = self.offsets[name]
        return [p + off for p in self.ptrs]

    def counter(self, i: int, rank: Optional[int] = None) -> int:
        base = self.ptrs[self.rank if rank is None else rank]
        return base + self.counter_off + 4 * i

    def counter_peers(self, i: int) -> List[int]:
        return [self.counter(i, r) for r in range(self.world)]

    def reset(self):
        """Zeroes the counters and the epoch on every rank; nothing of the group may be in flight."""
        torch.cuda.synchronize()
        dist.barrier(self.group)
        self.mem[self.counter_off:].zero_()
        self.epoch.zero_()
        torch.cuda.synchronize()
        dist.barrier(self.group)


class ShardedLayer:
    """The seven quantized linears of one decoder layer, sharded by output rows."""

    # matrices whose outputs are consumed together share one all-gather
    BOUNDARIES = (("q", "k", "v"), ("o",), ("gate", "up"), ("down",))

    def __init__(self, linear: Callable, shards: Dict[str, Tuple[torch.Tensor, torch.Tensor]], G: int, rank: int,
                 world: int, group=None, full: Optional[Dict[str, Tuple[torch.Tensor, torch.Tensor]]] = None):
        self.linear, self.shards, self.G = linear, shards, G
        self.rank, self.world, self.group = rank, world, group
        self.full = full if full is not None else (shards if world == 1 else None)
        self.kernels = None
        self.peer: Optional[PeerBuffers] = None

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

        layer = cls(linear, shards, G, rank, world)
        layer.kernels, layer.flags, layer.shapes = kernels, flags, dict(shapes)
        return layer

    def attach_peer_buffers(self, peer: "PeerBuffers", M: int):
        """Switches decode_pass to the fused all-gather: one gathered buffer per matrix (names of `shapes`, M rows
        each), one counter per layer boundary, shared by every layer that uses the same PeerBuffers (a boundary's
        buffers are consumed before the next pass reaches it: see decode_pass)."""
        from .ops import make_tp_desc
        self.peer, self.M = peer, M
        self.descs, self.waits = {}, []
        for b, names in enumerate(self.BOUNDARIES):
            per_epoch = 0
            for name in names:
                N, K = self.shapes[name]
                nl = N // self.world
                self.descs[name] = make_tp_desc(y_peers=peer.peers(name), sig_peers=peer.counter_peers(b), ld=N,
                                                pieces=[(nl, self.rank * nl)])
                per_epoch += self.world  # every launch of every rank signals once
            self.waits.append((peer.counter(b), per_epoch))

    # ------------------------------------------------------------------ four launches per pass
    # q | k | v and gate | up as one row-concatenated matrix each (rows of Wq / S are independent, so this is the same
    # arithmetic in fewer launches; the decode runner stores its weights this way).  Tensor parallel: every rank
    # concatenates ITS rows of the pieces, and the fused gather puts each piece at its own column of the gathered row.
    FUSED = (("qkv", ("q", "k", "v")), ("o", ("o",)), ("gu", ("gate", "up")), ("down", ("down",)))

    def fuse(self):
        """Builds the row-concatenated matrices (a copy: 7 matrices -> 4) and, with peer buffers attached, the
        descriptors of the four tensor-parallel launches.  Each launch also waits, before it reads its input, for
        the previous launch's gathered row -- the consumer-side wait of a decode step -- so a pass needs no wait
        kernels except one behind the last launch (which also advances the epoch)."""
        from .ops import make_tp_desc
        self.fused = {}
        for fname, names in self.FUSED:
            self.fused[fname] = (torch.cat([self.shards[n][0] for n in names]).contiguous(),
                                 torch.cat([self.shards[n][1] for n in names]).contiguous())
        if self.peer is None:
            return
        peer, P, r = self.peer, self.world, self.rank
        self.fdescs, prev = {}, None
        for b, (fname, names) in enumerate(self.FUSED):
            widths = [self.shapes[n][0] for n in names]
            pieces, col = [], 0
            for w in widths:
                pieces.append((w // P, col + r * (w // P)))
                col += w
            # deferred signal: a launch only stores; the next launch, which has seen it complete, announces it to
            # every rank and waits until every rank has announced its own
            wait = dict(wait_sig=peer.counter(prev), epoch=peer.epoch.data_ptr(), wait_per_epoch=P,
                        announce_peers=peer.counter_peers(prev)) if prev is not None else {}
            self.fdescs[fname] = make_tp_desc(y_peers=peer.peers(fname), ld=col, pieces=pieces, defer=True, **wait)
            prev = b
        # behind the last launch: announce it, wait for everybody's, close the epoch
        self.tail_desc = make_tp_desc(wait_sig=peer.counter(prev), epoch=peer.epoch.data_ptr(), wait_per_epoch=P,
                                      announce_peers=peer.counter_peers(prev))

    def decode_pass_fused4(self, x: torch.Tensor, act: torch.Tensor,
                           outs: Optional[List[torch.Tensor]] = None) -> List[torch.Tensor]:
        """One pass as four launches: q|k|v, o, gate|up take ``x``; down takes ``act``.  Returns the four full-width
        outputs [M, nq + 2 nkv], [M, hidden], [M, 2 I], [M, hidden] (written into ``outs`` when given, single GPU)."""
        k = self.kernels
        if self.peer is None:
            res = []
            for i, (fname, _) in enumerate(self.FUSED):
                Wq, S = self.fused[fname]
                res.append(k.w4_linear(act if fname == "down" else x, Wq, S, self.G, flags=self.flags,
                                       out=None if outs is None else outs[i]))
            return res
        outs = []
        peer = self.peer
        for fname, _ in self.FUSED:
            Wq, S = self.fused[fname]
            k.w4_linear_tp(act if fname == "down" else x, Wq, S, self.fdescs[fname], self.G, flags=self.flags)
            outs.append(peer.local(fname, self.M))
        k.tp_wait_desc(self.tail_desc, advance_epoch=True)
        return outs

    def host_step(self, M: int, stream: "torch.cuda.Stream", zero_copy_out: bool = False) -> "HostStep":
        """The pass as a serving loop calls it -- inputs and outputs in pinned host memory: see HostStep."""
        return HostStep(self, M, stream, zero_copy_out)

    def resident_bytes(self) -> int:
        return sum(w.numel() * 4 + s.numel() * 2 for w, s in self.shards.values())

    def decode_pass(self, x: torch.Tensor, act: torch.Tensor) -> List[torch.Tensor]:
        """One pass over the seven linears: q, k, v, o, gate, up take ``x [M, hidden]``; down takes
        ``act [M, intermediate]``.  Returns the seven full-width outputs in that order."""
        if self.peer is not None:
            return self._decode_pass_fused(x, act)
        outs = []
        for names in self.BOUNDARIES:
            local = []
            for name in names:
                Wq, S = self.shards[name]
                inp = act if Wq.shape[1] * 8 == act.shape[1] and name == "down" else x
                local.append(self.linear(inp, Wq, S, self.G))
            outs.extend(gather_rows(local, self.world, self.group))
        return outs

    def _decode_pass_fused(self, x: torch.Tensor, act: torch.Tensor) -> List[torch.Tensor]:
        """The same pass with the all-gather inside the GEMVs: every launch stores its rows into every rank's gathered
        buffer; at each boundary a one-thread kernel waits until all ranks' launches have counted themselves in.  The
        epoch advances once per pass.  A rank can run at most one boundary ahead of the slowest one (it needs
        everybody's rows to pass a wait), so a buffer is never overwritten while another rank still reads it."""
        k, peer = self.kernels, self.peer
        outs = []
        for b, names in enumerate(self.BOUNDARIES):
            for name in names:
                Wq, S = self.shards[name]
                inp = act if name == "down" else x
                k.w4_linear_tp(inp, Wq, S, self.descs[name], self.G, flags=self.flags)
                outs.append(peer.local(name, self.M))
            sig, per_epoch = self.waits[b]
            k.tp_wait(sig, peer.epoch.data_ptr(), per_epoch)
        peer.epoch.add_(1)
        return outs


class HostStep:
    """One decode pass of a fused ShardedLayer from host memory to host memory as ONE CUDA graph: the copy of the
    step's inputs from a pinned buffer (`x_host [M, hidden]`, `act_host [M, intermediate]`: views of one allocation,
    one copy), the four GEMV launches (and, tensor parallel, the wait behind them), the copy of all outputs into one
    pinned buffer (`out_host`, the four outputs back to back).  Calling the object replays the graph and waits for it:
    one graph launch and one stream synchronisation per step, whatever the number of kernels inside.  Fill the input
    views before the call; read `outs` (views of `out_host`) after it."""

    def __init__(self, layer: ShardedLayer, M: int, stream, zero_copy_out: bool = False):
        dev = layer.fused["qkv"][0].device
        hidden, inter = layer.shapes["q"][1], layer.shapes["down"][1]
        widths = [sum(layer.shapes[n][0] for n in names) for _, names in layer.FUSED]
        self.layer, self.M, self.stream = layer, M, stream
        self.in_host = torch.empty(M * (hidden + inter), dtype=torch.bfloat16).pin_memory()
        self.x_host = self.in_host[:M * hidden].view(M, hidden)
        self.act_host = self.in_host[M * hidden:].view(M, inter)
        self.out_host = torch.empty(M * sum(widths), dtype=torch.bfloat16).pin_memory()
        self.in_dev = torch.empty_like(self.in_host, device=dev)
        self.out_dev = torch.empty(M * sum(widths), dtype=torch.bfloat16, device=dev)
        self.outs, views, off = [], [], 0
        for w in widths:
            self.outs.append(self.out_host[off:off + M * w].view(M, w))
            views.append(self.out_dev[off:off + M * w].view(M, w))
            off += M * w
        self.h2d_bytes, self.d2h_bytes = self.in_host.numel() * 2, self.out_host.numel() * 2
        x_d, a_d = self.in_dev[:M * hidden].view(M, hidden), self.in_dev[M * hidden:].view(M, inter)

        def body():
            self.in_dev.copy_(self.in_host, non_blocking=True)
            if layer.peer is None and zero_copy_out:
                # the kernels store straight into the pinned output buffer: no copy node behind them
                layer.decode_pass_fused4(x_d, a_d, outs=self.outs)
                return
            if layer.peer is None:
                layer.decode_pass_fused4(x_d, a_d, outs=views)
            else:  # the gathered rows live in the symmetric buffers: bring them together for the one copy back
                for v, o in zip(views, layer.decode_pass_fused4(x_d, a_d)):
                    v.copy_(o)
            self.out_host.copy_(self.out_dev, non_blocking=True)

        with torch.cuda.stream(stream):
            body()  # every kernel variant loaded before the capture
            stream.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=stream):
                body()

    def __call__(self):
        # (a caller that already runs on `stream` saves the context switch: some microseconds of a step of eighty)
        if torch.cuda.current_stream(self.in_dev.device) == self.stream:
            self.graph.replay()
        else:
            with torch.cuda.stream(self.stream):
                self.graph.replay()
        self.stream.synchronize()
        return self.outs
