"""CPU tests (gloo, world_size 2) of the tensor-parallel host logic: row sharding and the packed all-gather.
The linear itself is supplied by the CPU oracle here; on GPUs it is the CUDA library."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from nanoserve_b200 import synth
from nanoserve_b200.tp import ShardedLayer, gather_rows

SHAPES = {"q": (64, 256), "k": (32, 256), "v": (32, 256), "o": (64, 256), "gate": (96, 256), "up": (96, 256),
          "down": (64, 384)}
ORDER = ["q", "k", "v", "o", "gate", "up", "down"]
G = 128


def _bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def _oracle_linear(x, Wq, S, G):
    y = oracle.w4_linear_bf16(_bits(x), Wq.numpy().view(np.uint32), _bits(S), G)
    return torch.from_numpy(y.view(np.int16)).view(torch.bfloat16)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shards = {}
        for name in ORDER:
            N, K = SHAPES[name]
            Wq, S = synth.synth_weight(N, K, G, seed=3)
            lo, hi = synth.shard_rows(N, rank, world)
            shards[name] = (torch.from_numpy(Wq[lo:hi].view(np.int32).copy()),
                            torch.from_numpy(S[lo:hi].view(np.int16).copy()).view(torch.bfloat16))
        layer = ShardedLayer(_oracle_linear, shards, G, rank, world)
        x = torch.from_numpy(synth.synth_x(M, 256, 1).view(np.int16)).view(torch.bfloat16)
        a = torch.from_numpy(synth.synth_x(M, 384, 2).view(np.int16)).view(torch.bfloat16)
        outs = layer.decode_pass(x, a)
        if rank == 0:
            q.put([_bits(o).copy() for o in outs])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("M", [1, 3])
def test_sharded_layer_equals_unsharded(M):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, M, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    x = synth.synth_x(M, 256, 1)
    a = synth.synth_x(M, 384, 2)
    for name, y in zip(ORDER, got):
        N, K = SHAPES[name]
        Wq, S = synth.synth_weight(N, K, G, seed=3)
        want = oracle.w4_linear_bf16(a if name == "down" else x, Wq, S, G)
        # row sharding leaves each output's arithmetic untouched: bit-exact
        assert np.array_equal(y, want), name


def test_shard_rows_partition():
    for N in (512, 3584, 18944, 100):
        for world in (1, 2, 4, 8):
            edges = [synth.shard_rows(N, r, world) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == N
            assert all(edges[i][1] == edges[i + 1][0] for i in range(world - 1))


def test_gather_rows_single_rank_is_identity():
    t = [torch.arange(6.0).view(2, 3)]
    assert gather_rows(t, 1)[0] is t[0]


def test_tp_descriptor_column_mapping():
    """make_tp_desc against the kernel's rule (tp_column in csrc/w4_gemv.cu): local column n of a shard made of up to
    three row-concatenated pieces goes to seg_dst[i] + (n - start of piece i).  Reassembling every rank's columns
    must give each gathered column exactly once, in q | k | v order."""
    from nanoserve_b200.ops import make_tp_desc

    def column(d, n):
        c = d.seg_dst[0] + n
        if n >= d.seg_end[0]:
            c = d.seg_dst[1] + (n - d.seg_end[0])
        if n >= d.seg_end[1]:
            c = d.seg_dst[2] + (n - d.seg_end[1])
        return c

    for world, widths in [(1, [64]), (2, [3584, 512, 512]), (4, [18944, 18944]), (8, [3584])]:
        total, seen = sum(widths), {}
        for r in range(world):
            pieces, off = [], 0
            for w in widths:
                pieces.append((w // world, off + r * (w // world)))
                off += w
            d = make_tp_desc(y_peers=[1] * world, sig_peers=[1] * world, ld=total, pieces=pieces)
            assert d.world == world and d.ld == total
            n_local = sum(w // world for w in widths)
            for n in range(n_local):
                c = column(d, n)
                assert c not in seen, (world, widths, r, n)
                seen[c] = (r, n)
        assert sorted(seen) == list(range(total))
        # piece i of rank r is contiguous and starts where the gathered piece starts plus r shards
        off = 0
        for i, w in enumerate(widths):
            for r in range(world):
                start_local = sum(x // world for x in widths[:i])
                assert seen[off + r * (w // world)] == (r, start_local)
            off += w
