"""GPU tests of the tensor-parallel GEMV entry point (b2_w4_linear_tp) on ONE GPU: the "ranks" are row shards of one
matrix launched one after the other on one stream, every rank's gathered buffer lives on the same device, so the peer
stores, the piece-wise column mapping, the arrival counters and the consumer-side wait are all exercised without a
second GPU.  (The launches are stream-ordered: a consumer never spins on a kernel that has not finished.)
"""
import numpy as np
import pytest
import torch

import oracle
from nanoserve_b200 import ops
from tests.util import bits_to_torch, check_bf16_output, torch_to_bits, u32_to_torch

pytestmark = pytest.mark.gpu


def _shards(Wq, S, world, pieces):
    """Row shards of a row-concatenated matrix: rank r gets rows [r w/P, (r+1) w/P) of every piece."""
    out = []
    for r in range(world):
        rows, off = [], 0
        for w in pieces:
            wl = w // world
            rows.append(torch.arange(off + r * wl, off + (r + 1) * wl))
            off += w
        idx = torch.cat(rows).to(Wq.device)
        out.append((Wq[idx].contiguous(), S[idx].contiguous()))
    return out


@pytest.mark.parametrize("M", [1, 4])
@pytest.mark.parametrize("world,pieces,K", [(1, [512], 512), (2, [256, 128, 128], 1024), (4, [1024, 1024], 512),
                                            (2, [3584], 3584)])
def test_fused_all_gather_matches_single_gpu(kernels, M, world, pieces, K):
    G, N = 128, sum(pieces)
    X, Wq, S = oracle.synth_inputs(M, N, K, G, seed=61)
    x, wq, s = bits_to_torch(X), u32_to_torch(Wq), bits_to_torch(S)
    want = kernels.w4_linear(x, wq, s, G).float()
    gathered = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    sig = torch.zeros(world, dtype=torch.int32, device="cuda")
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    grids = []
    for r, (wq_r, s_r) in enumerate(_shards(wq, s, world, pieces)):
        n_local = wq_r.shape[0]
        cols, off = [], 0
        for w in pieces:
            cols.append((w // world, off + r * (w // world)))
            off += w
        d = ops.make_tp_desc(y_peers=[g.data_ptr() for g in gathered],
                             sig_peers=[sig[i:].data_ptr() for i in range(world)], ld=N, pieces=cols)
        kernels.w4_linear_tp(x, wq_r, s_r, d, G)
        grids.append(kernels.gemv_grid(M, n_local, K, G))
    torch.cuda.synchronize()
    assert kernels.device_status() == 0
    assert sig.tolist() == [world] * world  # every launch counted itself in once on every rank
    assert all(g > 0 for g in grids)
    # rows are independent, but a shard may be planned with another K split than the whole matrix: the fp32 sums are
    # taken in another order, so the bound is one bf16 rounding plus summation noise; all ranks hold the same bits
    tol = want.abs() * 2.0**-7 + 1e-5 * want.abs().max()
    for g in gathered:
        assert torch.all((g.float() - want).abs() <= tol)
        assert torch.equal(g, gathered[0])
    check_bf16_output(torch_to_bits(gathered[0]), oracle.w4_linear_f32(X, Wq, S, G, threads=oracle.max_threads()), 2e-5)


def test_consumer_waits_on_the_counter_and_reads_the_gathered_row(kernels):
    """Producer -> consumer chain through a gathered buffer: the second GEMV (SwiGLU prologue) waits on the counter
    of the first and must reproduce the two-call result."""
    G, M, K1, I = 128, 2, 512, 1024
    _, Wa, Sa = oracle.synth_inputs(1, 2 * I, K1, G, seed=71)  # gate | up
    _, Wb, Sb = oracle.synth_inputs(1, 384, I, G, seed=72)     # down
    wa, sa, wb, sb = u32_to_torch(Wa), bits_to_torch(Sa), u32_to_torch(Wb), bits_to_torch(Sb)
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(M, K1, device="cuda", generator=g).to(torch.bfloat16)
    gu = kernels.w4_linear(x, wa, sa, G)
    want = kernels.w4_linear_fused(gu, wb, sb, G, prologue=2)

    buf = torch.zeros(M, 2 * I, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(M, 384, dtype=torch.bfloat16, device="cuda")
    sig = torch.zeros(2, dtype=torch.int32, device="cuda")
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    for step in range(3):  # counters only grow: the target follows the epoch
        epoch.fill_(step)
        buf.zero_()
        prod = ops.make_tp_desc(y_peers=[buf.data_ptr()], sig_peers=[sig.data_ptr()], ld=2 * I, pieces=[(2 * I, 0)])
        kernels.w4_linear_tp(x, wa, sa, prod, G)
        cons = ops.make_tp_desc(y_local=out.data_ptr(), wait_sig=sig.data_ptr(), epoch=epoch.data_ptr(),
                                wait_per_epoch=1)
        kernels.w4_linear_tp(buf, wb, sb, cons, G, prologue=2)
        torch.cuda.synchronize()
        assert torch.equal(out, want), step
    assert kernels.device_status() == 0


def test_deferred_signal_chain(kernels):
    """The cheaper protocol, one rank standing in for the group: the producer only stores (defer), the consumer behind
    it on the stream announces it on the arrival counter and waits on that counter; a wait kernel behind the consumer
    does the same for the consumer's own output and closes the epoch.  Three epochs in a row, no host-side reset."""
    G, M, K1, I = 128, 1, 512, 768
    _, Wa, Sa = oracle.synth_inputs(1, 2 * I, K1, G, seed=71)  # gate | up
    _, Wb, Sb = oracle.synth_inputs(1, 384, I, G, seed=72)     # down
    wa, sa, wb, sb = u32_to_torch(Wa), bits_to_torch(Sa), u32_to_torch(Wb), bits_to_torch(Sb)
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(M, K1, device="cuda", generator=g).to(torch.bfloat16)
    want = kernels.w4_linear_fused(kernels.w4_linear(x, wa, sa, G), wb, sb, G, prologue=2)
    buf = torch.zeros(M, 2 * I, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(M, 384, dtype=torch.bfloat16, device="cuda")
    sig = torch.zeros(2, dtype=torch.int32, device="cuda")
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    ep = epoch.data_ptr()
    prod = ops.make_tp_desc(y_peers=[buf.data_ptr()], ld=2 * I, pieces=[(2 * I, 0)], defer=True)
    cons = ops.make_tp_desc(y_peers=[out.data_ptr()], ld=384, pieces=[(384, 0)], defer=True, wait_sig=sig.data_ptr(),
                            epoch=ep, wait_per_epoch=1, announce_peers=[sig.data_ptr()])
    tail = ops.make_tp_desc(wait_sig=sig.data_ptr() + 4, epoch=ep, wait_per_epoch=1,
                            announce_peers=[sig.data_ptr() + 4])
    for step in range(3):
        buf.zero_()
        out.zero_()
        kernels.w4_linear_tp(x, wa, sa, prod, G)
        kernels.w4_linear_tp(buf, wb, sb, cons, G, prologue=2)
        kernels.tp_wait_desc(tail, advance_epoch=True)
        torch.cuda.synchronize()
        assert torch.equal(out, want), step
        assert sig.tolist() == [step + 1, step + 1] and int(epoch) == step + 1
    assert kernels.device_status() == 0


def test_swiglu_epilogue_into_gathered_row(kernels):
    """gate|up with SwiGLU in its epilogue as a tensor-parallel producer (deferred signal): the slice of the activation
    row lands at its column of the gathered row, 8 bytes at a time, bit-identical to the single-GPU epilogue; with an
    odd element offset of the row the two-byte fallback is taken."""
    G, K, I = 128, 1024, 1536
    _, Wq, S = oracle.synth_inputs(1, 2 * I, K, G, seed=91)
    wq, s = u32_to_torch(Wq), bits_to_torch(S)
    x = torch.randn(1, K, device="cuda", generator=torch.Generator(device="cuda").manual_seed(2)).to(torch.bfloat16)
    want = kernels.w4_linear_fused(x, wq, s, G, epilogue=ops.EPI_SWIGLU_PAIRS)
    for off in (0, 1):
        buf = torch.full((4 * I + 8,), 7.0, dtype=torch.bfloat16, device="cuda")
        row = buf[off:off + 4 * I]  # a gathered row of four ranks' slices; this "rank" is the third
        desc = ops.make_tp_desc(y_peers=[row.data_ptr()], ld=4 * I, pieces=[(I, 2 * I)], defer=True)
        kernels.w4_linear_tp(x, wq, s, desc, G, epilogue=ops.EPI_SWIGLU_PAIRS)
        torch.cuda.synchronize()
        assert torch.equal(row[2 * I:3 * I], want[0])
        assert torch.all(row[:2 * I] == 7.0) and torch.all(row[3 * I:] == 7.0)
    # without the deferred signal the register epilogue cannot serve a producer: refused, nothing launched
    sig = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="code -3"):
        kernels.w4_linear_tp(x, wq, s, ops.make_tp_desc(y_peers=[buf.data_ptr()], sig_peers=[sig.data_ptr()], ld=4 * I,
                                                        pieces=[(I, 0)]), G, epilogue=ops.EPI_SWIGLU_PAIRS)
    assert kernels.device_status() == 0


def test_bounded_wait_reports_a_time_out(kernels):
    """A counter nobody bumps: the consumer gives up after its bounded wait and the device status says so; the
    context stays usable."""
    G, M, N, K = 128, 1, 64, 256
    X, Wq, S = oracle.synth_inputs(M, N, K, G, seed=81)
    x, wq, s = bits_to_torch(X), u32_to_torch(Wq), bits_to_torch(S)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    sig = torch.zeros(1, dtype=torch.int32, device="cuda")
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    cons = ops.make_tp_desc(y_local=out.data_ptr(), wait_sig=sig.data_ptr(), epoch=epoch.data_ptr(), wait_per_epoch=1)
    kernels.w4_linear_tp(x, wq, s, cons, G)
    torch.cuda.synchronize()
    assert kernels.device_status() != 0
    kernels.clear_status()
    assert kernels.device_status() == 0
    y = kernels.w4_linear(x, wq, s, G)  # the library still works
    check_bf16_output(torch_to_bits(y), oracle.w4_linear_f32(X, Wq, S, G), 2e-5)


def test_tp_error_codes(kernels):
    x = torch.zeros(1, 256, dtype=torch.bfloat16, device="cuda")
    wq = torch.zeros(64, 32, dtype=torch.int32, device="cuda")
    s = torch.ones(64, 2, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="code -1"):  # neither producer nor consumer
        kernels.w4_linear_tp(x, wq, s, ops.make_tp_desc(), 128)
    buf = torch.zeros(1, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="code -4"):  # a peer without a counter
        kernels.w4_linear_tp(x, wq, s, ops.make_tp_desc(y_peers=[buf.data_ptr()], sig_peers=[None], ld=64,
                                                          pieces=[(64, 0)]), 128)
    with pytest.raises(RuntimeError, match="code -1"):  # gathered row narrower than the shard
        kernels.w4_linear_tp(x, wq, s, ops.make_tp_desc(y_peers=[buf.data_ptr()], sig_peers=[buf.data_ptr()], ld=32,
                                                          pieces=[(64, 0)]), 128)


def test_host_step_equals_the_device_pass(kernels):
    """ShardedLayer.host_step (one CUDA graph: copy in, four launches, copy out) against the same pass on device
    tensors; the inputs are changed between two calls to show that the graph reads the pinned buffer each time."""
    from nanoserve_b200 import synth
    from nanoserve_b200.tp import ShardedLayer
    shapes = {"q": (256, 256), "k": (64, 256), "v": (64, 256), "o": (256, 256), "gate": (512, 256), "up": (512, 256),
              "down": (256, 512)}
    order = ["q", "k", "v", "o", "gate", "up", "down"]
    layer = ShardedLayer.synthetic(kernels, shapes, order, 128, seed=3, rank=0, world=1, device=torch.device("cuda"))
    layer.fuse()
    st = torch.cuda.Stream()
    g = torch.Generator().manual_seed(1)
    for hs in (layer.host_step(1, st), layer.host_step(1, st, zero_copy_out=True)):
        for _ in range(2):
            x = torch.randn(1, 256, generator=g).to(torch.bfloat16)
            a = torch.randn(1, 512, generator=g).to(torch.bfloat16)
            hs.x_host.copy_(x)
            hs.act_host.copy_(a)
            outs = hs()
            want = layer.decode_pass_fused4(x.cuda(), a.cuda())
            torch.cuda.synchronize()
            for o, w in zip(outs, want):
                assert torch.equal(o, w.cpu())
    assert kernels.device_status() == 0
