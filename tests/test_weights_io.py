"""CPU tests of the packed-weight container: round trip, tensor-parallel row slices, corruption is detected."""
import numpy as np
import pytest

import oracle
from nanoserve_b200 import weights_io


def _layer(seed=0):
    W = oracle.fill_bf16(96 * 256, seed, 0.05).reshape(96, 256)
    Wq, S = oracle.w4_quantize(W, 128)
    emb = oracle.fill_bf16(50 * 64, seed + 1, 1.0).reshape(50, 64)
    return {"layers.0.q": (Wq, S), "embed": emb}, Wq, S, emb


def test_round_trip_and_alignment(tmp_path):
    tensors, Wq, S, emb = _layer()
    path = str(tmp_path / "model.nsw4")
    weights_io.save(path, tensors, meta={"model": "test", "group": 128})
    pw = weights_io.PackedWeights(path, verify=True)
    assert set(pw.names()) == {"layers.0.q", "embed"} and pw.meta["group"] == 128
    wq, s, G = pw.linear("layers.0.q")
    assert G == 128 and np.array_equal(wq, Wq) and np.array_equal(s, S)
    assert np.array_equal(pw.bf16("embed"), emb)
    for e in pw.tensors.values():
        for key in ("wq", "s", "data"):
            if key in e:
                assert e[key][0] % weights_io.ALIGN == 0
    # what was stored is what the oracle's linear consumes: same result from the file as from memory
    X = oracle.fill_bf16(2 * 256, 9, 1.0).reshape(2, 256)
    assert np.array_equal(oracle.w4_linear_f32(X, np.ascontiguousarray(wq), np.ascontiguousarray(s), 128),
                          oracle.w4_linear_f32(X, Wq, S, 128))


def test_row_shards_are_the_rows(tmp_path):
    tensors, Wq, S, _ = _layer(3)
    path = str(tmp_path / "m.nsw4")
    weights_io.save(path, tensors)
    pw = weights_io.PackedWeights(path)
    parts = [pw.linear("layers.0.q", r, 4) for r in range(4)]
    assert np.array_equal(np.concatenate([p[0] for p in parts]), Wq)
    assert np.array_equal(np.concatenate([p[1] for p in parts]), S)
    with pytest.raises(ValueError):
        pw.linear("layers.0.q", 0, 5)  # 96 rows do not split five ways
    with pytest.raises(KeyError):
        pw.linear("embed")


def test_corruption_and_foreign_files_are_rejected(tmp_path):
    tensors, *_ = _layer(5)
    path = str(tmp_path / "m.nsw4")
    weights_io.save(path, tensors)
    pw = weights_io.PackedWeights(path)
    off = pw.tensors["layers.0.q"]["wq"][0]
    del pw
    with open(path, "r+b") as f:
        f.seek(off + 7)
        b = f.read(1)
        f.seek(off + 7)
        f.write(bytes([b[0] ^ 0x10]))
    with pytest.raises(ValueError, match="checksum"):
        weights_io.PackedWeights(path, verify=True)
    other = tmp_path / "x.bin"
    other.write_bytes(b"not a weight file at all")
    with pytest.raises(ValueError, match="not a packed"):
        weights_io.PackedWeights(str(other))
    with pytest.raises(ValueError):
        weights_io.save(str(tmp_path / "bad.nsw4"), {"w": (np.zeros((4, 4), np.uint32), np.zeros((3, 1), np.uint16))})


@pytest.mark.gpu
def test_file_to_gpu_linear(tmp_path, kernels):
    """Quantize on the GPU, store, map, upload a rank's rows, run the linear: same bits as from memory."""
    import torch
    from tests.util import bits_to_torch, torch_to_bits, torch_to_u32
    W = bits_to_torch(oracle.fill_bf16(512 * 1024, 21, 0.05).reshape(512, 1024))
    Wq, S = kernels.w4_quantize(W, 128)
    path = str(tmp_path / "gpu.nsw4")
    weights_io.save(path, {"w": (torch_to_u32(Wq), torch_to_bits(S))})
    pw = weights_io.PackedWeights(path, verify=True)
    x = bits_to_torch(oracle.fill_bf16(3 * 1024, 22, 1.0).reshape(3, 1024))
    want = kernels.w4_linear(x, Wq, S, 128)
    wq2, s2 = pw.to_torch("w", "cuda")
    assert torch.equal(kernels.w4_linear(x, wq2, s2, 128), want)
    wq_r, s_r = pw.to_torch("w", "cuda", rank=1, world=4)
    assert torch.equal(kernels.w4_linear(x, wq_r, s_r, 128), want[:, 128:256])
