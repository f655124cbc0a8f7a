"""Small, self-contained runs of one kernel for profiler captures.

    python -m nanoserve_b200.profile_case gemv --m 1 --n 18944 --k 3584 --copies 16 --launches 6
    python -m nanoserve_b200.profile_case gemm --m 2048 --n 18944 --k 3584 --copies 2 --launches 3
    python -m nanoserve_b200.profile_case lm_head --m 1 --n 152064 --k 3584 --copies 1 --launches 4

Weights are random nibbles with the benchmark's scale distribution, generated on the device; `copies`
distinct matrices are used in rotation so that a launch reads DRAM rather than L2.  Each launch goes through
the library's C ABI exactly as the benchmark's do.  Keep the sizes small under a profiler.
"""
import argparse

import torch

from .ops import Kernels


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kind", choices=["gemv", "gemm", "lm_head"])
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--n", type=int, default=18944)
    ap.add_argument("--k", type=int, default=3584)
    ap.add_argument("--g", type=int, default=128)
    ap.add_argument("--copies", type=int, default=16)
    ap.add_argument("--launches", type=int, default=6)
    ap.add_argument("--flags", type=int, default=0)
    a = ap.parse_args()
    if a.kind == "gemv" and not 1 <= a.m <= 16:
        raise SystemExit("gemv: 1 <= m <= 16")
    if a.kind == "gemm" and a.m <= 16:
        raise SystemExit("gemm: m > 16")
    k = Kernels()
    k.init()
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(1)
    if a.kind == "lm_head":  # bf16 vocabulary projection with the block argmax (n = vocabulary rows)
        ws = [(torch.randn(a.n, a.k, device=dev, generator=gen) * 0.02).to(torch.bfloat16) for _ in range(a.copies)]
        x = torch.randn(a.m, a.k, device=dev, generator=gen).to(torch.bfloat16)
        nblk = k.lm_head_blocks(a.n)
        pv = torch.empty(nblk, dtype=torch.float32, device=dev)
        pi = torch.empty(nblk, dtype=torch.int32, device=dev)
        logits = torch.empty(a.m, a.n, dtype=torch.bfloat16, device=dev)
        for i in range(a.launches):
            k.lm_head(x, ws[i % a.copies], logits=logits, part_max=pv, part_idx=pi)
        torch.cuda.synchronize()
        if k.device_status() != 0:
            raise SystemExit("device status non-zero")
        print(f"lm_head m={a.m} v={a.n} k={a.k}: {a.launches} launches done")
        return
    ws = []
    for _ in range(a.copies):
        Wq = torch.randint(-2**31, 2**31 - 1, (a.n, a.k // 8), dtype=torch.int32, device=dev, generator=gen)
        S = (0.005 + (torch.randn(a.n, a.k // a.g, device=dev, generator=gen) * 0.01).abs()).to(torch.bfloat16)
        ws.append((Wq, S))
    x = torch.randn(a.m, a.k, device=dev, generator=gen).to(torch.bfloat16)
    y = torch.empty(a.m, a.n, dtype=torch.bfloat16, device=dev)
    for i in range(a.launches):
        Wq, S = ws[i % a.copies]
        k.w4_linear(x, Wq, S, a.g, flags=a.flags, out=y)
    torch.cuda.synchronize()
    if k.device_status() != 0:
        raise SystemExit("device status non-zero")
    print(f"{a.kind} m={a.m} n={a.n} k={a.k}: {a.launches} launches over {a.copies} weight copies done")


if __name__ == "__main__":
    main()
