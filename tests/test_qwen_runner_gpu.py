"""GPU test of the shape-only decode runner on a tiny configuration: logits of the prompt's last token and of the
first decode steps against a plain PyTorch fp32 forward on the dequantised weights (the torch reference is kept for
this floating-point path; bound: 3e-2 of the largest logit, bf16 activations between the operators), and graph replay
against eager stepping (identical tokens)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from nanoserve_b200.qwen import Qwen2Config, Qwen2Runner

pytestmark = pytest.mark.gpu

CFG = Qwen2Config(hidden=256, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=64, intermediate=512, vocab=1000,
                  rope_theta=1e4, rms_eps=1e-6, group=128)


def dequant(wt, G):
    Wq, S = wt
    sh = (4 * torch.arange(8, device=Wq.device, dtype=torch.int32))[None, None, :]
    q = ((Wq[:, :, None] >> sh) & 0xF).reshape(Wq.shape[0], -1).float() - 8.0
    return q * S.float().repeat_interleave(G, dim=1)


def torch_forward(r, ids, skip_mlp=False, skip_attn=False):
    """fp32 forward over the whole sequence `ids` (prompt + generated so far); returns logits of the last token.
    skip_mlp / skip_attn drop a sub-layer: used to show that the comparison would notice its absence."""
    cfg = r.cfg
    T, D, G = ids.shape[0], cfg.head_dim, cfg.group
    x = F.embedding(ids, r.embed).float()

    def norm(v, w):
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.rms_eps)) * w.float()

    pos = torch.arange(T, device=ids.device, dtype=torch.float32)
    fr = torch.outer(pos, r.inv_freq)
    cos, sin = torch.cat([fr, fr], -1).cos()[:, None, :], torch.cat([fr, fr], -1).sin()[:, None, :]

    def rope(v, H):
        v = v.view(T, H, D)
        rot = torch.cat([-v[..., D // 2:], v[..., :D // 2]], -1)
        return v * cos + rot * sin

    h = norm(x, r.layers[0]["ln_in"])
    for li, L in enumerate(r.layers):
        qkv = h @ dequant(L["qkv"], G).T + L["bias"].float()
        q = rope(qkv[:, :r.nq], cfg.n_heads).transpose(0, 1)[None]
        k = rope(qkv[:, r.nq:r.nq + r.nkv], cfg.n_kv_heads).transpose(0, 1)[None]
        v = qkv[:, r.nq + r.nkv:].view(T, cfg.n_kv_heads, D).transpose(0, 1)[None]
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)[0].transpose(0, 1).reshape(T, r.nq)
        if not skip_attn:
            x = x + a @ dequant(L["o"], G).T
        h = norm(x, L["ln_post"])
        # the runner stores gate|up as 16 gate rows, their 16 up rows, the next 16 gate rows ...
        gu = (h @ dequant(L["gu"], G).T).view(T, r.I // 16, 2, 16)
        act = F.silu(gu[:, :, 0].reshape(T, r.I)) * gu[:, :, 1].reshape(T, r.I)
        if not skip_mlp:
            x = x + act @ dequant(L["d"], G).T
        nxt = r.layers[li + 1]["ln_in"] if li + 1 < cfg.n_layers else r.final_norm
        h = norm(x, nxt)
    return h[-1:] @ r.lm_head.float().T


def test_decode_logits_and_graph(kernels):
    dev = torch.device("cuda")
    # norm gains large enough that attention and the MLP move the logits (the benchmark's model uses 0.001 so that
    # greedy decoding of a random model stays input-dependent; with that the layers would hardly show here)
    r = Qwen2Runner(CFG, kernels, dev, seed=3, max_len=96, norm_gain=1.0)
    prompt = torch.randint(0, CFG.vocab, (40,), device=dev, generator=torch.Generator(device=dev).manual_seed(5))
    with torch.cuda.stream(r.stream):
        first = int(r.prefill(prompt))
        seq = torch.cat([prompt, torch.tensor([first], device=dev)])
        for _ in range(3):
            logits = r.decode_step().float()  # logits for the token after `seq`
            ref = torch_forward(r, seq)
            scale = ref.abs().max()
            assert torch.all(torch.isfinite(logits))
            assert (logits - ref).abs().max() <= 3e-2 * scale, float((logits - ref).abs().max() / scale)
            # the bound means something only if a missing sub-layer would break it
            assert (torch_forward(r, seq, skip_mlp=True) - ref).abs().max() > 0.1 * scale
            assert (torch_forward(r, seq, skip_attn=True) - ref).abs().max() > 0.1 * scale
            seq = torch.cat([seq, r.tokens[int(r.step.item()) - 1:int(r.step.item())]])
    torch.cuda.synchronize()
    eager = r.generate(prompt, 12, use_graph=False)
    graphed = r.generate(prompt, 12, use_graph=True)
    assert eager == graphed
    assert eager[0] == first and len(eager) == 12
    assert kernels.device_status() == 0
