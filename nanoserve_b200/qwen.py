"""Shape-only Qwen2 (Llama-architecture) runner on the B200 library: random-init weights, greedy decode.

Mirrors the reference's ``python/nanoserve/qwen.py`` (``Qwen2Runner.forward / generate``, lines 136-178) for the
W4 configuration: every linear is int4 group-128 through ``ns_w4_linear``; embeddings and lm_head stay bf16.  There
are no checkpoints offline, so weights are seeded random nibbles and scales with the benchmark's distributions.
Differences from the reference, all on the host side of the boundary:
  * q/k/v and gate/up are stored as one row-concatenated matrix each (one GEMV instead of three / two): rows of
    ``Wq``/``S`` are independent, so this is the same arithmetic in fewer launches.
  * One decode step is captured in a CUDA graph; the position lives in device memory (``b2_decode_attention_fused``,
    ``b2_lm_head``, ``b2_greedy_pick``), so the same graph is replayed for every token.  The reference runs
    ~400 eager launches per token (README.md:227-228).
  * Tensor parallel: every matrix is sharded by output rows over the ranks, outputs are all-gathered at the four
    layer boundaries; attention, norms and RoPE run replicated on the gathered activations.  In the decode step the
    gather is fused into the GEMVs (``b2_w4_linear_tp``: peer stores into every rank's gathered row + arrival
    counters, the consumer waits on the counter); the prompt uses NCCL.
  * The bf16 lm_head runs through the library's own GEMV (``b2_lm_head``) with the final norm in its prologue and
    the argmax per 128 rows in its epilogue; ranks hold slices of the vocabulary and exchange only their
    (largest logit, index) pairs.
Batch size 1, as in the reference (qwen.py:12).
"""
import ctypes
import os
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .ops import EPI_SWIGLU_PAIRS, EPI_SWIGLU_PAIRS8, EPI_SWIGLU_STAGED, PRO_STAGED, Kernels, make_tp_desc


@dataclass
class Qwen2Config:
    hidden: int = 3584
    n_layers: int = 28
    n_heads: int = 28
    n_kv_heads: int = 4
    head_dim: int = 128
    intermediate: int = 18944
    vocab: int = 152064
    rope_theta: float = 1e6
    rms_eps: float = 1e-6
    group: int = 128

    @classmethod
    def qwen25_7b(cls):
        return cls()


def _rand_w4(N, K, G, gen, device):
    """Random-init int4 weights with the benchmark's distributions: uniform nibbles, scales 0.005 + |N(0, 0.01)|."""
    Wq = torch.randint(-2**31, 2**31 - 1, (N, K // 8), dtype=torch.int32, device=device, generator=gen)
    S = (0.005 + (torch.randn(N, K // G, device=device, generator=gen) * 0.01).abs()).to(torch.bfloat16)
    return Wq, S


class Qwen2Runner:
    def __init__(self, cfg: Qwen2Config, kernels: Kernels, device, rank: int = 0, world: int = 1, seed: int = 0,
                 max_len: int = 1024, group=None, fused_gather: bool = True, norm_gain: float = 0.001):
        self.cfg, self.k, self.dev = cfg, kernels, device
        self.rank, self.world, self.group = rank, world, group
        self.max_len = max_len
        H, D = cfg.hidden, cfg.head_dim
        self.nq, self.nkv, self.I = cfg.n_heads * D, cfg.n_kv_heads * D, cfg.intermediate
        for n in (self.nq, self.nkv, self.I, H, cfg.vocab):
            if n % world:
                raise ValueError(f"{n} rows do not split evenly over {world} ranks")
        gen = torch.Generator(device=device).manual_seed(seed)

        def shard(t):  # rows [rank * n / world, (rank + 1) * n / world)
            n = t.shape[0] // world
            return t[rank * n:(rank + 1) * n].contiguous()

        def w4(N, K):
            Wq, S = _rand_w4(N, K, cfg.group, gen, device)  # same seed on every rank, then each keeps its rows
            return shard(Wq), shard(S)

        # gate|up row blocks: 16 gate rows + their 16 up rows (8 + 8 with B2_QWEN_GU_BLOCK=8: the 16-rows-per-warp epilogue)
        self.gu_block = int(os.environ.get("B2_QWEN_GU_BLOCK", "16")) if world == 1 else 16
        # library flags of the down projection that takes the converted activations (diagnostics: plan choices)
        self.down_flags = int(os.environ.get("B2_QWEN_DOWN_FLAGS", "0"), 0)
        self.layers = []
        for _ in range(cfg.n_layers):
            q, k, v = w4(self.nq, H), w4(self.nkv, H), w4(self.nkv, H)
            o = w4(H, self.nq)
            g, u = w4(self.I, H), w4(self.I, H)
            d = w4(H, self.I)
            bias = (torch.randn(self.nq + 2 * self.nkv, device=device, generator=gen) * 0.02).to(torch.bfloat16)
            # 16 gate rows, their 16 up rows, the next 16 gate rows ... (of this rank's shard): the decode GEMV then
            # holds a gate value and its up value in the same lane and applies SwiGLU in its epilogue (same rows, same
            # arithmetic)
            def pairs(a, b, blk=self.gu_block):
                return torch.stack([a.view(a.shape[0] // blk, blk, -1), b.view(b.shape[0] // blk, blk, -1)],
                                   1).reshape(2 * a.shape[0], -1).contiguous()
            gu = (pairs(g[0], u[0]), pairs(g[1], u[1]))
            self.layers.append({
                "qkv": (torch.cat([q[0], k[0], v[0]]), torch.cat([q[1], k[1], v[1]])),
                "o": o, "gu": gu, "d": d,
                "bias": bias,  # full-width: applied after the gather (Qwen2 has q/k/v biases, qwen.py:76,147-148)
                "ln_in": (norm_gain * (1 + 0.02 * torch.randn(H, device=device, generator=gen))).to(torch.bfloat16),
                "ln_post": (norm_gain * (1 + 0.02 * torch.randn(H, device=device, generator=gen))).to(torch.bfloat16),
            })
        self.final_norm = (1 + 0.02 * torch.randn(H, device=device, generator=gen)).to(torch.bfloat16)
        # Random nibbles make every linear amplify its input (about 2.8x at K = 3584), and a stack of them drives the
        # residual stream to one direction whatever the token: greedy decoding of such a model repeats a single id.
        # To keep the generated sequence input-dependent -- so that a wrong kernel shows up as different tokens -- the
        # norm gains are small (the layers perturb the stream instead of replacing it), the embeddings have unit
        # scale, and the lm_head is the embedding table under a fixed permutation of the vocabulary: the next token is,
        # up to the layers' perturbation, the permutation's image of the current one.
        self.embed = torch.randn(cfg.vocab, H, device=device, generator=gen).to(torch.bfloat16)
        perm = torch.randperm(cfg.vocab, device=device, generator=gen)
        self.lm_head = shard((self.embed[perm].float() * 0.02).to(torch.bfloat16))
        self.inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, dtype=torch.int64, device=device).float() / D))
        self.cache_k = torch.zeros(cfg.n_layers, cfg.n_kv_heads, max_len, D, dtype=torch.bfloat16, device=device)
        self.cache_v = torch.zeros_like(self.cache_k)
        # decode state on the device
        self.pos = torch.zeros(1, dtype=torch.int32, device=device)
        self.step = torch.zeros(1, dtype=torch.int32, device=device)
        self.tokens = torch.zeros(max_len, dtype=torch.int64, device=device)
        self.x = torch.zeros(1, H, dtype=torch.bfloat16, device=device)  # residual stream of the current token
        self.x_alt = torch.zeros_like(self.x)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.stream = torch.cuda.Stream(device=device)
        self.scratch = torch.empty(int(kernels.lib.b2_decode_workspace_bytes(cfg.n_heads, D)), dtype=torch.uint8,
                                   device=device)
        self.attn_flags = int(os.environ.get("B2_QWEN_ATTN_FLAGS", "2"))  # 1: merge inside the launch; 2: early cache reads
        # partials and arrival counters (zero between launches) of the fused attention kernel
        self.attn_ws = torch.zeros(int(kernels.lib.b2_decode_attention_fused_workspace_bytes(
            cfg.n_heads, cfg.n_kv_heads, D)), dtype=torch.uint8, device=device)
        # vocabulary projection: this rank's logits and one (largest logit, index) pair per 128 rows of its shard
        self.v_local = cfg.vocab // world
        self.nblk = kernels.lm_head_blocks(self.v_local)
        self.logits = torch.zeros(1, self.v_local, dtype=torch.bfloat16, device=device)
        self.part_max = torch.zeros(world, self.nblk, dtype=torch.float32, device=device)
        self.part_idx = torch.zeros(world, self.nblk, dtype=torch.int32, device=device)
        kernels.init()
        self.peer = None
        if world > 1 and fused_gather:
            self._setup_fused_gather()

    def _setup_fused_gather(self):
        """Symmetric buffers for the four gathered rows of a layer (shared by all layers: a rank cannot pass a wait
        before every rank has delivered, so it is never more than one boundary ahead of the slowest rank and a buffer
        is consumed everywhere before anyone overwrites it), four arrival counters per layer, and the descriptors of
        every tensor-parallel launch.  Signals are deferred: a GEMV only stores into the peers' rows; the kernel behind
        it on the stream announces it (one release per rank) before waiting for its own input."""
        from .tp import PeerBuffers
        cfg, k, P, r = self.cfg, self.k, self.world, self.rank
        H, I, nq, nkv, G = cfg.hidden, self.I, self.nq, self.nkv, cfg.group
        self.peer = peer = PeerBuffers({"qkv": nq + 2 * nkv, "o": H, "act": I, "d": H}, 4 * cfg.n_layers,
                                       self.dev, self.group)
        ep = peer.epoch.data_ptr()
        self.tp_desc = []

        def after(c):
            """Consumer side of boundary c: announce this rank's producer of c (the kernel in front on the stream),
            then wait until every rank has announced its own."""
            return dict(wait_sig=peer.counter(c), epoch=ep, wait_per_epoch=P, announce_peers=peer.counter_peers(c))

        for li in range(cfg.n_layers):
            c = 4 * li
            self.tp_desc.append({
                "qkv": make_tp_desc(peer.peers("qkv"), ld=nq + 2 * nkv, defer=True,
                                    pieces=[(nq // P, r * nq // P), (nkv // P, nq + r * nkv // P),
                                            (nkv // P, nq + nkv + r * nkv // P)], **(after(c - 1) if li > 0 else {})),
                "attn": make_tp_desc(**after(c)),
                "o": make_tp_desc(peer.peers("o"), ld=H, pieces=[(H // P, r * H // P)], defer=True),
                # gate|up with SwiGLU in its epilogue: this rank's slice of the activation row
                "gu": make_tp_desc(peer.peers("act"), ld=I, defer=True, pieces=[(I // P, r * I // P)], **after(c + 1)),
                "d": make_tp_desc(peer.peers("d"), ld=H, pieces=[(H // P, r * H // P)], defer=True, **after(c + 2)),
            })
        self.tp_tail = make_tp_desc(**after(4 * cfg.n_layers - 1))

    # ------------------------------------------------------------------ helpers
    def weight_bytes_per_token(self) -> int:
        """Bytes of weights one decode step streams on this rank (packed + scales + bf16 lm_head shard)."""
        n = 0
        for L in self.layers:
            for name in ("qkv", "o", "gu", "d"):
                Wq, S = L[name]
                n += Wq.numel() * 4 + S.numel() * 2
        return n + self.lm_head.numel() * 2

    def _st(self):
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def _gather(self, local: torch.Tensor) -> torch.Tensor:
        """[T, n / world] -> [T, n] (rank-major along the feature axis)."""
        if self.world == 1:
            return local
        T, n = local.shape
        out = torch.empty(self.world, T, n, dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=self.group)
        return out.permute(1, 0, 2).reshape(T, self.world * n)

    def _gather_parts(self, local: torch.Tensor, widths: List[int]) -> torch.Tensor:
        """Local output of a row-concatenated matrix ([T, sum(w_i / world)]) -> full [T, sum(w_i)] with each part
        contiguous (q | k | v order)."""
        if self.world == 1:
            return local
        T = local.shape[0]
        out = torch.empty(self.world, T, local.shape[1], dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=self.group)
        parts, off = [], 0
        for w in widths:
            wl = w // self.world
            parts.append(out[:, :, off:off + wl].permute(1, 0, 2).reshape(T, w))
            off += wl
        return torch.cat(parts, dim=1)

    def linear(self, x, wt):
        return self.k.w4_linear(x, wt[0], wt[1], self.cfg.group)

    # ------------------------------------------------------------------ prompt (eager, GEMM path)
    @torch.no_grad()
    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        """Runs the prompt, fills the KV cache, leaves the device state ready for decoding.  Returns the first
        generated token (tensor on the device)."""
        cfg, k = self.cfg, self.k
        T, D = ids.shape[0], cfg.head_dim
        assert T < self.max_len
        x = F.embedding(ids, self.embed).contiguous()
        h = k.rmsnorm(x, None, self.layers[0]["ln_in"], cfg.rms_eps)
        for li, L in enumerate(self.layers):
            qkv = self._gather_parts(self.linear(h, L["qkv"]), [self.nq, self.nkv, self.nkv])
            qkv = qkv + L["bias"]
            q, kk, v = qkv[:, :self.nq], qkv[:, self.nq:self.nq + self.nkv], qkv[:, self.nq + self.nkv:]
            k.rope(q, kk, self.inv_freq, cfg.n_heads, cfg.n_kv_heads, D, 0)
            self.cache_k[li, :, :T] = kk.reshape(T, cfg.n_kv_heads, D).transpose(0, 1)
            self.cache_v[li, :, :T] = v.reshape(T, cfg.n_kv_heads, D).transpose(0, 1)
            qh = q.reshape(T, cfg.n_heads, D).transpose(0, 1)[None]
            kh = kk.reshape(T, cfg.n_kv_heads, D).transpose(0, 1)[None]
            vh = v.reshape(T, cfg.n_kv_heads, D).transpose(0, 1)[None]
            a = F.scaled_dot_product_attention(qh, kh, vh, is_causal=True, enable_gqa=True)
            a = a[0].transpose(0, 1).reshape(T, self.nq).contiguous()
            h = k.rmsnorm(x, self._gather(self.linear(a, L["o"])), L["ln_post"], cfg.rms_eps)
            gu = self.linear(h, L["gu"])
            il = self.I // self.world
            gu = gu.view(T, il // self.gu_block, 2, self.gu_block)  # gate and up row blocks alternate (see __init__)
            act = self._gather(k.swiglu(gu[:, :, 0].reshape(T, il), gu[:, :, 1].reshape(T, il)))
            nxt = self.layers[li + 1]["ln_in"] if li + 1 < cfg.n_layers else self.final_norm
            h = k.rmsnorm(x, self._gather(self.linear(act, L["d"])), nxt, cfg.rms_eps)
        self.pos.fill_(T - 1)  # the pick advances it to T, the position of the first generated token
        self.step.zero_()
        if self.peer is not None:
            self.peer.reset()  # counters and epoch restart together, on every rank
        self._lm_head_and_pick(h[-1:].contiguous(), None, None)
        return self.tokens[0]

    def _lm_head_and_pick(self, x, r, wn):
        """Vocabulary projection of this rank's rows (final add + RMSNorm in its prologue, argmax per 128 rows in its
        epilogue), then the pick over all ranks' (value, index) pairs: two all-gathers of a few hundred bytes
        instead of one of the 152064 logits.  Returns this rank's logits."""
        cfg, k, w = self.cfg, self.k, self.world
        mine_v, mine_i = self.part_max[self.rank], self.part_idx[self.rank]
        k.lm_head(x, self.lm_head, logits=self.logits, part_max=mine_v, part_idx=mine_i,
                  idx_offset=self.rank * self.v_local, r=r, wn=wn, eps=cfg.rms_eps)
        if w > 1:
            dist.all_gather_into_tensor(self.part_max, mine_v, group=self.group)
            dist.all_gather_into_tensor(self.part_idx, mine_i, group=self.group)
        rc = k.lib.b2_greedy_pick(self.part_max.data_ptr(), self.part_idx.data_ptr(), w * self.nblk, cfg.vocab,
                                  self.embed.data_ptr(), cfg.hidden, self.pos.data_ptr(), self.tokens.data_ptr(),
                                  self.step.data_ptr(), self.x.data_ptr(), self._st())
        k._check(rc, "b2_greedy_pick")
        return self.logits

    def _greedy_next(self, logits):
        rc = self.k.lib.b2_greedy_next(logits.data_ptr(), self.cfg.vocab, self.embed.data_ptr(), self.cfg.hidden,
                                       self.pos.data_ptr(), self.tokens.data_ptr(), self.step.data_ptr(),
                                       self.x.data_ptr(), self.scratch.data_ptr(), self._st())
        self.k._check(rc, "b2_greedy_next")

    # ------------------------------------------------------------------ one decode step (graph-capturable)
    def _fused(self, x, wt, prologue, r=None, wn=None, x_out=None):
        return self.k.w4_linear_fused(x, wt[0], wt[1], self.cfg.group, prologue=prologue, r=r, wn=wn,
                                      eps=self.cfg.rms_eps, x_out=x_out)

    @torch.no_grad()
    def decode_step(self):
        """One token.  Six launches per layer on one GPU: qkv GEMV (residual add + RMSNorm folded in), attention
        (bias, RoPE, KV store and the pass over the cache in one kernel, then the merge), o GEMV, gate|up GEMV (add + norm
        in its prologue, SwiGLU in its epilogue), down GEMV.
        The residual stream alternates between two buffers because a fused GEMV may not overwrite the X other CTAs
        are still reading; every step starts again from `self.x`, where b2_greedy_next puts the next embedding."""
        if self.peer is not None:
            return self._decode_step_fused_gather()
        cfg, k, lib = self.cfg, self.k, self.k.lib
        D = cfg.head_dim
        x, x_alt = self.x, self.x_alt
        r, wn = None, self.layers[0]["ln_in"]  # pending residual and the norm that follows it
        for li, L in enumerate(self.layers):
            y = self._fused(x, L["qkv"], 1, r=r, wn=wn, x_out=x_alt if r is not None else None)
            if r is not None:
                x, x_alt = x_alt, x
            qkv = self._gather_parts(y, [self.nq, self.nkv, self.nkv]).contiguous()
            a = torch.empty(1, self.nq, dtype=torch.bfloat16, device=self.dev)
            rc = lib.b2_decode_attention_fused(qkv.data_ptr(), L["bias"].data_ptr(), self.inv_freq.data_ptr(),
                                               self.pos.data_ptr(), self.cache_k[li].data_ptr(),
                                               self.cache_v[li].data_ptr(), a.data_ptr(), self.attn_ws.data_ptr(),
                                               cfg.n_heads, cfg.n_kv_heads, D, self.max_len, None, self.attn_flags,
                                               self._st())
            k._check(rc, "b2_decode_attention_fused")
            o = self._gather(self.linear(a, L["o"]))
            if self.world == 1 and self.gu_block == 8:
                act = self.k.w4_linear_fused(x, L["gu"][0], L["gu"][1], cfg.group, prologue=1, r=o, wn=L["ln_post"],
                                             eps=cfg.rms_eps, x_out=x_alt, epilogue=EPI_SWIGLU_PAIRS8)
                x, x_alt = x_alt, x
                d = self.linear(act, L["d"])
            elif self.world == 1 and self.I % 128 == 0:
                # SwiGLU in the epilogue of gate|up, written in the converted form the down projection copies into
                # its shared memory (no conversion of 18944 activations in every CTA of the down projection)
                staged = self.k.w4_linear_fused(x, L["gu"][0], L["gu"][1], cfg.group, prologue=1, r=o, wn=L["ln_post"],
                                                eps=cfg.rms_eps, x_out=x_alt, epilogue=EPI_SWIGLU_STAGED)
                x, x_alt = x_alt, x
                d = self.k.w4_linear_fused(staged, L["d"][0], L["d"][1], cfg.group, prologue=PRO_STAGED,
                                           flags=self.down_flags)
            else:  # SwiGLU in the epilogue; the activation is gathered by NCCL
                act = self._gather(self.k.w4_linear_fused(x, L["gu"][0], L["gu"][1], cfg.group, prologue=1, r=o,
                                                          wn=L["ln_post"], eps=cfg.rms_eps, x_out=x_alt,
                                                          epilogue=EPI_SWIGLU_PAIRS))
                x, x_alt = x_alt, x
                d = self._gather(self.linear(act, L["d"]))
            r = d
            wn = self.layers[li + 1]["ln_in"] if li + 1 < cfg.n_layers else self.final_norm
        # final add + RMSNorm folded into the vocabulary projection, argmax partials in its epilogue.  The residual
        # stream is not needed after this: the next step starts from the embedding the pick writes into self.x.
        return self._lm_head_and_pick(x, r, wn)

    @torch.no_grad()
    def _decode_step_fused_gather(self):
        """The decode step on more than one GPU with the all-gathers inside the GEMVs: the same five launches per
        layer as on one GPU, no collective.  Every GEMV stores its rows into the gathered row of every rank and counts
        itself in; the kernel that consumes the row (the next GEMV, or the attention kernel) waits on the counter."""
        cfg, k, lib, peer = self.cfg, self.k, self.k.lib, self.peer
        D, G, eps = cfg.head_dim, cfg.group, cfg.rms_eps
        ep = peer.epoch.data_ptr()
        qkv_buf, o_buf = peer.local("qkv", 1), peer.local("o", 1)
        act_buf, d_buf = peer.local("act", 1), peer.local("d", 1)
        x, x_alt = self.x, self.x_alt
        for li, L in enumerate(self.layers):
            dsc = self.tp_desc[li]
            if li == 0:
                k.w4_linear_tp(x, L["qkv"][0], L["qkv"][1], dsc["qkv"], G, prologue=1, wn=L["ln_in"], eps=eps)
            else:
                k.w4_linear_tp(x, L["qkv"][0], L["qkv"][1], dsc["qkv"], G, prologue=1, r=d_buf, wn=L["ln_in"], eps=eps,
                               x_out=x_alt)
                x, x_alt = x_alt, x
            a = torch.empty(1, self.nq, dtype=torch.bfloat16, device=self.dev)
            rc = lib.b2_decode_attention_fused(qkv_buf.data_ptr(), L["bias"].data_ptr(), self.inv_freq.data_ptr(),
                                               self.pos.data_ptr(), self.cache_k[li].data_ptr(),
                                               self.cache_v[li].data_ptr(), a.data_ptr(), self.attn_ws.data_ptr(),
                                               cfg.n_heads, cfg.n_kv_heads, D, self.max_len,
                                               ctypes.byref(dsc["attn"]), self.attn_flags, self._st())
            k._check(rc, "b2_decode_attention_fused")
            k.w4_linear_tp(a, L["o"][0], L["o"][1], dsc["o"], G)
            k.w4_linear_tp(x, L["gu"][0], L["gu"][1], dsc["gu"], G, prologue=1, r=o_buf, wn=L["ln_post"], eps=eps,
                           x_out=x_alt, epilogue=EPI_SWIGLU_PAIRS)
            x, x_alt = x_alt, x
            k.w4_linear_tp(act_buf, L["d"][0], L["d"][1], dsc["d"], G)
        k.tp_wait_desc(self.tp_tail, advance_epoch=True)  # the last down projection; closes the step's epoch
        return self._lm_head_and_pick(x, d_buf, self.final_norm)

    def capture(self):
        """Warms up and captures one decode step.  The warm-up steps advance the device state; callers that
        need clean state re-run prefill afterwards."""
        with torch.cuda.stream(self.stream):
            for _ in range(2):
                self.decode_step()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=self.stream):
                self.decode_step()
        self.graph = g

    @torch.no_grad()
    def generate(self, prompt_ids: torch.Tensor, n_new: int, use_graph: bool = True) -> List[int]:
        """Greedy decoding.  Returns the generated ids (list), as the reference's generate does (qwen.py:166-178)."""
        assert prompt_ids.shape[0] + n_new <= self.max_len
        # Everything runs on the runner's own stream: split-K launches of one device share scratch memory and arrival
        # counters, so a prefill on the caller's stream must never overlap the warm-up steps of capture().
        with torch.cuda.stream(self.stream):
            if use_graph and self.graph is None:
                self.prefill(prompt_ids)
                torch.cuda.synchronize()
                self.capture()
            self.prefill(prompt_ids)
            for _ in range(n_new - 1):
                if use_graph:
                    self.graph.replay()
                else:
                    self.decode_step()
        torch.cuda.synchronize()
        self.check_status()
        return self.tokens[:n_new].tolist()

    def check_status(self):
        """Raises if a kernel gave up on a bounded wait (a ring slot, a tensor-parallel arrival counter): the tokens
        generated since the last check are then meaningless."""
        rc = self.k.device_status()
        if rc != 0:
            raise RuntimeError(f"device status {rc}: a kernel reported a time-out during decoding")


def decode_rate(kernels: Kernels, device, rank: int = 0, world: int = 1, cfg: Optional[Qwen2Config] = None,
                prompt_len: int = 512, n_new: int = 256, seed: int = 0, fused_gather: bool = True) -> dict:
    """Greedy decode of `n_new` tokens after a `prompt_len`-token prompt of uniform random ids, batch 1: the
    reference's decode-rate measurement ((G - 1) tokens over the time after the first one, python/bench_e2e.py:210-213)
    with CUDA events around the G - 1 graph replays.  Every rank must call it; returns the numbers of this rank."""
    cfg = cfg or Qwen2Config.qwen25_7b()
    r = Qwen2Runner(cfg, kernels, device, rank=rank, world=world, seed=seed, max_len=prompt_len + n_new + 8,
                    fused_gather=fused_gather)
    gen = torch.Generator(device=device).manual_seed(4)
    prompt = torch.randint(0, cfg.vocab, (prompt_len,), device=device, generator=gen)
    r.generate(prompt, 4)  # warms every kernel variant and captures the decode graph
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    with torch.cuda.stream(r.stream):
        e0.record(r.stream)
        r.prefill(prompt)
        e1.record(r.stream)
        for _ in range(n_new - 1):
            r.graph.replay()
        e2.record(r.stream)
    torch.cuda.synchronize()
    r.check_status()
    t_prefill, t_decode = e0.elapsed_time(e1) * 1e-3, e1.elapsed_time(e2) * 1e-3
    tokens = r.tokens[:n_new].tolist()
    import hashlib
    sha = hashlib.sha1(",".join(map(str, tokens)).encode()).hexdigest()[:16]
    # tensor parallel == single GPU: rank 0 builds the same model unsharded and compares the logits of the first
    # generated token (its own slice of the vocabulary) and the whole generated sequence
    tp_check = None
    if world > 1:
        with torch.cuda.stream(r.stream):
            r.prefill(prompt)
        torch.cuda.synchronize()
        mine = r.logits.float().clone()
        if rank == 0:
            r1 = Qwen2Runner(cfg, kernels, device, rank=0, world=1, seed=seed, max_len=prompt_len + n_new + 8)
            toks1 = r1.generate(prompt, n_new)
            with torch.cuda.stream(r1.stream):
                r1.prefill(prompt)
            torch.cuda.synchronize()
            want = r1.logits.float()[:, :mine.shape[1]]
            scale = want.abs().max()
            tp_check = {"logits_max_rel": float(((mine - want).abs() / scale).max()), "tokens_equal": toks1 == tokens,
                        "first_difference": next((i for i, (a, b) in enumerate(zip(toks1, tokens)) if a != b), None)}
            tp_check["ok"] = tp_check["logits_max_rel"] <= 2e-2 and tp_check["tokens_equal"]
            del r1
            torch.cuda.empty_cache()
        dist.barrier()
        # The benchmark's model has small norm gains (so that greedy decoding of random weights stays input-dependent),
        # which also means its logits say little about attention and the MLP.  A second, short comparison with unit
        # gains, where every sub-layer moves the logits: four layers, 64-token prompt, six decode steps.
        import copy
        c4 = copy.copy(cfg)
        c4.n_layers = min(4, cfg.n_layers)
        short = prompt[:64]
        rs = Qwen2Runner(c4, kernels, device, rank=rank, world=world, seed=seed + 1, max_len=96,
                         fused_gather=fused_gather, norm_gain=1.0)
        toks_s = rs.generate(short, 6)
        torch.cuda.synchronize()
        rs.check_status()
        mine_s = rs.logits.float().clone()
        if rank == 0:
            r1s = Qwen2Runner(c4, kernels, device, rank=0, world=1, seed=seed + 1, max_len=96, norm_gain=1.0)
            toks_1 = r1s.generate(short, 6)
            torch.cuda.synchronize()
            want_s = r1s.logits.float()[:, :mine_s.shape[1]]
            rel = float(((mine_s - want_s).abs() / want_s.abs().max()).max())
            tp_check["unit_gain"] = {"layers": c4.n_layers, "logits_max_rel": rel, "tokens_equal": toks_1 == toks_s}
            tp_check["ok"] = bool(tp_check["ok"] and rel <= 2e-2 and toks_1 == toks_s)
            del r1s
        del rs
        torch.cuda.empty_cache()
        dist.barrier()
    return {"tp_check": tp_check, "tokens_sha1": sha, "distinct_tokens": len(set(tokens)), "tok_s": (n_new - 1) / t_decode, "ms_per_token": t_decode / (n_new - 1) * 1e3,
            "prefill_tok_s": prompt_len / t_prefill, "prompt_len": prompt_len, "n_new": n_new,
            "weight_bytes_per_token_per_rank": r.weight_bytes_per_token(), "first_tokens": tokens[:8],
            "launches_per_token": "6 per layer + lm_head (final norm and block argmax folded in) + the pick, one CUDA graph; " +
                                  ("all-gathers fused into the GEMVs" if r.peer is not None else
                                   "NCCL all-gathers at the layer boundaries" if world > 1 else "one GPU")}


if __name__ == "__main__":
    import argparse
    import json

    ap = argparse.ArgumentParser(description="greedy-decode rate of a random-init Qwen2.5-7B-shaped W4 model, one GPU")
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--layers", type=int, default=28)
    a = ap.parse_args()
    c = Qwen2Config.qwen25_7b()
    c.n_layers = a.layers
    print(json.dumps(decode_rate(Kernels(), torch.device("cuda"), cfg=c, prompt_len=a.prompt, n_new=a.new)))
