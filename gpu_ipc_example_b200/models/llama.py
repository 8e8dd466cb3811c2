"""Llama-3-shaped decoder, tensor-parallel, for inference (decode) benchmarks of the fused collectives.

One `LlamaTP` object drives all ranks its communicator drives: one rank in a multi-process job, every
rank of an emulated world on one GPU - so every tensor below is a list with one entry per local rank.

Per layer there are exactly two all-reduces (after the attention output projection and after the MLP
down projection); each is fused with the residual add and the RMSNorm that follows it, in one of
three ways (`fusion=`):

  "gemm"       the row-parallel projection itself is part of the kernel: tcgen05/TMA GEMM whose
               epilogue reduce-scatters into the peers, owner reduce + residual + RMSNorm, all-gather
               (`Communicator.linear_allreduce`)
  "allreduce"  cuBLAS projection, then one one-shot all-reduce + residual + RMSNorm kernel
               (`Communicator.allreduce_residual_rmsnorm`)
  "nccl"       the baseline: cuBLAS projection, `torch.distributed.all_reduce`, separate add and norm

What lies between the GEMMs and the collectives runs in three hand-written kernels when the head
dimension is 128 (`kernels=True`, the default there): rotary embedding fused with the KV-cache append,
attention of the new token over the cache (grouped-query, split over the context), SiLU(gate) * up.
With `kernels=False` the same steps are plain PyTorch ops (the reference path of the tests).

The reference has no model code; its smoke script all-reduces decode-sized fp16 activations the way a
tensor-parallel decoder does (script/gpu_inference_test.py:29-45).  Weights are random N(0, 0.02).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn.functional as F


@dataclass
class LlamaConfig:
    layers: int = 80
    hidden: int = 8192
    n_heads: int = 64
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 28672
    vocab: int = 128256
    eps: float = 1e-5
    rope_theta: float = 5e5
    dtype: torch.dtype = torch.float16

    @classmethod
    def llama3_70b(cls) -> "LlamaConfig":
        return cls()

    @classmethod
    def tiny(cls) -> "LlamaConfig":
        return cls(layers=2, hidden=512, n_heads=8, n_kv_heads=8, head_dim=64, ffn=1024, vocab=2048)

    @classmethod
    def tiny128(cls) -> "LlamaConfig":
        """Small, but with the 70B model's head dimension and grouped-query ratio (the hand-written decode kernels)."""
        return cls(layers=2, hidden=1024, n_heads=16, n_kv_heads=8, head_dim=128, ffn=2048, vocab=2048)


def rms_norm(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    v = x.float()
    return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * gamma


def apply_rope(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """x: [B, heads, D]; pos: [B] absolute positions.  Rotates pairs (i, i + D/2)."""
    B, H, D = x.shape
    half = D // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, device=x.device, dtype=torch.float32) / half))
    ang = pos.float()[:, None] * inv[None, :]  # [B, half]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x[..., :half].float(), x[..., half:].float()
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


class LlamaTP:
    def __init__(self, cfg: LlamaConfig, comm, batch: int, max_ctx: int, fusion: str = "allreduce", seed: int = 0,
                 device: Optional[torch.device] = None, kernels: Optional[bool] = None, pack_weights: bool = False,
                 local_gemm=None):
        assert fusion in ("gemm", "allreduce", "nccl")
        self.cfg, self.comm, self.fusion = cfg, comm, fusion
        # QKV and gate/up projections on the library's weight-streaming kernel instead of the framework's matmul
        # (off by default: measured level with cuBLAS at these shapes, a little behind it once the step is a graph)
        # True / False, or "qkv" / "gate_up" for one of the two projections only
        self.local_gemm = local_gemm if comm is not None else False
        # the decode kernels are written for head_dim 128 and 1/2/4/8 query heads per KV head
        can = cfg.head_dim == 128 and (cfg.n_heads // cfg.n_kv_heads) in (1, 2, 4, 8) and cfg.ffn % 8 == 0
        self.kernels = can if kernels is None else (kernels and can)
        self.world = comm.world if comm is not None else 1
        self.nlocal = comm.nlocal if comm is not None else 1
        self.ranks = [comm._C.rank(comm._h, i) for i in range(self.nlocal)] if comm is not None else [0]
        W = self.world
        assert cfg.n_heads % W == 0 and cfg.n_kv_heads % W == 0 and cfg.ffn % W == 0, "heads and FFN must divide by the world size"
        self.hq, self.hkv, self.ffn_local = cfg.n_heads // W, cfg.n_kv_heads // W, cfg.ffn // W
        self.batch, self.max_ctx = batch, max_ctx
        dev = device or torch.device("cuda", torch.cuda.current_device())
        self.dev = dev
        dt, D, H = cfg.dtype, cfg.head_dim, cfg.hidden

        def rnd(gen, *shape):
            return (torch.randn(*shape, device=dev, generator=gen) * 0.02).to(dt)

        # replicated tensors come from one generator, sharded ones from a per-rank generator
        g_rep = torch.Generator(device=dev).manual_seed(seed)
        self.embed = rnd(g_rep, cfg.vocab, H)
        self.norm_attn = [torch.ones(H, device=dev, dtype=dt) for _ in range(cfg.layers)]
        self.norm_mlp = [torch.ones(H, device=dev, dtype=dt) for _ in range(cfg.layers)]
        self.norm_final = torch.ones(H, device=dev, dtype=dt)
        self.wqkv, self.wo, self.wgu, self.wdown, self.lm_head, self.kcache, self.vcache = [], [], [], [], [], [], []
        for r in self.ranks:
            g = torch.Generator(device=dev).manual_seed(seed * 1000 + 17 + r)
            self.wqkv.append([rnd(g, (self.hq + 2 * self.hkv) * D, H) for _ in range(cfg.layers)])
            self.wo.append([rnd(g, H, self.hq * D) for _ in range(cfg.layers)])           # row-parallel: [N, K_local]
            self.wgu.append([rnd(g, 2 * self.ffn_local, H) for _ in range(cfg.layers)])
            self.wdown.append([rnd(g, H, self.ffn_local) for _ in range(cfg.layers)])     # row-parallel
            self.lm_head.append(rnd(g, cfg.vocab // W, H))
            self.kcache.append([torch.zeros(batch, self.hkv, max_ctx, D, device=dev, dtype=dt) for _ in range(cfg.layers)])
            self.vcache.append([torch.zeros(batch, self.hkv, max_ctx, D, device=dev, dtype=dt) for _ in range(cfg.layers)])
        self.pos = 0
        self.stage_events = None  # a list: decode() then appends (stage name, start event, end event)
        if self.kernels:
            from .._ext import load

            C = load()
            dev_index = dev.index if dev.index is not None else torch.cuda.current_device()
            self.attn_splits = C.attention_splits(batch, self.hkv, max_ctx, dev_index)
            nbytes = C.attention_workspace_bytes(batch, self.hq, self.hkv, self.attn_splits)
            self.attn_ws = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(self.nlocal)]
        if pack_weights and fusion == "gemm":
            # row-parallel weights in the layout the fused GEMM streams fastest (done once, at load time)
            from ..parallel.communicator import Communicator

            self.wo_run = [[Communicator.pack_weight(w) for w in ws] for ws in self.wo]
            self.wdown_run = [[Communicator.pack_weight(w) for w in ws] for ws in self.wdown]
        else:
            self.wo_run, self.wdown_run = self.wo, self.wdown

    # ------------------------------------------------------------------ collectives
    def _reduce_norm(self, residual: List[torch.Tensor], gamma: torch.Tensor, x: List[torch.Tensor], w: List[torch.Tensor]):
        """Returns (normed, new_residual) for partial = x @ w.T summed over ranks."""
        eps = self.cfg.eps
        gam = [gamma] * self.nlocal
        if self.world == 1 and self.fusion != "gemm":
            s = [x[0] @ w[0].t() + residual[0]]
            return [rms_norm(s[0], gamma, eps)], s
        if self.fusion == "gemm":
            out, res = self.comm.linear_allreduce(x if self.nlocal > 1 else x[0], w if self.nlocal > 1 else w[0],
                                                  residual if self.nlocal > 1 else residual[0], gam if self.nlocal > 1 else gamma, eps)
            # the library alternates between two sets of output buffers per shape, so `res` stays valid as the
            # residual of the next call and `out` until the call after that: no copies
            return (out, res) if isinstance(out, list) else ([out], [res])
        assert w[0].dim() == 2, "packed weights are for fusion='gemm'"
        parts = [xi @ wi.t() for xi, wi in zip(x, w)]
        if self.fusion == "allreduce":
            out, res = self.comm.allreduce_residual_rmsnorm(parts if self.nlocal > 1 else parts[0],
                                                            residual if self.nlocal > 1 else residual[0],
                                                            gam if self.nlocal > 1 else gamma, eps)
            return (out, res) if isinstance(out, list) else ([out], [res])
        import torch.distributed as dist

        assert self.nlocal == 1, "the NCCL baseline needs one process per rank"
        dist.all_reduce(parts[0])
        s = parts[0].add_(residual[0])
        return [F.rms_norm(s, (s.shape[-1],), gamma, eps)], [s]  # the framework's one-kernel norm: a fair baseline

    def _stage(self, name):
        """Context manager that brackets a stage of the step with CUDA events when `stage_events` is a list."""
        import contextlib

        if self.stage_events is None:
            return contextlib.nullcontext()

        @contextlib.contextmanager
        def cm():
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            yield
            b.record()
            self.stage_events.append((name, a, b))

        return cm()

    def _linear(self, xs, ws, which="qkv"):
        """Column-parallel projection of every local rank: the library's weight-streaming kernel when `local_gemm`
        is on and the shape fits it, else the framework's matmul."""
        if self.local_gemm in (True, which) and xs[0].shape[0] <= 32 and ws[0].shape[0] % 128 == 0:
            if self.nlocal == 1 and not self.comm._virtual:
                return [self.comm.linear(xs[0], ws[0])]
            return self.comm.linear(list(xs), list(ws))
        return [x @ w.t() for x, w in zip(xs, ws)]

    # ------------------------------------------------------------------ one decode step
    @torch.no_grad()
    def decode(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens: [batch] int64 ids of the newest position.  Returns the next ids [batch] (greedy)."""
        cfg = self.cfg
        B, D = tokens.shape[0], cfg.head_dim
        pos = self.pos
        posv = torch.full((B,), pos, device=self.dev, dtype=torch.int64)
        h = [self.embed[tokens] for _ in range(self.nlocal)]                       # residual stream, replicated
        normed = [rms_norm(h[i], self.norm_attn[0], cfg.eps) for i in range(self.nlocal)]
        for l in range(cfg.layers):
            attn_out = []
            with self._stage("qkv_gemm"):
                qkv_all = self._linear(normed, [self.wqkv[i][l] for i in range(self.nlocal)])
            for i in range(self.nlocal):
                qkv = qkv_all[i]
                if self.kernels:
                    with self._stage("rope_append"):
                        torch.ops.b200ipc.rope_kv_append(qkv, self.kcache[i][l], self.vcache[i][l], self.hq, self.hkv, pos, cfg.rope_theta)
                    with self._stage("attention"):
                        attn_out.append(torch.ops.b200ipc.decode_attention(qkv, self.kcache[i][l], self.vcache[i][l], self.attn_ws[i],
                                                                           self.hq, self.hkv, pos + 1, self.attn_splits))
                    continue
                q, k, v = qkv.split([self.hq * D, self.hkv * D, self.hkv * D], dim=-1)
                q = apply_rope(q.view(B, self.hq, D), posv, cfg.rope_theta)
                k = apply_rope(k.view(B, self.hkv, D), posv, cfg.rope_theta)
                self.kcache[i][l][:, :, pos] = k
                self.vcache[i][l][:, :, pos] = v.view(B, self.hkv, D)
                kk = self.kcache[i][l][:, :, :pos + 1]
                vv = self.vcache[i][l][:, :, :pos + 1]
                o = F.scaled_dot_product_attention(q.unsqueeze(2), kk, vv, enable_gqa=self.hq != self.hkv)  # [B, hq, 1, D]
                attn_out.append(o.reshape(B, self.hq * D))
            with self._stage("o_proj_allreduce_norm"):
                normed, h = self._reduce_norm(h, self.norm_mlp[l], attn_out, [self.wo_run[i][l] for i in range(self.nlocal)])
            act = []
            with self._stage("gate_up_gemm"):
                gu_all = self._linear(normed, [self.wgu[i][l] for i in range(self.nlocal)], "gate_up")
            for i in range(self.nlocal):
                gu = gu_all[i]
                if self.kernels:
                    with self._stage("silu_mul"):
                        act.append(torch.ops.b200ipc.silu_mul(gu))
                    continue
                gate, up = gu.split(self.ffn_local, dim=-1)
                act.append(F.silu(gate) * up)
            gamma_next = self.norm_attn[l + 1] if l + 1 < cfg.layers else self.norm_final
            with self._stage("down_proj_allreduce_norm"):
                normed, h = self._reduce_norm(h, gamma_next, act, [self.wdown_run[i][l] for i in range(self.nlocal)])
        self.last_hidden = normed  # final-norm output of every local rank (replicated values)
        # vocabulary-parallel head: local arg-max, then the global one over ranks
        best_val, best_idx = [], []
        for i in range(self.nlocal):
            logits = (normed[i] @ self.lm_head[i].t()).float()
            v, ix = logits.max(dim=-1)
            best_val.append(v)
            best_idx.append(ix + self.ranks[i] * (cfg.vocab // self.world))
        self.pos += 1
        if self.world == 1:
            return best_idx[0]
        if self.nlocal > 1:
            vals = torch.stack(best_val)                       # [world, B]
            idxs = torch.stack(best_idx)
            return idxs.gather(0, vals.argmax(0, keepdim=True))[0]
        import torch.distributed as dist

        vals = [torch.empty_like(best_val[0]) for _ in range(self.world)]
        idxs = [torch.empty_like(best_idx[0]) for _ in range(self.world)]
        dist.all_gather(vals, best_val[0])
        dist.all_gather(idxs, best_idx[0])
        return torch.stack(idxs).gather(0, torch.stack(vals).argmax(0, keepdim=True))[0]

    def weight_bytes_per_rank(self) -> int:
        cfg, D = self.cfg, self.cfg.head_dim
        per_layer = ((self.hq + 2 * self.hkv) * D * cfg.hidden + cfg.hidden * self.hq * D + 2 * self.ffn_local * cfg.hidden +
                     cfg.hidden * self.ffn_local)
        return 2 * (cfg.layers * per_layer + cfg.vocab // self.world * cfg.hidden)


def full_weights_from_shards(m: LlamaTP):
    """Assembles the unsharded weights of an emulated-world model (all ranks local) for a single-device
    reference computation."""
    assert m.nlocal == m.world
    cfg, D = m.cfg, m.cfg.head_dim
    out = []
    for l in range(cfg.layers):
        wq = torch.cat([m.wqkv[i][l][:m.hq * D] for i in range(m.world)])
        wk = torch.cat([m.wqkv[i][l][m.hq * D:(m.hq + m.hkv) * D] for i in range(m.world)])
        wv = torch.cat([m.wqkv[i][l][(m.hq + m.hkv) * D:] for i in range(m.world)])
        wo = torch.cat([m.wo[i][l] for i in range(m.world)], dim=1)
        wg = torch.cat([m.wgu[i][l][:m.ffn_local] for i in range(m.world)])
        wu = torch.cat([m.wgu[i][l][m.ffn_local:] for i in range(m.world)])
        wd = torch.cat([m.wdown[i][l] for i in range(m.world)], dim=1)
        out.append((wq, wk, wv, wo, wg, wu, wd))
    head = torch.cat([m.lm_head[i] for i in range(m.world)])
    return out, head


@torch.no_grad()
def dense_decode_reference(m: LlamaTP, token_steps: List[torch.Tensor]) -> List[torch.Tensor]:
    """fp32 single-device re-computation of the same decode steps from the assembled weights; returns the
    hidden state before the LM head for every step (for numerical comparison)."""
    cfg, D = m.cfg, m.cfg.head_dim
    layers, _ = full_weights_from_shards(m)
    B = token_steps[0].shape[0]
    kc = [torch.zeros(B, cfg.n_kv_heads, len(token_steps), D, device=m.dev) for _ in range(cfg.layers)]
    vc = [torch.zeros(B, cfg.n_kv_heads, len(token_steps), D, device=m.dev) for _ in range(cfg.layers)]
    outs = []
    for pos, tokens in enumerate(token_steps):
        posv = torch.full((B,), pos, device=m.dev, dtype=torch.int64)
        h = m.embed[tokens].float()
        for l, (wq, wk, wv, wo, wg, wu, wd) in enumerate(layers):
            x = rms_norm(h, m.norm_attn[l].float(), cfg.eps)
            q = apply_rope((x @ wq.float().t()).view(B, cfg.n_heads, D), posv, cfg.rope_theta)
            k = apply_rope((x @ wk.float().t()).view(B, cfg.n_kv_heads, D), posv, cfg.rope_theta)
            v = (x @ wv.float().t()).view(B, cfg.n_kv_heads, D)
            kc[l][:, :, pos], vc[l][:, :, pos] = k, v
            o = F.scaled_dot_product_attention(q.unsqueeze(2), kc[l][:, :, :pos + 1], vc[l][:, :, :pos + 1],
                                               enable_gqa=cfg.n_heads != cfg.n_kv_heads)
            h = h + o.reshape(B, -1) @ wo.float().t()
            x = rms_norm(h, m.norm_mlp[l].float(), cfg.eps)
            h = h + (F.silu(x @ wg.float().t()) * (x @ wu.float().t())) @ wd.float().t()
        outs.append(rms_norm(h, m.norm_final.float(), cfg.eps))
    return outs
