"""Llama-3-shaped decoder stack with tensor + sequence parallelism.

The shape of the benchmark model: hidden 8192, 64 query heads, 8 KV heads, head
dim 128, SwiGLU FFN 28672, RMSNorm, RoPE theta 500000, vocab 128256.  Between
blocks the activations are sharded over the sequence; QKV and gate/up
projections are column-parallel (AllGather->Matmul), o_proj and down_proj are
row-parallel (Matmul->ReduceScatter).
"""
from __future__ import annotations

import dataclasses
import math

import torch
import torch.nn.functional as F

from ..ops import fused
from ..parallel.tp_layers import ColumnParallelLinear, RowParallelLinear, TPContext


@dataclasses.dataclass
class LlamaConfig:
    hidden: int = 8192
    n_heads: int = 64
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 28672
    n_layers: int = 8
    vocab: int = 128256
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5
    init_std: float = 0.02

    @staticmethod
    def llama3_70b_8layers():
        return LlamaConfig()

    @staticmethod
    def tiny(n_layers=2):
        return LlamaConfig(hidden=1024, n_heads=8, n_kv_heads=8, head_dim=128, ffn=2048, n_layers=n_layers, vocab=1024)


def rope_tables(seq, dim, theta, device):
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, device=device, dtype=torch.float32) / dim))
    t = torch.arange(seq, device=device, dtype=torch.float32)
    f = torch.outer(t, inv)
    return f.cos(), f.sin()


class DecoderLayer(torch.nn.Module):
    def __init__(self, cfg: LlamaConfig, ctx: TPContext, idx: int):
        super().__init__()
        self.cfg, self.ctx = cfg, ctx
        p = ctx.world
        assert cfg.n_heads % p == 0 and cfg.n_kv_heads % p == 0 and cfg.ffn % p == 0
        self.hq, self.hkv = cfg.n_heads // p, cfg.n_kv_heads // p
        dev = "cuda"
        self.attn_norm = torch.nn.Parameter(torch.ones(cfg.hidden, device=dev, dtype=torch.bfloat16))
        self.ffn_norm = torch.nn.Parameter(torch.ones(cfg.hidden, device=dev, dtype=torch.bfloat16))
        # Column-parallel layers keep their gathered input (a persistent symmetric buffer, saved for the backward pass),
        # so their keys are per layer; the row-parallel layers' symmetric buffers are transient and shared.
        self.qkv = ColumnParallelLinear(cfg.hidden, (cfg.n_heads + 2 * cfg.n_kv_heads) * cfg.head_dim, ctx, f"qkv{idx}", cfg.init_std)
        self.o = RowParallelLinear(cfg.n_heads * cfg.head_dim, cfg.hidden, ctx, "o", cfg.init_std)
        self.gate_up = ColumnParallelLinear(cfg.hidden, 2 * cfg.ffn, ctx, f"gate_up{idx}", cfg.init_std)
        self.down = RowParallelLinear(cfg.ffn, cfg.hidden, ctx, "down", cfg.init_std)

    def forward(self, x, delta, cos, sin):
        """x: residual stream [S/P, hidden]; delta: the previous block's output still to be added to it (or None).
        Returns the updated stream and this layer's pending addition, so that every residual add is fused into the
        RMSNorm that follows it."""
        cfg, k_ = self.cfg, self.ctx.fused_ops
        d = cfg.head_dim
        x, h = fused.add_rms_norm(x, delta, self.attn_norm, cfg.norm_eps, use_kernels=k_)
        qkv = self.qkv(h)                                                     # [S, (hq + 2 hkv) * D]
        s = qkv.shape[0]
        q = fused.rope(qkv[:, :self.hq * d].view(s, self.hq, d), cos, sin, use_kernels=k_)
        k = fused.rope(qkv[:, self.hq * d:(self.hq + self.hkv) * d].view(s, self.hkv, d), cos, sin, use_kernels=k_)
        v = qkv[:, (self.hq + self.hkv) * d:].view(s, self.hkv, d)
        attn = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None], is_causal=True,
                                              enable_gqa=self.hq != self.hkv)
        attn = attn[0].transpose(0, 1).reshape(s, self.hq * d)
        x, h = fused.add_rms_norm(x, self.o(attn), self.ffn_norm, cfg.norm_eps, use_kernels=k_)
        return x, self.down(fused.swiglu(self.gate_up(h), use_kernels=k_))


class LlamaStack(torch.nn.Module):
    """Embedding -> n decoder layers -> final norm; returns the sequence-sharded hidden states."""

    def __init__(self, cfg: LlamaConfig, ctx: TPContext):
        super().__init__()
        self.cfg, self.ctx = cfg, ctx
        self.embed = torch.nn.Parameter(torch.randn(cfg.vocab, cfg.hidden, device="cuda", dtype=torch.float32).mul_(cfg.init_std).to(torch.bfloat16))
        self.layers = torch.nn.ModuleList(DecoderLayer(cfg, ctx, i) for i in range(cfg.n_layers))
        self.final_norm = torch.nn.Parameter(torch.ones(cfg.hidden, device="cuda", dtype=torch.bfloat16))
        self._rope = None

    def forward(self, token_ids):
        # token_ids [S] (the full sequence on every rank); each rank embeds its own sequence shard
        s = token_ids.shape[0]
        p, r = self.ctx.world, self.ctx.rank
        assert s % p == 0
        shard = token_ids[r * (s // p):(r + 1) * (s // p)]
        x = F.embedding(shard, self.embed)
        if self._rope is None or self._rope[0].shape[0] != s:
            self._rope = rope_tables(s, self.cfg.head_dim, self.cfg.rope_theta, x.device)
        cos, sin = self._rope
        delta = None
        for layer in self.layers:
            x, delta = layer(x, delta, cos, sin)
        return fused.add_rms_norm(x, delta, self.final_norm, self.cfg.norm_eps, use_kernels=self.ctx.fused_ops)[1]

    def loss(self, token_ids):
        """Scalar training signal with non-trivial gradients: the mean product of neighbouring features of the final
        hidden states of this rank's sequence shard.  (The mean SQUARE of an RMS-normalised output is constant, so its
        gradients would be rounding noise.)"""
        h = self.forward(token_ids).float()
        return (h * h.roll(1, dims=-1)).mean()
