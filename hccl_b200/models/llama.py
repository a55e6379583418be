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


def apply_rope(x, cos, sin):
    # x [S, H, D]; rotate pairs (first half, second half)
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d].float(), x[..., d:].float()
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1).to(x.dtype)


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
        # keys are shared between layers: the symmetric staging buffers are reused layer after layer
        self.qkv = ColumnParallelLinear(cfg.hidden, (cfg.n_heads + 2 * cfg.n_kv_heads) * cfg.head_dim, ctx, "qkv", cfg.init_std)
        self.o = RowParallelLinear(cfg.n_heads * cfg.head_dim, cfg.hidden, ctx, "o", cfg.init_std)
        self.gate_up = ColumnParallelLinear(cfg.hidden, 2 * cfg.ffn, ctx, "gate_up", cfg.init_std)
        self.down = RowParallelLinear(cfg.ffn, cfg.hidden, ctx, "down", cfg.init_std)

    def forward(self, x, cos, sin):
        cfg = self.cfg
        h = F.rms_norm(x, (cfg.hidden,), self.attn_norm, cfg.norm_eps)
        qkv = self.qkv(h)                                                     # [S, (hq + 2 hkv) * D]
        s = qkv.shape[0]
        q, k, v = qkv.split([self.hq * cfg.head_dim, self.hkv * cfg.head_dim, self.hkv * cfg.head_dim], dim=-1)
        q = apply_rope(q.view(s, self.hq, cfg.head_dim), cos, sin)
        k = apply_rope(k.view(s, self.hkv, cfg.head_dim), cos, sin)
        v = v.view(s, self.hkv, cfg.head_dim)
        attn = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None], is_causal=True,
                                              enable_gqa=self.hq != self.hkv)
        attn = attn[0].transpose(0, 1).reshape(s, self.hq * cfg.head_dim)
        x = x + self.o(attn)
        h = F.rms_norm(x, (cfg.hidden,), self.ffn_norm, cfg.norm_eps)
        gu = self.gate_up(h)
        g, u = gu.chunk(2, dim=-1)
        x = x + self.down(F.silu(g) * u)
        return x


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
        for layer in self.layers:
            x = layer(x, cos, sin)
        return F.rms_norm(x, (self.cfg.hidden,), self.final_norm, self.cfg.norm_eps)

    def loss(self, token_ids):
        """Scalar training signal: mean square of the final hidden states of this rank's sequence shard."""
        return self.forward(token_ids).float().pow(2).mean()
