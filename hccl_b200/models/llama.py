"""Llama-3-shaped decoder stack with tensor + sequence parallelism.

The shape of the benchmark model: hidden 8192, 64 query heads, 8 KV heads, head
dim 128, SwiGLU FFN 28672, RMSNorm, RoPE theta 500000, vocab 128256.  Between
blocks the activations are sharded over the sequence; QKV and gate/up
projections are column-parallel (AllGather->Matmul), o_proj and down_proj are
row-parallel (Matmul->ReduceScatter).

Nothing large is replicated.  The embedding table is cut along the hidden
dimension: every rank looks all tokens up in its column slice and one AlltoAll
turns ``[S, hidden / P]`` into the rank's sequence shard ``[S / P, hidden]``
(1/P of the bytes a vocabulary-parallel reduce-scatter would move); the
backward pass runs the same exchange the other way and accumulates into a
``[vocab, hidden / P]`` gradient.  The RMSNorm weights are the only replicated
parameters; each rank sees the gradient of its own sequence shard only, so
``sync_replicated_grads`` sums them over the group before the optimizer step.
The loss of a rank is its shard's share of the mean over the WHOLE sequence:
the per-rank losses add up to the loss of the unsharded model and the
gradients match it.
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
        self.attn_norm = torch.nn.Parameter(torch.ones(cfg.hidden, device=ctx.device, dtype=ctx.dtype))
        self.ffn_norm = torch.nn.Parameter(torch.ones(cfg.hidden, device=ctx.device, dtype=ctx.dtype))
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


class _ShardedEmbedding(torch.autograd.Function):
    """Embedding whose table is cut along the hidden dimension, producing this rank's sequence shard."""

    @staticmethod
    def forward(fctx, token_ids, table, ctx: TPContext):
        # table [vocab, hidden / P]; token_ids [S] (the whole sequence on every rank)
        p = ctx.world
        s, hp = token_ids.shape[0], table.shape[1]
        cols = F.embedding(token_ids, table)                               # [S, hidden / P]: rows grouped by destination rank
        got = ctx.all_to_all(cols.view(p, s // p, hp), "embed_fwd")         # block q: rank q's columns of my tokens
        fctx.save_for_backward(token_ids)
        fctx.ctx, fctx.vocab = ctx, table.shape[0]
        return got.permute(1, 0, 2).reshape(s // p, p * hp)

    @staticmethod
    def backward(fctx, dx):
        (token_ids,) = fctx.saved_tensors
        ctx, p = fctx.ctx, fctx.ctx.world
        sp, hidden = dx.shape
        send = dx.view(sp, p, hidden // p).permute(1, 0, 2).contiguous()   # block q: my tokens' gradient of rank q's columns
        got = ctx.all_to_all(send, "embed_bwd").view(sp * p, hidden // p)  # every token's gradient of my columns
        dtable = torch.ops.aten.embedding_dense_backward(got, token_ids, fctx.vocab, -1, False)
        return None, dtable, None


class LlamaStack(torch.nn.Module):
    """Embedding -> n decoder layers -> final norm; returns the sequence-sharded hidden states."""

    def __init__(self, cfg: LlamaConfig, ctx: TPContext):
        super().__init__()
        self.cfg, self.ctx = cfg, ctx
        assert cfg.hidden % ctx.world == 0
        self.embed = torch.nn.Parameter(torch.randn(cfg.vocab, cfg.hidden // ctx.world, device=ctx.device, dtype=torch.float32)
                                        .mul_(cfg.init_std).to(ctx.dtype))
        self.layers = torch.nn.ModuleList(DecoderLayer(cfg, ctx, i) for i in range(cfg.n_layers))
        self.final_norm = torch.nn.Parameter(torch.ones(cfg.hidden, device=ctx.device, dtype=ctx.dtype))
        self._rope = None

    def replicated_parameters(self):
        """Parameters every rank holds a full copy of (the RMSNorm weights)."""
        out = []
        for layer in self.layers:
            out += [layer.attn_norm, layer.ffn_norm]
        return out + [self.final_norm]

    def sync_replicated_grads(self):
        """Sums the gradients of the replicated parameters over the group: one flat all-reduce.  Call between
        ``backward`` and the optimizer step; without it the copies drift apart."""
        if self.ctx.world == 1:
            return
        params = [p for p in self.replicated_parameters() if p.grad is not None]
        if not params:
            return
        grads = [p.grad for p in params]
        flat = self.ctx.flat_buffer("replicated_grads", sum(g.numel() for g in grads), grads[0].dtype)
        torch.cat([g.reshape(-1) for g in grads], out=flat)
        self.ctx.all_reduce_(flat, "replicated_grads")
        torch._foreach_copy_(grads, [c.view_as(g) for c, g in zip(flat.split([g.numel() for g in grads]), grads)])

    @torch.no_grad()
    def load_full(self, full: "LlamaStack"):
        """Takes this rank's slices of an unsharded model's parameters (tests compare the two)."""
        p, r = self.ctx.world, self.ctx.rank
        cfg = self.cfg
        d = cfg.head_dim

        def rows(w, n_per):     # [n_per * p rows] -> this rank's n_per rows
            return w[r * n_per:(r + 1) * n_per]

        self.embed.copy_(full.embed[:, r * (cfg.hidden // p):(r + 1) * (cfg.hidden // p)])
        self.final_norm.copy_(full.final_norm)
        for mine, ref in zip(self.layers, full.layers):
            mine.attn_norm.copy_(ref.attn_norm)
            mine.ffn_norm.copy_(ref.ffn_norm)
            hq, hkv = cfg.n_heads // p, cfg.n_kv_heads // p
            wq, wk, wv = ref.qkv.weight.split([cfg.n_heads * d, cfg.n_kv_heads * d, cfg.n_kv_heads * d])
            mine.qkv.weight.copy_(torch.cat([rows(wq, hq * d), rows(wk, hkv * d), rows(wv, hkv * d)]))
            wg, wu = ref.gate_up.weight.chunk(2)
            mine.gate_up.weight.copy_(torch.cat([rows(wg, cfg.ffn // p), rows(wu, cfg.ffn // p)]))
            mine.o.weight.copy_(ref.o.weight[:, r * hq * d:(r + 1) * hq * d])
            mine.down.weight.copy_(ref.down.weight[:, r * (cfg.ffn // p):(r + 1) * (cfg.ffn // p)])

    def forward(self, token_ids):
        # token_ids [S] (the full sequence on every rank)
        s = token_ids.shape[0]
        p = self.ctx.world
        assert s % p == 0
        x = F.embedding(token_ids, self.embed) if p == 1 else _ShardedEmbedding.apply(token_ids, self.embed, self.ctx)
        if self._rope is None or self._rope[0].shape[0] != s:
            self._rope = rope_tables(s, self.cfg.head_dim, self.cfg.rope_theta, x.device)
        cos, sin = self._rope
        delta = None
        for layer in self.layers:
            x, delta = layer(x, delta, cos, sin)
        return fused.add_rms_norm(x, delta, self.final_norm, self.cfg.norm_eps, use_kernels=self.ctx.fused_ops)[1]

    def loss(self, token_ids):
        """Scalar training signal with non-trivial gradients: the mean, over the WHOLE sequence, of the product of
        neighbouring features of the final hidden states; a rank returns its sequence shard's share of it, so the
        ranks' losses add up to the unsharded model's.  (The mean SQUARE of an RMS-normalised output is constant, so
        its gradients would be rounding noise.)"""
        h = self.forward(token_ids).float()
        return (h * h.roll(1, dims=-1)).sum() / (token_ids.shape[0] * h.shape[-1])
