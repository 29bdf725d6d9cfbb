"""Llama-2/3 decoder: architecture description, size presets and the eager module.

``Transformer`` here is the *framework-level* statement of the model: plain autograd modules
whose hot ops route through :mod:`prime_b200.ops.functional` (hand-written sm_100a kernels on
CUDA tensors, fp32 torch math on CPU tensors). It defines parameter names, shapes and
initialisation, runs the CPU/gloo DiLoCo slice, and is the oracle for the fused training engine
(:mod:`prime_b200.engine`), which executes the same network as an explicit kernel schedule.

Parity with the reference (paths inside the reference project):
  ModelArgs / presets   src/zeroband/models/llama/model.py:45-66, llama/__init__.py:15-82
  hidden-size rule      src/zeroband/models/llama/model.py:322-338
  init                  src/zeroband/models/llama/model.py:234-237, 343-346, 386-389, 463-494
  parameter FQNs        tok_embeddings, layers.{i}.attention.{wq,wk,wv,wo}, layers.{i}.feed_forward.{w1,w2,w3},
                        layers.{i}.{attention_norm,ffn_norm}, norm, output (+ complex buffer freqs_cis)
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace

import torch
import torch.nn as nn

from ..ops import functional as F_


@dataclass
class ModelArgs:
    dim: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int | None = None
    vocab_size: int = -1
    multiple_of: int = 256
    ffn_dim_multiplier: float | None = None
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_batch_size: int = 32
    max_seq_len: int = 2048
    depth_init: bool = True
    norm_type: str = "fused_rmsnorm"
    fused_linear_ce: bool = False
    attn_fn: str = "flex"
    # explicit SwiGLU width; overrides the multiple_of / ffn_dim_multiplier rule when set
    ffn_hidden: int | None = None
    # "reference": depth-scaled truncated normal; "normal": plain N(0, init_std) everywhere
    init_mode: str = "reference"
    init_std: float = 0.02

    @property
    def kv_heads(self) -> int:
        return self.n_kv_heads if self.n_kv_heads is not None else self.n_heads

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads

    @property
    def hidden_dim(self) -> int:
        if self.ffn_hidden is not None:
            return self.ffn_hidden
        h = int(2 * (4 * self.dim) / 3)
        if self.ffn_dim_multiplier is not None:
            h = int(self.ffn_dim_multiplier * h)
        return self.multiple_of * ((h + self.multiple_of - 1) // self.multiple_of)

    def num_params(self, exclude_embedding: bool = False) -> int:
        d, f, hd = self.dim, self.hidden_dim, self.head_dim
        per_layer = d * (self.n_heads * hd) * 2 + d * (self.kv_heads * hd) * 2 + 3 * d * f + 2 * d
        n = self.n_layers * per_layer + d + self.vocab_size * d
        if not exclude_embedding:
            n += self.vocab_size * d
        return n


llama2_configs: dict[str, ModelArgs] = {
    "debugmodel": ModelArgs(dim=256, n_layers=2, n_heads=8),
    "70M": ModelArgs(dim=512, n_layers=6, n_heads=8),
    "150M": ModelArgs(dim=1024, n_layers=12, n_heads=16),
    "271M": ModelArgs(dim=1024, n_layers=16, n_heads=8),
    "1B": ModelArgs(dim=2048, n_layers=18, n_heads=16),
    "7B": ModelArgs(dim=4096, n_layers=32, n_heads=32),
    "10B": ModelArgs(dim=5120, n_layers=32, n_heads=40),
    "13B": ModelArgs(dim=5120, n_layers=40, n_heads=40),
    "26B": ModelArgs(dim=5120, n_layers=80, n_heads=40),
    "70B": ModelArgs(dim=8192, n_layers=80, n_heads=64, n_kv_heads=8, ffn_dim_multiplier=1.3, multiple_of=4096),
}

llama3_configs: dict[str, ModelArgs] = {
    "debugmodel": ModelArgs(dim=256, n_layers=8, n_heads=16, rope_theta=500000),
    "1B": ModelArgs(dim=2048, n_layers=18, n_heads=16, n_kv_heads=8, ffn_dim_multiplier=1.3, multiple_of=512,
                    rope_theta=500000),
    "8B": ModelArgs(dim=4096, n_layers=32, n_heads=32, n_kv_heads=8, ffn_dim_multiplier=1.3, multiple_of=1024,
                    rope_theta=500000),
    "10B": ModelArgs(dim=4096, n_layers=42, n_heads=32, n_kv_heads=8, ffn_dim_multiplier=1.3, multiple_of=1024,
                     rope_theta=500000),
    "70B": ModelArgs(dim=8192, n_layers=80, n_heads=64, n_kv_heads=8, ffn_dim_multiplier=1.3, multiple_of=4096,
                     rope_theta=500000),
    "405B": ModelArgs(dim=16384, n_layers=126, n_heads=128, n_kv_heads=8, ffn_dim_multiplier=1.2, multiple_of=4096,
                      rope_theta=500000),
}

# Shapes named by the benchmark configurations that are not reference presets.
bench_configs: dict[str, ModelArgs] = {
    "tiny": ModelArgs(dim=256, n_layers=2, n_heads=4, ffn_hidden=704, vocab_size=1024, max_seq_len=128,
                      init_mode="normal"),
    "150M": ModelArgs(dim=1024, n_layers=12, n_heads=16, ffn_hidden=4096, vocab_size=32000, max_seq_len=1024,
                      init_mode="normal"),
    "1B": ModelArgs(dim=2048, n_layers=18, n_heads=16, ffn_hidden=8192, vocab_size=32000, max_seq_len=2048,
                    init_mode="normal"),
    "10B": replace(llama3_configs["10B"], vocab_size=128256, max_seq_len=8192, init_mode="normal"),
}


def get_model_args(type_model: str, name_model: str, vocab_size: int, seq_length: int, attn_fn: str = "flex",
                   fused_linear_ce: bool = False) -> ModelArgs:
    table = {"llama2": llama2_configs, "llama3": llama3_configs}.get(type_model)
    if table is None:
        raise ValueError(f"Model type {type_model} not supported")
    if name_model not in table:
        raise ValueError(f"Model {name_model} is not a {type_model} preset (have {sorted(table)})")
    return replace(table[name_model], vocab_size=vocab_size, max_seq_len=seq_length, attn_fn=attn_fn,
                   fused_linear_ce=fused_linear_ce)


def get_model(config, vocab_size: int) -> tuple["Transformer", ModelArgs]:
    """Build the model named by a :class:`prime_b200.config.Config` (reference: llama/__init__.py:85-103)."""
    args = get_model_args(config.type_model, config.name_model, vocab_size, config.data.seq_length,
                          config.train.attn_fn, config.train.fused_linear_ce)
    return Transformer(args), args


def precompute_freqs_cis(dim: int, end: int, theta: float = 10000.0) -> torch.Tensor:
    """complex64 [end, dim/2] rotation table (the reference's persistent ``freqs_cis`` buffer)."""
    freqs = 1.0 / (theta ** (torch.arange(0, dim, 2)[: dim // 2].float() / dim))
    t = torch.arange(end, device=freqs.device)
    return torch.polar(torch.ones(end, dim // 2), torch.outer(t, freqs).float())


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        return F_.rmsnorm(x, self.weight, self.eps)

    def reset_parameters(self):
        nn.init.ones_(self.weight)


def build_norm(norm_type: str, dim: int, eps: float = 1e-5) -> nn.Module:
    """Norm factory (reference: models/norms.py:24-51). ``rmsnorm`` and ``fused_rmsnorm`` are the
    same module here: one implementation, kernel on CUDA, fp32 torch math on CPU."""
    norm_type = norm_type.lower()
    if norm_type == "layernorm":
        return nn.LayerNorm(dim, eps=eps, bias=False)
    if norm_type == "np_layernorm":
        return nn.LayerNorm(dim, eps=eps, elementwise_affine=False, bias=False)
    if norm_type in ("rmsnorm", "fused_rmsnorm"):
        return RMSNorm(dim, eps)
    raise NotImplementedError(f"Unknown norm_type: '{norm_type}'")


class Attention(nn.Module):
    def __init__(self, args: ModelArgs):
        super().__init__()
        self.n_heads, self.n_kv_heads, self.head_dim = args.n_heads, args.kv_heads, args.head_dim
        self.wq = nn.Linear(args.dim, args.n_heads * self.head_dim, bias=False)
        self.wk = nn.Linear(args.dim, self.n_kv_heads * self.head_dim, bias=False)
        self.wv = nn.Linear(args.dim, self.n_kv_heads * self.head_dim, bias=False)
        self.wo = nn.Linear(args.n_heads * self.head_dim, args.dim, bias=False)

    def init_weights(self, init_std: float):
        for lin in (self.wq, self.wk, self.wv):
            nn.init.trunc_normal_(lin.weight, mean=0.0, std=0.02)
        nn.init.trunc_normal_(self.wo.weight, mean=0.0, std=init_std)

    def forward(self, x2d, rope_table, seq_len, seq_start):
        qkv = torch.cat([F_.linear(x2d, self.wq.weight), F_.linear(x2d, self.wk.weight), F_.linear(x2d, self.wv.weight)], -1)
        qkv = F_.rope(qkv, rope_table, seq_len, self.n_heads + self.n_kv_heads, self.head_dim)
        o = F_.attention(qkv, seq_start, self.n_heads, self.n_kv_heads, self.head_dim)
        return F_.linear(o, self.wo.weight)


class FeedForward(nn.Module):
    def __init__(self, dim: int, hidden_dim: int):
        super().__init__()
        self.w1 = nn.Linear(dim, hidden_dim, bias=False)
        self.w2 = nn.Linear(hidden_dim, dim, bias=False)
        self.w3 = nn.Linear(dim, hidden_dim, bias=False)

    def forward(self, x):
        return F_.linear(F_.swiglu(torch.cat([F_.linear(x, self.w1.weight), F_.linear(x, self.w3.weight)], -1)), self.w2.weight)

    def init_weights(self, init_std: float):
        nn.init.trunc_normal_(self.w1.weight, mean=0.0, std=0.02)
        for lin in (self.w2, self.w3):
            nn.init.trunc_normal_(lin.weight, mean=0.0, std=init_std)


class TransformerBlock(nn.Module):
    def __init__(self, layer_id: int, args: ModelArgs):
        super().__init__()
        self.attention = Attention(args)
        self.feed_forward = FeedForward(args.dim, args.hidden_dim)
        self.layer_id = layer_id
        self.attention_norm = build_norm(args.norm_type, args.dim, args.norm_eps)
        self.ffn_norm = build_norm(args.norm_type, args.dim, args.norm_eps)
        self.weight_init_std = 0.02 / (2 * (layer_id + 1)) ** 0.5 if args.depth_init else 0.02 / (2 * args.n_layers) ** 0.5

    def forward(self, x2d, rope_table, seq_len, seq_start):
        h = x2d + self.attention(self.attention_norm(x2d), rope_table, seq_len, seq_start)
        return h + self.feed_forward(self.ffn_norm(h))

    def init_weights(self):
        for norm in (self.attention_norm, self.ffn_norm):
            norm.reset_parameters()
        self.attention.init_weights(self.weight_init_std)
        self.feed_forward.init_weights(self.weight_init_std)


class Transformer(nn.Module):
    """Decoder-only Llama. ``forward(tokens, seqlens=None)`` returns fp32 logits ``[B, T, V]``
    (or the final hidden states when ``args.fused_linear_ce``), like the reference's
    ``Transformer.forward(tokens, block_mask)``; document masking is driven by per-sample
    ``seqlens`` (or a prebuilt ``seq_start`` row map) instead of a BlockMask."""

    def __init__(self, args: ModelArgs):
        super().__init__()
        assert args.vocab_size > 0, "vocab_size must be set"
        self.model_args = args
        self.vocab_size, self.n_layers = args.vocab_size, args.n_layers
        self.tok_embeddings = nn.Embedding(args.vocab_size, args.dim)
        self.register_buffer("freqs_cis", precompute_freqs_cis(args.head_dim, args.max_seq_len * 2, args.rope_theta),
                             persistent=True)
        self.layers = nn.ModuleDict({str(i): TransformerBlock(i, args) for i in range(args.n_layers)})
        self.norm = build_norm(args.norm_type, args.dim, args.norm_eps)
        self.output = nn.Linear(args.dim, args.vocab_size, bias=False)
        self.init_weights()

    def init_weights(self, generator: torch.Generator | None = None):
        args = self.model_args
        if args.init_mode == "normal":
            for name, p in self.named_parameters():
                if "norm" in name:
                    nn.init.ones_(p)
                else:
                    nn.init.normal_(p, 0.0, args.init_std, generator=generator)
            return
        nn.init.normal_(self.tok_embeddings.weight)
        for layer in self.layers.values():
            layer.init_weights()
        self.norm.reset_parameters()
        std = args.dim ** -0.5
        nn.init.trunc_normal_(self.output.weight, mean=0.0, std=std, a=-3 * std, b=3 * std)

    def rope_table(self) -> torch.Tensor:
        """[2*max_seq_len, head_dim/2, 2] fp32 (cos, sin) view of ``freqs_cis``."""
        return torch.view_as_real(self.freqs_cis).contiguous()

    def forward(self, tokens: torch.Tensor, seqlens=None, seq_start: torch.Tensor | None = None):
        B, T = tokens.shape
        if seq_start is None:
            from ..ops.attention import seq_start_from_batch, seq_start_from_seqlens
            seq_start = (seq_start_from_seqlens(seqlens, T, tokens.device) if seqlens is not None
                         else seq_start_from_batch(B, T, tokens.device))
        h = self.tok_embeddings(tokens).reshape(B * T, -1)
        table = self.rope_table()
        for layer in self.layers.values():
            h = layer(h, table, T, seq_start)
        h = self.norm(h)
        if self.model_args.fused_linear_ce:
            return h.reshape(B, T, -1)
        return F_.linear(h, self.output.weight).float().reshape(B, T, -1)

    @classmethod
    def from_model_args(cls, args: ModelArgs) -> "Transformer":
        return cls(args)


def get_num_flop_per_token(num_params: int, args: ModelArgs, seq_len: int) -> int:
    """6N + 12 L H hd T (reference: src/zeroband/utils/__init__.py:51-66)."""
    return 6 * num_params + 12 * args.n_layers * args.n_heads * args.head_dim * seq_len


def get_num_params(model: nn.Module, exclude_embedding: bool = False) -> int:
    n = sum(p.numel() for p in model.parameters())
    if exclude_embedding and hasattr(model, "tok_embeddings"):
        n -= model.tok_embeddings.weight.numel()
    return n
