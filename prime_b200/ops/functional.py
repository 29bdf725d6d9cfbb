"""Autograd-aware ops used by the eager modules.

CPU tensors: ordinary differentiable torch math (fp32 internally) — this is also the numerical
oracle. CUDA tensors: ``torch.autograd.Function`` wrappers whose forward and backward are the
hand-written sm_100a kernels (bf16 activations / weights, fp32 accumulation). fp32 CUDA inputs are
cast to bf16 at the op boundary, which mirrors the reference's FSDP2 mixed-precision policy
(param_dtype=bf16, src/zeroband/train.py:144-146).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import attention as A
from . import kernels as K


def _bf16(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16)


# ------------------------------------------------------------------------------------------ linear
class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        xb, wb = _bf16(x).contiguous(), _bf16(w).contiguous()
        ctx.save_for_backward(xb, wb)
        ctx.w_dtype = w.dtype
        return K.gemm(xb, wb)

    @staticmethod
    def backward(ctx, dy):
        xb, wb = ctx.saved_tensors
        dy = _bf16(dy).contiguous()
        dx = K.gemm(dy, wb, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            dw = K.gemm(dy, xb, a_mn=True, b_mn=True, out_dtype=torch.float32).to(ctx.w_dtype)
        return dx, dw


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` for 2-D ``x``."""
    if not x.is_cuda:
        return F.linear(x, w.to(x.dtype))
    return _Linear.apply(x, w)


# ------------------------------------------------------------------------------------------ rmsnorm
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        xb, wb = _bf16(x).contiguous(), _bf16(w).contiguous()
        y, rstd = K.rmsnorm_fwd(xb, wb, eps)
        ctx.save_for_backward(xb, wb, rstd)
        ctx.w_dtype = w.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        xb, wb, rstd = ctx.saved_tensors
        dw = torch.zeros(wb.numel(), dtype=torch.float32, device=xb.device)
        dx = K.rmsnorm_bwd(xb, wb, rstd, _bf16(dy).contiguous(), dw, accumulate_dw=False)
        return dx, dw.to(ctx.w_dtype), None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    if not x.is_cuda:
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)
    shp = x.shape
    return _RMSNorm.apply(x.reshape(-1, shp[-1]), w, eps).reshape(shp)


# ------------------------------------------------------------------------------------------ rope
class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, table, seq_len, n_rot, hd):
        ctx.save_for_backward(table)
        ctx.meta = (seq_len, n_rot, hd)
        return K.rope_(_bf16(qkv).contiguous().clone(), table, seq_len, n_rot, hd)

    @staticmethod
    def backward(ctx, d):
        (table,) = ctx.saved_tensors
        seq_len, n_rot, hd = ctx.meta
        return K.rope_(_bf16(d).contiguous().clone(), table, seq_len, n_rot, hd, backward=True), None, None, None, None


def rope(qkv: torch.Tensor, table: torch.Tensor, seq_len: int, n_rot_heads: int, head_dim: int) -> torch.Tensor:
    """Rotate the first ``n_rot_heads`` heads of each row (interleaved pairs); position = row % seq_len."""
    if qkv.is_cuda:
        return _Rope.apply(qkv, table, seq_len, n_rot_heads, head_dim)
    M = qkv.shape[0]
    rot = qkv[:, : n_rot_heads * head_dim].float().reshape(M, n_rot_heads, head_dim // 2, 2)
    cs = table[torch.arange(M, device=qkv.device) % seq_len][:, None].to(rot.dtype)
    re = rot[..., 0] * cs[..., 0] - rot[..., 1] * cs[..., 1]
    im = rot[..., 0] * cs[..., 1] + rot[..., 1] * cs[..., 0]
    out = torch.stack([re, im], -1).reshape(M, -1).to(qkv.dtype)
    return torch.cat([out, qkv[:, n_rot_heads * head_dim:]], -1)


# ------------------------------------------------------------------------------------------ swiglu
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h13):
        hb = _bf16(h13).contiguous()
        ctx.save_for_backward(hb)
        return K.swiglu_fwd(hb)

    @staticmethod
    def backward(ctx, d):
        (hb,) = ctx.saved_tensors
        return K.swiglu_bwd(hb, _bf16(d).contiguous())


def swiglu(h13: torch.Tensor) -> torch.Tensor:
    """``silu(h13[:, :F]) * h13[:, F:]``."""
    if h13.is_cuda:
        return _SwiGLU.apply(h13)
    Fdim = h13.shape[1] // 2
    return F.silu(h13[:, :Fdim]) * h13[:, Fdim:]


# ------------------------------------------------------------------------------------------ attention
class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, seq_start, H, KV, hd):
        qb = _bf16(qkv).contiguous()
        o, lse2 = A.attention_fwd(qb, seq_start, H, KV, hd)
        ctx.save_for_backward(qb, o, lse2, seq_start)
        ctx.meta = (H, KV, hd)
        return o

    @staticmethod
    def backward(ctx, do):
        qb, o, lse2, seq_start = ctx.saved_tensors
        H, KV, hd = ctx.meta
        return A.attention_bwd(qb, o, _bf16(do).contiguous(), lse2, seq_start, H, KV, hd), None, None, None, None


def attention(qkv: torch.Tensor, seq_start: torch.Tensor, H: int, KV: int, hd: int) -> torch.Tensor:
    if qkv.is_cuda:
        return _Attention.apply(qkv, seq_start, H, KV, hd)
    return A.attention_reference(qkv, seq_start, H, KV, hd).to(qkv.dtype)
