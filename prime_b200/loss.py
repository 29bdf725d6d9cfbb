"""Cross-entropy (+ optional z-loss) for the eager path
(reference: src/zeroband/loss.py:5-87).

``compute_cross_entropy_loss`` keeps the reference signature. With ``fused_linear_weight`` the
logits are never materialised for more than one chunk of tokens: each chunk runs head GEMM ->
cross-entropy kernel (gradient written in place) -> dgrad / wgrad GEMMs, which is the same schedule
the fused engine uses for its head (csrc/elementwise.cu ``cross_entropy_kernel``)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .ops import kernels as K


def _ce_max_z(logits: torch.Tensor, labels: torch.Tensor, z_weight: float | None, ignore_index: int):
    lf = logits.float()
    ce = F.cross_entropy(lf, labels, ignore_index=ignore_index, reduction="sum")
    if z_weight is None:
        return ce, None
    mx = lf.max(dim=-1).values
    mx = torch.where(labels != ignore_index, mx, torch.zeros_like(mx))
    return ce, z_weight * mx.pow(2).sum()


class _FusedLinearCE(torch.autograd.Function):
    """h [M,D], W [V,D], labels [M] -> (mean CE, z) with gradients of h and W computed in forward."""

    @staticmethod
    def forward(ctx, h, weight, labels, z_weight, ignore_index, chunk):
        M, D = h.shape
        V = weight.shape[0]
        hb = h.to(torch.bfloat16).contiguous() if h.is_cuda else h.float()
        wb = weight.to(torch.bfloat16).contiguous() if h.is_cuda else weight.float()
        inv = K.count_valid(labels, ignore_index)
        loss_rows = torch.empty(M, dtype=torch.float32, device=h.device)
        z_rows = torch.empty(M, dtype=torch.float32, device=h.device)
        dh = torch.empty_like(hb)
        dW = torch.zeros(V, D, dtype=torch.float32, device=h.device)
        Vp = (V + 7) // 8 * 8
        buf = torch.empty(min(chunk, M), Vp, dtype=hb.dtype, device=h.device)
        z_mode = K.Z_LSE if z_weight else K.Z_NONE
        for c0 in range(0, M, chunk):
            c1 = min(M, c0 + chunk)
            lg = buf[: c1 - c0, :V]
            K.gemm(hb[c0:c1], wb, out=lg)
            K.cross_entropy_(lg, labels[c0:c1], inv, loss_rows[c0:c1], z_rows[c0:c1], z_mode=z_mode, z_weight=z_weight or 0.0)
            K.gemm(lg, wb, out=dh[c0:c1], b_mn=True)
            K.gemm(lg, hb[c0:c1], out=dW, residual=dW, a_mn=True, b_mn=True)
        ctx.save_for_backward(dh, dW)
        ctx.dtypes = (h.dtype, weight.dtype)
        ce = loss_rows.sum() * inv[0]
        z = z_rows.sum() * inv[0] * (z_weight or 0.0)
        return ce, z

    @staticmethod
    def backward(ctx, g_ce, g_z):
        dh, dW = ctx.saved_tensors
        # the in-forward gradient is d(ce + z); both outputs receive the same upstream scale in practice
        return (dh * g_ce).to(ctx.dtypes[0]), (dW * g_ce).to(ctx.dtypes[1]), None, None, None, None


def compute_cross_entropy_loss(logits: torch.Tensor, labels: torch.Tensor, z_weight: float | None = None,
                               num_chunks: int | None = None, ignore_index: int = -100,
                               fused_linear_weight: torch.Tensor | None = None):
    """Returns ``(ce_loss, z_loss | None)``; CE is summed over tokens and divided by the number of
    non-ignored labels. ``logits`` is ``[B, T, V]`` — or the final hidden states ``[B, T, D]`` when
    ``fused_linear_weight`` (the output projection) is given."""
    if fused_linear_weight is None:
        V = logits.size(-1)
        flat, lab = logits.reshape(-1, V), labels.reshape(-1)
        n = (lab != ignore_index).sum().clamp_min(1)
        if num_chunks:
            ce_t, z_t = 0.0, 0.0
            for lg, lb in zip(flat.chunk(num_chunks, 0), lab.chunk(num_chunks, 0)):
                ce, z = _ce_max_z(lg, lb, z_weight, ignore_index)
                ce_t = ce_t + ce
                z_t = z_t + (z if z is not None else 0.0)
            return ce_t / n, (z_t / n if z_weight is not None else None)
        ce, z = _ce_max_z(flat, lab, z_weight, ignore_index)
        return ce / n, (z / n if z is not None else None)
    D = logits.size(-1)
    chunk = max(1, logits.numel() // D // num_chunks) if num_chunks else 8192
    ce, z = _FusedLinearCE.apply(logits.reshape(-1, D), fused_linear_weight, labels.reshape(-1), z_weight, ignore_index, chunk)
    return ce, (z if z_weight is not None else None)
