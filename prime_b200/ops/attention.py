"""Causal, document-masked GQA attention over a packed token stream.

``qkv`` is the fused projection ``[M, (H + 2*KV) * hd]`` (q heads, then k heads, then v heads)
with RoPE already applied. ``seq_start[m]`` (int32) is the first row that query row ``m`` may
attend to; row ``m`` itself is the last. A batch of B independent sequences of length T is the
special case ``seq_start[m] = (m // T) * T``; packed documents (the reference's
``create_block_mask_from_seqlens``, src/zeroband/models/llama/model.py:168-198) use the document
start instead. On CUDA the tcgen05 kernels in csrc/attn_fwd_sm100.cu / attn_bwd_sm100.cu run;
on CPU a dense fp32 statement of the same math.
"""
from __future__ import annotations

import torch

from .. import native
from ..native import check, ptr, stream_ptr
from .kernels import _scratch_buf, status_word

native.register_cuda_sigs({
    "pb_attn_fwd": [native.vp, native.vp, native.vp, native.vp, native.i32, native.i32, native.i32, native.i32,
                    native.i64, native.i64, native.f32, native.vp, native.vp],
    "pb_attn_bwd": [native.vp] * 9 + [native.i32] * 5 + [native.i64] * 4 + [native.f32, native.vp, native.vp, native.vp],
})


def seq_start_from_batch(batch: int, seq_len: int, device) -> torch.Tensor:
    return (torch.arange(batch * seq_len, device=device, dtype=torch.int32) // seq_len) * seq_len


def seq_start_from_seqlens(seqlens: list[list[int]] | list[torch.Tensor], seq_len: int, device) -> torch.Tensor:
    """Per-row document starts for a batch of packed samples; ``seqlens[b]`` sums to ``seq_len``."""
    out = torch.empty(len(seqlens) * seq_len, dtype=torch.int32)
    for b, lens in enumerate(seqlens):
        pos = b * seq_len
        for n in (lens.tolist() if isinstance(lens, torch.Tensor) else lens):
            out[pos: pos + n] = pos
            pos += n
        assert pos == (b + 1) * seq_len, "seqlens of a sample must sum to seq_len"
    return out.to(device)


def _dense_mask(seq_start: torch.Tensor) -> torch.Tensor:
    M = seq_start.numel()
    r = torch.arange(M, device=seq_start.device)
    return (r[None, :] <= r[:, None]) & (r[None, :] >= seq_start[:, None].long())


def attention_reference(qkv: torch.Tensor, seq_start: torch.Tensor, H: int, KV: int, hd: int, scale: float | None = None):
    """Dense fp32 attention (autograd-capable); returns o [M, H*hd] in fp32."""
    M = qkv.shape[0]
    scale = scale if scale is not None else hd ** -0.5
    x = qkv.float()
    q = x[:, : H * hd].reshape(M, H, hd).transpose(0, 1)
    k = x[:, H * hd: (H + KV) * hd].reshape(M, KV, hd).transpose(0, 1)
    v = x[:, (H + KV) * hd:].reshape(M, KV, hd).transpose(0, 1)
    k = k.repeat_interleave(H // KV, dim=0)
    v = v.repeat_interleave(H // KV, dim=0)
    s = (q @ k.transpose(1, 2)) * scale
    s = s.masked_fill(~_dense_mask(seq_start)[None], float("-inf"))
    p = torch.softmax(s, -1)
    return (p @ v).transpose(0, 1).reshape(M, H * hd)


_warned_small_head = False


def _padded_hd(hd: int) -> int:
    """Kernel head size that a head of ``hd`` columns is zero-padded to (0: none fits)."""
    return 64 if hd < 64 else 128 if hd < 128 else 0


def _pad_heads(x: torch.Tensor, n_heads: int, hd: int, to: int) -> torch.Tensor:
    """[M, n_heads * hd] -> [M, n_heads * to], every head zero-padded on the right."""
    M = x.shape[0]
    out = x.new_zeros(M, n_heads, to)
    out[:, :, :hd] = x.reshape(M, n_heads, hd)
    return out.view(M, n_heads * to)


def _cut_heads(x: torch.Tensor, n_heads: int, hd: int, padded: int) -> torch.Tensor:
    return x.view(x.shape[0], n_heads, padded)[:, :, :hd].reshape(x.shape[0], n_heads * hd)


def _small_head_fwd(qkv, seq_start, H, KV, hd, scale, out):
    """Head sizes other than 64 / 128 (the debug presets: 16 and 32). Heads that fit are zero-padded to the next kernel
    head size, which changes neither the scores nor the real output columns, so these models run the same tcgen05
    kernels; larger heads run the dense fp32 statement on the device."""
    to = _padded_hd(hd)
    if to and hd % 8 == 0:
        o_p, lse2 = attention_fwd(_pad_heads(qkv, H + 2 * KV, hd, to), seq_start, H, KV, to, scale)
        o = _cut_heads(o_p, H, hd, to)
        if out is not None:
            out.copy_(o)
            o = out
        return o, lse2
    global _warned_small_head
    if not _warned_small_head:
        import warnings
        warnings.warn(f"head_dim={hd} has no tcgen05 attention kernel (64 and 128 do); using dense attention")
        _warned_small_head = True
    M = qkv.shape[0]
    x = qkv.float()
    q = x[:, : H * hd].reshape(M, H, hd).transpose(0, 1)
    k = x[:, H * hd: (H + KV) * hd].reshape(M, KV, hd).transpose(0, 1).repeat_interleave(H // KV, dim=0)
    s = ((q @ k.transpose(1, 2)) * scale).masked_fill(~_dense_mask(seq_start)[None], float("-inf"))
    lse2 = torch.logsumexp(s, -1) * 1.4426950408889634
    o = attention_reference(qkv, seq_start, H, KV, hd, scale).to(qkv.dtype)
    if out is not None:
        out.copy_(o)
        o = out
    return o, lse2


def _small_head_bwd(qkv, o, dout, lse2, seq_start, H, KV, hd, scale, dqkv, rope_table, seq_len, row_dots):
    to = _padded_hd(hd)
    if to and hd % 8 == 0:
        g_p = attention_bwd(_pad_heads(qkv, H + 2 * KV, hd, to), _pad_heads(o, H, hd, to), _pad_heads(dout, H, hd, to), lse2,
                            seq_start, H, KV, to, scale, row_dots=row_dots)
        g = _cut_heads(g_p, H + 2 * KV, hd, to).contiguous()
        if rope_table is not None:      # the kernel's own inverse rotation pairs columns of the padded head: done here instead
            from .kernels import rope_
            g = rope_(g, rope_table, seq_len, H + KV, hd, backward=True)
        dqkv.copy_(g)
        return dqkv
    with torch.enable_grad():
        x = qkv.detach().float().requires_grad_(True)
        ref = attention_reference(x, seq_start, H, KV, hd, scale)
        (g,) = torch.autograd.grad(ref, x, dout.float())
    g = g.to(torch.bfloat16).contiguous()
    if rope_table is not None:
        from .kernels import rope_
        g = rope_(g, rope_table, seq_len, H + KV, hd, backward=True)
    dqkv.copy_(g)
    return dqkv


def attention_fwd(qkv: torch.Tensor, seq_start: torch.Tensor, H: int, KV: int, hd: int, scale: float | None = None,
                  out: torch.Tensor | None = None):
    """Returns (o [M, H*hd] bf16/fp32, lse2 [H, M] fp32 in log2 units of the scaled scores)."""
    M = qkv.shape[0]
    scale = scale if scale is not None else hd ** -0.5
    if not qkv.is_cuda:
        x = qkv.float()
        q = x[:, : H * hd].reshape(M, H, hd).transpose(0, 1)
        k = x[:, H * hd: (H + KV) * hd].reshape(M, KV, hd).transpose(0, 1).repeat_interleave(H // KV, dim=0)
        s = (q @ k.transpose(1, 2)) * scale
        s = s.masked_fill(~_dense_mask(seq_start)[None], float("-inf"))
        lse2 = torch.logsumexp(s, -1) * 1.4426950408889634
        o = attention_reference(qkv, seq_start, H, KV, hd, scale).to(qkv.dtype)
        if out is not None:
            out.copy_(o)
            o = out
        return o, lse2
    assert qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and seq_start.dtype == torch.int32
    if hd not in (64, 128):
        return _small_head_fwd(qkv, seq_start, H, KV, hd, scale, out)
    if out is None:
        out = torch.empty(M, H * hd, dtype=torch.bfloat16, device=qkv.device)
    lse2 = torch.empty(H, M, dtype=torch.float32, device=qkv.device)
    check(native.cuda().pb_attn_fwd(ptr(qkv), ptr(seq_start), ptr(out), ptr(lse2), M, H, KV, hd, qkv.stride(0),
                                    out.stride(0), scale, ptr(status_word(qkv.device)), stream_ptr()), "pb_attn_fwd")
    return out, lse2


def row_dots_buffer(device, M: int, H: int) -> torch.Tensor:
    """fp32 [H * M] scratch for the dO . O row sums (shared with the backward kernel's own pre-pass)."""
    return _scratch_buf(device, "attn_D", M * H)


def attention_bwd(qkv: torch.Tensor, o: torch.Tensor, dout: torch.Tensor, lse2: torch.Tensor, seq_start: torch.Tensor,
                  H: int, KV: int, hd: int, scale: float | None = None, dqkv: torch.Tensor | None = None,
                  rope_table: torch.Tensor | None = None, seq_len: int = 0, row_dots: torch.Tensor | None = None):
    """Gradient of the fused qkv buffer. With ``rope_table`` the inverse rotation of dq and dk is
    folded into the final pass (so the result is the gradient w.r.t. the *unrotated* projection).
    ``row_dots`` ([H, M] fp32 = sum over a head's columns of dout * o), when the caller already has it
    (``kernels.gemm_rowdot``), replaces the kernel's own pre-pass over ``o`` and ``dout``."""
    M = qkv.shape[0]
    scale = scale if scale is not None else hd ** -0.5
    if dqkv is None:
        dqkv = torch.empty_like(qkv)
    if not qkv.is_cuda:
        with torch.enable_grad():
            x = qkv.detach().float().requires_grad_(True)
            ref = attention_reference(x, seq_start, H, KV, hd, scale)
            (g,) = torch.autograd.grad(ref, x, dout.float())
        if rope_table is not None:
            from .kernels import rope_
            g = rope_(g.contiguous(), rope_table, seq_len, H + KV, hd, backward=True)
        dqkv.copy_(g.to(dqkv.dtype))
        return dqkv
    assert dout.stride(1) == 1 and o.stride(1) == 1 and dqkv.stride(1) == 1
    if hd not in (64, 128):
        return _small_head_bwd(qkv, o, dout, lse2, seq_start, H, KV, hd, scale, dqkv, rope_table, seq_len, row_dots)
    dq_acc = _scratch_buf(qkv.device, "attn_dq", M * H * hd)
    D = row_dots if row_dots is not None else _scratch_buf(qkv.device, "attn_D", M * H)
    tiles = _scratch_buf(qkv.device, "attn_tiles", (M + 127) // 128 + 1, torch.int32)
    assert rope_table is None or seq_len > 0
    check(native.cuda().pb_attn_bwd(ptr(qkv), ptr(o) if row_dots is None else None, ptr(dout), ptr(lse2), ptr(seq_start), ptr(dqkv), ptr(dq_acc), ptr(D),
                                    ptr(rope_table), max(int(seq_len), 1), M, H, KV, hd, qkv.stride(0),
                                    o.stride(0), dout.stride(0), dqkv.stride(0), scale, ptr(tiles), ptr(status_word(qkv.device)),
                                    stream_ptr()), "pb_attn_bwd")
    return dqkv
