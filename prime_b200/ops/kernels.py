"""Functional (non-autograd) wrappers over the sm_100a kernels, with plain-PyTorch CPU twins.

Every function dispatches on the device of its inputs: CUDA tensors go to the hand-written
kernels through :mod:`prime_b200.native` (hard error if the library is missing); CPU tensors
run the same math with torch ops in fp32, which is what the CPU tests and the CPU DiLoCo slice
use and what the GPU numerics tests compare against.
"""
from __future__ import annotations

import torch

from .. import native
from ..native import check, ptr, stream_ptr

import os as _os

# PRIME_B200_GEMM=single forces the single-CTA kernel (A/B measurements); default uses the CTA-pair kernel when it fits
_GEMM_PAIR = _os.environ.get("PRIME_B200_GEMM", "pair") != "single"
_status: dict[int, torch.Tensor] = {}
_scratch: dict[tuple[int, str], torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 word kernels write a non-zero code into when a bounded wait expires."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _status[idx]


def check_status(device: torch.device | None = None) -> None:
    """Synchronising check of the device status word; raises if any kernel reported a timeout."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    code = int(status_word(device).item())
    if code != 0:
        status_word(device).zero_()
        raise native.NativeError(f"device kernel reported error code {code & 0xff} (cta {code >> 8})")


def _scratch_buf(device, key: str, numel: int, dtype=torch.float32) -> torch.Tensor:
    k = (device.index or 0, key)
    t = _scratch.get(k)
    if t is None or t.numel() < numel or t.dtype != dtype:
        t = torch.empty(numel, dtype=dtype, device=device)
        _scratch[k] = t
    return t


# ---------------------------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------------------------
def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, residual: torch.Tensor | None = None,
         a_mn: bool = False, b_mn: bool = False, out_dtype: torch.dtype = torch.bfloat16, bn: int = 0,
         max_ctas: int = 0) -> torch.Tensor:
    """``out[M,N] = op(a) @ op(b).T (+ residual)`` with fp32 accumulation.

    ``a`` is ``[M,K]`` (or ``[K,M]`` when ``a_mn``); ``b`` is ``[N,K]`` (or ``[K,N]`` when ``b_mn``).
    ``residual`` has the shape and dtype of ``out`` and may be ``out`` itself (accumulate).
    On CUDA this is the tcgen05/TMEM kernel (csrc/gemm_sm100.cu).
    """
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    assert K == Kb, f"inner dimensions differ: {K} vs {Kb}"
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    if not a.is_cuda:
        af = (a.t() if a_mn else a).float()
        bf = (b.t() if b_mn else b).float()
        r = af @ bf.t()
        if residual is not None:
            r = r + residual.float()
        out.copy_(r.to(out.dtype))
        return out
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.stride(-1) == 1 and b.stride(-1) == 1 and out.stride(-1) == 1
    assert out.dtype in (torch.bfloat16, torch.float32)
    if residual is not None:
        assert residual.dtype == out.dtype and residual.shape == out.shape and residual.stride(-1) == 1
    ldr = residual.stride(0) if residual is not None else 0
    # bn: 0 = choose; 128 / 256 = single-CTA tile width; 512 = the CTA-pair (cta_group::2) 256x256 kernel
    use_pair = bn == 512 or (bn == 0 and _GEMM_PAIR and M >= 512 and N >= 256)
    if use_pair:
        slices = _splitk_slices(M, N, K, a.device) if bn == 0 else 1
        if slices > 1:
            # few output tiles, long K (weight gradients): K slices as extra work items, fp32 partials, one reduce
            ws = _splitk_ws(slices * M * N, a.device)
            rc = native.cuda().pb_gemm_bf16_pair_splitk(ptr(a), ptr(b), ptr(ws), M, N, K, a.stride(0), b.stride(0), int(a_mn),
                                                        int(b_mn), slices, max_ctas, ptr(status_word(a.device)), stream_ptr())
            check(rc, f"pb_gemm_bf16_pair_splitk(M={M},N={N},K={K},slices={slices})")
            used = native.cuda().pb_gemm_splitk_slices(K, slices)
            rc = native.cuda().pb_splitk_reduce(ptr(ws), used, M, N, ptr(residual), ldr, ptr(out), out.stride(0),
                                                int(out.dtype == torch.float32), stream_ptr())
            check(rc, "pb_splitk_reduce")
            return out
        if (residual is not None and out.dtype == torch.bfloat16 and residual.stride(0) % 8 == 0 and residual.data_ptr() % 16 == 0
                and max_ctas == 0):
            # bf16 residual / accumulate: the addend tiles come in by TMA and the sum leaves by TMA (staged epilogue)
            _gemm_epi(a, b, out, M, N, K, b_mn, 5, 0, 0, 0, residual, "add", a_mn=a_mn)
            return out
        rc = native.cuda().pb_gemm_bf16_pair(ptr(a), ptr(b), ptr(out), ptr(residual), M, N, K, a.stride(0), b.stride(0),
                                             out.stride(0), ldr, int(a_mn), int(b_mn), int(out.dtype == torch.float32), max_ctas,
                                             ptr(status_word(a.device)), stream_ptr())
        check(rc, f"pb_gemm_bf16_pair(M={M},N={N},K={K},a_mn={a_mn},b_mn={b_mn})")
        return out
    rc = native.cuda().pb_gemm_bf16(
        ptr(a), ptr(b), ptr(out), ptr(residual), M, N, K, a.stride(0), b.stride(0), out.stride(0), ldr, int(a_mn), int(b_mn),
        int(out.dtype == torch.float32), bn if bn in (128, 256) else 0, max_ctas, ptr(status_word(a.device)), stream_ptr())
    check(rc, f"pb_gemm_bf16(M={M},N={N},K={K},a_mn={a_mn},b_mn={b_mn})")
    return out


_SPLITK_WS: dict = {}
_N_PAIRS: dict = {}


def _splitk_ws(numel: int, device) -> torch.Tensor:
    t = _SPLITK_WS.get(device)
    if t is None or t.numel() < numel:
        t = torch.empty(numel, dtype=torch.float32, device=device)
        _SPLITK_WS[device] = t
    return t


def _splitk_slices(M: int, N: int, K: int, device) -> int:
    """K slices for the CTA-pair GEMM: 1 unless the product has too few 256x256 tiles to fill the GPU and a long
    K. Minimises waves x k-blocks per slice (0.42 us per k-block) plus the fp32 partials' round trip."""
    if N % 4 or K < 4096:
        return 1
    pairs = _N_PAIRS.get(device)
    if pairs is None:
        pairs = _N_PAIRS[device] = torch.cuda.get_device_properties(device).multi_processor_count // 2
    tiles = ((M + 255) // 256) * ((N + 255) // 256)
    if tiles * 4 > pairs * 3:
        return 1
    kb = (K + 63) // 64
    best, best_t = 1, -(-tiles // pairs) * kb * 0.42
    for s_ in range(2, 17):
        if s_ * M * N * 4 > (256 << 20):
            break
        t = -(-tiles * s_ // pairs) * -(-kb // s_) * 0.42 + s_ * M * N * 8 / 5e6 + 5.0
        if t < best_t:
            best, best_t = s_, t
    return best


def _pair_ok(M: int, N: int) -> bool:
    return _GEMM_PAIR and M >= 512 and N >= 256


def _gemm_epi(a, b, out, M, N, K, b_mn, epi, i0, i1, i2, aux, what, aux2=None, a_mn=False):
    rc = native.cuda().pb_gemm_bf16_pair_epi(ptr(a), ptr(b), ptr(out), None, M, N, K, a.stride(0), b.stride(0),
                                             out.stride(0) if out is not None else 0, 0, int(a_mn), int(b_mn), 0, 0, epi, i0, i1, i2,
                                             ptr(aux), aux.stride(0) if aux.dim() == 2 else 0, ptr(aux2),
                                             ptr(status_word(a.device)), stream_ptr())
    check(rc, f"pb_gemm_bf16_pair_epi[{what}](M={M},N={N},K={K})")


def gemm_swiglu(x: torch.Tensor, w13: torch.Tensor, h13: torch.Tensor, act: torch.Tensor):
    """``h13 = x @ w13.T`` (``w13 = [w1; w3]``, ``[2F, K]``) and ``act = silu(h13[:, :F]) * h13[:, F:]`` in one
    kernel: the SwiGLU runs in the GEMM epilogue on the fp32 accumulators (csrc/gemm2_sm100.cu). Falls
    back to GEMM + swiglu_fwd where the fused kernel does not apply (CPU, small or odd shapes)."""
    M, K = x.shape
    F = w13.shape[0] // 2
    if x.is_cuda and _pair_ok(M, 2 * F) and F % 128 == 0 and h13.stride(-1) == 1 and act.stride(-1) == 1:
        _gemm_epi(x, w13, h13, M, 2 * F, K, False, 1, F, 0, 0, act, "swiglu")
        return h13, act
    gemm(x, w13, out=h13)
    swiglu_fwd(h13, out=act)
    return h13, act


def gemm_dswiglu(dout: torch.Tensor, w2: torch.Tensor, h13: torch.Tensor, dact_ws: torch.Tensor | None = None):
    """In place ``h13 <- d(h13)`` for ``out = act @ w2.T``: ``d(act) = dout @ w2`` never leaves the GEMM, its
    epilogue reads gate | up from ``h13`` and writes d gate | d up back. ``w2`` is ``[D, F]``. Falls back to
    GEMM (into ``dact_ws``) + swiglu_bwd where the fused kernel does not apply."""
    M = dout.shape[0]
    F = w2.shape[1]
    if dout.is_cuda and _pair_ok(M, F) and F % 64 == 0 and h13.stride(-1) == 1:
        _gemm_epi(dout, w2, None, M, F, dout.shape[1], True, 3, F, 0, 0, h13, "dswiglu")
        return h13
    if dact_ws is None:
        dact_ws = torch.empty(M, F, dtype=h13.dtype, device=h13.device)
    gemm(dout, w2, out=dact_ws, b_mn=True)
    swiglu_bwd(h13, dact_ws, dh13=h13)
    return h13


def gemm_rope(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, table: torch.Tensor, seq_len: int, n_rot_heads: int,
              head_dim: int):
    """``out = x @ w.T`` with the rotary embedding applied to the leading ``n_rot_heads`` heads of every output
    row (position = row index modulo ``seq_len``) before the store. Falls back to GEMM + rope_."""
    M, K = x.shape
    N = w.shape[0]
    if x.is_cuda and _pair_ok(M, N) and head_dim % 64 == 0 and out.stride(-1) == 1 and table.shape[0] >= seq_len:
        _gemm_epi(x, w, out, M, N, K, False, 2, seq_len, n_rot_heads * head_dim, head_dim, table, "rope")
        return out
    gemm(x, w, out=out)
    rope_(out, table, seq_len, n_rot_heads, head_dim)
    return out


def gemm_rowdot(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, other: torch.Tensor, dots: torch.Tensor, group: int,
                b_mn: bool = False) -> bool:
    """``out = a @ op(b).T`` (bf16) and ``dots[g, m] = sum_{c in group g} out_fp32[m, c] * other[m, c]`` for column groups of
    ``group`` columns, in one kernel (the dO . O row sums of the attention backward, taken in the epilogue of the
    GEMM that produces dO). Returns False without touching anything when the fused kernel does not apply."""
    M = a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    if not (a.is_cuda and _pair_ok(M, N) and group == 64 and N % 64 == 0 and out.stride(-1) == 1 and other.stride(-1) == 1
            and other.shape == out.shape and dots.is_contiguous() and dots.numel() >= (N // 64) * M):
        return False
    _gemm_epi(a, b, out, M, N, a.shape[1], b_mn, 4, 64, 0, 0, other, "rowdot", aux2=dots)
    return True


# ---------------------------------------------------------------------------------------------
# RMSNorm
# ---------------------------------------------------------------------------------------------
def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor | None = None,
                rstd: torch.Tensor | None = None):
    M, N = x.shape
    if out is None:
        out = torch.empty_like(x)
    if rstd is None:
        rstd = torch.empty(M, dtype=torch.float32, device=x.device)
    if not x.is_cuda:
        xf = x.float()
        r = torch.rsqrt(xf.pow(2).mean(-1) + eps)
        out.copy_((xf * r[:, None] * w.float()).to(out.dtype))
        rstd.copy_(r)
        return out, rstd
    check(native.cuda().pb_rmsnorm_fwd(ptr(x), ptr(w), ptr(out), ptr(rstd), M, N, eps, stream_ptr()), "pb_rmsnorm_fwd")
    return out, rstd


def rmsnorm_bwd(x, w, rstd, dy, dw: torch.Tensor, dres: torch.Tensor | None = None, dx: torch.Tensor | None = None,
                accumulate_dw: bool = True):
    """Returns dx (= norm input gradient + ``dres``) and adds the weight gradient into ``dw``."""
    M, N = x.shape
    if dx is None:
        dx = torch.empty_like(x)
    if not x.is_cuda:
        xh = x.float() * rstd[:, None]
        g = dy.float() * w.float()
        d = (g - xh * (g * xh).mean(-1, keepdim=True)) * rstd[:, None]
        if dres is not None:
            d = d + dres.float()
        dx.copy_(d.to(dx.dtype))
        dwv = (dy.float() * xh).sum(0)
        dw.copy_(((dw.float() + dwv) if accumulate_dw else dwv).to(dw.dtype))
        return dx
    lib = native.cuda()
    ctas = lib.pb_rmsnorm_bwd_ctas()
    part = _scratch_buf(x.device, "rms_bwd", ctas * N)
    check(lib.pb_rmsnorm_bwd(ptr(x), ptr(w), ptr(rstd), ptr(dy), ptr(dres), ptr(dx), ptr(part), ptr(dw),
                             int(dw.dtype == torch.float32), int(accumulate_dw), M, N, stream_ptr()), "pb_rmsnorm_bwd")
    return dx


# ---------------------------------------------------------------------------------------------
# RoPE (interleaved pairs), in place on the first `n_rot_heads` heads of each row
# ---------------------------------------------------------------------------------------------
def rope_table(seq_len: int, head_dim: int, theta: float, device) -> torch.Tensor:
    """[seq_len, head_dim/2, 2] fp32 (cos, sin) — the real form of the reference's complex
    ``freqs_cis`` (src/zeroband/models/llama/model.py:69-89)."""
    freqs = 1.0 / (theta ** (torch.arange(0, head_dim, 2)[: head_dim // 2].float() / head_dim))
    t = torch.arange(seq_len).float()
    ang = torch.outer(t, freqs)
    return torch.stack([ang.cos(), ang.sin()], dim=-1).contiguous().to(device)


def rope_(qkv: torch.Tensor, table: torch.Tensor, seq_len: int, n_rot_heads: int, head_dim: int, backward: bool = False):
    M = qkv.shape[0]
    if not qkv.is_cuda:
        x = qkv[:, : n_rot_heads * head_dim].float().reshape(M, n_rot_heads, head_dim // 2, 2)
        pos = torch.arange(M) % seq_len
        cs = table[pos][:, None]  # [M,1,hd/2,2]
        co, si = cs[..., 0], cs[..., 1] * (-1.0 if backward else 1.0)
        re = x[..., 0] * co - x[..., 1] * si
        im = x[..., 0] * si + x[..., 1] * co
        qkv[:, : n_rot_heads * head_dim] = torch.stack([re, im], -1).reshape(M, -1).to(qkv.dtype)
        return qkv
    check(native.cuda().pb_rope(ptr(qkv), ptr(table), M, seq_len, n_rot_heads, head_dim, qkv.stride(0), int(backward),
                                stream_ptr()), "pb_rope")
    return qkv


# ---------------------------------------------------------------------------------------------
# SwiGLU
# ---------------------------------------------------------------------------------------------
def swiglu_fwd(h13: torch.Tensor, out: torch.Tensor | None = None):
    M, F2 = h13.shape
    F = F2 // 2
    if out is None:
        out = torch.empty(M, F, dtype=h13.dtype, device=h13.device)
    if not h13.is_cuda:
        g, u = h13[:, :F].float(), h13[:, F:].float()
        out.copy_((torch.nn.functional.silu(g) * u).to(out.dtype))
        return out
    check(native.cuda().pb_swiglu_fwd(ptr(h13), ptr(out), M, F, stream_ptr()), "pb_swiglu_fwd")
    return out


def swiglu_bwd(h13: torch.Tensor, dact: torch.Tensor, dh13: torch.Tensor | None = None):
    M, F2 = h13.shape
    F = F2 // 2
    if dh13 is None:
        dh13 = torch.empty_like(h13)
    if not h13.is_cuda:
        g, u, d = h13[:, :F].float(), h13[:, F:].float(), dact.float()
        s = torch.sigmoid(g)
        dg = d * u * s * (1 + g * (1 - s))
        du = d * g * s
        dh13.copy_(torch.cat([dg, du], 1).to(dh13.dtype))
        return dh13
    check(native.cuda().pb_swiglu_bwd(ptr(h13), ptr(dact), ptr(dh13), M, F, stream_ptr()), "pb_swiglu_bwd")
    return dh13


# ---------------------------------------------------------------------------------------------
# Embedding
# ---------------------------------------------------------------------------------------------
def embedding_fwd(tokens: torch.Tensor, E: torch.Tensor, out: torch.Tensor | None = None):
    M = tokens.numel()
    D = E.shape[1]
    if out is None:
        out = torch.empty(M, D, dtype=E.dtype, device=E.device)
    if not E.is_cuda:
        out.copy_(E[tokens.reshape(-1)])
        return out
    check(native.cuda().pb_embedding_fwd(ptr(tokens), ptr(E), ptr(out), M, D, stream_ptr()), "pb_embedding_fwd")
    return out


def embedding_bwd(tokens: torch.Tensor, dout: torch.Tensor, dE: torch.Tensor):
    M = tokens.numel()
    D = dE.shape[1]
    if not dE.is_cuda:
        dE.index_add_(0, tokens.reshape(-1), dout.to(dE.dtype))
        return dE
    check(native.cuda().pb_embedding_bwd(ptr(tokens), ptr(dout), ptr(dE), M, D, int(dE.dtype == torch.float32),
                                         stream_ptr()), "pb_embedding_bwd")
    return dE


# ---------------------------------------------------------------------------------------------
# Cross-entropy on a chunk of logits, gradient written in place
# ---------------------------------------------------------------------------------------------
Z_NONE, Z_MAX, Z_LSE = 0, 1, 2


def count_valid(labels: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """[2] fp32 tensor: (1/count, count) of labels != ignore_index (count clamped to >= 1 for the inverse)."""
    out = torch.empty(2, dtype=torch.float32, device=labels.device)
    if not labels.is_cuda:
        n = int((labels != ignore_index).sum())
        out[0] = 1.0 / max(n, 1)
        out[1] = n
        return out
    check(native.cuda().pb_count_valid(ptr(labels), labels.numel(), ignore_index, ptr(out), stream_ptr()), "pb_count_valid")
    return out


def cross_entropy_(logits: torch.Tensor, labels: torch.Tensor, inv_count: torch.Tensor, loss_rows: torch.Tensor,
                   z_rows: torch.Tensor | None, grad_scale: float = 1.0, ignore_index: int = -100,
                   z_mode: int = Z_NONE, z_weight: float = 0.0, write_grad: bool = True):
    """Per-row loss / z terms into ``loss_rows`` / ``z_rows``; ``logits`` is overwritten with
    ``d(mean CE + z_weight * mean z)/dlogits * grad_scale`` when ``write_grad``."""
    rows, V = logits.shape
    if not logits.is_cuda:
        lf = logits.float()
        lse = torch.logsumexp(lf, -1)
        mx, arg = lf.max(-1)
        valid = labels != ignore_index
        safe = labels.clamp_min(0)
        li = (lse - lf.gather(1, safe[:, None])[:, 0]) * valid
        loss_rows.copy_(li)
        zi = {Z_NONE: torch.zeros_like(lse), Z_MAX: mx * mx, Z_LSE: lse * lse}[z_mode] * valid
        if z_rows is not None:
            z_rows.copy_(zi)
        if write_grad:
            scale = valid.float() * float(inv_count[0]) * grad_scale
            soft = torch.exp(lf - lse[:, None])
            coef = scale * (1.0 + (2 * z_weight * lse if z_mode == Z_LSE else 0.0))
            g = soft * coef[:, None]
            g[torch.arange(rows), safe] -= scale
            if z_mode == Z_MAX:
                g[torch.arange(rows), arg] += scale * 2 * z_weight * mx
            logits.copy_(g.to(logits.dtype))
        return
    check(native.cuda().pb_cross_entropy(ptr(logits), ptr(labels), ptr(loss_rows), ptr(z_rows), ptr(inv_count),
                                         grad_scale, rows, V, logits.stride(0), ignore_index, z_mode, z_weight,
                                         int(write_grad), stream_ptr()), "pb_cross_entropy")


def sum_f32(x: torch.Tensor, out: torch.Tensor, scale_ptr: torch.Tensor | None = None, scale: float = 1.0,
            accumulate: bool = False):
    """out[0] (+)= scale * scale_ptr[0] * sum(x), fixed summation order."""
    if not x.is_cuda:
        v = x.sum() * scale * (float(scale_ptr[0]) if scale_ptr is not None else 1.0)
        out[0] = out[0] + v if accumulate else v
        return out
    scr = _scratch_buf(x.device, "sum", 1024)
    check(native.cuda().pb_sum_f32(ptr(x), x.numel(), ptr(scr), ptr(scale_ptr), scale, ptr(out), int(accumulate),
                                   stream_ptr()), "pb_sum_f32")
    return out


def sumsq(x: torch.Tensor, out: torch.Tensor, accumulate: bool = False):
    if not x.is_cuda:
        v = x.float().pow(2).sum()
        out[0] = out[0] + v if accumulate else v
        return out
    scr = _scratch_buf(x.device, "sumsq", 1024)
    check(native.cuda().pb_sumsq(ptr(x), x.numel(), int(x.dtype == torch.float32), ptr(scr), ptr(out), int(accumulate),
                                 stream_ptr()), "pb_sumsq")
    return out


# ---------------------------------------------------------------------------------------------
# AdamW on flat buffers
# ---------------------------------------------------------------------------------------------
def adamw_(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, p_lowp: torch.Tensor | None, lr: float,
           beta1: float, beta2: float, eps: float, wd: float, step: int, gnorm: torch.Tensor | None = None,
           max_norm: float = 1.0, gscale: float = 1.0):
    """In-place decoupled-weight-decay Adam (torch.optim.AdamW semantics) on flat fp32 state,
    with optional global-norm clipping (``gnorm`` = device scalar holding the total norm) and
    a refreshed low-precision copy of the parameters."""
    n = p.numel()
    if not p.is_cuda:
        gf = g.float() * gscale
        if gnorm is not None:
            gf = gf * min(1.0, max_norm / (float(gnorm) + 1e-6))
        p.mul_(1 - lr * wd)
        m.mul_(beta1).add_(gf, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
        bc1 = 1 - beta1 ** step
        bc2 = (1 - beta2 ** step) ** 0.5
        p.addcdiv_(m, v.sqrt() / bc2 + eps, value=-lr / bc1)
        if p_lowp is not None:
            p_lowp.copy_(p.to(p_lowp.dtype))
        return
    check(native.cuda().pb_adamw(ptr(p), ptr(g), int(g.dtype == torch.float32), ptr(m), ptr(v), ptr(p_lowp), n, lr, beta1,
                                 beta2, eps, wd, step, ptr(gnorm), max_norm, gscale, stream_ptr()), "pb_adamw")


def cast_to_bf16(src: torch.Tensor, dst: torch.Tensor):
    if not src.is_cuda:
        dst.copy_(src.to(dst.dtype))
        return dst
    check(native.cuda().pb_cast_f32_bf16(ptr(src), ptr(dst), src.numel(), stream_ptr()), "pb_cast_f32_bf16")
    return dst
