"""GPU numerics: every sm_100a kernel against a plain PyTorch fp32 statement of the same op."""
import pytest
import torch

from prime_b200.ops import kernels as ops

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (384, 512, 320), (1000, 776, 200), (4096, 1024, 4096)])
@pytest.mark.parametrize("bn", [128, 256, 512])
def test_gemm_layouts(M, N, K, a_mn, b_mn, bn):
    torch.manual_seed(0)
    dev = "cuda"
    if a_mn and M % 8:
        pytest.skip("M-major A needs M % 8 == 0")
    a = torch.randn((K, M) if a_mn else (M, K), device=dev, dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device=dev, dtype=torch.bfloat16)
    out = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bn=bn)
    ref = (a.t() if a_mn else a).float() @ (b if b_mn else b.t()).float()
    torch.cuda.synchronize()
    ops.check_status()
    assert _rel(out, ref) < 1e-2
    # fp32 output with accumulate
    acc = torch.randn(M, N, device=dev, dtype=torch.float32)
    ref2 = acc + ref
    ops.gemm(a, b, out=acc, residual=acc, a_mn=a_mn, b_mn=b_mn, bn=bn)
    assert _rel(acc, ref2) < 1e-3
    # bf16 residual
    r = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
    o3 = ops.gemm(a, b, residual=r, a_mn=a_mn, b_mn=b_mn, bn=bn)
    assert _rel(o3, ref + r.float()) < 1e-2
    ops.check_status()


@pytest.mark.parametrize("M", [2304, 4352])
def test_gemm_banded_tile_order(M):
    """A B operand of 48 MB or more switches the CTA-pair kernel to tile numbering in bands of 16 tile rows: 9 rows
    (one short band) and 17 rows (a full band and a band of one), plain, residual and fp32 epilogues."""
    torch.manual_seed(0)
    dev = "cuda"
    N, K = 12544, 2048                                              # B = 51 MB, 49 tile columns
    a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    b = (torch.randn(N, K, device=dev) * K ** -0.5).bfloat16()
    ref = a.float() @ b.float().t()
    out = ops.gemm(a, b)
    r = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
    out_r = ops.gemm(a, b, residual=r)
    out_f = ops.gemm(a, b, out_dtype=torch.float32)
    torch.cuda.synchronize()
    ops.check_status()
    assert _rel(out, ref) < 1e-2 and _rel(out_r, ref + r.float()) < 1e-2 and _rel(out_f, ref) < 1e-3
    # the same through the N-major layout of B (input-gradient form) and with the SwiGLU epilogue (w13 = 50 MB)
    bt = b.t().contiguous()
    assert _rel(ops.gemm(a, bt, b_mn=True), ref) < 1e-2
    F = 6144
    w13 = (torch.randn(2 * F, K, device=dev) * K ** -0.5).bfloat16()
    h13 = torch.empty(M, 2 * F, device=dev, dtype=torch.bfloat16)
    act = torch.empty(M, F, device=dev, dtype=torch.bfloat16)
    ops.gemm_swiglu(a, w13, h13, act)
    ref13 = a.float() @ w13.float().t()
    torch.cuda.synchronize()
    ops.check_status()
    assert _rel(h13, ref13) < 1e-2
    assert _rel(act, torch.nn.functional.silu(ref13[:, :F]) * ref13[:, F:]) < 1e-2


@pytest.mark.parametrize("M,F,K", [(1024, 256, 192), (2000, 1024, 512), (4096, 4096, 1024)])
def test_gemm_fused_swiglu_epilogues(M, F, K):
    """SwiGLU forward and backward fused into the CTA-pair GEMM epilogue vs plain fp32 math."""
    torch.manual_seed(0)
    dev = "cuda"
    x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    w13 = (torch.randn(2 * F, K, device=dev) * K ** -0.5).bfloat16()
    h13 = torch.empty(M, 2 * F, device=dev, dtype=torch.bfloat16)
    act = torch.empty(M, F, device=dev, dtype=torch.bfloat16)
    ops.gemm_swiglu(x, w13, h13, act)
    ref = x.float() @ w13.float().t()
    g, u = ref[:, :F], ref[:, F:]
    torch.cuda.synchronize()
    ops.check_status()
    assert _rel(h13, ref) < 1e-2
    assert _rel(act, torch.nn.functional.silu(g) * u) < 1e-2
    # backward: out = act @ w2.T, d(h13) from dout
    D = 256
    w2 = (torch.randn(D, F, device=dev) * F ** -0.5).bfloat16()
    dout = torch.randn(M, D, device=dev, dtype=torch.bfloat16)
    gb, ub = h13[:, :F].float(), h13[:, F:].float()
    dact = dout.float() @ w2.float()
    sg = torch.sigmoid(gb)
    ref_d = torch.cat([dact * ub * sg * (1 + gb * (1 - sg)), dact * gb * sg], 1)
    ops.gemm_dswiglu(dout, w2, h13)
    torch.cuda.synchronize()
    ops.check_status()
    assert _rel(h13, ref_d) < 1.5e-2


@pytest.mark.parametrize("M,H,KV,hd,K,T", [(1024, 4, 4, 64, 256, 256), (3000, 8, 2, 128, 512, 1000), (4096, 16, 16, 64, 1024, 1024)])
def test_gemm_fused_rope_epilogue(M, H, KV, hd, K, T):
    torch.manual_seed(0)
    dev = "cuda"
    N = (H + 2 * KV) * hd
    x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    w = (torch.randn(N, K, device=dev) * K ** -0.5).bfloat16()
    table = ops.rope_table(T, hd, 10000.0, dev)
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    ops.gemm_rope(x, w, out, table, T, H + KV, hd)
    ref = (x.float() @ w.float().t())
    ref = ops.rope_(ref.cpu(), table.cpu(), T, H + KV, hd).to(dev)      # CPU twin rotates fp32 in place
    torch.cuda.synchronize()
    ops.check_status()
    assert _rel(out, ref) < 1e-2
    # the rotated part really differs from the unrotated product
    assert _rel(out[:, : (H + KV) * hd], (x.float() @ w.float().t())[:, : (H + KV) * hd]) > 0.1


@pytest.mark.parametrize("M,N,K,res", [(1024, 1024, 8192, False), (768, 1024, 32768, True), (3072, 1024, 16384, True)])
def test_gemm_split_k_weight_gradient(M, N, K, res):
    """Few output tiles + long K: the K slices run as separate work items, partials are reduced in fp32."""
    torch.manual_seed(0)
    dev = "cuda"
    a = torch.randn(K, M, device=dev, dtype=torch.bfloat16)      # dy [tokens, M] read M-major
    b = torch.randn(K, N, device=dev, dtype=torch.bfloat16)
    assert ops._splitk_slices(M, N, K, torch.device(dev, torch.cuda.current_device())) > 1
    ref = a.float().t() @ b.float()
    for dt in (torch.bfloat16, torch.float32):
        r = torch.randn(M, N, device=dev, dtype=dt) if res else None
        out = torch.empty(M, N, device=dev, dtype=dt)
        ops.gemm(a, b, out=out, residual=r, a_mn=True, b_mn=True)
        torch.cuda.synchronize()
        ops.check_status()
        assert _rel(out, ref + (r.float() if res else 0)) < (1e-2 if dt == torch.bfloat16 else 1e-3)
    # accumulate in place (residual aliases the output)
    acc = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
    want = ref + acc.float()
    ops.gemm(a, b, out=acc, residual=acc, a_mn=True, b_mn=True)
    assert _rel(acc, want) < 1e-2


@pytest.mark.parametrize("M,N,K", [(1024, 256, 256), (3000, 1024, 512), (4096, 1024, 1024)])
def test_gemm_fused_rowdot_epilogue(M, N, K):
    """dO = dh @ wo with the dO . O row sums of every 64-column head taken in the same kernel."""
    torch.manual_seed(0)
    dev = "cuda"
    dh = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    wo = (torch.randn(K, N, device=dev) * K ** -0.5).bfloat16()          # [D, H*hd], used N-major (dgrad)
    o = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    dots = torch.full(((N // 64) * M,), float("nan"), device=dev)
    assert ops.gemm_rowdot(dh, wo, out, o, dots, 64, b_mn=True)
    ref = dh.float() @ wo.float()
    ref_d = (ref * o.float()).reshape(M, N // 64, 64).sum(-1).t().contiguous()      # [heads, M]
    torch.cuda.synchronize()
    ops.check_status()
    assert _rel(out, ref) < 1e-2
    assert _rel(dots.view(N // 64, M), ref_d) < 1e-2


def test_gemm_persistent_many_tiles():
    torch.manual_seed(1)
    a = torch.randn(8192, 1024, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(4096, 1024, device="cuda", dtype=torch.bfloat16)
    out = ops.gemm(a, b)
    ref = a.float() @ b.float().t()
    assert _rel(out, ref) < 1e-2
    ops.check_status()


# widths with one (<= 1024), two (1536, 2048) and four (3072, 4096) warps per row in the backward; row counts that
# leave some of a CTA's row slots empty in the last iteration
@pytest.mark.parametrize("M,N", [(1000, 1024), (64, 256), (300, 4096), (1201, 768), (3, 512), (2501, 2048), (1999, 1536),
                                 (4099, 3072), (9001, 4096)])
def test_rmsnorm(M, N):
    torch.manual_seed(0)
    x = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(N, device="cuda")).bfloat16()
    dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    dres = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    y, rstd = ops.rmsnorm_fwd(x, w, 1e-5)
    yc, rc = ops.rmsnorm_fwd(x.cpu(), w.cpu(), 1e-5)
    assert _rel(y.cpu(), yc) < 1e-2
    assert _rel(rstd.cpu(), rc) < 1e-4
    dw = torch.zeros(N, device="cuda", dtype=torch.float32)
    dx = ops.rmsnorm_bwd(x, w, rstd, dy, dw, dres=dres)
    dwc = torch.zeros(N, dtype=torch.float32)
    dxc = ops.rmsnorm_bwd(x.cpu(), w.cpu(), rc, dy.cpu(), dwc, dres=dres.cpu())
    assert _rel(dx.cpu(), dxc) < 1e-2
    assert _rel(dw.cpu(), dwc) < 1e-3


def test_rope_roundtrip_and_ref():
    torch.manual_seed(0)
    T, H, KV, hd, B = 128, 4, 2, 64, 3
    qkv = torch.randn(B * T, (H + 2 * KV) * hd, device="cuda", dtype=torch.bfloat16)
    tab = ops.rope_table(T, hd, 10000.0, "cuda")
    ref = ops.rope_(qkv.cpu().clone(), tab.cpu(), T, H + KV, hd)
    got = ops.rope_(qkv.clone(), tab, T, H + KV, hd)
    assert _rel(got.cpu(), ref) < 1e-2
    assert torch.equal(got[:, (H + KV) * hd:], qkv[:, (H + KV) * hd:])
    back = ops.rope_(got.clone(), tab, T, H + KV, hd, backward=True)
    assert _rel(back, qkv) < 2e-2


def test_swiglu():
    torch.manual_seed(0)
    h = torch.randn(777, 2 * 512, device="cuda", dtype=torch.bfloat16)
    d = torch.randn(777, 512, device="cuda", dtype=torch.bfloat16)
    assert _rel(ops.swiglu_fwd(h).cpu(), ops.swiglu_fwd(h.cpu())) < 1e-2
    assert _rel(ops.swiglu_bwd(h, d).cpu(), ops.swiglu_bwd(h.cpu(), d.cpu())) < 1e-2


@pytest.mark.parametrize("fp32", [True, False])
def test_embedding(fp32):
    torch.manual_seed(0)
    V, D, M = 1000, 256, 4096
    E = torch.randn(V, D, device="cuda", dtype=torch.bfloat16)
    tok = torch.randint(0, V, (M,), device="cuda")
    out = ops.embedding_fwd(tok, E)
    assert torch.equal(out, E[tok])
    dout = torch.randn(M, D, device="cuda", dtype=torch.bfloat16)
    dE = torch.zeros(V, D, device="cuda", dtype=torch.float32 if fp32 else torch.bfloat16)
    ops.embedding_bwd(tok, dout, dE)
    ref = torch.zeros(V, D, dtype=torch.float32).index_add_(0, tok.cpu(), dout.cpu().float())
    assert _rel(dE.cpu(), ref) < (1e-5 if fp32 else 3e-2)


@pytest.mark.parametrize("z_mode", [ops.Z_NONE, ops.Z_MAX, ops.Z_LSE])
@pytest.mark.parametrize("V", [1024, 32000, 1003])
def test_cross_entropy(z_mode, V):
    torch.manual_seed(0)
    rows = 257
    ld = (V + 7) // 8 * 8
    buf = (torch.randn(rows, ld, device="cuda") * 3).bfloat16()
    logits = buf[:, :V]
    orig = logits.cpu().float().clone()
    labels = torch.randint(0, V, (rows,), device="cuda")
    labels[::7] = -100
    inv = ops.count_valid(labels)
    assert int(inv[1].item()) == int((labels != -100).sum())
    lc = logits.cpu().clone().contiguous()
    loss_c, z_c = torch.empty(rows), torch.empty(rows)
    ops.cross_entropy_(lc, labels.cpu(), inv.cpu(), loss_c, z_c, grad_scale=0.5, z_mode=z_mode, z_weight=1e-2)
    loss_g = torch.empty(rows, device="cuda")
    z_g = torch.empty(rows, device="cuda")
    ops.cross_entropy_(logits, labels, inv, loss_g, z_g, grad_scale=0.5, z_mode=z_mode, z_weight=1e-2)
    assert _rel(loss_g.cpu(), loss_c) < 1e-3
    assert _rel(z_g.cpu(), z_c) < 1e-3 or z_mode == ops.Z_NONE
    assert _rel(logits.cpu(), lc) < 2e-2
    # autograd cross-check of the CPU twin itself
    x = orig.requires_grad_(True)
    ce = torch.nn.functional.cross_entropy(x, labels.cpu(), reduction="sum") / float(inv[1])
    lse = torch.logsumexp(x, -1)
    valid = (labels.cpu() != -100).float()
    if z_mode == ops.Z_MAX:
        ce = ce + 1e-2 * ((x.max(-1).values ** 2) * valid).sum() / float(inv[1])
    if z_mode == ops.Z_LSE:
        ce = ce + 1e-2 * ((lse ** 2) * valid).sum() / float(inv[1])
    (0.5 * ce).backward()
    assert _rel(lc, x.grad) < 2e-2


@pytest.mark.parametrize("g_dtype", [torch.float32, torch.bfloat16])
def test_adamw_matches_torch(g_dtype):
    torch.manual_seed(0)
    n = 100_003
    p0 = torch.randn(n)
    p = p0.clone().cuda()
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    pl = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ref_p = torch.nn.Parameter(p0.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1, eps=1e-8)
    for step in range(1, 4):
        g = torch.randn(n).to(g_dtype)
        ref_p.grad = g.float().clone()
        opt.step()
        ops.adamw_(p, g.cuda(), m, v, pl, 1e-3, 0.9, 0.95, 1e-8, 0.1, step)
    assert _rel(p.cpu(), ref_p.data) < 1e-5
    assert _rel(pl.cpu(), ref_p.data) < 1e-2


def test_sumsq_and_clip():
    x = torch.randn(1_000_001, device="cuda")
    out = torch.zeros(1, device="cuda")
    ops.sumsq(x, out)
    assert abs(out.item() - x.double().pow(2).sum().item()) / out.item() < 1e-5
    ops.sumsq(x.bfloat16(), out, accumulate=True)
    assert abs(out.item() - 2 * x.double().pow(2).sum().item()) / out.item() < 1e-2


@pytest.mark.parametrize("n", [1000, 1 << 20, 3_000_001])
def test_gpu_quantizer_matches_host(n):
    from prime_b200.compression import host
    from prime_b200.ops.quant import dequantize_cuda, uniform_8bit_quantize_cuda
    torch.manual_seed(0)
    x = torch.randn(n, device="cuda") * 1e-3
    q, lut = uniform_8bit_quantize_cuda(x)
    deq = dequantize_cuda(q, lut)
    assert ((deq - x).norm() / x.norm()).item() < 0.05
    from prime_b200 import native
    chunk = native.cuda().pb_dl_chunk()
    xc = x.cpu()
    for c in range(min(2, lut.shape[0])):
        sl = slice(c * chunk, min(n, (c + 1) * chunk))
        qh, luth = host.uniform_8bit_quantize(xc[sl])
        diff = (q[sl].cpu().int() - qh.int()).abs()
        assert diff.max() <= 1 and (diff > 0).float().mean() < 1e-3
        assert torch.allclose(lut[c].cpu(), luth, atol=1e-6, rtol=1e-3)
    q2, lut2 = uniform_8bit_quantize_cuda(x)     # bit-reproducible
    assert torch.equal(q, q2) and torch.equal(lut, lut2)
