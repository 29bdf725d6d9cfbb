"""The fused engine's hand-written backward and update against autograd on the eager model (CPU, fp32)."""
import copy

import pytest
import torch

from prime_b200.engine.fused_llama import FusedLlama
from prime_b200.models.llama import ModelArgs, Transformer


def _tiny(**kw):
    base = dict(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, ffn_hidden=128, vocab_size=96, max_seq_len=16, init_mode="normal",
                init_std=0.2)
    base.update(kw)
    return ModelArgs(**base)


class _F32Engine(FusedLlama):
    """fp32 replicas / activations so the CPU comparison is tight."""

    def _buf(self, name, shape, dtype=torch.bfloat16):
        return super()._buf(name, shape, torch.float32 if dtype == torch.bfloat16 else dtype)


def _mk(args, ac=False, z=(0, 0.0)):
    torch.manual_seed(0)
    model = Transformer(args)
    eng = _F32Engine(args, device="cpu", grad_dtype=torch.float32, ac_ckpt=ac, ce_chunk_tokens=24, z_mode=z[0], z_weight=z[1])
    eng.params = eng.params.float()
    for p in eng.layout.params:
        eng.w[p.name] = eng.params[p.offset: p.offset + p.numel].view(p.shape)
    H, KV, hd, D, F = args.n_heads, args.kv_heads, args.head_dim, args.dim, args.hidden_dim
    for i in range(args.n_layers):
        q = eng.layout.params[eng.layout.by_name[f"layers.{i}.attention.wq.weight"]]
        eng.wqkv[i] = eng.params[q.offset: q.offset + (H + 2 * KV) * hd * D].view(-1, D)
        w1 = eng.layout.params[eng.layout.by_name[f"layers.{i}.feed_forward.w1.weight"]]
        eng.w13[i] = eng.params[w1.offset: w1.offset + 2 * F * D].view(2 * F, D)
    eng._rope = model.rope_table()
    eng.load_from_module(model)
    for name, v in eng.named_master_shards():   # fp32 publish
        s = eng.layout.segments[0][eng.layout.by_name[name]]
        eng.params[s.full_offset: s.full_offset + s.numel].copy_(v.reshape(-1))
    return model, eng


@pytest.mark.parametrize("ac", [False, True, 2])
@pytest.mark.parametrize("packed", [False, True])
def test_engine_grads_match_autograd(ac, packed):
    args = _tiny()
    model, eng = _mk(args, ac=ac)
    B, T = 3, 16
    tokens = torch.randint(0, args.vocab_size, (B, T))
    labels = torch.randint(0, args.vocab_size, (B, T))
    labels[0, :3] = -100
    seqlens = [[5, 11], [16], [1, 7, 8]] if packed else None
    from prime_b200.ops.attention import seq_start_from_seqlens
    ss = seq_start_from_seqlens(seqlens, T, "cpu") if packed else None
    out = eng.forward_backward(tokens, labels, seq_start=ss)
    logits = model(tokens, seqlens=seqlens)
    ref = torch.nn.functional.cross_entropy(logits.reshape(-1, args.vocab_size), labels.reshape(-1), ignore_index=-100)
    ref.backward()
    assert abs(out["loss"].item() - ref.item()) < 1e-4
    for name, p in model.named_parameters():
        g = eng.g[name]
        err = (g - p.grad).norm() / (p.grad.norm() + 1e-12)
        assert err < 1e-4, (name, err.item())
    assert torch.allclose(eng.forward_logits(tokens, seq_start=ss), logits, atol=1e-4)


def test_engine_grad_accumulation_and_adamw_step():
    args = _tiny()
    model, eng = _mk(args)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    B, T = 2, 16
    for step in range(2):
        for mb in range(2):
            tokens = torch.randint(0, args.vocab_size, (B, T))
            labels = torch.randint(0, args.vocab_size, (B, T))
            eng.forward_backward(tokens, labels, loss_scale=0.5)
            loss = torch.nn.functional.cross_entropy(model(tokens).reshape(-1, args.vocab_size), labels.reshape(-1)) * 0.5
            loss.backward()
        ref_norm = torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad()
        norm = eng.optimizer_step(1e-2, (0.9, 0.95), 1e-8, 0.1, 1.0)
        assert abs(norm.item() - ref_norm.item()) / ref_norm.item() < 1e-4
        for name, v in eng.named_master_shards():   # republish in fp32 for the next comparison
            s = eng.layout.segments[0][eng.layout.by_name[name]]
            eng.params[s.full_offset: s.full_offset + s.numel].copy_(v.reshape(-1))
    sd = dict(model.named_parameters())
    for name, v in eng.named_master_shards():
        # Adam normalises the update, so elements whose gradient is ~0 amplify round-off: compare in norm
        assert (v - sd[name]).norm() / sd[name].norm() < 1e-3, name


def test_z_loss_modes_match_autograd():
    from prime_b200.ops import kernels as K
    args = _tiny()
    for mode in (K.Z_MAX, K.Z_LSE):
        model, eng = _mk(args, z=(mode, 1e-2))
        tokens = torch.randint(0, args.vocab_size, (2, 16))
        labels = torch.randint(0, args.vocab_size, (2, 16))
        out = eng.forward_backward(tokens, labels)
        lg = model(tokens).reshape(-1, args.vocab_size)
        z = (lg.max(-1).values ** 2).mean() if mode == K.Z_MAX else (torch.logsumexp(lg, -1) ** 2).mean()
        ref = torch.nn.functional.cross_entropy(lg, labels.reshape(-1)) + 1e-2 * z
        ref.backward()
        assert abs((out["loss"] + out["z_loss"]).item() - ref.item()) < 1e-4
        for name, p in model.named_parameters():
            assert (eng.g[name] - p.grad).norm() / (p.grad.norm() + 1e-12) < 1e-4, name


def test_segment_tables_merge_contiguous_runs():
    """With one rank neighbouring parameters are contiguous in both the full and the shard buffer and collapse
    into few runs; with two ranks every parameter keeps its own row-shard segment."""
    from prime_b200.engine.fused_llama import _SegArrays
    from prime_b200.engine.layout import llama_layout
    args = ModelArgs(dim=64, n_layers=2, n_heads=4, ffn_hidden=128, vocab_size=96, max_seq_len=32)
    for world in (1, 2):
        lay = llama_layout(args, world)
        segs = [s for g in range(len(lay.groups)) for s in lay.group_segments(0, g)]
        sa = _SegArrays(segs)
        assert sa.total == sum(s.numel for s in segs)
        covered = sorted((sa.full[i], sa.numel[i]) for i in range(sa.n))
        for (o0, n0), (o1, _) in zip(covered, covered[1:]):
            assert o0 + n0 <= o1
        if world == 1:
            assert sa.n < len([s for s in segs if s.numel > 0])
        else:
            assert sa.n <= len(segs)


def test_optimizer_cta_ranges_cover_every_segment():
    """The reduce / AdamW launches give each non-empty segment its own CTA range: a segment without one would
    silently keep stale gradients. Ranges are monotone, end at the grid size and follow the segment sizes."""
    import ctypes as C

    from prime_b200 import native
    try:
        lib = native.cuda()
    except native.NativeError:
        pytest.skip("CUDA library not built")
    gen = torch.Generator().manual_seed(0)
    cases = [[5], [1, 1, 1], [0, 7, 0, 9, 0], [1 << 24, 512, 1 << 21, 0, 3, 1 << 24],
             torch.randint(1, 1 << 22, (111,), generator=gen).tolist(), [1] * 128]
    for numel in cases:
        n = len(numel)
        arr = (C.c_longlong * n)(*numel)
        for ctas in (1, n, 148, 640, 4096):
            out = (C.c_int * (n + 1))()
            grid = lib.pb_zero_cta_ranges(n, arr, ctas, out)
            begins = list(out)
            nonempty = sum(1 for x in numel if x > 0)
            assert grid == begins[-1] and grid >= nonempty
            if nonempty:
                assert grid == max(ctas, n)
            total = sum(numel)
            for i, x in enumerate(numel):
                width = begins[i + 1] - begins[i]
                assert width >= (1 if x > 0 else 0) and (x > 0 or width == 0)
                share = x / total * grid if total else 0.0
                if share >= 4.0:                # large segments get about their share of the grid
                    assert 0.5 * share <= width <= 1.5 * share + 1


def test_soap_runs_as_a_shard_optimizer_of_the_fused_engine(tmp_path):
    """``optim.type = "soap"`` with the fused engine: the engine produces the reduced fp32 gradient shard and the global
    norm, SOAP steps the fp32 master shards in place, the bf16 replica is refreshed. Checked against SOAP applied by hand
    to copies of the same shards with the same clipped gradients, over enough steps to cross a basis refresh; then the
    optimizer state round-trips through the flat state dict a checkpoint uses."""
    from prime_b200.backend import FusedBackend
    from prime_b200.config import SoapConfig
    from prime_b200.lr_scheduler import get_scheduler
    from prime_b200.optimizers import SOAP
    args = ModelArgs(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, ffn_hidden=128, vocab_size=200, max_seq_len=32,
                     init_mode="normal", init_std=0.05)
    cfg = SoapConfig(lr=3e-3, weight_decay=0.01, precondition_frequency=3, max_preconditioner_dim=256)
    eng = FusedLlama(args, device="cpu", grad_dtype=torch.float32, ce_chunk_tokens=64)
    eng.init_weights(seed=2)
    backend = FusedBackend(eng, cfg, lambda o: get_scheduler("cosine", o, 1, 0, 100), max_norm=0.5)
    assert backend.shard_optimizer is not None and eng._shard_opt is backend.shard_optimizer
    # the hand-run twin: copies of the shards, their own SOAP
    twin = [torch.nn.Parameter(t.clone()) for _, t in eng.named_master_shards()]
    opt = SOAP(twin, lr=cfg.lr, betas=(cfg.betas1, cfg.betas2), eps=1e-12, weight_decay=cfg.weight_decay,
               max_preconditioner_dim=cfg.max_preconditioner_dim, precondition_frequency=cfg.precondition_frequency)
    g = torch.Generator().manual_seed(0)
    losses = []
    for step in range(5):
        tok = torch.randint(0, args.vocab_size, (2, 33), generator=g)
        batch = {"input_ids": tok[:, :-1].contiguous(), "labels": tok[:, 1:].contiguous()}
        lr = backend.current_lr()
        out = backend.train_step(batch, micro_bs=2)
        losses.append(out["loss"])
        # grad_shard still holds the clipped gradients the shard optimizer consumed
        for q, (name, _) in zip(twin, eng.named_master_shards()):
            q.grad = eng.shard_view(eng.grad_shard, name).clone()
        for group in opt.param_groups:
            group["lr"] = lr
        opt.step()
        for q, (name, t) in zip(twin, eng.named_master_shards()):
            assert torch.allclose(q.data, t, rtol=1e-5, atol=1e-6), (step, name)
        # the bf16 replica follows the master shard
        name0, t0 = next(iter(eng.named_master_shards()))
        assert torch.allclose(eng.w[name0].float(), t0, atol=2e-2)
    assert out["grad_norm"] > 0 and all(torch.isfinite(torch.tensor(losses)))
    # state dict: every tensor of the shard optimizer's state, keyed by rank and parameter; loading fills them in place
    sd = backend.optimizer_state_dict()
    assert any(k.endswith(".Q_L") for k in sd) and any(k.endswith(".GG_R") for k in sd) and "state.step" in sd
    saved = {k: v.clone() for k, v in sd.items()}
    eng2 = FusedLlama(args, device="cpu", grad_dtype=torch.float32, ce_chunk_tokens=64)
    eng2.init_weights(seed=2)
    backend2 = FusedBackend(eng2, cfg, lambda o: get_scheduler("cosine", o, 1, 0, 100), max_norm=0.5)
    sd2 = backend2.optimizer_state_dict()
    assert set(sd2) == set(sd)
    for k, v in sd2.items():
        v.copy_(saved[k])                     # what the checkpoint loader does
    backend2.load_optimizer_state_dict(sd2)
    assert eng2.opt_step == eng.opt_step
    q0 = eng2._shard_params[0]
    assert backend2.shard_optimizer.state[q0]["step"] == 5
