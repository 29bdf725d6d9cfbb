"""Fused engine on the GPU (bf16 kernels) against the same engine on the CPU (fp32 torch math)."""
import pytest
import torch

from prime_b200.engine.fused_llama import FusedLlama
from prime_b200.models.llama import ModelArgs, Transformer
from prime_b200.ops.kernels import check_status

pytestmark = pytest.mark.gpu


def _args(**kw):
    base = dict(dim=256, n_layers=2, n_heads=4, n_kv_heads=2, ffn_hidden=512, vocab_size=1000, max_seq_len=256,
                init_mode="normal", init_std=0.05)
    base.update(kw)
    return ModelArgs(**base)


@pytest.mark.parametrize("ac", [False, True])
def test_engine_gpu_matches_cpu(ac):
    args = _args()
    torch.manual_seed(0)
    model = Transformer(args)
    gpu = FusedLlama(args, device="cuda", ac_ckpt=ac, ce_chunk_tokens=256)
    cpu = FusedLlama(args, device="cpu", grad_dtype=torch.float32, ce_chunk_tokens=256)
    gpu.load_from_module(model)
    cpu.load_from_module(model)
    B, T = 3, 256
    tokens = torch.randint(0, args.vocab_size, (B, T))
    labels = torch.randint(0, args.vocab_size, (B, T))
    og = gpu.forward_backward(tokens.cuda(), labels.cuda())
    oc = cpu.forward_backward(tokens, labels)
    check_status()
    assert abs(og["loss"].item() - oc["loss"].item()) < 3e-2
    worst = 0.0
    for name in cpu.g:
        a, b = gpu.g[name].float().cpu(), cpu.g[name].float()
        err = ((a - b).norm() / (b.norm() + 1e-12)).item()
        worst = max(worst, err)
        assert err < 6e-2, (name, err)
    n_g = gpu.optimizer_step(1e-3)
    n_c = cpu.optimizer_step(1e-3)
    assert abs(n_g.item() - n_c.item()) / n_c.item() < 3e-2
    for (name, a), (_, b) in zip(gpu.named_master_shards(), cpu.named_master_shards()):
        assert ((a.cpu() - b).norm() / b.norm()).item() < 6e-3, name  # one Adam step of size lr on bf16-vs-fp32 gradients
    check_status()


def test_engine_gpu_loss_decreases_and_logits():
    args = _args(n_kv_heads=4)
    eng = FusedLlama(args, device="cuda", ce_chunk_tokens=512)
    eng.init_weights(seed=1)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, args.vocab_size, (4, 257), generator=g)
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    first = last = None
    for i in range(6):
        loss, _ = eng.train_step(x, y, lr=2e-3, micro_bs=2)
        first = loss if first is None else first
        last = loss
    assert last < first - 0.1
    logits = eng.forward_logits(x.cuda())
    assert logits.shape == (4, 256, args.vocab_size) and torch.isfinite(logits).all()
    check_status()


def test_smoke_entry():
    import __graft_entry__ as ge
    ge.smoke()
