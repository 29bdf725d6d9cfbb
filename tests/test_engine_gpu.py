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


class _SilentPeerComm:
    """Single-rank communicator whose device barrier waits for a second 'peer' that never signals: pad 1 is this
    GPU's own zero-filled memory. The wait runs out after its (short) budget and the kernel returns with
    PB_ERR_TIMEOUT_PEER in the status word; nothing traps, faults or spins forever."""
    world, rank = 1, 0

    def __init__(self, device):
        import ctypes as C
        from prime_b200.engine.fused_llama import LocalComm
        self._local = LocalComm()
        self.device = torch.device(device)
        self.pads = torch.zeros(2, 64 * 16, dtype=torch.int32, device=device)
        self._ptrs = (C.c_void_p * 2)(self.pads[0].data_ptr(), self.pads[1].data_ptr())
        self.epoch = 0
        self.silent = False

    def alloc(self, *a, **k):
        return self._local.alloc(*a, **k)

    def peer_ptrs(self, t):
        return self._local.peer_ptrs(t)

    def host_barrier(self):
        pass

    def allreduce_scalars(self, src, dst, n):
        dst[:n].copy_(src[:n])

    def barrier(self, slot=0, stream=None):
        if not self.silent:
            return
        from prime_b200 import native
        from prime_b200.native import check, ptr, stream_ptr
        from prime_b200.ops.kernels import status_word
        self.epoch += 1
        check(native.cuda().pb_peer_barrier(self._ptrs, 2, 0, 0, self.epoch, ptr(status_word(self.device)), stream_ptr(stream)),
              "pb_peer_barrier")


def test_peer_wait_runs_out_and_train_step_raises():
    """A device-side wait for a peer that never arrives gives up after its budget, the status word carries
    PB_ERR_TIMEOUT_PEER, train_step turns it into an exception, and the context keeps working afterwards."""
    import time
    from prime_b200 import native
    from prime_b200.ops.kernels import status_word
    lib = native.cuda()
    native.register_cuda_sigs({"pb_set_peer_wait_budget_ns": [native.i64], "pb_get_peer_wait_budget_ns": []})
    lib.pb_get_peer_wait_budget_ns.restype = __import__("ctypes").c_longlong
    old = lib.pb_get_peer_wait_budget_ns()
    assert old == 2_000_000_000
    assert lib.pb_set_peer_wait_budget_ns(20_000_000) == 0            # 20 ms
    try:
        args = _args()
        comm = _SilentPeerComm("cuda")
        eng = FusedLlama(args, device="cuda", comm=comm, ce_chunk_tokens=256)
        eng.init_weights(seed=0)
        tok = torch.randint(0, args.vocab_size, (2, 257))
        x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
        loss0, _ = eng.train_step(x, y, lr=1e-3)                       # healthy step
        comm.silent = True
        t0 = time.perf_counter()
        with pytest.raises(native.NativeError, match="error code 5"):
            eng.train_step(x, y, lr=1e-3)
        assert time.perf_counter() - t0 < 5.0                          # two 20 ms waits, not a hang
        assert int(status_word(torch.device("cuda", 0)).item()) == 0   # cleared by the raise
        comm.silent = False
        loss1, _ = eng.train_step(x, y, lr=1e-3)                       # the context is still usable
        assert loss1 == loss1 and loss1 < loss0 + 1.0
        # the bare kernel: status word holds code 5 with the silent peer's index in the upper bits
        comm.silent = True
        comm.barrier()
        torch.cuda.synchronize()
        code = int(status_word(torch.device("cuda", 0)).item())
        assert code & 0xff == 5 and code >> 8 == 1
        with pytest.raises(native.NativeError):
            check_status()
        check_status()
    finally:
        lib.pb_set_peer_wait_budget_ns(old)


class _OneWorkerMesh:
    """What Diloco needs from an ElasticDeviceMesh for a single worker whose 'all-reduce' is the identity."""

    class _PG:
        def size(self):
            return 1

        def rank(self):
            return 0

    def __init__(self):
        self.global_pg = self._PG()

    def maybe_reinit_global_pg(self, *a, **k):
        return False

    def get_global_pg(self, maybe_reinit=False):
        return self.global_pg

    def monitored_barrier(self, flag):
        return None


def test_outer_step_with_device_resident_state_matches_host_path(monkeypatch):
    """With ``outer_state_resident`` the fused engine keeps fp32 outer parameters and momentum on the device, forms the
    pseudo-gradient there and applies Nesterov there; the host copies are refreshed on demand. Three outer steps must
    leave the same inner shard, outer parameters and momentum as the host path (host subtraction, torch SGD on the
    host), and a host copy rewritten in between (as a checkpoint load does) must be picked up."""
    from prime_b200 import diloco as diloco_mod
    from prime_b200.config import DilocoConfig
    from prime_b200.diloco import Diloco
    monkeypatch.setattr(diloco_mod, "all_reduce", lambda compression, tensor, op, group: None)   # one worker: identity
    args = _args()
    engines, dls = [], []
    for resident in (True, False):
        eng = FusedLlama(args, device="cuda", ce_chunk_tokens=256)
        eng.init_weights(seed=3)
        engines.append(eng)
        dls.append(Diloco(DilocoConfig(inner_steps=2, outer_state_resident=resident), eng, _OneWorkerMesh()))
    assert dls[0]._device_state(engines[0]) is not None and dls[1]._device_state(engines[1]) is None
    g = torch.Generator(device="cuda").manual_seed(5)
    for step in range(3):
        delta = torch.randn(engines[0].master.numel(), device="cuda", generator=g) * 1e-3
        for eng, dl in zip(engines, dls):
            eng.master.add_(delta)                      # "inner training"
            dl.step(eng, flag=f"s{step}")
        if step == 1:                                   # the host copies are rewritten between outer steps
            for eng, dl in zip(engines, dls):
                dl.wait_host_state()
                dl.offloaded_data_flat_tensor.mul_(0.5)
                dl.mark_host_state_written()
                eng.master.copy_(dl.offloaded_data_flat_tensor)
    check_status()
    dls[0].wait_host_state()
    assert torch.allclose(engines[0].master, engines[1].master, rtol=0, atol=1e-6)
    assert torch.allclose(dls[0].offloaded_data_flat_tensor, dls[1].offloaded_data_flat_tensor, rtol=0, atol=1e-6)
    assert torch.allclose(dls[0]._momentum_flat(), dls[1]._momentum_flat(), rtol=0, atol=1e-6)
    assert torch.equal(engines[0].master.cpu(), dls[0].offloaded_data_flat_tensor)
    # the optimizer object that checkpoints serialise sees the refreshed momentum
    p0 = dls[0].param_list_cpu[0]
    assert torch.equal(dls[0].outer_optimizer.state[p0]["momentum_buffer"].reshape(-1), dls[0]._momentum_flat()[: p0.numel()])


def test_soap_shard_optimizer_on_gpu():
    """``optim.type = "soap"`` on the GPU: gradients, reduce and clip come from the engine's kernels, SOAP steps the fp32
    shards with torch's CUDA ops, the bf16 replica is refreshed by the push kernel. Same check as on the CPU: a hand-run
    SOAP on copies of the shards, fed the clipped gradient shard, stays equal to the engine's master weights."""
    from prime_b200.backend import FusedBackend
    from prime_b200.config import SoapConfig
    from prime_b200.lr_scheduler import get_scheduler
    from prime_b200.optimizers import SOAP
    args = _args()
    cfg = SoapConfig(lr=2e-3, weight_decay=0.01, precondition_frequency=2, max_preconditioner_dim=1024)
    eng = FusedLlama(args, device="cuda", ce_chunk_tokens=512)
    eng.init_weights(seed=4)
    backend = FusedBackend(eng, cfg, lambda o: get_scheduler("cosine", o, 1, 0, 100), max_norm=1.0)
    twin = [torch.nn.Parameter(t.clone()) for _, t in eng.named_master_shards()]
    opt = SOAP(twin, lr=cfg.lr, betas=(cfg.betas1, cfg.betas2), eps=1e-12, weight_decay=cfg.weight_decay,
               max_preconditioner_dim=cfg.max_preconditioner_dim, precondition_frequency=cfg.precondition_frequency)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, args.vocab_size, (4, 257), generator=g)
    batch = {"input_ids": tok[:, :-1].contiguous(), "labels": tok[:, 1:].contiguous()}
    losses = []
    for step in range(4):
        lr = backend.current_lr()
        out = backend.train_step(batch, micro_bs=2)
        losses.append(out["loss"])
        for q, (name, _) in zip(twin, eng.named_master_shards()):
            q.grad = eng.shard_view(eng.grad_shard, name).clone()
        for group in opt.param_groups:
            group["lr"] = lr
        opt.step()
        for q, (name, t) in zip(twin, eng.named_master_shards()):
            assert torch.allclose(q.data, t, rtol=1e-3, atol=1e-4), (step, name)
    check_status()
    assert losses[-1] < losses[0]
    name0, t0 = next(iter(eng.named_master_shards()))
    assert torch.allclose(eng.w[name0].float(), t0, atol=2e-2)
