"""Small units: schedulers, loss, state-dict shipping, top-k retention, signatures, utils, model invariants."""
import math
import multiprocessing as mp
import os

import pytest
import torch

from prime_b200.checkpoint import delete_topk, get_checkpoints_to_delete
from prime_b200.loss import compute_cross_entropy_loss
from prime_b200.lr_scheduler import get_scheduler
from prime_b200.models.llama import ModelArgs, Transformer, llama2_configs, llama3_configs
from prime_b200.utils import (FakeTokenizer, PerfCounter, get_module_signature, get_peak_flops, get_random_available_port_list,
                              get_tensor_signature)
from prime_b200.utils.ip import parse_iperf_output
from prime_b200.utils.state_dict_send_recv import _get_sendable_state_dict, _load_sendable_state_dict


def test_schedulers():
    p = torch.nn.Parameter(torch.zeros(1))
    for kind in ("cosine", "linear", "wsd-sqrt"):
        opt = torch.optim.SGD([p], lr=1.0)
        s = get_scheduler(kind, opt, num_warmup_steps=10, num_stable_steps=50, num_training_steps=100)
        lrs = []
        for _ in range(100):
            lrs.append(s.get_last_lr()[0])
            opt.step()
            s.step()
        assert lrs[0] == 0.0 and abs(lrs[10] - 1.0) < 1e-9 and lrs[5] == pytest.approx(0.5)
        if kind == "wsd-sqrt":
            assert all(abs(x - 1) < 1e-9 for x in lrs[10:50]) and lrs[75] == pytest.approx(1 - math.sqrt(0.5))
        if kind == "cosine":
            assert lrs[55] == pytest.approx(0.5, abs=1e-6)
        if kind == "linear":
            assert lrs[55] == pytest.approx(0.5, abs=1e-6)
        assert lrs[-1] < 0.05


def test_loss_matches_torch_and_chunking_and_fused():
    torch.manual_seed(0)
    B, T, V, D = 2, 16, 50, 32
    h = torch.randn(B, T, D, requires_grad=True)
    W = torch.randn(V, D, requires_grad=True) * 0.3
    W.retain_grad()
    labels = torch.randint(0, V, (B, T))
    labels[0, :4] = -100
    logits = h @ W.t()
    ce, z = compute_cross_entropy_loss(logits, labels)
    ref = torch.nn.functional.cross_entropy(logits.reshape(-1, V), labels.reshape(-1), ignore_index=-100)
    assert z is None and torch.allclose(ce, ref, atol=1e-6)
    ce2, z2 = compute_cross_entropy_loss(logits, labels, z_weight=1e-2, num_chunks=4)
    assert torch.allclose(ce2, ref, atol=1e-6) and z2 is not None and z2.item() > 0
    # fused linear + CE: same value and gradients as the plain path
    ce3, z3 = compute_cross_entropy_loss(h, labels, fused_linear_weight=W, num_chunks=2)
    assert torch.allclose(ce3, ref, atol=1e-5) and z3 is None
    gh, gW = torch.autograd.grad(ref, [h, W], retain_graph=True)
    fh, fW = torch.autograd.grad(ce3, [h, W])
    assert torch.allclose(gh, fh, atol=1e-5) and torch.allclose(gW, fW, atol=1e-5)


def test_state_dict_split_merge_roundtrip():
    sd = {"a": torch.randn(3, 4), "b": {"c": torch.arange(5), "d": "text", "e": [torch.ones(2), 3, {"f": torch.zeros(1)}]}, "g": 1.5}
    skel, tensors = _get_sendable_state_dict(sd)
    assert len(tensors) == 4 and isinstance(skel["a"], str) and skel["b"]["d"] == "text"
    import pickle
    pickle.dumps(skel)   # tensor free
    back = _load_sendable_state_dict(tensors, skel)
    assert torch.equal(back["a"], sd["a"]) and torch.equal(back["b"]["e"][2]["f"], sd["b"]["e"][2]["f"]) and back["g"] == 1.5
    with pytest.raises(ValueError):
        _load_sendable_state_dict([torch.zeros(1)] * 4, skel)


def _p2p(rank, port, q):
    import torch.distributed as dist
    from prime_b200.utils.state_dict_send_recv import recv_state_dict, send_state_dict
    store = dist.TCPStore("127.0.0.1", port, 2, rank == 0)
    from datetime import timedelta
    pg = dist.ProcessGroupGloo(store, rank, 2, timedelta(seconds=60))
    sd = {"w": torch.arange(6.).reshape(2, 3), "opt": {"step": 3, "m": torch.ones(4) * 2}}
    if rank == 0:
        send_state_dict(pg, sd, 1)
        q.put("sent")
    else:
        like = {"w": torch.zeros(2, 3), "opt": {"step": 0, "m": torch.zeros(4)}}
        got = recv_state_dict(pg, 0, like)
        q.put(bool(torch.equal(got["w"], sd["w"]) and got["opt"]["step"] == 3 and torch.equal(got["opt"]["m"], sd["opt"]["m"])))


def test_state_dict_send_recv_between_processes():
    (port,) = get_random_available_port_list(1)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_p2p, args=(r, port, q)) for r in range(2)]
    [p.start() for p in ps]
    res = [q.get(timeout=120) for _ in ps]
    [p.join(timeout=20) for p in ps]
    assert True in res and "sent" in res


def test_topk_retention(tmp_path):
    for s in (5, 10, 15, 20, 100):
        (tmp_path / f"step_{s}").mkdir()
    (tmp_path / "other").mkdir()
    assert [os.path.basename(p) for p in get_checkpoints_to_delete(str(tmp_path), 2)] == ["step_5", "step_10", "step_15"]
    import logging
    delete_topk(logging.getLogger("t"), str(tmp_path), 2)
    assert sorted(os.listdir(tmp_path)) == ["other", "step_100", "step_20"]


def test_utils():
    assert get_peak_flops("NVIDIA B200") == 2.25e15 and get_peak_flops("NVIDIA H100 80GB HBM3") == 989e12
    assert get_peak_flops("NVIDIA H100 NVL") == 835e12 and get_peak_flops("something else") == 312e12
    assert parse_iperf_output("... 1.0 sec  5.25 GBytes  45.1 Gbits/sec") == int(45.1e9)
    t = FakeTokenizer()
    assert len(t) == 1000 and t.eos_token_id == 1
    a, b = torch.arange(1000.), torch.arange(1000.)
    assert get_tensor_signature(a) == get_tensor_signature(b)
    b[500] = -1
    assert get_tensor_signature(a) != get_tensor_signature(b)
    pc = PerfCounter(3)
    assert pc.get_tokens_per_second() is None
    for _ in range(5):
        pc.count_tokens(100)
    assert pc.get_tokens_per_second() > 0 and len(pc.tokens) == 3
    assert len(set(get_random_available_port_list(4))) == 4


def test_model_presets_shapes():
    assert llama2_configs["150M"].hidden_dim == 2816 and llama3_configs["10B"].hidden_dim == 14336
    assert llama3_configs["1B"].hidden_dim == 7168 and llama2_configs["7B"].hidden_dim == 11008
    from dataclasses import replace
    n = replace(llama3_configs["10B"], vocab_size=128256).num_params()
    assert abs(n - 10.21e9) / 10.21e9 < 0.01


def _tiny():
    return ModelArgs(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, ffn_hidden=128, vocab_size=100, max_seq_len=64)


def test_model_forward_and_packing_invariants():
    torch.manual_seed(0)
    m = Transformer(_tiny())
    assert set(dict(m.named_parameters())) >= {"tok_embeddings.weight", "layers.0.attention.wq.weight", "layers.1.feed_forward.w2.weight",
                                               "norm.weight", "output.weight"}
    assert m.freqs_cis.dtype == torch.complex64 and m.freqs_cis.shape == (128, 8)
    x = torch.randint(0, 100, (2, 32))
    out = m(x)
    assert out.shape == (2, 32, 100) and out.dtype == torch.float32
    # the same 16-token sequence packed twice gives equal halves ...
    half = torch.randint(0, 100, (1, 16))
    packed = torch.cat([half, half], 1)
    o = m(packed, seqlens=[[16, 16]])
    # document isolation is exact: changing document 2 never changes the logits of document 1
    other = packed.clone()
    other[0, 16:] = torch.randint(0, 100, (16,))
    o2 = m(other, seqlens=[[16, 16]])
    assert torch.allclose(o[:, :16], o2[:, :16], atol=1e-6)
    # without the document mask it does leak
    o3, o4 = m(packed), m(other)
    assert torch.allclose(o3[:, :16], o4[:, :16], atol=1e-6)           # causal: still no leak backwards
    assert not torch.allclose(o[:, 16:], o3[:, 16:], atol=1e-4)        # but doc 2 sees doc 1 when unmasked
    # packed first document == the same document alone
    alone = m(half)
    assert torch.allclose(o[:, :16], alone, atol=1e-5)


def test_model_backward_and_ac_wrapper():
    from prime_b200.utils.activation_ckpt import apply_ac_ckpt
    torch.manual_seed(0)
    m = Transformer(_tiny())
    x = torch.randint(0, 100, (2, 16))
    loss = m(x).float().pow(2).mean()
    loss.backward()
    g0 = m.layers["0"].attention.wq.weight.grad.clone()
    m.zero_grad()
    apply_ac_ckpt(m, 1)
    loss2 = m(x).float().pow(2).mean()
    loss2.backward()
    g1 = dict(m.named_parameters())
    key = next(k for k in g1 if k.endswith("layers.0._checkpoint_wrapped_module.attention.wq.weight") or k.endswith("layers.0.attention.wq.weight"))
    assert torch.allclose(g0, g1[key].grad, atol=1e-6) and torch.allclose(loss, loss2)
    sig = get_module_signature(m)
    assert isinstance(sig, str) and len(sig) == 32


def test_soap_optimizer_matches_adam_in_a_fixed_basis_and_converges():
    """SOAP with identity factors (sides wider than max_preconditioner_dim) is exactly AdamW; with real
    factors it drives an ill-conditioned least-squares problem down faster than AdamW at the same lr."""
    import copy
    from prime_b200.config import SoapConfig
    from prime_b200.optimizers import SOAP, get_optimizer
    torch.manual_seed(0)
    w0 = torch.randn(6, 5)
    g = [torch.randn(6, 5) for _ in range(4)]
    wa, ws = torch.nn.Parameter(w0.clone()), torch.nn.Parameter(w0.clone())
    adam = torch.optim.AdamW([wa], lr=1e-2, betas=(0.9, 0.95), eps=1e-12, weight_decay=0.1)
    soap = SOAP([ws], lr=1e-2, betas=(0.9, 0.95), eps=1e-12, weight_decay=0.1, max_preconditioner_dim=1)
    for gi in g:
        wa.grad, ws.grad = gi.clone(), gi.clone()
        adam.step()
        soap.step()
    assert torch.allclose(wa, ws, atol=1e-6)
    # ill-conditioned quadratic: f(W) = || A W B - T ||^2
    A = torch.diag(torch.logspace(0, 2, 8)) @ torch.linalg.qr(torch.randn(8, 8)).Q
    B = torch.linalg.qr(torch.randn(6, 6)).Q @ torch.diag(torch.logspace(0, 1.5, 6))
    T = torch.randn(8, 6)

    def run(opt_fn, steps=300):
        w = torch.nn.Parameter(torch.zeros(8, 6))
        b = torch.nn.Parameter(torch.zeros(6))
        opt = opt_fn([w, b])
        for _ in range(steps):
            opt.zero_grad()
            loss = ((A @ w @ B + b - T) ** 2).mean()
            loss.backward()
            opt.step()
        return loss.item(), opt
    l_soap, opt = run(lambda ps: get_optimizer(ps, SoapConfig(lr=3e-2, weight_decay=0.0, precondition_frequency=10)))
    l_adam, _ = run(lambda ps: torch.optim.AdamW(ps, lr=3e-2, betas=(0.9, 0.95), weight_decay=0.0))
    assert isinstance(opt, SOAP)
    assert l_soap < l_adam
    # state round trip
    sd = copy.deepcopy(opt.state_dict())
    opt.load_state_dict(sd)


def test_convert_dl_state_positions_from_both_reference_layouts():
    from prime_b200.cli.convert_dl_state import source_positions, transfer
    streaming = {"_snapshot": {"_worker_snapshots": {
        "worker_0": {"dataset_state": {"ex_iterable": {"ex_iterables": [{"ex_iterable": {"shard_idx": 4, "shard_example_idx": 10}},
                                                                         {"ex_iterable": {"shard_idx": 1, "shard_example_idx": 0}}]}}},
        "worker_1": {"dataset_state": {"ex_iterable": {"ex_iterables": [{"ex_iterable": {"shard_idx": 6, "shard_example_idx": 3}},
                                                                         {"ex_iterable": {"shard_idx": 0, "shard_example_idx": 9}}]}}}}}}
    assert source_positions(streaming) == [{"file_index": 7, "row_index": None}, {"file_index": 2, "row_index": None}]
    parquet = {"_snapshot": {"_worker_snapshots": {"worker_0": {"dataset_state": {"dataset": {
        "dataset_0": {"files": ["a", "b", "c"], "file_index": 2, "row_index": 40, "increment": 4, "init_row_index": 0},
        "dataset_1": {"files": ["d"], "file_index": 0, "row_index": 8, "increment": 4, "init_row_index": 0}}}}}}}
    new = {"loader": {"dataset": {"dataset": {"dataset_0": {"files": ["a", "b", "c"], "file_index": 0, "row_index": 1, "init_row_index": 1},
                                              "dataset_1": {"files": ["d"], "file_index": 0, "row_index": 1, "init_row_index": 1}}},
                      "batches_yielded": 1}, "ready_batch": None, "started": False}
    assert transfer(parquet, new) == 2
    d = new["loader"]["dataset"]["dataset"]
    assert (d["dataset_0"]["file_index"], d["dataset_0"]["row_index"]) == (2, 40)
    assert transfer(streaming, new) == 2
    assert (d["dataset_0"]["file_index"], d["dataset_0"]["row_index"]) == (7 % 3, 1)       # next shard, from its first row
    assert (d["dataset_1"]["file_index"], d["dataset_1"]["row_index"]) == (0, 1)


@pytest.mark.parametrize("sanitizer", ["address,undefined", "thread"])
def test_host_library_under_sanitizers(sanitizer, tmp_path):
    """The host quantiser and TCP ring, built with ASan+UBSan and with TSan, run their own C++ driver
    (tests/native/host_sanitize.cpp: odd sizes, tails, a 3-rank loopback ring on threads) without a report."""
    import shutil
    import subprocess
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = str(tmp_path / "host_san")
    src = [os.path.join(root, "tests/native/host_sanitize.cpp"), os.path.join(root, "prime_b200/csrc/host/quantize.cpp"),
           os.path.join(root, "prime_b200/csrc/host/tcp_ring.cpp")]
    cc = subprocess.run(["g++", "-std=c++17", "-O1", "-g", f"-fsanitize={sanitizer}", "-fno-omit-frame-pointer", *src, "-o", exe,
                         "-lpthread"], capture_output=True, text=True)
    if cc.returncode != 0 and "sanitize" in cc.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert cc.returncode == 0, cc.stderr[-2000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, (run.stdout + run.stderr)[-3000:]
    assert "0 failure(s)" in run.stdout


def test_wget_refuses_names_outside_destination(tmp_path, monkeypatch):
    """A peer's listing is untrusted: entries that would land outside the destination are refused."""
    import io
    import json
    import urllib.request

    from prime_b200.utils import wget as W

    def fake_open(url, timeout=None):
        if url.endswith("?list=1"):
            return io.BytesIO(json.dumps(["ok.bin", "../escape.bin"]).encode())
        return io.BytesIO(b"data")

    monkeypatch.setattr(urllib.request, "urlopen", fake_open)
    dest = tmp_path / "dst"
    with pytest.raises(ValueError):
        W.wget("http://127.0.0.1:1/latest/", str(dest))
    assert (dest / "ok.bin").read_bytes() == b"data" and not (tmp_path / "escape.bin").exists()
    monkeypatch.setattr(urllib.request, "urlopen", lambda url, timeout=None: io.BytesIO(json.dumps(["/abs.bin"]).encode()))
    with pytest.raises(ValueError):
        W.wget("http://127.0.0.1:1/latest/", str(dest))


def test_wandb_logger_reads_run_name_from_inner_config(monkeypatch):
    import sys
    import types
    seen = {}
    fake = types.SimpleNamespace(init=lambda **kw: seen.update(kw), log=lambda m: None, finish=lambda: None)
    monkeypatch.setitem(sys.modules, "wandb", fake)
    from prime_b200.utils.metric_logger import WandbMetricLogger
    WandbMetricLogger(project="p", config={"config": {"run_name": "r1"}, "world_info": {}}, resume=False)
    assert seen["name"] == "r1"


def test_engine_flag_checks():
    """Reference flags that the kernel engine cannot honour are refused or reported, not silently accepted."""
    import logging
    from prime_b200.config import Config
    from prime_b200.train import _check_engine_flags
    log = logging.getLogger("flagtest")
    seen = []
    log.warning = lambda msg, *a: seen.append(msg)
    base = {"data": {"fake": True}, "name_model": "debugmodel", "type_model": "llama2", "optim": {}}
    mk = lambda **t: Config(**base, train={"micro_bs": 1, **t})  # noqa: E731
    with pytest.raises(ValueError, match="fsdp_cpu_offload"):
        _check_engine_flags(mk(fsdp_cpu_offload=True), True, log)
    _check_engine_flags(mk(attn_fn="math", torch_compile=True, reshard_after_forward=True), True, log)
    assert len(seen) == 2
    seen.clear()
    _check_engine_flags(mk(), True, log)                    # defaults: nothing to say
    _check_engine_flags(mk(attn_fn="math"), False, log)     # eager path honours attn_fn
    assert not seen


def test_bench_allreduce_arms_print_one_json_line_on_cpu_ranks():
    """``bench.py --config allreduce --impl reference`` runs on CPU ranks over gloo (that is where the reference's outer
    all-reduce runs): two ranks, one small size. It prints one JSON line that either holds the reference ring's row or
    says in one line why the reference is unavailable; the same line shape as the GPU arms."""
    import json
    import subprocess
    import sys
    from prime_b200.utils import get_random_available_port
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(get_random_available_port()), os.path.join(root, "bench.py"), "--gpus", "2", "--config", "allreduce",
           "--impl", "reference", "--sizes-mb", "1"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=root)
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert out.returncode == 0 and len(lines) == 1, out.stderr[-2000:]
    d = json.loads(lines[0])
    assert d["impl"] == "reference"
    if "unavailable" in d:
        assert isinstance(d["unavailable"], str) and d["unavailable"]
    else:
        assert d["n_gpus"] == 2 and d["higher_is_better"] is False
        row = d["rows"][0]
        assert row["ref_py_uint8_ring"]["rel_err"] < 0.1 and row["gloo_fp32"]["rel_err"] < 1e-6
