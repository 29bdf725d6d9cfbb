"""Training entry point on GPUs: fused engine through `prime_b200.train` (1 GPU and, when the box has
them, 2 GPUs with the symmetric-memory ZeRO path), plus 2-GPU numerical agreement with 1 GPU."""
import os
import pickle
import subprocess
import sys

import pytest
import torch

from prime_b200.utils import get_random_available_port

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(nproc, argv, log, extra_env=None, module="prime_b200.train", timeout=900):
    env = dict(os.environ)
    env.update({"WANDB_MODE": "disabled", "NCCL_NVLS_ENABLE": "0"})
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(get_random_available_port()), "-m", module] + argv
    with open(log, "w") as f:
        rc = subprocess.call(cmd, cwd=ROOT, env=env, stdout=f, stderr=subprocess.STDOUT, timeout=timeout)
    assert rc == 0, open(log).read()[-4000:]


ARGS = ["@configs/debug/normal.toml", "--optim.total_steps", "6", "--train.micro_bs", "4", "--optim.batch_size", "8",
        "--data.seq_length", "256", "--no-data.sequence_packing", "--optim.optim.lr", "1e-3", "--optim.warmup_steps", "2"]


def _losses(pkl):
    with open(pkl, "rb") as f:
        return [x["Loss"] for x in pickle.load(f) if "Loss" in x]


def test_train_one_gpu(tmp_path):
    _torchrun(1, ARGS + ["--project", str(tmp_path / "m1.pkl")], tmp_path / "l1.log")
    l1 = _losses(tmp_path / "m1.pkl")
    assert len(l1) == 6 and l1[-1] < l1[0]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_train_two_gpus_matches_one(tmp_path):
    _torchrun(1, ARGS + ["--project", str(tmp_path / "m1.pkl")], tmp_path / "l1.log")
    _torchrun(2, ARGS + ["--project", str(tmp_path / "m2.pkl"), "--train.micro_bs", "2"], tmp_path / "l2.log")
    l1, l2 = _losses(tmp_path / "m1.pkl"), _losses(tmp_path / "m2.pkl")
    assert len(l2) == 6
    # every rank reads its own data stream, so only the level is comparable (exact equivalence of the
    # sharded step is checked by test_zero_sharded_step_matches_single_rank)
    assert all(abs(a - b) < 0.3 for a, b in zip(l1, l2))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("mode", [[], ["--reshard"], ["--reshard", "--ac"]], ids=["replica", "reshard", "reshard-ac"])
def test_zero_sharded_step_matches_single_rank(tmp_path, mode):
    n = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(get_random_available_port()), os.path.join(ROOT, "tests", "multi_gpu", "zero_equivalence.py")] + mode
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout + r.stderr)[-4000:]


def test_train_one_gpu_diloco_ckpt_resume(tmp_path):
    ck = tmp_path / "ck"
    common = ["@configs/debug/diloco.toml", "--optim.total_steps", "8", "--diloco.inner_steps", "2", "--train.micro_bs", "4",
              "--optim.batch_size", "8", "--data.seq_length", "256", "--train.log_model_hash", "--ckpt.path", str(ck),
              "--ckpt.interval", "4"]
    _torchrun(1, common + ["--project", str(tmp_path / "a.pkl")], tmp_path / "a.log")
    assert (ck / "step_4" / ".metadata").exists()
    _torchrun(1, common + ["--project", str(tmp_path / "b.pkl"), "--ckpt.resume", str(ck / "step_4")], tmp_path / "b.log")
    with open(tmp_path / "a.pkl", "rb") as f:
        a = pickle.load(f)
    with open(tmp_path / "b.pkl", "rb") as f:
        b = pickle.load(f)
    saved = next(x for x in a if x.get("step") == 4 and "inner_model_hash_save" in x)
    resumed = next(x for x in b if "inner_model_hash_resume" in x)
    for k in ("inner_model_hash", "inner_optimizer_hash", "outer_optimizer_hash", "outer_model_hash"):
        assert saved[f"{k}_save"] == resumed[f"{k}_resume"], k
    la = {x["step"]: x["Loss"] for x in a if "Loss" in x}
    lb = {x["step"]: x["Loss"] for x in b if "Loss" in x}
    for s in lb:
        assert abs(la[s] - lb[s]) < 2e-2


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_nvlink_uint8_allreduce_and_fused_outer_step(tmp_path):
    n = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(get_random_available_port()), os.path.join(ROOT, "tests", "multi_gpu", "diloco_nvlink.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout + r.stderr)[-4000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("compression", ["uint8", "no"])
def test_diloco_workers_inside_one_job_over_nvlink(tmp_path, compression):
    """Two DiLoCo workers as sub-groups of one launcher; the outer step runs on the NVLink kernels."""
    n = 4 if torch.cuda.device_count() >= 4 else 2
    argv = ["@configs/debug/diloco.toml", "--optim.total_steps", "4", "--diloco.inner_steps", "2", "--train.micro_bs", "4",
            "--optim.batch_size", "8", "--data.seq_length", "256", "--diloco.compression", compression, "--train.log_model_hash",
            "--project", str(tmp_path / "m.pkl")]
    _torchrun(n, argv, tmp_path / "job.log", extra_env={"PRIME_B200_WORKERS_PER_JOB": "2"})
    out = []
    for w in range(2):
        with open(str(tmp_path / "m.pkl") + f".w{w}", "rb") as f:
            out.append(pickle.load(f))
    for m in out:
        assert len([x for x in m if "Loss" in x]) == 4 and all(x["num_peers"] == 2 for x in m if "Loss" in x)
    ha = [x for x in out[0] if "outer_model_hash_outer_step" in x]
    hb = [x for x in out[1] if "outer_model_hash_outer_step" in x]
    assert len(ha) == 2
    for x, y in zip(ha, hb):
        assert x["outer_model_hash_outer_step"] == y["outer_model_hash_outer_step"]
        assert x["inner_model_hash_outer_step"] == y["inner_model_hash_outer_step"]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_allgather_fused_gemm(tmp_path):
    n = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(get_random_available_port()), os.path.join(ROOT, "tests", "multi_gpu", "ag_gemm.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout + r.stderr)[-4000:]
    print(r.stdout[-500:])
