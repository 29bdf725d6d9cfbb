"""End-to-end training runs on CPU ranks (gloo): plain, DiLoCo across two workers with the uint8 ring,
activation checkpointing / z-loss flags, and checkpoint save -> resume equivalence."""
import os
import pickle
import subprocess
import sys

import pytest

from prime_b200.utils import get_random_available_port_list

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _launch(argv, env_extra, log_path):
    env = dict(os.environ)
    env.update({"CUDA_VISIBLE_DEVICES": "", "WANDB_MODE": "disabled", "ZERO_BAND_LOG_LEVEL": "INFO", "OMP_NUM_THREADS": "2"})
    env.update(env_extra)
    f = open(log_path, "w")
    return subprocess.Popen([sys.executable, "-m", "prime_b200.train"] + argv, cwd=ROOT, env=env, stdout=f, stderr=subprocess.STDOUT)


def _local_env(rank, world, port):
    return {"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank), "LOCAL_WORLD_SIZE": str(world),
            "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)}


_PORT_TROUBLE = ("Address already in use", "EADDRINUSE", "Connection refused", "Connection reset")


def _run_job(tmp_path, name, n_workers, n_local, argv, timeout=420):
    """Run one training job as child processes; a job that died because one of its freshly picked ports was taken by
    another process in the meantime is started once more on new ports."""
    try:
        return _run_job_once(tmp_path, name, n_workers, n_local, argv, timeout)
    except AssertionError as e:
        if not any(t in str(e) for t in _PORT_TROUBLE):
            raise
    return _run_job_once(tmp_path, name + "_again", n_workers, n_local, argv, timeout)


def _run_job_once(tmp_path, name, n_workers, n_local, argv, timeout):
    ports = get_random_available_port_list(2 + n_workers)
    procs, logs = [], []
    for w in range(n_workers):
        for r in range(n_local):
            env = _local_env(r, n_local, ports[2 + w])
            if n_workers > 1:
                env.update({"GLOBAL_UNIQUE_ID": str(w), "GLOBAL_ADDR": "127.0.0.1", "GLOBAL_PORT": str(ports[0]), "GLOBAL_RANK": str(w),
                            "GLOBAL_WORLD_SIZE": str(n_workers), "ZERO_BAND_GLOBAL_PG_TIMEOUT_SECONDS": "120"})
            log = tmp_path / f"{name}_w{w}_r{r}.log"
            logs.append(log)
            extra = ["--project", str(tmp_path / f"{name}_w{w}.pkl")]
            if n_workers > 1:
                extra += ["--data.data_rank", str(w), "--data.data_world_size", str(n_workers)]
            procs.append(_launch(argv + extra, env, log))
    for p, log in zip(procs, logs):
        try:
            rc = p.wait(timeout=timeout)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise AssertionError(f"timeout; log tail:\n{log.read_text()[-3000:]}")
        if rc != 0:
            for q in procs:
                if q.poll() is None:
                    q.kill()
            raise AssertionError(f"{log}:\n{log.read_text()[-3000:]}")
    out = []
    for w in range(n_workers):
        with open(tmp_path / f"{name}_w{w}.pkl", "rb") as f:
            out.append(pickle.load(f))
    return out


BASE = ["@configs/debug/normal.toml", "--optim.total_steps", "4", "--train.micro_bs", "4", "--optim.batch_size", "8",
        "--data.seq_length", "128"]


def test_single_process_training(tmp_path):
    (m,) = _run_job(tmp_path, "plain", 1, 1, BASE)
    steps = [x for x in m if "Loss" in x]
    assert [x["step"] for x in steps] == [1, 2, 3, 4]
    assert all(0 < x["Loss"] < 20 for x in steps) and "grad_norm" in steps[0] and "inner_lr" in steps[0]
    assert steps[-1]["total_tokens"] == 4 * 8 * 128


def test_two_local_ranks_ac_zloss_no_packing(tmp_path):
    (m,) = _run_job(tmp_path, "dp2", 1, 2, BASE + ["--train.ac_ckpt", "--optim.z_loss", "--no-data.sequence_packing"])
    steps = [x for x in m if "Loss" in x]
    assert len(steps) == 4 and "z_loss" in steps[0]


@pytest.mark.parametrize("compression", ["no", "uint8"])
def test_diloco_two_workers(tmp_path, compression):
    argv = ["@configs/debug/diloco.toml", "--optim.total_steps", "4", "--diloco.inner_steps", "2", "--train.micro_bs", "4",
            "--optim.batch_size", "8", "--diloco.compression", compression, "--train.log_model_hash", "--data.seq_length", "128"]
    a, b = _run_job(tmp_path, f"diloco_{compression}", 2, 1, argv)
    for m in (a, b):
        inner = [x for x in m if "Loss" in x]
        outer = [x for x in m if "outer_step" in x]
        assert len(inner) == 4 and len(outer) == 2 and all(x["num_peers"] == 2 for x in inner)
        assert inner[-1]["total_tokens"] == 4 * 8 * 128 * 2
    # after every outer step all workers hold the same model and the same outer state
    ha = [x for x in a if "outer_model_hash_outer_step" in x]
    hb = [x for x in b if "outer_model_hash_outer_step" in x]
    assert len(ha) == 2
    for x, y in zip(ha, hb):
        assert x["outer_model_hash_outer_step"] == y["outer_model_hash_outer_step"]
        assert x["inner_model_hash_outer_step"] == y["inner_model_hash_outer_step"]


def test_checkpoint_resume_equivalence(tmp_path):
    ck = tmp_path / "ckpt"
    common = ["@configs/debug/diloco.toml", "--optim.total_steps", "8", "--diloco.inner_steps", "2", "--train.micro_bs", "4",
              "--optim.batch_size", "8", "--train.log_model_hash", "--no-data.sequence_packing", "--train.attn_fn", "math",
              "--ckpt.path", str(ck), "--ckpt.interval", "4", "--ckpt.topk", "5", "--data.seq_length", "128"]
    (full,) = _run_job(tmp_path, "full", 1, 1, common)
    assert (ck / "step_4" / ".metadata").exists() and (ck / "step_4" / "__0_0.pt").exists() and (ck / "step_4" / "data" / "_0.pt").exists()
    (res,) = _run_job(tmp_path, "resumed", 1, 1, common + ["--ckpt.resume", str(ck / "step_4")])
    saved = next(x for x in full if x.get("step") == 4 and "inner_model_hash_save" in x)
    resumed = next(x for x in res if "inner_model_hash_resume" in x)
    for k in ("inner_model_hash", "inner_optimizer_hash", "outer_optimizer_hash", "outer_model_hash"):
        assert saved[f"{k}_save"] == resumed[f"{k}_resume"], k
    lf = {x["step"]: x for x in full if "Loss" in x}
    lr_ = {x["step"]: x for x in res if "Loss" in x}
    assert sorted(lr_) == [5, 6, 7, 8]
    for s in lr_:
        assert abs(lf[s]["Loss"] - lr_[s]["Loss"]) < 1e-3
        assert lf[s]["inner_lr"] == lr_[s]["inner_lr"] and lf[s]["total_tokens"] == lr_[s]["total_tokens"]


def test_late_joiner_recovers_from_sidecar_and_enters_with_zero_pseudo_gradient(tmp_path):
    """Two workers train with a checkpoint staged at every outer step; a third starts later with
    ``--ckpt.live_recovery_url auto``: it downloads the newest staged checkpoint from worker 0's sidecar while the
    members keep training, skips the inner steps of that outer iteration, contributes a zero pseudo-gradient, and
    from that outer step on holds the same outer model and optimizer state as the members."""
    import time
    ports = get_random_available_port_list(5)
    total = 24
    common = ["@configs/debug/diloco.toml", "--optim.total_steps", str(total), "--diloco.inner_steps", "2", "--train.micro_bs", "4",
              "--optim.batch_size", "8", "--train.log_model_hash", "--data.seq_length", "128", "--ckpt.interval", "2", "--ckpt.topk", "2"]
    genv = {"GLOBAL_ADDR": "127.0.0.1", "GLOBAL_PORT": str(ports[0]), "GLOBAL_WORLD_SIZE": "2",
            "ZERO_BAND_GLOBAL_PG_TIMEOUT_SECONDS": "120", "PRIME_B200_CKPT_STAGING": str(tmp_path / "shm")}
    procs, logs = [], []

    def start(uid, grank, port, extra):
        env = _local_env(0, 1, port)
        env.update(genv)
        env.update({"GLOBAL_UNIQUE_ID": uid, "GLOBAL_RANK": str(grank)})
        log = tmp_path / f"join_{uid}.log"
        logs.append(log)
        argv = common + ["--project", str(tmp_path / f"join_{uid}.pkl"), "--ckpt.path", str(tmp_path / f"ck_{uid}"),
                         "--data.data_rank", str(min(grank, 2)), "--data.data_world_size", "3"] + extra
        procs.append(_launch(argv, env, log))

    for w in range(2):
        start(str(w), w, ports[1 + w], [])
    deadline = time.time() + 240
    while "step: 4," not in (logs[0].read_text() if logs[0].exists() else ""):      # members are past their first saves
        assert time.time() < deadline and procs[0].poll() is None, logs[0].read_text()[-3000:]
        time.sleep(0.5)
    start("J", 100, ports[3], ["--ckpt.live_recovery_url", "auto"])
    for p, log in zip(procs, logs):
        try:
            rc = p.wait(timeout=600)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise AssertionError(f"timeout; log tail:\n{log.read_text()[-3000:]}")
        assert rc == 0, f"{log}:\n{log.read_text()[-3000:]}"
    m0, m1, mj = [pickle.load(open(tmp_path / f"join_{u}.pkl", "rb")) for u in ("0", "1", "J")]
    outer = lambda m: {x["step"]: x for x in m if "outer_model_hash_outer_step" in x}  # noqa: E731
    o0, o1, oj = outer(m0), outer(m1), outer(mj)
    assert oj, "the joiner never took part in an outer step"
    first = min(oj)
    assert first > 4 and first % 2 == 0
    # the joiner ran no inner step before its first outer step ...
    assert min(x["step"] for x in mj if "Loss" in x) == first + 1
    # ... and from that outer step on everyone holds the same outer model / momentum and the same inner model
    for s in sorted(oj):
        for k in ("outer_model_hash_outer_step", "outer_optimizer_hash_outer_step", "inner_model_hash_outer_step"):
            assert oj[s][k] == o0[s][k] == o1[s][k], (s, k)
    peers = {x["step"]: x["num_peers"] for x in m0 if "num_peers" in x}
    assert peers[first + 1] == 3 and peers[1] == 2
    assert max(x["step"] for x in mj if "Loss" in x) == total
