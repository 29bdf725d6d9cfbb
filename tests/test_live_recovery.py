"""Live recovery on CPU: (a) a joiner downloads a running worker's staged checkpoint from its HTTP
sidecar and ends with identical state; (b) the point-to-point transfer over the worker group."""
import multiprocessing as mp
import os
import traceback

import pytest
import torch

from prime_b200.utils import get_random_available_port_list


def _mk_backend(seed):
    from prime_b200.backend import EagerBackend
    from prime_b200.lr_scheduler import get_scheduler
    from prime_b200.models.llama import ModelArgs, Transformer
    torch.manual_seed(seed)
    args = ModelArgs(dim=32, n_layers=1, n_heads=2, ffn_hidden=64, vocab_size=50, max_seq_len=16)
    model = Transformer(args)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
    sched = get_scheduler("cosine", opt, 2, 10, 20)
    return EagerBackend(model, opt, sched), args


class _DL:
    def __init__(self):
        self.pos = 0

    def state_dict(self):
        return {"pos": self.pos}

    def load_state_dict(self, sd):
        self.pos = sd["pos"]


def _train_a_bit(backend, args, steps=3):
    g = torch.Generator().manual_seed(0)
    for _ in range(steps):
        tok = torch.randint(0, args.vocab_size, (2, 17), generator=g)
        backend.train_step({"input_ids": tok[:, :-1], "labels": tok[:, 1:], "seq_start": None}, micro_bs=2)


def _env(uid, grank, gport, lport, staging):
    return dict(WORLD_SIZE="1", RANK="0", LOCAL_RANK="0", LOCAL_WORLD_SIZE="1", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(lport),
                GLOBAL_UNIQUE_ID=uid, GLOBAL_ADDR="127.0.0.1", GLOBAL_PORT=str(gport), GLOBAL_WORLD_SIZE="2", GLOBAL_RANK=str(grank),
                ZERO_BAND_GLOBAL_PG_TIMEOUT_SECONDS="60", ZERO_BAND_LOG_LEVEL="ERROR", PRIME_B200_CKPT_STAGING=staging)


def _sig(backend, diloco):
    from prime_b200 import utils
    return (utils.get_dict_signature({n: t for n, t in backend.named_master_shards()}),
            utils.get_tensor_list_signature([p.data for p in diloco.param_list_cpu]),
            utils.get_optimizer_signature(diloco.outer_optimizer))


def _worker(role, env, q, tmp, mode):
    os.environ.update(env)
    try:
        import torch.distributed as dist
        from prime_b200.checkpoint import CkptManager, TrainingProgress
        from prime_b200.comms import ElasticDeviceMesh
        from prime_b200.config import CkptConfig, DilocoConfig
        from prime_b200.diloco import Diloco
        edm = ElasticDeviceMesh()
        backend, args = _mk_backend(seed=1 if role == "src" else 2)
        diloco = Diloco(DilocoConfig(inner_steps=2), backend, edm)
        prog = TrainingProgress(0, 0, 0)
        cfg = CkptConfig(path=os.path.join(tmp, role), interval=2, live_recovery_rank_src=0 if role == "dst" else None)
        mgr = CkptManager(cfg, backend, backend.lr_scheduler, _DL(), prog, None, diloco.param_list_cpu, diloco.outer_optimizer, diloco=diloco)
        if role == "src":
            _train_a_bit(backend, args)
            diloco.outer_optimizer.step()               # momentum buffers exist
            diloco.set_outer_from_inner(backend)
            prog.step, prog.outer_step, prog.total_tokens = 6, 3, 1234
            if mode == "http":
                mgr.save()
                port = mgr.start_sidecar()
                edm.global_store.set("sidecar_port", str(port))
                edm.global_pg.barrier().wait()          # joiner has finished downloading
            else:
                edm.global_pg.barrier().wait()
                mgr.send_ckpt_to_peer(edm.global_pg, 1, blocking=True)
            out = (_sig(backend, diloco), prog.state_dict(), backend.lr_scheduler.state_dict()["last_epoch"])
        else:
            if mode == "http":
                port = int(edm.global_store.get("sidecar_port").decode())
                mgr.recover_from_sidecar(f"http://127.0.0.1:{port}/latest/")
                edm.global_pg.barrier().wait()
            else:
                diloco.outer_optimizer.step()
                edm.global_pg.barrier().wait()
                mgr.recv_ckpt_from_peer(edm.global_pg)
            out = (_sig(backend, diloco), prog.state_dict(), backend.lr_scheduler.state_dict()["last_epoch"])
        q.put((role, out))
        edm.global_pg.barrier().wait()
        import time
        if role == "src":
            time.sleep(1.0)
        mgr.close()
        edm.close()
    except Exception:
        q.put((role, "ERR " + traceback.format_exc()))


@pytest.mark.parametrize("mode", ["http", "p2p"])
def test_joiner_recovers_state_from_running_worker(tmp_path, mode):
    ports = get_random_available_port_list(3)
    staging = str(tmp_path / "shm")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_worker, args=(role, _env(role, i, ports[0], ports[1 + i], staging), q, str(tmp_path), mode))
          for i, role in enumerate(["src", "dst"])]
    [p.start() for p in ps]
    out = dict(q.get(timeout=180) for _ in ps)
    [p.join(timeout=30) for p in ps]
    for v in out.values():
        assert not (isinstance(v, str) and v.startswith("ERR")), v
    (sig_s, prog_s, ep_s), (sig_d, prog_d, ep_d) = out["src"], out["dst"]
    assert sig_s[0] == sig_d[0], "inner model"
    assert sig_s[1] == sig_d[1], "outer model"
    assert sig_s[2] == sig_d[2], "outer optimizer"
    assert prog_s == prog_d and ep_s == ep_d
