"""ElasticDeviceMesh on CPU ranks: static worker group, join, clean leave (deathrattle), killed
worker (heartbeat timeout), monitored-barrier eviction, ring-order solver."""
import multiprocessing as mp
import os
import signal
import time
import traceback

import pytest
import torch

from prime_b200.comms import solve_ring_order
from prime_b200.utils import get_random_available_port_list


def _env(uid, grank, gworld, gport, lport, extra=None):
    e = dict(WORLD_SIZE="1", RANK="0", LOCAL_RANK="0", LOCAL_WORLD_SIZE="1", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(lport),
             GLOBAL_UNIQUE_ID=uid, GLOBAL_ADDR="127.0.0.1", GLOBAL_PORT=str(gport), GLOBAL_WORLD_SIZE=str(gworld),
             GLOBAL_RANK=str(grank), ZERO_BAND_EDM_HEARTBEAT_INTERVAL_SECONDS="1", ZERO_BAND_EDM_HEARTBEAT_TIMEOUT_SECONDS="3",
             ZERO_BAND_GLOBAL_PG_TIMEOUT_SECONDS="6", ZERO_BAND_GLOBAL_STORE_TIMEOUT_SECONDS="30", ZERO_BAND_LOG_LEVEL="ERROR")
    e.update(extra or {})
    return e


def _run(target, env, q, *args):
    os.environ.update(env)
    try:
        q.put((env["GLOBAL_UNIQUE_ID"], target(*args)))
    except Exception:
        q.put((env["GLOBAL_UNIQUE_ID"], "ERR " + traceback.format_exc()))


def _allreduce_check(edm, value):
    from prime_b200.config import Compression
    t = torch.full((1000,), float(value))
    edm.global_pg.all_reduce_tensor(t, Compression.NO)
    return t[0].item()


def _finish(edm):
    """Leave together: the leader hosts the store, so it must be the last to go."""
    edm.global_pg.barrier().wait()
    if edm.world_info.global_rank == 0:
        time.sleep(1.5)
    edm.close()


# ---------------------------------------------------------------- scenarios (module level: spawn-picklable)
def _static_worker(value):
    from prime_b200.comms import ElasticDeviceMesh
    edm = ElasticDeviceMesh()
    out = (edm.global_pg.size(), edm.mesh_count, _allreduce_check(edm, value))
    edm.monitored_barrier("b0")
    assert edm.maybe_reinit_global_pg(admit_joiners=True) is False
    _finish(edm)
    return out


def _ramp_worker(role, ev_joined, ev_leave):
    from prime_b200.comms import ElasticDeviceMesh
    edm = ElasticDeviceMesh()
    log = []
    if role == "joiner":
        log.append(("joined", edm.global_pg.size(), edm.mesh_count))
        log.append(("sum", _allreduce_check(edm, 100)))
        edm.monitored_barrier("after_join")
        # phase 2: leader resolves (nothing changes) ; then this worker leaves cleanly
        edm.maybe_reinit_global_pg(admit_joiners=False)
        edm.close()
        return log
    log.append(("start", edm.global_pg.size(), edm.mesh_count))
    log.append(("sum", _allreduce_check(edm, 1)))
    changed = False
    for _ in range(120):                # poll like the training loop does at each outer step, until the joiner shows up
        changed = edm.maybe_reinit_global_pg(admit_joiners=True)
        if changed:
            break
        time.sleep(0.5)
    log.append(("after_join", changed, edm.global_pg.size(), edm.mesh_count))
    log.append(("sum", _allreduce_check(edm, 1)))
    edm.monitored_barrier("after_join")
    edm.maybe_reinit_global_pg(admit_joiners=False)
    changed = False
    for _ in range(120):                # ... and until its deathrattle is seen
        changed = edm.maybe_reinit_global_pg(admit_joiners=False)
        if changed:
            break
        time.sleep(0.5)
    log.append(("after_leave", changed, edm.global_pg.size(), edm.mesh_count))
    log.append(("sum", _allreduce_check(edm, 1)))
    _finish(edm)
    return log


def _kill_worker(role):
    from prime_b200.comms import ElasticDeviceMesh
    edm = ElasticDeviceMesh()
    if role == "victim":
        os.kill(os.getpid(), signal.SIGKILL)     # no deathrattle, no cleanup: heartbeats just stop
    time.sleep(5.0)                              # > heartbeat timeout
    changed = edm.maybe_reinit_global_pg(admit_joiners=False)
    out = (changed, edm.global_pg.size(), _allreduce_check(edm, 2))
    _finish(edm)
    return out


def _barrier_worker(role):
    from prime_b200.comms import ElasticDeviceMesh
    edm = ElasticDeviceMesh()
    failed = False
    if role == "late":
        time.sleep(9.0)                          # never reaches the barrier in time, but keeps beating
        edm._stop_heartbeat(deathrattle=False)
        return "late"
    try:
        edm.monitored_barrier("x")
    except RuntimeError:
        failed = True
    changed = edm.maybe_reinit_global_pg(admit_joiners=False)
    # the retry of the outer step: same flag again, now among the survivors, then the reduction itself
    edm.monitored_barrier("x")
    total = _allreduce_check(edm, 1 + edm.world_info.global_rank)
    out = (failed, changed, edm.global_pg.size(), total)
    _finish(edm)
    return out


def _collect(procs, q, n, timeout=120):
    out = {}
    for _ in range(n):
        k, v = q.get(timeout=timeout)
        out[k] = v
    for p in procs:
        p.join(timeout=20)
    for v in out.values():
        assert not (isinstance(v, str) and v.startswith("ERR")), v
    return out


def test_static_worker_group():
    ports = get_random_available_port_list(4)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_run, args=(_static_worker, _env(f"w{i}", i, 2, ports[0], ports[1 + i]), q, i + 1)) for i in range(2)]
    [p.start() for p in procs]
    out = _collect(procs, q, 2)
    for size, mesh_count, total in out.values():
        assert size == 2 and mesh_count == 1 and total == 3.0     # one re-mesh for the ring order


def test_on_ramp_then_off_ramp():
    ports = get_random_available_port_list(5)
    ctx = mp.get_context("spawn")
    q, ev_joined, ev_leave = ctx.Queue(), ctx.Event(), ctx.Event()
    procs = [ctx.Process(target=_run, args=(_ramp_worker, _env(f"w{i}", i, 2, ports[0], ports[1 + i]), q, "member", ev_joined, ev_leave))
             for i in range(2)]
    [p.start() for p in procs]
    time.sleep(8.0)     # members are up and running
    joiner = ctx.Process(target=_run, args=(_ramp_worker, _env("A", 100, 2, ports[0], ports[4]), q, "joiner", ev_joined, ev_leave))
    joiner.start()
    k, v = q.get(timeout=120)          # the joiner finishes first (it leaves)
    assert k == "A" and not (isinstance(v, str) and v.startswith("ERR")), v
    assert v[0][0] == "joined" and v[0][1] == 3 and v[1] == ("sum", 102.0)
    joiner.join(timeout=20)
    ev_leave.set()
    out = _collect(procs, q, 2)
    for log in out.values():
        assert log[0][:2] == ("start", 2) and log[1] == ("sum", 2.0)
        assert log[2][0] == "after_join" and log[2][1] is True and log[2][2] == 3
        assert log[3] == ("sum", 102.0)
        assert log[4][0] == "after_leave" and log[4][1] is True and log[4][2] == 2
        assert log[5] == ("sum", 2.0)
        assert log[4][3] > log[2][3] > log[0][2]        # mesh_count grows with every re-mesh


def test_killed_worker_is_detected_by_heartbeat_timeout():
    ports = get_random_available_port_list(5)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    roles = ["member", "member", "victim"]
    procs = [ctx.Process(target=_run, args=(_kill_worker, _env(f"w{i}", i, 3, ports[0], ports[1 + i]), q, roles[i])) for i in range(3)]
    [p.start() for p in procs]
    out = _collect(procs[:2], q, 2)
    procs[2].join(timeout=10)
    for changed, size, total in out.values():
        assert changed is True and size == 2 and total == 4.0


def test_monitored_barrier_evicts_late_worker():
    ports = get_random_available_port_list(5)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    roles = ["member", "member", "late"]
    procs = [ctx.Process(target=_run, args=(_barrier_worker, _env(f"w{i}", i, 3, ports[0], ports[1 + i]), q, roles[i])) for i in range(3)]
    [p.start() for p in procs]
    out = _collect(procs, q, 3)
    for uid in ("w0", "w1"):
        failed, changed, size, total = out[uid]
        assert failed is True and changed is True and size == 2 and total == 3.0


def test_ring_order_solver():
    cost = [[0, 1, 9, 9], [9, 0, 1, 9], [9, 9, 0, 1], [1, 9, 9, 0]]
    c, path = solve_ring_order(cost)
    assert c == 4 and path == [0, 1, 2, 3, 0]
    import random
    rng = random.Random(0)
    n = 12
    big = [[0 if i == j else rng.randint(1, 100) for j in range(n)] for i in range(n)]
    c, path = solve_ring_order(big)
    assert sorted(path[:-1]) == list(range(n)) and path[0] == path[-1] == 0
