"""ElasticDeviceMesh: a fixed intra-worker group plus a worker group that grows and shrinks while
training runs (reference: src/zeroband/comms.py:32-609).

Topology is the reference's: one launcher (torchrun) per DiLoCo worker; inside a worker the default
process group carries ZeRO-3; across workers, rank ``r`` of every worker forms its own group (one
store per local rank on the leader), so only ranks that hold the same shard ever talk.

The store protocol is kept key for key, because it is the observable behaviour of the mesh:
``status`` in {init, running, reinit}, ``world_size``, ``mesh_count``, ``rank_{uid}``, ``gid_{rank}``,
``joiner_{i}`` (null-terminated queue), ``heartbeat_{uid}`` (wall time, or -100 as a deathrattle),
``barrier_{rank}``, ``resolved_time``, ``ping_{a}_{b}`` and ``iperf_{uid}`` (on the leader's local-rank-0
store), ``live_recovery/rank_{r}``; process-group rendezvous happens under ``mesh_{mesh_count}/``.

What differs, deliberately:
  * the data plane of the worker group is this package's C++ TCP ring (or NVLink peer kernels for
    workers inside one box), not gloo; a gloo group on the same store remains for barriers and for
    object / tensor point-to-point (live recovery);
  * heartbeats come from a daemon thread with its own store connection, so a killed process stops
    beating immediately (the reference forks a child process that can outlive its parent);
  * eviction after a failed monitored barrier works on unique ids (the reference mixes ranks and
    ids, so it never evicts anyone);
  * non-leaders wait for the leader with a timeout instead of forever;
  * link bandwidth is probed with an in-process TCP sink instead of the `iperf` binary, and the ring
    order is solved in-process (exact for up to 9 workers, 2-opt beyond).
"""
from __future__ import annotations

import itertools
import os
import socket
import threading
import time
from datetime import timedelta
from typing import List, Optional
from uuid import uuid4

import torch
import torch.distributed as dist
from torch.distributed.device_mesh import init_device_mesh

from .collectives import TcpRing, _my_ip
from .config import Compression
from .utils.logger import get_logger
from .utils.world_info import get_world_info


def _env_int(name: str, default: str) -> int:
    return int(os.getenv(name, default))


TCPSTORE_TIMEOUT = timedelta(seconds=_env_int("ZERO_BAND_GLOBAL_STORE_TIMEOUT_SECONDS", "300"))
TCPSTORE_POLLING_INTERVAL = float(os.getenv("ZERO_BAND_GLOBAL_STORE_POLLING_INTERVAL_SECONDS", "0.1"))
GLOBAL_PG_TIMEOUT = timedelta(seconds=_env_int("ZERO_BAND_GLOBAL_PG_TIMEOUT_SECONDS", "600"))
MAX_JOINERS = 100
HEARTBEAT_INTERVAL = float(os.getenv("ZERO_BAND_EDM_HEARTBEAT_INTERVAL_SECONDS", "2"))
HEARTBEAT_TIMEOUT = float(os.getenv("ZERO_BAND_EDM_HEARTBEAT_TIMEOUT_SECONDS", "10"))
IPERF_PORT = _env_int("ZERO_BAND_IPERF_PORT", "10101")
PING_UNKNOWN = 1_000_000_000


# ---------------------------------------------------------------------------------------------
# worker-group objects
# ---------------------------------------------------------------------------------------------
class _DoneWork:
    def wait(self, *a, **k):
        return True


class SingleWorkerGroup:
    """Placeholder worker group of size 1 (DiLoCo disabled, or a lone worker)."""

    def __init__(self, rank: int = 0):
        self._rank = rank

    def size(self) -> int:
        return 1

    def rank(self) -> int:
        return 0

    def barrier(self):
        return _DoneWork()

    def all_reduce_tensor(self, tensor, compression=Compression.NO, average=False):
        return None


class WorkerGroup:
    """The resizable cross-worker group: a gloo group for control / point-to-point plus the TCP ring
    for the pseudo-gradient payload."""

    def __init__(self, store, rank: int, world: int, timeout: timedelta, host: str | None, nconn: int = 4):
        self._rank, self._world = rank, world
        self.pg = dist.ProcessGroupGloo(store, rank, world, timeout)
        self.ring = TcpRing(dist.PrefixStore("ring", store), rank, world, host=host, nconn=nconn,
                            timeout_s=max(5.0, timeout.total_seconds()))

    def size(self) -> int:
        return self._world

    def rank(self) -> int:
        return self._rank

    def barrier(self):
        return self.pg.barrier()

    def all_reduce_tensor(self, tensor: torch.Tensor, compression: Compression = Compression.NO, average: bool = False) -> None:
        self.ring.all_reduce(tensor, compression, average)

    def allreduce(self, tensors, *a, **k):
        return self.pg.allreduce(tensors, *a, **k)

    def send(self, tensors, dst: int, tag: int = 0):
        return self.pg.send(tensors, dst, tag)

    def recv(self, tensors, src: int, tag: int = 0):
        return self.pg.recv(tensors, src, tag)

    def close(self):
        self.ring.close()


# ---------------------------------------------------------------------------------------------
# ring ordering
# ---------------------------------------------------------------------------------------------
def solve_ring_order(cost: List[List[int]]) -> tuple[int, List[int]]:
    """Cheapest Hamiltonian cycle through all workers starting at 0 (``cost[i][j]`` = time to push a
    fixed payload from i to j). Returns (cycle cost, path with the start repeated at the end)."""
    n = len(cost)
    if n <= 2:
        path = list(range(n)) + [0]
        return sum(cost[a][b] for a, b in zip(path, path[1:])), path
    if n <= 9:
        best, best_path = None, None
        for perm in itertools.permutations(range(1, n)):
            path = (0,) + perm + (0,)
            c = sum(cost[a][b] for a, b in zip(path, path[1:]))
            if best is None or c < best:
                best, best_path = c, list(path)
        return best, best_path
    left, path = set(range(1, n)), [0]
    while left:
        nxt = min(left, key=lambda j: cost[path[-1]][j])
        left.remove(nxt)
        path.append(nxt)
    improved = True
    while improved:
        improved = False
        for i in range(1, n - 1):
            for j in range(i + 1, n):
                cand = path[:i] + path[i:j + 1][::-1] + path[j + 1:]
                old = sum(cost[a][b] for a, b in zip(path + [0], (path + [0])[1:]))
                new = sum(cost[a][b] for a, b in zip(cand + [0], (cand + [0])[1:]))
                if new < old:
                    path, improved = cand, True
    path = path + [0]
    return sum(cost[a][b] for a, b in zip(path, path[1:])), path


class _BandwidthSink(threading.Thread):
    """Accepts connections and discards whatever arrives (the target of the peers' probes)."""

    def __init__(self, port: int):
        super().__init__(daemon=True)
        self.sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self.sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        try:
            self.sock.bind(("", port))
        except OSError:
            self.sock.bind(("", 0))
        self.port = self.sock.getsockname()[1]
        self.sock.listen(64)
        self._stop = threading.Event()

    def run(self):
        self.sock.settimeout(0.5)
        while not self._stop.is_set():
            try:
                conn, _ = self.sock.accept()
            except (socket.timeout, OSError):
                continue
            threading.Thread(target=self._drain, args=(conn,), daemon=True).start()

    @staticmethod
    def _drain(conn):
        conn.settimeout(5.0)
        try:
            while conn.recv(1 << 20):
                pass
        except OSError:
            pass
        finally:
            conn.close()

    def stop(self):
        self._stop.set()
        try:
            self.sock.close()
        except OSError:
            pass


def probe_bits_per_second(host: str, port: int, seconds: float = 0.25) -> float:
    """Push bytes to a peer's sink for ``seconds`` and return the achieved bits/s (0 on failure)."""
    buf = b"\x01" * (1 << 20)
    try:
        with socket.create_connection((host, port), timeout=3.0) as s:
            s.settimeout(3.0)
            sent, t0 = 0, time.perf_counter()
            while time.perf_counter() - t0 < seconds:
                sent += s.send(buf)
            dt = time.perf_counter() - t0
        return sent * 8 / dt if dt > 0 else 0.0
    except OSError:
        return 0.0


# ---------------------------------------------------------------------------------------------
# the mesh
# ---------------------------------------------------------------------------------------------
class ElasticDeviceMesh:
    """See module docstring. Attributes: ``global_pg`` (worker group), ``local_pg``, ``mesh``,
    ``cuda_local_mesh``, ``cpu_local_mesh``, ``live_recovery``, ``mesh_count``."""

    def __init__(self, backend: str = "cpu:gloo,cuda:nccl", enable: bool = True, live_recovery_rank_src: int | None = None):
        self._logger = get_logger()
        self.world_info = get_world_info()
        self.live_recovery_rank_src = live_recovery_rank_src
        # runtime knobs are read when the mesh is built (not at import), so a launcher can set them late
        self.store_timeout = timedelta(seconds=_env_int("ZERO_BAND_GLOBAL_STORE_TIMEOUT_SECONDS", "300"))
        self.polling_interval = float(os.getenv("ZERO_BAND_GLOBAL_STORE_POLLING_INTERVAL_SECONDS", "0.1"))
        self.pg_timeout = timedelta(seconds=_env_int("ZERO_BAND_GLOBAL_PG_TIMEOUT_SECONDS", "600"))
        self.heartbeat_interval = float(os.getenv("ZERO_BAND_EDM_HEARTBEAT_INTERVAL_SECONDS", "2"))
        self.heartbeat_timeout = float(os.getenv("ZERO_BAND_EDM_HEARTBEAT_TIMEOUT_SECONDS", "10"))
        self.global_pg = SingleWorkerGroup(self.world_info.rank)
        self.mesh_count = 0
        self._in_job = self.world_info.workers_in_job > 1
        if self._in_job:
            self._init_workers_in_job(backend, enable)
            return
        if enable and self.world_info.global_addr is None:
            self._logger.warning("DiLoCo is enabled but GLOBAL_ADDR / GLOBAL_PORT are not set: running as a single worker")
            enable = False
        self.enable = enable
        self.live_recovery = _NullLiveRecovery()
        self._heartbeat_thread: threading.Thread | None = None
        self._sink: _BandwidthSink | None = None
        if enable:
            self._init_global_pg()
        # intra-worker group
        if not dist.is_initialized():
            if not torch.cuda.is_available():
                backend = "gloo"
            dist.init_process_group(backend=backend)
        dev_type = "cuda" if torch.cuda.is_available() and "nccl" in dist.get_backend() else "cpu"
        self.mesh = init_device_mesh(dev_type, (self.world_info.nnodes, self.world_info.local_world_size),
                                     mesh_dim_names=("internode", "intranode"))
        self.local_pg = self.mesh.get_group("intranode")
        self.cuda_local_mesh = init_device_mesh(dev_type, mesh_shape=(self.local_pg.size(),))
        self.cpu_local_mesh = init_device_mesh("cpu", mesh_shape=(self.local_pg.size(),))
        if self.enable:
            self._optimize_ring_ranks()
            if self.live_recovery_rank_src is not None:
                self.live_recovery.ask_for_live_ckpt(self.live_recovery_rank_src)
            self.global_pg.barrier().wait()
            self._logger.info(f"global_pg size : {self.global_pg.size()}, local_pg size: {self.local_pg.size()}")

    # ------------------------------------------------------------------ several workers inside one launcher
    def _init_workers_in_job(self, backend: str, enable: bool) -> None:
        """Static worker layout inside one job on one NVSwitch domain: sub-groups of the job's NCCL
        group; the worker group runs on this package's NVLink kernels. Membership never changes in
        this mode (elastic join / leave is the TCP worker group's job)."""
        wi = self.world_info
        self.enable = False                      # no stores, no heartbeat; the methods below become no-ops
        self.live_recovery = _NullLiveRecovery()
        self._heartbeat_thread = None
        self._sink = None
        if not dist.is_initialized():
            dist.init_process_group(backend="nccl", device_id=torch.device("cuda", wi.device_index))
        k, per = wi.workers_in_job, wi.local_world_size
        self.local_pg = None
        for w in range(k):
            g = dist.new_group([w * per + r for r in range(per)])
            if w == wi.global_rank:
                self.local_pg = g
        self._worker_pg = None
        for r in range(per):
            g = dist.new_group([w * per + r for w in range(k)])
            if r == wi.local_rank:
                self._worker_pg = g
        from torch.distributed.device_mesh import DeviceMesh
        mine = [wi.global_rank * per + r for r in range(per)]
        self.mesh = self.cuda_local_mesh = DeviceMesh.from_group(self.local_pg, "cuda", torch.tensor(mine))
        self.cpu_local_mesh = None
        if enable:
            from .parallel.diloco_comm import NvlinkWorkerGroup
            from .parallel.symm import SymmComm
            self.global_pg = NvlinkWorkerGroup(SymmComm(self._worker_pg, torch.device("cuda", wi.device_index)), 1 << 20)
        self.mesh_count = 0
        self._logger.info(f"workers-in-job mesh: worker {wi.global_rank}/{k}, shard rank {wi.local_rank}/{per}")

    # ------------------------------------------------------------------ teardown
    def close(self, destroy_local: bool = True):
        """Leave the mesh cleanly: deathrattle, stop helper threads, drop the groups."""
        self._stop_heartbeat()
        if self._sink is not None:
            self._sink.stop()
            self._sink = None
        if isinstance(self.global_pg, WorkerGroup):
            self.global_pg.close()
        if destroy_local and dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:  # noqa: BLE001
                pass

    def __del__(self):
        try:
            self._stop_heartbeat()
        except Exception:  # noqa: BLE001
            pass

    # ------------------------------------------------------------------ stores
    def _init_global_store(self):
        wi = self.world_info
        self._logger.info(f"[{wi.global_unique_id}](Leader: {self._global_leader}) TCPStore init: Connecting via "
                          f"{wi.global_addr}:{wi.global_port + wi.rank}")
        self.global_store = dist.TCPStore(host_name=wi.global_addr, port=wi.global_port + wi.rank, timeout=self.store_timeout,
                                          is_master=self._global_leader, wait_for_workers=False)
        # the leader's local-rank-0 store doubles as the box-wide notice board (pings, sink addresses)
        if wi.rank == 0:
            self.god_store = self.global_store
        else:
            self.god_store = dist.TCPStore(host_name=wi.global_addr, port=wi.global_port, timeout=self.store_timeout,
                                           is_master=False, wait_for_workers=False)

    def _get(self, key: str) -> str:
        return self.global_store.get(key).decode("utf-8")

    def _init_global_store_values(self):
        wi = self.world_info
        self.global_store.set(f"gid_{wi.global_rank}", wi.global_unique_id)
        self.global_store.set(f"rank_{wi.global_unique_id}", str(wi.global_rank))
        if self._global_leader:
            self.global_store.set("mesh_count", "0")
            self.global_store.set("world_size", str(wi.global_world_size))
            self.global_store.set("joiner_0", "null")
            for i in range(wi.global_world_size):
                self.global_store.set(f"barrier_{i}", "null")
            self._global_ids = [self._get(f"gid_{i}") for i in range(wi.global_world_size)]
            for a in self._global_ids:
                for b in self._global_ids:
                    self.god_store.set(f"ping_{a}_{b}", str(PING_UNKNOWN))
            self.global_store.set("status", "init")
            self.global_status = "init"
        else:
            self.global_status = self._wait_for_status()
            if self.global_status != "running":
                self._global_ids = [self._get(f"gid_{i}") for i in range(wi.global_world_size)]

    def _wait_for_status(self, status: Optional[str] = None) -> str:
        deadline = time.monotonic() + self.store_timeout.total_seconds()
        while True:
            try:
                ret = self._get("status")
                if status is None or ret == status:
                    return ret
            except Exception:  # noqa: BLE001  key not there yet
                if status is not None:
                    raise
            if time.monotonic() > deadline:
                raise TimeoutError(f"status never became {status!r}")
            time.sleep(self.polling_interval)

    # ------------------------------------------------------------------ group creation
    def _create_global_pg(self):
        wi = self.world_info
        if isinstance(getattr(self, "global_pg", None), WorkerGroup):
            self.global_pg.close()
        self.global_pg = None
        wi.global_rank = int(self._get(f"rank_{wi.global_unique_id}"))
        wi.global_world_size = int(self._get("world_size"))
        self.mesh_count = int(self._get("mesh_count"))
        self._logger.debug(f"New global rank: {wi.global_rank}, New global world size: {wi.global_world_size} "
                           f"New mesh count: {self.mesh_count}")
        prefix_store = dist.PrefixStore(f"mesh_{self.mesh_count}", self.global_store)
        host = "127.0.0.1" if wi.global_addr in ("localhost", "127.0.0.1") else _my_ip()
        self.global_pg = WorkerGroup(prefix_store, wi.global_rank, wi.global_world_size, self.pg_timeout, host)
        self._logger.debug("Global pg created with %d peers. Timeout of %s", self.global_pg.size(), self.pg_timeout)

    def _local_barrier(self):
        if dist.is_initialized() and getattr(self, "local_pg", None) is not None:
            dist.barrier(self.local_pg)

    def _optimize_ring_ranks(self):
        wi = self.world_info
        self._global_ids = [self._get(f"gid_{i}") for i in range(wi.global_world_size)]
        if wi.local_rank == 0:
            self._measure_connectivity()
        self._local_barrier()
        self.global_pg.barrier().wait()
        if self._global_leader:
            pings = self.get_pings()
            min_dist, path = solve_ring_order(pings)
            self._logger.debug(f"Ring order cost {min_dist}, path {path}")
            new_gids = [self._global_ids[i] for i in path[:-1]]
            assert set(new_gids) == set(self._global_ids)
            for i, gid in enumerate(new_gids):
                self.global_store.set(f"rank_{gid}", str(i))
                self.global_store.set(f"gid_{i}", gid)
            self.global_store.set("mesh_count", str(self.mesh_count + 1))
        self._local_barrier()
        self.global_pg.barrier().wait()
        self._global_ids = [self._get(f"gid_{i}") for i in range(wi.global_world_size)]
        self._create_global_pg()

    # ------------------------------------------------------------------ join queue
    def _queue_join(self):
        for i in range(MAX_JOINERS):
            if self._get(f"joiner_{i}") == "null":
                self.global_store.set(f"joiner_{i}", self.world_info.global_unique_id)
                self.global_store.set(f"joiner_{i + 1}", "null")
                return
        raise RuntimeError("Too many joiners")

    def _get_joiners(self) -> List[str]:
        out = []
        for i in range(MAX_JOINERS):
            j = self._get(f"joiner_{i}")
            if j == "null":
                break
            out.append(j)
        return out

    def _clear_joiners(self):
        self.global_store.set("joiner_0", "null")

    # ------------------------------------------------------------------ init
    def _init_global_pg(self) -> None:
        t0 = time.perf_counter()
        wi = self.world_info
        self._global_leader = wi.global_rank == 0
        self._init_global_store()
        self._init_global_store_values()
        self.live_recovery = LiveRecovery(store=self.global_store)
        if self.global_status == "running":          # joiner path
            self._logger.info("Waiting to join")
            self._queue_join()
            self._wait_for_status("reinit")
        self._create_global_pg()
        if self._global_leader:
            self.global_store.set("status", "running")
            self._resolve_seq = 0
            self.global_store.set("resolved_time", f"0:{uuid4().hex}")
        self.global_status = "running"
        self._last_resolve_seq = self._resolution_seq(self._wait_key("resolved_time"))
        self._start_heartbeat()
        self._logger.info(f"Elastic Device mesh init done with {self.global_pg.size()} peers in {time.perf_counter() - t0} seconds")
        if wi.local_rank == 0:
            self._start_bandwidth_sink()
        self._evicted_nodes: list[str] = []

    @staticmethod
    def _resolution_seq(value: str) -> int:
        """Sequence number of a ``resolved_time`` value (``"<seq>:<uuid>"``)."""
        return int(value.split(":", 1)[0])

    def _wait_key(self, key: str) -> str:
        deadline = time.monotonic() + self.store_timeout.total_seconds()
        while True:
            try:
                return self._get(key)
            except Exception:  # noqa: BLE001
                if time.monotonic() > deadline:
                    raise
                time.sleep(self.polling_interval)

    # ------------------------------------------------------------------ heartbeat
    def _start_heartbeat(self):
        self._heartbeat_stop = threading.Event()
        wi = self.world_info
        uid, addr, port = wi.global_unique_id, wi.global_addr, wi.global_port + wi.rank
        store_timeout, interval = self.store_timeout, self.heartbeat_interval

        def loop(stop: threading.Event):
            try:
                store = dist.TCPStore(host_name=addr, port=port, timeout=store_timeout, is_master=False, wait_for_workers=False)
            except Exception:  # noqa: BLE001
                return
            while not stop.is_set():
                try:
                    store.set(f"heartbeat_{uid}", str(time.time()))
                except Exception:  # noqa: BLE001
                    pass
                stop.wait(interval)

        self._send_heartbeat()
        self._heartbeat_thread = threading.Thread(target=loop, args=(self._heartbeat_stop,), daemon=True)
        self._heartbeat_thread.start()

    def _stop_heartbeat(self, deathrattle: bool = True):
        if self._heartbeat_thread is not None:
            self._heartbeat_stop.set()
            self._heartbeat_thread.join(timeout=5)
            self._heartbeat_thread = None
            if deathrattle:
                self._send_deathrattle()

    def _send_heartbeat(self):
        try:
            self.global_store.set(f"heartbeat_{self.world_info.global_unique_id}", str(time.time()))
        except Exception:  # noqa: BLE001
            self._logger.error("Error sending heartbeat", exc_info=True)

    def _send_deathrattle(self):
        if hasattr(self, "global_store"):
            try:
                self.global_store.set(f"heartbeat_{self.world_info.global_unique_id}", "-100")
            except Exception:  # noqa: BLE001
                pass

    def _check_heartbeats(self) -> List[str]:
        dead, now = [], time.time()
        for gid in self._global_ids:
            try:
                if not self.global_store.check([f"heartbeat_{gid}"]):
                    self._logger.warning(f"Node {gid} has no heartbeat")
                    continue
                last = float(self._get(f"heartbeat_{gid}"))
                if now - last > self.heartbeat_timeout:
                    dead.append(gid)
                    self.global_store.delete_key(f"heartbeat_{gid}")
            except Exception:  # noqa: BLE001
                self._logger.warning(f"Node {gid} has no heartbeat")
        return dead

    # ------------------------------------------------------------------ world resolution
    def _resolve_world(self, admit_joiners: bool = False) -> bool:
        joiners = self._get_joiners() if admit_joiners else []
        dead = self._check_heartbeats()
        self._logger.debug("Joiners (%sadmitting): %s, Dead nodes: %s, Evicting nodes: %s", "" if admit_joiners else "not ",
                           joiners, dead, self._evicted_nodes)
        dead.extend(self._evicted_nodes)
        self._evicted_nodes = []
        if not joiners and not dead:
            return False
        leaving = set(dead)
        live = [g for g in self._global_ids if g not in leaving]
        for i, gid in enumerate(live):
            self.global_store.set(f"rank_{gid}", str(i))
            self.global_store.set(f"gid_{i}", gid)
        n = len(live)
        for j in joiners:
            if j in live:
                continue
            self.global_store.set(f"rank_{j}", str(n))
            self.global_store.set(f"gid_{n}", j)
            live.append(j)
            n += 1
        self._global_ids = live
        for a in live:
            for b in live:
                self.god_store.set(f"ping_{a}_{b}", str(PING_UNKNOWN))
        # barrier_0 too: a failed monitored barrier leaves "error" there, and the survivors' retry (same flag)
        # must not read that stale value
        for i in range(n):
            self.global_store.set(f"barrier_{i}", "null")
        self.global_store.set("world_size", str(n))
        self.global_store.set("mesh_count", str(self.mesh_count + 1))
        self.global_store.set("status", "reinit")
        return True

    def maybe_reinit_global_pg(self, admit_joiners: bool = False, _depth: int = 0) -> bool:
        """Resolve joins / departures; rebuild the worker group if membership changed."""
        if not self.enable:
            return False
        t0 = time.perf_counter()
        if self._global_leader:
            changed = self._resolve_world(admit_joiners=admit_joiners)
            if _depth > 0 and not changed:
                # a retry after a failed group creation with unchanged membership: move to a fresh store prefix, so that
                # nobody reads the rendezvous keys (addresses of sockets that are closed by now) the failed attempt left
                self.global_store.set("mesh_count", str(int(self._get("mesh_count")) + 1))
            self._resolve_seq += 1
            self.global_store.set("resolved_time", f"{self._resolve_seq}:{uuid4().hex}")
        else:
            # Resolutions are counted, not just noticed: the leader bumps the sequence number once per call and does
            # not wait for anyone when membership is unchanged, so it can be two calls ahead of a worker that was busy
            # (writing a checkpoint, say). A worker that only waited for "the value changed" would take both bumps for
            # one and then wait for a third that never comes. One resolution of the leader's lead is kept in credit.
            deadline = time.monotonic() + self.pg_timeout.total_seconds()
            while (seq := self._resolution_seq(self._get("resolved_time"))) <= self._last_resolve_seq:
                if time.monotonic() > deadline:
                    raise TimeoutError("the leader did not resolve the world in time")
                time.sleep(self.polling_interval)
            self._last_resolve_seq = max(self._last_resolve_seq + 1, seq - 1)
        self._logger.debug("World resolved in %s seconds", time.perf_counter() - t0)
        if self._get("status") == "running":
            return False
        try:
            self._create_global_pg()
            self._optimize_ring_ranks()
            self.global_pg.barrier().wait()
        except Exception as e:  # noqa: BLE001
            self._logger.error(f"Error recreating process group: {e}. Retrying...")
            if _depth >= 8:
                raise
            return self.maybe_reinit_global_pg(admit_joiners=admit_joiners, _depth=_depth + 1)
        if self._global_leader:
            self._clear_joiners()
            self.global_store.set("status", "running")
        self._stop_heartbeat(deathrattle=False)
        self._start_heartbeat()
        return True

    def get_global_pg(self, maybe_reinit: bool = False):
        if maybe_reinit:
            self.maybe_reinit_global_pg()
        return self.global_pg

    # ------------------------------------------------------------------ monitored barrier
    def monitored_barrier(self, flag: str):
        """Store-based barrier across the worker group. The leader waits up to the group timeout for
        everyone; workers that did not arrive are remembered for eviction at the next resolution and
        the barrier fails for all."""
        if not self.enable:
            if getattr(self, "_in_job", False):
                self.global_pg.barrier()
            return
        flag = str(flag)
        t0 = time.perf_counter()
        wi = self.world_info
        limit = self.pg_timeout.total_seconds()
        if self._global_leader:
            while True:
                late = [i for i in range(1, wi.global_world_size) if self._get(f"barrier_{i}") != flag]
                if not late:
                    break
                if time.perf_counter() - t0 > limit:
                    self._evicted_nodes = [self._get(f"gid_{i}") for i in late]
                    self._logger.error("Monitored barrier failed due to timeout; evicting %s", self._evicted_nodes)
                    self.global_store.set(f"barrier_{wi.global_rank}", "error")
                    raise RuntimeError("Monitored barrier failed due to timeout")
                time.sleep(self.polling_interval)
            self.global_store.set(f"barrier_{wi.global_rank}", flag)
        else:
            self.global_store.set(f"barrier_{wi.global_rank}", flag)
            while (ans := self._get("barrier_0")) != flag:
                if ans == "error":
                    raise RuntimeError("Monitored barrier failed due to error")
                if time.perf_counter() - t0 > 2 * limit:
                    raise RuntimeError("Monitored barrier failed: leader unreachable")
                time.sleep(self.polling_interval)
        self._logger.debug("Monitored barrier resolved in %s seconds", time.perf_counter() - t0)

    # ------------------------------------------------------------------ bandwidth probing
    def get_pings(self) -> List[List[int]]:
        n = self.world_info.global_world_size
        pings = [[PING_UNKNOWN] * n for _ in range(n)]
        for i, a in enumerate(self._global_ids):
            for j, b in enumerate(self._global_ids):
                if i != j:
                    try:
                        pings[i][j] = int(self.god_store.get(f"ping_{a}_{b}"))
                    except Exception:  # noqa: BLE001
                        pass
        return pings

    def _start_bandwidth_sink(self):
        if self._sink is not None:
            return
        self._sink = _BandwidthSink(IPERF_PORT + self.world_info.global_rank)
        self._sink.start()
        host = "127.0.0.1" if self.world_info.global_addr in ("localhost", "127.0.0.1") else _my_ip()
        self.god_store.set(f"iperf_{self.world_info.global_unique_id}", f"{host}:{self._sink.port}")

    def _measure_connectivity(self):
        me = self.world_info.global_unique_id
        for gid in self._global_ids:
            if gid == me:
                continue
            try:
                if not self.god_store.check([f"iperf_{gid}"]):
                    continue
                host, port = self.god_store.get(f"iperf_{gid}").decode().rsplit(":", 1)
                bps = probe_bits_per_second(host, int(port))
                cost = min(PING_UNKNOWN, int(1e13 / bps)) if bps > 0 else PING_UNKNOWN
                self.god_store.set(f"ping_{me}_{gid}", str(cost))
            except Exception:  # noqa: BLE001
                self._logger.debug("bandwidth probe to %s failed", gid)

    def measure_bandwidth(self) -> List[List[int]]:
        """Probe every peer's sink and return the current ping matrix (time to move 10 Tb, in s)."""
        self._measure_connectivity()
        return self.get_pings()


class _NullLiveRecovery:
    """Stand-in when there is no worker group (single worker)."""

    def reset(self):
        pass

    def should_send_ckpt_to(self):
        return None

    def ask_for_live_ckpt(self, rank: int):
        pass


class LiveRecovery:
    """Mailbox through which a joining worker asks a running one for a live checkpoint
    (reference: src/zeroband/comms.py:585-609)."""

    def __init__(self, store):
        self.store = dist.PrefixStore("live_recovery", store)
        self.world_info = get_world_info()

    def _key(self, rank: int) -> str:
        return f"rank_{rank}"

    def reset(self):
        self.store.set(self._key(self.world_info.global_rank), "null")

    def should_send_ckpt_to(self) -> int | None:
        """Rank of a joiner that asked this worker for a checkpoint, if any (polled once per outer step)."""
        try:
            if not self.store.check([self._key(self.world_info.global_rank)]):
                return None
            data = self.store.get(self._key(self.world_info.global_rank)).decode("utf-8")
        except Exception:  # noqa: BLE001
            return None
        if data == "null" or not data:
            return None
        try:
            return int(data)
        except ValueError:
            return None

    def ask_for_live_ckpt(self, rank: int):
        self.store.set(self._key(rank), str(self.world_info.global_rank))
