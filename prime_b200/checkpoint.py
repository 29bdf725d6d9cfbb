"""Checkpointing: distributed checkpoint (DCP) of model / optimizer / scheduler / progress, per-rank
sidecar files for the outer optimizer and the dataloader, RAM-staged asynchronous persistence,
top-k retention, remote push and live recovery for joining workers
(reference: src/zeroband/checkpoint.py:46-563).

On-disk layout (unchanged, so checkpoints interchange and the HF exporter works)::

    {ckpt.path}/step_{N}/.metadata, __{rank}_{i}.distcp ... dcp.save({"model","optimizer","scheduler","training_progress"})
    {ckpt.path}/step_{N}/__{local_rank}_0.pt                {"optimizer": outer SGD state, local tensors}
    {ckpt.path}/step_{N}/data/_{local_rank}.pt              {"data_loader": dataloader.state_dict()}
    {ckpt.remote.path}/step_{N}/...                         copy of the above
    {ckpt.remote_data_path}/data_{data_rank}/{step_N,latest}/_{r}.pt

What is built here that the reference only describes in its README (lines 12-19):
  * ``save`` writes into a RAM-backed staging directory (``/dev/shm``) so the training loop is blocked
    only for the in-memory write; background processes then copy the step directory to
    ``ckpt.path`` and to the remote, and prune old steps;
  * every worker runs a small HTTP sidecar over its newest staged checkpoint; a joining worker
    downloads it (``download_live_ckpt``), loads it, skips the inner steps and enters the next outer
    step with a zero pseudo-gradient. Address / port come from ``ZERO_BAND_LIVE_RECO_ADDR`` /
    ``ZERO_BAND_LIVE_RECO_PORT``.
The reference's point-to-point transfer over the worker group (``send_ckpt_to_peer`` /
``recv_ckpt_from_peer``) is kept as well; after it, both the inner shards and the host-side outer
copy equal the sender's outer parameters (the reference leaves the outer copy stale).
"""
from __future__ import annotations

import functools
import http.server
import json
import logging
import multiprocessing
import os
import shutil
import threading
import time
import urllib.request
import uuid
import warnings
from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp
from torch.distributed.checkpoint.stateful import Stateful

from .config import CkptConfig
from .utils.logger import get_logger
from .utils.state_dict_send_recv import recv_state_dict, send_state_dict, send_tensor_and_state_dict
from .utils.world_info import get_world_info

SHM_ROOT = os.environ.get("PRIME_B200_CKPT_STAGING", "/dev/shm/prime_b200_ckpt")


@dataclass
class TrainingProgress(Stateful):
    total_tokens: int
    outer_step: int
    step: int

    def state_dict(self) -> dict[str, Any]:
        return {"total_tokens": self.total_tokens, "outer_step": self.outer_step, "step": self.step}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        self.total_tokens = state_dict["total_tokens"]
        self.outer_step = state_dict["outer_step"]
        self.step = state_dict["step"]


class ModelWrapper(Stateful):
    def __init__(self, backend) -> None:
        self.backend = backend

    def state_dict(self) -> dict[str, Any]:
        return self.backend.model_state_dict()

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        self.backend.load_model_state_dict(state_dict)


class OptimizerWrapper(Stateful):
    def __init__(self, backend) -> None:
        self.backend = backend

    def state_dict(self) -> dict[str, Any]:
        return self.backend.optimizer_state_dict()

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        self.backend.load_optimizer_state_dict(state_dict)


def cast_dtensor_to_tensor(state_dict: dict[str, Any]) -> dict[str, Any]:
    out = {}
    for k, v in state_dict.items():
        if isinstance(v, dict):
            out[k] = cast_dtensor_to_tensor(v)
        elif hasattr(v, "to_local"):
            out[k] = v.to_local()
        else:
            out[k] = v
    return out


class OuterOptimizerWrapper(Stateful):
    """State of the host-side outer SGD as plain local tensors."""

    def __init__(self, optimizer: torch.optim.Optimizer) -> None:
        self.optimizer = optimizer

    def state_dict(self) -> dict[str, Any]:
        return cast_dtensor_to_tensor(self.optimizer.state_dict())

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        # load values into existing momentum buffers when they exist (they may be views of a pinned
        # flat buffer); otherwise let torch create them
        params = [p for g in self.optimizer.param_groups for p in g["params"]]
        for idx, st in state_dict.get("state", {}).items():
            p = params[int(idx)]
            cur = self.optimizer.state[p]
            for k, v in st.items():
                if isinstance(v, torch.Tensor) and isinstance(cur.get(k), torch.Tensor):
                    cur[k].copy_(v)
                else:
                    cur[k] = v.clone() if isinstance(v, torch.Tensor) else v
        for g_new, g in zip(state_dict.get("param_groups", []), self.optimizer.param_groups):
            for k, v in g_new.items():
                if k != "params":
                    g[k] = v


def non_error_barrier(group=None):
    try:
        if dist.is_initialized():
            dist.barrier(group)
    except Exception as e:  # noqa: BLE001
        get_logger().info(f"Error in data checkpointing barrier: {e}, continuing training")


def get_checkpoints_to_delete(ckpt_path: str, topk: int) -> list[str]:
    """Step directories beyond the newest ``topk``."""
    if not os.path.isdir(ckpt_path):
        return []
    steps = []
    for d in os.listdir(ckpt_path):
        if d.startswith("step_"):
            try:
                steps.append((int(d.split("_")[1]), d))
            except ValueError:
                continue
    steps.sort()
    return [os.path.join(ckpt_path, d) for _, d in steps[:-topk]] if topk > 0 else []


def delete_topk(logger: logging.Logger, ckpt_path: str, topk: int) -> list[str]:
    gone = get_checkpoints_to_delete(ckpt_path, topk)
    for d in gone:
        shutil.rmtree(d, ignore_errors=True)
    if gone:
        logger.info(f"Deleted {gone}")
    return gone


# ---------------------------------------------------------------------------------------------
# background copy jobs (run in child processes)
# ---------------------------------------------------------------------------------------------
def _copy_tree(src: str, dst: str) -> None:
    """Copy a step directory; ``dst`` may be any fsspec URL."""
    if "://" not in dst:
        os.makedirs(os.path.dirname(dst) or ".", exist_ok=True)
        tmp = f"{dst}.partial.{os.getpid()}"      # unique per copier: two jobs never share a temporary tree
        shutil.rmtree(tmp, ignore_errors=True)
        shutil.copytree(src, tmp)
        shutil.rmtree(dst, ignore_errors=True)
        os.replace(tmp, dst)
        return
    import fsspec
    fs, root = fsspec.core.url_to_fs(dst)
    for base, _, files in os.walk(src):
        rel = os.path.relpath(base, src)
        fs.makedirs(os.path.join(root, rel) if rel != "." else root, exist_ok=True)
        for f in files:
            fs.put_file(os.path.join(base, f), os.path.join(root, rel, f) if rel != "." else os.path.join(root, f))


def _persist_job(src: str, dst: str, prune_root: str | None, topk: int | None) -> None:
    _copy_tree(src, dst)
    if prune_root is not None and topk is not None:
        delete_topk(logging.getLogger("prime_b200.ckpt"), prune_root, topk)


# ---------------------------------------------------------------------------------------------
# live-recovery sidecar
# ---------------------------------------------------------------------------------------------
class _SidecarHandler(http.server.SimpleHTTPRequestHandler):
    def log_message(self, *a):  # silence
        pass

    def do_GET(self):
        if self.path.endswith("?resolve=1"):
            # the real name behind a symlinked directory ("latest" -> "step_N"), so a client can pin one step
            real = os.path.basename(os.path.realpath(self.translate_path(self.path.split("?", 1)[0])))
            body = json.dumps(real).encode()
            self.send_response(200)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)
            return
        if self.path.endswith("?list=1"):
            root = self.translate_path(self.path.split("?", 1)[0])
            files = []
            for base, _, names in os.walk(root):
                for n in names:
                    files.append(os.path.relpath(os.path.join(base, n), root))
            body = json.dumps(sorted(files)).encode()
            self.send_response(200)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)
            return
        return super().do_GET()


class LiveRecoverySidecar:
    """Static-file HTTP server over the staging directory; ``/latest/`` is a symlink to the newest
    complete step. One per training process (port = base port + local rank)."""

    def __init__(self, root: str, host: str = "0.0.0.0", port: int = 0):
        os.makedirs(root, exist_ok=True)
        handler = functools.partial(_SidecarHandler, directory=root)
        self.httpd = http.server.ThreadingHTTPServer((host, port), handler)
        self.port = self.httpd.server_address[1]
        self.thread = threading.Thread(target=self.httpd.serve_forever, daemon=True)
        self.thread.start()

    def stop(self):
        self.httpd.shutdown()
        self.httpd.server_close()


def _default_sidecar_addr() -> str:
    """Address the sidecar binds when ZERO_BAND_LIVE_RECO_ADDR is unset: the interface the worker group talks over
    (loopback for single-host groups, the GLOO_SOCKET_IFNAME interface otherwise); every interface only as a last
    resort."""
    if os.environ.get("GLOBAL_ADDR", "127.0.0.1") in ("localhost", "127.0.0.1"):
        return "127.0.0.1"
    ifname = os.environ.get("GLOO_SOCKET_IFNAME")
    if ifname:
        try:
            from .utils.ip import get_ip_address
            return get_ip_address(ifname)
        except OSError:
            pass
    return "0.0.0.0"


def download_live_ckpt(url: str, destination: str) -> str:
    """Fetch a peer's newest staged checkpoint (``http://addr:port/latest/``) into ``destination``."""
    from .utils.wget import wget
    # pin the step behind ".../latest/" first: the link may move to a newer step while the files are being fetched
    base = url.rstrip("/")
    if base.endswith("/latest"):
        try:
            with urllib.request.urlopen(base + "/?resolve=1", timeout=60) as r:
                step = json.loads(r.read().decode())
            if isinstance(step, str) and step.startswith("step_"):
                url = base[: -len("latest")] + step + "/"
        except (OSError, ValueError):
            pass
    wget(url, destination)
    return destination


# ---------------------------------------------------------------------------------------------
# manager
# ---------------------------------------------------------------------------------------------
class CkptManager:
    """Saves / loads / ships the training state. ``backend`` is a training backend
    (:mod:`prime_b200.backend`); ``diloco`` (optional) provides ``param_list_cpu`` and
    ``outer_optimizer``."""

    states: dict[str, Stateful]

    def __init__(self, config: CkptConfig, backend, scheduler, dataloader, training_progress: TrainingProgress,
                 data_rank: int | None, diloco_offloaded_param_list: list | None = None,
                 diloco_offloaded_optimizer: torch.optim.Optimizer | None = None, diloco=None, use_staging: bool = True,
                 process_group=None, subdir: str | None = None):
        if subdir is not None and config.path is not None:      # several workers in one job: one tree per worker
            config = config.model_copy(update={"path": os.path.join(config.path, subdir)})
        self.process_group = process_group
        self.config = config
        self.backend, self.scheduler, self.dataloader = backend, scheduler, dataloader
        self.training_progress, self.data_rank = training_progress, data_rank
        assert (diloco_offloaded_param_list is None) == (diloco_offloaded_optimizer is None), \
            "diloco_offloaded_model and diloco_offloaded_optimizer must be both None or both have values"
        self.diloco = diloco
        self.diloco_offloaded_param_list = diloco_offloaded_param_list
        self.diloco_offloaded_optimizer = diloco_offloaded_optimizer
        self._init_state()
        self._logger = get_logger(config if hasattr(config, "log_level") else None)
        self.world_info = get_world_info()
        self.non_blocking_process: list[multiprocessing.Process] = []
        self.blocking_process: list[multiprocessing.Process] = []
        self._live_reco_thread: threading.Thread | None = None
        self._sidecar: LiveRecoverySidecar | None = None
        self.use_staging = use_staging and os.path.isdir("/dev/shm") and config.path is not None
        self._staging_root = os.path.join(SHM_ROOT, uuid.uuid5(uuid.NAMESPACE_URL, os.path.abspath(config.path)).hex) \
            if config.path is not None else None
        if self.world_info.local_rank == 0:
            for p in (config.path, config.remote.path if config.remote is not None else None, config.remote_data_path):
                if p is not None:
                    self.check_path_access(p)

    def check_path_access(self, ckpt_path: str) -> None:
        import fsspec
        probe = os.path.join(ckpt_path, f".dummy_file_{uuid.uuid4()}.txt")
        try:
            fs, _ = fsspec.core.url_to_fs(ckpt_path)
            fs.makedirs(ckpt_path, exist_ok=True)
            with fsspec.open(probe, "w") as f:
                f.write("This is a dummy file for testing access.")
            fs.rm(probe)
        except Exception as e:  # noqa: BLE001
            self._logger.error(f"Error checking path access {ckpt_path}: {e}, aborting training")
            raise

    def _init_state(self) -> None:
        self.states = {"model": ModelWrapper(self.backend), "optimizer": OptimizerWrapper(self.backend), "scheduler": self.scheduler,
                       "training_progress": self.training_progress}

    # ------------------------------------------------------------------ save
    @torch.no_grad()
    def save(self, remote: bool = False) -> None:
        """Write ``step_{step}``. With staging the call returns after the RAM write; persistence to
        ``ckpt.path`` (and the remote) continues in child processes."""
        step_dir = os.path.join(self.config.path, f"step_{self.training_progress.step}")
        remote_dir = os.path.join(self.config.remote.path, f"step_{self.training_progress.step}") \
            if (remote and self.config.remote is not None) else None
        t0 = time.perf_counter()
        write_dir = os.path.join(self._staging_root, f"step_{self.training_progress.step}") if self.use_staging else step_dir
        self._save(write_dir)
        self._logger.info(f"Saved checkpoint to {write_dir} in {time.perf_counter() - t0} seconds")
        non_error_barrier(self.process_group)
        if self.world_info.local_rank == 0:
            if self.use_staging:
                self._point_latest(write_dir)
                self._spawn(_persist_job, (write_dir, step_dir, self.config.path, self.config.topk), blocking=True)
                self._prune_staging(keep=os.path.basename(write_dir))
            elif self.config.topk is not None:
                delete_topk(self._logger, self.config.path, self.config.topk)
            if remote_dir is not None:
                self._async_save_remote(write_dir, remote_dir)

    def _spawn(self, fn, args, blocking: bool) -> None:
        ctx = multiprocessing.get_context("spawn")
        p = ctx.Process(target=fn, args=args, daemon=True)
        p.start()
        (self.blocking_process if blocking else self.non_blocking_process).append(p)

    def _point_latest(self, step_dir: str) -> None:
        link = os.path.join(self._staging_root, "latest")
        tmp = link + ".tmp"
        try:
            if os.path.lexists(tmp):
                os.remove(tmp)
            os.symlink(os.path.basename(step_dir), tmp)
            os.replace(tmp, link)
        except OSError:
            pass

    def _prune_staging(self, keep: str) -> None:
        """RAM is precious: keep only the newest staged step (older ones are on disk by now or are
        being copied from by a child that holds its files open)."""
        self.wait_for_copy_jobs(exclude_last=True)
        for d in os.listdir(self._staging_root):
            if d.startswith("step_") and d != keep:
                shutil.rmtree(os.path.join(self._staging_root, d), ignore_errors=True)

    @torch.no_grad()
    def _save(self, ckpt_path: str) -> None:
        self.wait_for_blocking_job()
        quiet = self._logger.getEffectiveLevel() >= logging.INFO
        with warnings.catch_warnings():
            if quiet:
                warnings.simplefilter("ignore")
            os.makedirs(ckpt_path, exist_ok=True)
            # several writer threads per rank (every parameter shard is an item of its own), and no fsync for files
            # that land in the in-memory staging directory: the blocking part of a save is this call
            staged = self.use_staging and ckpt_path.startswith(SHM_ROOT)
            writer = dcp.FileSystemWriter(ckpt_path, thread_count=max(1, int(os.environ.get("PRIME_B200_CKPT_WRITER_THREADS", "4"))),
                                          sync_files=not staged)
            dcp.save(self.states, storage_writer=writer, process_group=self.process_group)
            if self.diloco_offloaded_optimizer is not None:
                if self.diloco is not None:
                    self.diloco.wait_host_state()      # the host copy of the outer momentum may still be on its way
                with open(os.path.join(ckpt_path, f"__{self.world_info.local_rank}_0.pt"), "wb") as f:
                    torch.save({"optimizer": OuterOptimizerWrapper(self.diloco_offloaded_optimizer).state_dict()}, f)
            data_dir = os.path.join(ckpt_path, "data")
            self.save_data(data_dir, self.dataloader, self.world_info.local_rank)
            non_error_barrier(self.process_group)
            # after the barrier data_dir holds every local rank's file: one copier per destination, from local rank 0
            if self.config.remote_data_path is not None and self.world_info.local_rank == 0:
                base = os.path.join(self.config.remote_data_path, f"data_{self.data_rank}")
                for name in (f"step_{self.training_progress.step}", "latest"):
                    self._spawn(_copy_tree, (data_dir, os.path.join(base, name)), blocking=False)

    @staticmethod
    def save_data(data_path: str, dataloader, local_rank: int) -> None:
        os.makedirs(data_path, exist_ok=True)
        with open(os.path.join(data_path, f"_{local_rank}.pt"), "wb") as f:
            torch.save({"data_loader": dataloader.state_dict()}, f)

    def _async_save_remote(self, ckpt_path: str, remote_ckpt_path: str, blocking: bool = True) -> None:
        """Push a step directory to the remote without blocking training."""
        self._spawn(_copy_tree, (ckpt_path, remote_ckpt_path), blocking=blocking)

    def wait_for_copy_jobs(self, exclude_last: bool = False) -> None:
        jobs = self.blocking_process[:-1] if exclude_last else self.blocking_process
        for p in jobs:
            p.join()
        self.blocking_process = self.blocking_process[-1:] if exclude_last else []

    def wait_for_blocking_job(self) -> None:
        """Join the persistence jobs of the previous save (called before the next one and at exit)."""
        for p in self.blocking_process:
            p.join()
        self.blocking_process = []
        if self.world_info.local_rank == 0 and self.config.topk is not None and self.config.path is not None:
            delete_topk(self._logger, self.config.path, self.config.topk)

    def close(self) -> None:
        self.wait_for_blocking_job()
        for p in self.non_blocking_process:
            p.join(timeout=60)
        if self._sidecar is not None:
            self._sidecar.stop()
            self._sidecar = None
        # the staged copy lives in RAM (/dev/shm): once the persistence jobs have joined it is on disk, so free it
        if self.use_staging and self._staging_root is not None and self.world_info.local_rank == 0:
            shutil.rmtree(self._staging_root, ignore_errors=True)

    def __del__(self):
        try:
            self.wait_for_blocking_job()
        except Exception:  # noqa: BLE001
            pass

    # ------------------------------------------------------------------ load
    def _load_data(self, resume_ckpt_path: str) -> None:
        self._logger.debug(f"loading data from {resume_ckpt_path}")
        p = os.path.join(resume_ckpt_path, "data", f"_{self.world_info.local_rank}.pt")
        if not os.path.exists(p):
            p = os.path.join(resume_ckpt_path, f"_{self.world_info.local_rank}.pt")
        with open(p, "rb") as f:
            self.dataloader.load_state_dict(torch.load(f, weights_only=False)["data_loader"])

    @torch.no_grad()
    def load(self, resume_ckpt_path: str, skip_dataloader: bool = False, data_path: str | None = None) -> None:
        """Restore model / optimizer / scheduler / progress, re-derive the outer parameters from the
        inner ones, load the outer momentum and the dataloader position."""
        t0 = time.perf_counter()
        world_info = self.world_info
        files = os.listdir(resume_ckpt_path)
        if len(files) == 1 and files[0].startswith("diloco_"):      # legacy layout: one sub-folder
            resume_ckpt_path = os.path.join(resume_ckpt_path, files[0])
        dcp.load(self.states, checkpoint_id=resume_ckpt_path, process_group=self.process_group)
        if self.config.token_count is not None:
            self.training_progress.total_tokens = self.config.token_count
        self._logger.debug("sync inner model")
        if self.diloco is not None:
            self.diloco.set_outer_from_inner(self.backend)
        elif self.diloco_offloaded_param_list is not None:
            for p_off, (_, t) in zip(self.diloco_offloaded_param_list, self.backend.named_master_shards()):
                p_off.data.copy_(t)
        if self.diloco_offloaded_optimizer is not None:
            with open(os.path.join(resume_ckpt_path, f"__{world_info.local_rank}_0.pt"), "rb") as f:
                rank_state = torch.load(f, weights_only=True)     # tensors and plain values only
            OuterOptimizerWrapper(self.diloco_offloaded_optimizer).load_state_dict(rank_state["optimizer"])
            if self.diloco is not None:
                self.diloco.mark_host_state_written()
        if not skip_dataloader:
            if self.config.remote_data_load:
                self.remote_data_load()
            else:
                self._load_data(data_path if data_path is not None else resume_ckpt_path)
        self._init_state()
        self._logger.info(f"Loaded checkpoint from {resume_ckpt_path} in {time.perf_counter() - t0} seconds")

    def remote_data_load(self) -> None:
        import fsspec
        remote = os.path.join(self.config.remote_data_path, f"data_{self.data_rank}", "latest", f"_{self.world_info.local_rank}.pt")
        with fsspec.open(remote, "rb") as f:
            self.dataloader.load_state_dict(torch.load(f, weights_only=False)["data_loader"])

    # ------------------------------------------------------------------ live recovery: HTTP sidecar
    def start_sidecar(self) -> int | None:
        """Serve this worker's staged checkpoints; returns the port (None if staging is off)."""
        if not self.use_staging or self._sidecar is not None:
            return self._sidecar.port if self._sidecar is not None else None
        base = int(os.environ.get("ZERO_BAND_LIVE_RECO_PORT", "0"))
        port = base + self.world_info.local_rank if base else 0
        self._sidecar = LiveRecoverySidecar(self._staging_root, os.environ.get("ZERO_BAND_LIVE_RECO_ADDR", _default_sidecar_addr()), port)
        return self._sidecar.port

    def recover_from_sidecar(self, url: str, scratch_dir: str | None = None) -> None:
        """Joiner side: download ``url`` (a peer's ``.../latest/``) and load it (dataloader state excluded:
        the joiner reads its own data shard)."""
        scratch_dir = scratch_dir or os.path.join(SHM_ROOT, f"recv_{uuid.uuid4().hex}")
        try:
            download_live_ckpt(url, scratch_dir)
            self.load(scratch_dir, skip_dataloader=True)
        finally:
            shutil.rmtree(scratch_dir, ignore_errors=True)

    # ------------------------------------------------------------------ live recovery: point-to-point over the worker group
    @torch.no_grad()
    def recv_ckpt_from_peer(self, global_pg) -> None:
        assert self.diloco_offloaded_param_list is not None, "recv_ckpt_from_peers is only supported with diloco"
        t0 = time.perf_counter()
        src = self.config.live_recovery_rank_src
        self._logger.debug(f"Start receiving ckpt from rank {src}")
        if self.diloco is not None:
            self.diloco.wait_host_state()
        jobs, bufs = [], []
        for i, p in enumerate(self.diloco_offloaded_param_list):
            buf = torch.empty_like(p.data)
            bufs.append(buf)
            jobs.append(global_pg.recv([buf], src, i))
        for j in jobs:
            j.wait()
        # both copies take the sender's outer parameters: the host-side outer copy and the inner shards
        for p, buf, (_, shard) in zip(self.diloco_offloaded_param_list, bufs, self.backend.named_master_shards()):
            p.data.copy_(buf)
            shard.copy_(buf)
        self.backend.publish_params()
        self._logger.debug("live recovery progress: offloaded model received 1/5")
        outer = recv_state_dict(global_pg, src, OuterOptimizerWrapper(self.diloco_offloaded_optimizer).state_dict())
        OuterOptimizerWrapper(self.diloco_offloaded_optimizer).load_state_dict(outer)
        if self.diloco is not None:
            self.diloco.mark_host_state_written()
        self._logger.debug("live recovery progress: outer optimizer state dict received 2/5")
        self.training_progress.load_state_dict(recv_state_dict(global_pg, src, self.training_progress.state_dict()))
        self._logger.debug("live recovery progress: training progress state dict received 3/5")
        like = cast_dtensor_to_tensor(self.backend.optimizer_state_dict())
        got = recv_state_dict(global_pg, src, like)
        self._load_inner_optimizer_local(got)
        self._logger.debug("live recovery progress: inner optimizer state dict received 4/5")
        self.scheduler.load_state_dict(recv_state_dict(global_pg, src, self.scheduler.state_dict()))
        self._logger.debug(f"live recovery progress: scheduler state dict received 5/5; done in {time.perf_counter() - t0} seconds")

    def _load_inner_optimizer_local(self, flat_local: dict[str, Any]) -> None:
        cur = self.backend.optimizer_state_dict()
        for k, v in flat_local.items():
            tgt = cur.get(k)
            if isinstance(v, torch.Tensor) and isinstance(tgt, torch.Tensor):
                (tgt.to_local() if hasattr(tgt, "to_local") else tgt).copy_(v)
            else:
                cur[k] = v
        self.backend.load_optimizer_state_dict(cur)

    @torch.no_grad()
    def send_ckpt_to_peer(self, global_pg, dest_rank: int, blocking: bool = False) -> None:
        def _send():
            assert self.diloco_offloaded_param_list is not None, "send_ckpt_to_peer is only supported with diloco"
            t0 = time.perf_counter()
            self._logger.debug(f"Start sending ckpt to rank {dest_rank}")
            if self.diloco is not None:
                self.diloco.wait_host_state()
            try:
                jobs = [global_pg.send([p.data.contiguous()], dest_rank, i) for i, p in enumerate(self.diloco_offloaded_param_list)]
                for j in jobs:
                    j.wait()
                send_state_dict(global_pg, OuterOptimizerWrapper(self.diloco_offloaded_optimizer).state_dict(), dest_rank)
                send_state_dict(global_pg, self.training_progress.state_dict(), dest_rank)
                send_state_dict(global_pg, cast_dtensor_to_tensor(self.backend.optimizer_state_dict()), dest_rank)
                send_state_dict(global_pg, self.scheduler.state_dict(), dest_rank)
            except RuntimeError as e:
                self._logger.error(f"Error sending ckpt to rank {dest_rank}: {e}")
            else:
                self._logger.debug(f"Sent ckpt to rank {dest_rank} in {time.perf_counter() - t0} seconds")

        thread = threading.Thread(target=_send)
        thread.start()
        self._logger.debug("Live recovery thread started")
        if blocking:
            thread.join()
        else:
            self._live_reco_thread = thread
