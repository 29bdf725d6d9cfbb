"""Training entry point: ``torchrun ... -m prime_b200.train @configs/150M/B200.toml --a.b value``
(reference: src/zeroband/train.py:79-567).

One launcher per DiLoCo worker; inside a worker the ranks form a ZeRO-3 group. The loop is the
reference's: outer iterations of ``diloco.inner_steps`` optimizer steps (1 without DiLoCo), each of
``batch_size / local_world / micro_bs`` micro-steps; metrics per inner and per outer step;
checkpoints only at outer-step boundaries; exit after ``optim.total_steps``.

On CUDA the model is the fused engine (hand-written kernels, symmetric-memory collectives) fed by the
GPU prefetcher; on CPU (gloo) it is the eager module — same loop, same checkpoints, same metrics.
"""
from __future__ import annotations

import os
import sys
import time
from functools import partial

import torch
import torch.distributed as dist

from . import utils
from .backend import EagerBackend, FusedBackend
from .checkpoint import CkptManager, TrainingProgress
from .comms import ElasticDeviceMesh
from .config import Config, load_config
from .data import TEST_VOCAB_SIZE, get_dataloader
from .diloco import Diloco
from .lr_scheduler import get_scheduler
from .models.llama import Transformer, get_model_args, get_num_flop_per_token
from .optimizers import get_optimizer
from .utils import FakeTokenizer, PerfCounter, get_peak_flops
from .utils.logger import get_logger
from .utils.metric_logger import DummyMetricLogger, WandbMetricLogger
from .utils.profiler import MemoryProfiler
from .utils.stopwatch import Stopwatch
from .utils.world_info import get_world_info


def log_hash_training_state(config: Config, backend, diloco: Diloco | None, metric_logger, step: int, id: str = "") -> None:
    """md5 signatures of inner model / inner optimizer / outer optimizer / outer model, logged and (on
    rank 0) recorded as metrics; used to check save / resume / live-recovery equality."""
    if not config.train.log_model_hash:
        return
    logger = get_logger()
    from .checkpoint import cast_dtensor_to_tensor
    inner_model = utils.get_dict_signature({n: t for n, t in backend.named_master_shards()})
    inner_opt = utils.get_dict_signature({k: v for k, v in cast_dtensor_to_tensor(backend.optimizer_state_dict()).items()
                                          if k.startswith("state.")})
    logger.debug(f"inner diloco model {id} : {inner_model}")
    logger.debug(f"inner optimizer hash {id} : {inner_opt}")
    metrics = {"step": step, f"inner_model_hash_{id}": inner_model, f"inner_optimizer_hash_{id}": inner_opt}
    if config.diloco is not None and diloco is not None:
        diloco.wait_host_state()
        outer_opt = utils.get_optimizer_signature(diloco.outer_optimizer)
        outer_model = utils.get_tensor_list_signature([p.data for p in diloco.param_list_cpu])
        logger.debug(f"outer diloco optimizer hash {id} : {outer_opt}")
        logger.debug(f"outer diloco model hash {id} : {outer_model}")
        metrics.update({f"outer_optimizer_hash_{id}": outer_opt, f"outer_model_hash_{id}": outer_model})
    if get_world_info().rank == 0 and metric_logger is not None:
        metric_logger.log(metrics)


def _get_tokenizer(config: Config):
    if config.data.fake and config.name_model == "debugmodel":
        return FakeTokenizer()
    from transformers import AutoTokenizer
    name = {"llama2": "mistralai/Mistral-7B-v0.1", "llama3": "meta-llama/Meta-Llama-3-8B"}.get(config.type_model)
    if name is None:
        raise ValueError(f"Model type {config.type_model} not supported")
    if config.data.fake:
        try:
            return AutoTokenizer.from_pretrained(name, use_fast=True, local_files_only=True)
        except Exception:  # noqa: BLE001  offline box with fake data: ids only need to be in range
            return FakeTokenizer()
    return AutoTokenizer.from_pretrained(name, use_fast=True)


def _resolve_sidecar_url(config: Config, edm: ElasticDeviceMesh) -> str:
    """``ckpt.live_recovery_url`` as given, or for "auto" the address the source worker published in the store."""
    url = config.ckpt.live_recovery_url
    if url != "auto":
        return url
    src = config.ckpt.live_recovery_rank_src or 0
    uid = edm.global_store.get(f"gid_{src}").decode()
    return f"http://{edm.global_store.get(f'sidecar_{uid}').decode()}/latest/"


def _recover_from_sidecar_with_retry(ckpt_manager: CkptManager, url: str, limit_s: float) -> None:
    """The source may not have staged a checkpoint yet (it saves at outer-step boundaries): poll until it has."""
    deadline = time.monotonic() + limit_s
    while True:
        try:
            ckpt_manager.recover_from_sidecar(url)
            return
        except Exception:  # noqa: BLE001
            if time.monotonic() > deadline:
                raise
            time.sleep(1.0)


def _check_engine_flags(config: Config, fused_path: bool, logger) -> None:
    """Flags of the reference's FSDP2 / torch.compile stack that mean something else (or nothing) here: say so once
    instead of accepting them silently."""
    t = config.train
    if t.fsdp_cpu_offload:
        raise ValueError("train.fsdp_cpu_offload is not supported: the engine keeps the sharded fp32 master weights and AdamW "
                         "moments in HBM (12 bytes per parameter divided by the number of GPUs); only the DiLoCo outer state "
                         "lives in (pinned) host memory")
    if not fused_path:
        return
    fields = t.model_fields_set
    if "torch_compile" in fields and t.torch_compile:
        logger.warning("train.torch_compile has no effect on the GPU path: the model is a fixed schedule of hand-written kernels")
    if "attn_fn" in fields:
        logger.warning(f"train.attn_fn={t.attn_fn!r} has no effect on the GPU path: attention always runs the tcgen05 flash "
                       "kernels (document mask from seq_start)")
    if "reshard_after_forward" not in fields:
        logger.info("bf16 parameter replica resident on every GPU (set train.reshard_after_forward=true to keep only the row "
                    "shards and re-gather each block when it runs)")


def train(config: Config) -> None:
    world_info = get_world_info()
    logger = get_logger(config)
    sw = Stopwatch(config)
    sw.start("train()")
    assert config.optim.batch_size % world_info.local_world_size == 0
    batch_size = config.optim.batch_size // world_info.local_world_size
    assert batch_size % config.train.micro_bs == 0, \
        f"The micro batch size ({config.train.micro_bs}) must divide the number of samples on each GPU ({batch_size})."
    gradient_accumulation_steps = batch_size // config.train.micro_bs
    if config.ckpt is not None and config.ckpt.interval is not None and config.diloco is not None:
        assert config.ckpt.interval % config.diloco.inner_steps == 0, \
            "ckpt interval must be a multiple of diloco inner steps as we only save at the end of an outer step"
    use_cuda = torch.cuda.is_available()
    device = torch.device("cuda", world_info.device_index) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)

    if world_info.workers_in_job > 1 and config.data.data_rank is None:
        config.data.data_rank, config.data.data_world_size = world_info.global_rank, world_info.workers_in_job
    with sw.record_block("Get Tokenizer"):
        tokenizer = _get_tokenizer(config)
    vocab_size = len(tokenizer) if (config.name_model != "debugmodel" or not config.data.fake) else TEST_VOCAB_SIZE

    with sw.record_block("Get Dataloader"):
        train_dataloader = get_dataloader(tokenizer=tokenizer, world_size=world_info.world_size, rank=world_info.rank,
                                          batch_size=batch_size, data_config=config.data, device=device)
        train_iter = iter(train_dataloader)

    margs = get_model_args(config.type_model, config.name_model, vocab_size, config.data.seq_length, config.train.attn_fn,
                           config.train.fused_linear_ce)
    gpu_peak_flops = get_peak_flops(torch.cuda.get_device_name(device) if use_cuda else "cpu")
    num_params = margs.num_params(exclude_embedding=True)
    num_flop_per_token = get_num_flop_per_token(num_params, margs, config.data.seq_length)
    logger.info(f"Number of parameters: {num_params}")

    # a joiner that recovers from a sidecar does not ask the source for a point-to-point transfer
    sidecar_join = config.ckpt.live_recovery_url is not None
    with sw.record_block("Elastic Device Mesh"):
        elastic_device_mesh = ElasticDeviceMesh(enable=config.diloco is not None,
                                                live_recovery_rank_src=None if sidecar_join else config.ckpt.live_recovery_rank_src)

    sched = partial(get_scheduler, config.optim.sched_type, num_warmup_steps=config.optim.warmup_steps,
                    num_stable_steps=config.optim.stable_steps, num_training_steps=config.optim.total_steps)
    z_weight = config.optim.z_loss_weight if config.optim.z_loss else None
    # both optimizers run on the fused engine: AdamW as its sharded kernel, SOAP as a shard optimizer on the engine's fp32
    # row shards (every rank preconditions its own rows; see FusedBackend)
    fused_path = use_cuda and config.optim.optim.type in ("adam", "soap")
    _check_engine_flags(config, fused_path, logger)
    want_reshard = "reshard_after_forward" in config.train.model_fields_set and config.train.reshard_after_forward
    if fused_path and want_reshard and config.optim.optim.type == "soap":
        logger.warning("train.reshard_after_forward has no effect with optim.type = soap: the shard optimizer refreshes the resident "
                       "bf16 replica after its step")
        want_reshard = False
    with sw.record_block("Get Model"):
        if fused_path:
            from .engine.fused_llama import FusedLlama
            from .ops import kernels as K
            comm = None
            if world_info.local_world_size > 1:
                from .parallel.symm import SymmComm
                comm = SymmComm(elastic_device_mesh.local_pg, device)
            engine = FusedLlama(margs, device=device, comm=comm,
                                grad_dtype=torch.float32 if config.train.reduce_fp32 else torch.bfloat16,
                                reshard=want_reshard,
                                ac_ckpt=config.train.ac_ckpt, z_mode=K.Z_LSE if (z_weight and config.train.fused_linear_ce) else
                                (K.Z_MAX if z_weight else K.Z_NONE), z_weight=z_weight or 0.0)
            torch.manual_seed(42)
            engine.load_from_module(Transformer(margs))
            backend = FusedBackend(engine, config.optim.optim, lambda opt: sched(opt), mesh=elastic_device_mesh.cuda_local_mesh)
        else:
            torch.manual_seed(42)
            model = Transformer(margs).to(device)
            inner_optimizer = get_optimizer(model.parameters(), config.optim.optim)
            backend = EagerBackend(model, inner_optimizer, sched(inner_optimizer), elastic_device_mesh.local_pg, z_loss_weight=z_weight,
                                   num_chunks=config.optim.num_chunks, fused_linear_ce=config.train.fused_linear_ce)

    diloco = Diloco(config.diloco, backend, elastic_device_mesh) if config.diloco is not None else None
    training_progress = TrainingProgress(total_tokens=0, outer_step=0, step=0)
    ckpt_manager = CkptManager(config=config.ckpt, backend=backend, scheduler=backend.lr_scheduler, dataloader=train_dataloader,
                               training_progress=training_progress, data_rank=config.data.data_rank,
                               diloco_offloaded_optimizer=diloco.outer_optimizer if diloco is not None else None,
                               diloco_offloaded_param_list=diloco.param_list_cpu if diloco is not None else None, diloco=diloco,
                               process_group=elastic_device_mesh.local_pg if world_info.workers_in_job > 1 else None,
                               subdir=f"worker_{world_info.global_rank}" if world_info.workers_in_job > 1 else None)
    if diloco is not None and config.ckpt.path is not None:
        port = ckpt_manager.start_sidecar()
        if port is not None and elastic_device_mesh.enable:
            # address book for joiners: same-shard ranks of every worker share one store, so one key per worker id
            from .checkpoint import _default_sidecar_addr
            addr = os.environ.get("ZERO_BAND_LIVE_RECO_ADDR") or _default_sidecar_addr()
            if addr == "0.0.0.0":
                from .collectives import _my_ip
                addr = _my_ip()
            elastic_device_mesh.global_store.set(f"sidecar_{world_info.global_unique_id}", f"{addr}:{port}")

    metric_logger = None
    if world_info.rank == 0:
        cls = WandbMetricLogger if config.metric_logger_type == "wandb" else DummyMetricLogger
        if world_info.workers_in_job > 1 and config.metric_logger_type == "dummy":
            config.project = f"{config.project}.w{world_info.global_rank}"      # one metrics file per worker
        metric_logger = cls(project=config.project, config={"config": config.model_dump(), "world_info": world_info.json()},
                            resume=config.wandb_resume)

    if config.ckpt.resume is not None:
        with sw.record_block("Resume Checkpoint"):
            ckpt_manager.load(resume_ckpt_path=config.ckpt.resume, skip_dataloader=config.ckpt.skip_dataloader,
                              data_path=config.ckpt.data_path)
            train_iter = iter(train_dataloader)
            log_hash_training_state(config, backend, diloco, metric_logger, step=training_progress.step, id="resume")

    memory_profiler = MemoryProfiler(config.train.memory_profiler.freq, config.train.memory_profiler.snapshot_dir,
                                     barrier=lambda: dist.barrier()) if config.train.memory_profiler is not None else None
    num_inner_steps = config.diloco.inner_steps if config.diloco is not None else 1
    perf_counter = PerfCounter(window_size=10)
    device_meter = utils.DeviceThroughputMeter(window_size=10)
    logger.debug("Finished setup in %f seconds", sw.elapsed())
    need_live_recovery = config.ckpt.live_recovery_rank_src is not None and not sidecar_join
    need_sidecar_recovery = sidecar_join
    fake_outer_step = False

    while True:
        if num_inner_steps > 1:
            logger.info(f"outer_step step: {training_progress.outer_step}")
        time_start_outer = time.perf_counter()
        if diloco is not None:
            if need_sidecar_recovery:
                # README join: fetch the newest staged checkpoint of a running worker over HTTP while the members train,
                # skip this outer iteration's inner steps and enter the outer step with a zero pseudo-gradient
                t0 = time.perf_counter()
                url = _resolve_sidecar_url(config, elastic_device_mesh)
                logger.info(f"Start live recovery from sidecar {url}")
                _recover_from_sidecar_with_retry(ckpt_manager, url, elastic_device_mesh.pg_timeout.total_seconds())
                log_hash_training_state(config, backend, diloco, metric_logger, step=training_progress.step, id="live_reco_recv")
                need_sidecar_recovery = False
                fake_outer_step = True
                logger.info("sidecar live recovery done in %f", time.perf_counter() - t0)
            elif not need_live_recovery:
                elastic_device_mesh.maybe_reinit_global_pg(admit_joiners=True)
                dest = elastic_device_mesh.live_recovery.should_send_ckpt_to()
                if dest is not None:
                    logger.info(f"Start live recovery to rank {dest}")
                    ckpt_manager.send_ckpt_to_peer(elastic_device_mesh.global_pg, dest, blocking=True)
                    elastic_device_mesh.live_recovery.reset()
            else:
                t0 = time.perf_counter()
                logger.info(f"Start live recovery from rank {config.ckpt.live_recovery_rank_src}")
                ckpt_manager.recv_ckpt_from_peer(elastic_device_mesh.global_pg)
                log_hash_training_state(config, backend, diloco, metric_logger, step=training_progress.step, id="live_reco_recv")
                need_live_recovery = False
                if config.ckpt.remote_data_load:
                    ckpt_manager.remote_data_load()
                logger.info("live recovery done in %f", time.perf_counter() - t0)

        if fake_outer_step:
            # the members run these steps; the joiner only keeps its counters and schedule aligned with theirs
            for _ in range(num_inner_steps):
                backend.lr_scheduler.step()
            training_progress.step += num_inner_steps
            training_progress.total_tokens += (num_inner_steps * config.data.seq_length * config.optim.batch_size
                                               * elastic_device_mesh.global_pg.size())
        for inner_step in range(0 if fake_outer_step else num_inner_steps):
            sw.start("inner_step")
            with sw.record_block("Load batch"):
                batch = next(train_iter)
            with sw.record_block("Train step"):
                out = backend.train_step(batch, micro_bs=config.train.micro_bs)
            training_progress.step += 1
            new_tokens = config.data.seq_length * config.optim.batch_size
            perf_counter.count_tokens(new_tokens)
            device_meter.step(new_tokens)
            training_progress.total_tokens += new_tokens * (elastic_device_mesh.global_pg.size() if diloco is not None else 1)
            loss = out["loss"]
            metrics = {"Loss": loss, "step": training_progress.step, "inner_lr": backend.current_lr(),
                       "Perplexity": float(torch.exp(torch.tensor(loss))), "total_tokens": training_progress.total_tokens,
                       "time": time.time(), "grad_norm": out["grad_norm"]}
            if config.optim.z_loss:
                metrics["z_loss"] = out["z_loss"]
            log = f"step: {training_progress.step}, loss: {loss:.4f}"
            tps = perf_counter.get_tokens_per_second()
            if tps is not None:
                metrics["tokens_per_second"] = tps
                metrics["mfu"] = 100 * num_flop_per_token * tps / gpu_peak_flops / world_info.local_world_size
                log += f", tokens_per_second: {tps:.2f}, mfu: {metrics['mfu']:.2f}"
            dtps = device_meter.tokens_per_second()
            if dtps is not None:
                metrics["device_tokens_per_second"] = dtps
            if diloco is not None:
                metrics["num_peers"] = elastic_device_mesh.global_pg.size()
                log += f", diloco_peers: {metrics['num_peers']}"
            if world_info.rank == 0:
                metric_logger.log(metrics)
            logger.info(log)
            if memory_profiler is not None:
                memory_profiler.step()
            sw.stop("inner_step")

        if diloco is not None:
            t0 = time.perf_counter()
            diloco.step(model=backend, fake=fake_outer_step, flag=str(training_progress.outer_step))
            fake_outer_step = False
            diloco_time = time.perf_counter() - t0
            log_hash_training_state(config, backend, diloco, metric_logger, step=training_progress.step, id="outer_step")
        training_progress.outer_step += 1

        if config.ckpt.interval is not None and training_progress.step > 0 and training_progress.step % config.ckpt.interval == 0:
            do_remote = config.ckpt.remote is not None and training_progress.step % config.ckpt.remote.interval == 0
            ckpt_manager.save(remote=do_remote)
            log_hash_training_state(config, backend, diloco, metric_logger, step=training_progress.step, id="save")

        if diloco is not None:
            tps = config.optim.batch_size * config.diloco.inner_steps * config.data.seq_length / (time.perf_counter() - time_start_outer)
            mfu = 100 * num_flop_per_token * tps / gpu_peak_flops / world_info.local_world_size
            logger.info(f"effective mfu: {mfu}")
            if world_info.rank == 0:
                metric_logger.log({"outer_mfu": mfu, "step": training_progress.step, "outer_step": training_progress.outer_step,
                                   "outer_tokens_per_second": tps, "all_reduce_step": diloco_time})
        if training_progress.step >= config.optim.total_steps:
            break

    if world_info.rank == 0:
        metric_logger.finish()
    ckpt_manager.close()
    elastic_device_mesh.close()
    logger.info("Training finished, exiting ...")


def main(argv: list[str] | None = None) -> None:
    torch.manual_seed(42)
    config = load_config(argv)
    world_info = get_world_info()
    logger = get_logger(config)
    if torch.cuda.is_available():
        torch.cuda.set_device(world_info.device_index)

    def run():
        try:
            train(config)
        except Exception as e:  # noqa: BLE001
            import multiprocessing
            logger.info("Caught an exception, terminating children")
            logger.info(e)
            for p in multiprocessing.active_children():
                p.terminate()
            raise

    if config.train.torch_profiler and world_info.rank == 0:
        from torch.profiler import ProfilerActivity, profile
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
        os.makedirs("logs", exist_ok=True)
        with profile(activities=acts, record_shapes=True) as prof:
            run()
        prof.export_chrome_trace("logs/profile.json.gz")
        logger.info(prof.key_averages().table(sort_by="self_cpu_time_total", row_limit=10))
    else:
        run()


if __name__ == "__main__":
    main()
