"""Typed configuration: TOML files, dotted command-line overrides and ``ZERO_BAND_*`` environment overrides.

Schema, defaults and validators are those of the reference (src/zeroband/config.py:10-194) so its
TOML files load unchanged. The argument grammar is implemented here (the reference delegates to an
external package): ``@file.toml`` loads a file, ``--a.b.c value`` overrides a key, a bare ``--a.b``
sets a boolean true, ``--no-a.b`` sets it false; later arguments win and the command line beats the
file. Unknown keys are rejected. Every field is also addressable as ``ZERO_BAND_<PATH>``
(``ZERO_BAND_TRAIN_MICRO_BS``); unlike the reference (config.py:197-274, which rejects them) the
runtime knobs of the elastic mesh that share the prefix are allowed through.
"""
from __future__ import annotations

import os
import sys
import tomllib
from enum import Enum
from typing import Any, Literal, TypeAlias, Union, get_args, get_origin

from pydantic import BaseModel, ConfigDict, create_model, model_validator

AttnFnType: TypeAlias = Literal["flex", "math"]


class BaseConfig(BaseModel):
    model_config = ConfigDict(extra="forbid", validate_assignment=False)


class Compression(Enum):
    NO = "no"
    UINT8 = "uint8"


class DataConfig(BaseConfig):
    dataset_name_or_paths: str = "datasets/fineweb-edu"
    val_dataset_name_or_paths: str | None = None
    sequence_packing: bool = True
    seq_length: int = 1024
    fake: bool = False
    num_workers: int = 4
    max_train_samples: int | None = None
    max_eval_samples: int | None = None
    dataset_ratio: str | None = None
    data_rank: int | None = None
    data_world_size: int | None = None
    reverse_data_files: bool = False
    split_by_data_rank: bool = True


class AdamConfig(BaseConfig):
    type: Literal["adam"] = "adam"
    lr: float = 4e-4
    weight_decay: float = 0.1
    betas1: float = 0.9
    betas2: float = 0.95


class SoapConfig(BaseConfig):
    type: Literal["soap"] = "soap"
    lr: float = 4e-4
    weight_decay: float = 1e-05
    betas1: float = 0.9
    betas2: float = 0.95
    max_preconditioner_dim: int = 8192
    precondition_frequency: int = 100


OptimizersConfig: TypeAlias = AdamConfig | SoapConfig


class OptimConfig(BaseConfig):
    optim: OptimizersConfig = AdamConfig()
    sched_type: Literal["cosine", "linear", "wsd-sqrt"] = "cosine"
    warmup_steps: int = 1000
    stable_steps: int = 80_000
    total_steps: int = 88_000
    batch_size: int = 512
    z_loss: bool = False
    z_loss_weight: float = 2e-4
    num_chunks: int | None = None


class DilocoConfig(BaseConfig):
    outer_lr: float = 0.7
    inner_steps: int
    compression: Compression = Compression.NO
    retry_all_reduce: int = 3
    # NVLink worker groups only: keep the fp32 outer parameters and momentum resident in device memory between outer
    # steps. The pinned host copies are then written only when somebody reads them (checkpoint save, live recovery,
    # the hash log) instead of inside every outer step. False = stage both ways on every outer step.
    outer_state_resident: bool = True


class MemoryProfilerConfig(BaseConfig):
    freq: int = 10
    snapshot_dir: str


class TrainConfig(BaseConfig):
    micro_bs: int = 1
    ac_ckpt: bool | int = False
    reshard_after_forward: bool = True
    reduce_fp32: bool = False
    log_model_hash: bool = False
    memory_profiler: MemoryProfilerConfig | None = None
    torch_profiler: bool = False
    torch_compile: bool = True
    fused_linear_ce: bool = False
    fsdp_cpu_offload: bool = False
    attn_fn: AttnFnType = "flex"


class MonitorConfig(BaseConfig):
    log_flush_interval: int = 10
    base_url: str | None = None
    auth_token: str | None = None


class RemoteConfig(BaseConfig):
    path: str
    interval: int


class CkptConfig(BaseConfig):
    path: str | None = None
    interval: int | None = None
    topk: int | None = None
    remote: RemoteConfig | None = None
    remote_data_path: str | None = None
    remote_data_load: bool = False
    resume: str | None = None
    skip_dataloader: bool = False
    live_recovery_rank_src: int | None = None
    # joiner side of the sidecar recovery: URL of a running worker's sidecar (".../latest/"), or "auto" to look the
    # address up in the worker-group store (source = live_recovery_rank_src, default rank 0). The joiner downloads the
    # newest staged checkpoint, skips the inner steps of that outer iteration and enters the outer step with a zero
    # pseudo-gradient.
    live_recovery_url: str | None = None
    data_path: str | None = None
    token_count: int | None = None

    @model_validator(mode="after")
    def validate_path_and_interval(self):
        if (self.path is None) != (self.interval is None):
            raise ValueError("path and interval must be both set or both None")
        if self.path is None and self.remote is not None:
            raise ValueError("remote_path is set but path is not set")
        return self

    @model_validator(mode="after")
    def validate_remote_data_path(self):
        if self.remote_data_load and self.data_path is not None:
            raise ValueError("remote_data_load and data_path are mutually exclusive")
        if self.remote_data_load and self.remote_data_path is None:
            raise ValueError("remote_data_load is set but remote_data_path is not set")
        return self


ENV_VAR_PREFIX = "ZERO_BAND_"

# Runtime knobs read directly from the environment by the elastic mesh / trainer; they share the
# prefix but are not config fields.
RUNTIME_ENV_VARS = frozenset({
    "ZERO_BAND_GLOBAL_STORE_TIMEOUT_SECONDS", "ZERO_BAND_GLOBAL_PG_TIMEOUT_SECONDS",
    "ZERO_BAND_GLOBAL_STORE_POLLING_INTERVAL_SECONDS", "ZERO_BAND_EDM_HEARTBEAT_INTERVAL_SECONDS",
    "ZERO_BAND_EDM_HEARTBEAT_TIMEOUT_SECONDS", "ZERO_BAND_IPERF_PORT", "ZERO_BAND_DEV",
    "ZERO_BAND_LIVE_RECO_PORT", "ZERO_BAND_LIVE_RECO_ADDR", "ZERO_BAND_LOG_LEVEL", "ZERO_BAND_LOG_ALL_RANK",
})


class Config(BaseConfig):
    name_model: Literal["debugmodel", "70M", "150M", "271M", "1B", "7B", "10B", "13B", "26B", "70B"] = "150M"
    type_model: Literal["llama2", "llama3"] = "llama3"
    project: str = "zeroband"
    run_id: str | None = None
    run_name: str | None = None
    metric_logger_type: Literal["wandb", "dummy"] = "wandb"
    wandb_resume: bool = False
    log_level: Literal["NOTSET", "DEBUG", "INFO", "WARNING", "ERROR", "CRITICAL"] = "INFO"
    log_all_rank: bool = False
    diloco: DilocoConfig | None = None
    data: DataConfig = DataConfig()
    optim: OptimConfig = OptimConfig()
    train: TrainConfig
    monitor: MonitorConfig | None = None
    ckpt: CkptConfig = CkptConfig()

    @model_validator(mode="after")
    def ckpt_diloco_step(self):
        if self.ckpt is not None and self.ckpt.interval is not None and self.diloco is not None:
            assert self.ckpt.interval % self.diloco.inner_steps == 0, \
                "ckpt interval must be a multiple of diloco inner steps as we only save at the end of an outer step"
        return self

    @model_validator(mode="after")
    def validate_live_recovery_rank_src(self):
        if self.ckpt is not None and self.ckpt.live_recovery_rank_src is not None and self.diloco is None:
            raise ValueError("live_recovery_rank_src is only supported with diloco")
        if self.ckpt is not None and self.ckpt.live_recovery_url is not None and self.diloco is None:
            raise ValueError("live_recovery_url is only supported with diloco")
        return self


# ---------------------------------------------------------------------------------------------
# command line
# ---------------------------------------------------------------------------------------------
def _set_nested(d: dict, dotted: str, value: Any) -> None:
    keys = dotted.split(".")
    for k in keys[:-1]:
        nxt = d.get(k)
        if not isinstance(nxt, dict):
            nxt = {}
            d[k] = nxt
        d = nxt
    d[keys[-1]] = value


def _merge(dst: dict, src: dict) -> dict:
    for k, v in src.items():
        if isinstance(v, dict) and isinstance(dst.get(k), dict):
            _merge(dst[k], v)
        else:
            dst[k] = v
    return dst


def parse_argv(argv: list[str] | None = None) -> dict:
    """Turn ``@cfg.toml --a.b v --flag --no-x.y`` into a nested dict (values stay strings; pydantic
    coerces them). Dashes in key names are accepted as underscores."""
    argv = list(sys.argv[1:] if argv is None else argv)
    out: dict = {}
    i = 0
    while i < len(argv):
        arg = argv[i]
        if arg.startswith("@"):
            with open(arg[1:].strip() or argv[i + 1], "rb") as f:
                _merge(out, tomllib.load(f))
            i += 1 if arg[1:].strip() else 2
            continue
        if not arg.startswith("--"):
            raise ValueError(f"unexpected positional argument {arg!r} (config files are passed as @file.toml)")
        key = arg[2:]
        if "=" in key:
            key, val = key.split("=", 1)
            _set_nested(out, key.replace("-", "_"), val)
            i += 1
            continue
        key = key.replace("-", "_")
        if key.startswith("no_") or key.startswith("no-"):
            _set_nested(out, key[3:], False)
            i += 1
            continue
        nxt = argv[i + 1] if i + 1 < len(argv) else None
        if nxt is None or nxt.startswith("--") or nxt.startswith("@"):
            _set_nested(out, key, True)
            i += 1
        else:
            _set_nested(out, key, nxt)
            i += 2
    return out


def load_config(argv: list[str] | None = None, env: bool = True) -> Config:
    cfg = Config(**parse_argv(argv))
    if env:
        resolve_env_vars(cfg)
    return cfg


# ---------------------------------------------------------------------------------------------
# environment overrides
# ---------------------------------------------------------------------------------------------
def _is_model(tp) -> bool:
    return isinstance(tp, type) and issubclass(tp, BaseModel)


def _submodels(annotation) -> list[type[BaseModel]]:
    if _is_model(annotation):
        return [annotation]
    if get_origin(annotation) in (Union, getattr(__import__("types"), "UnionType")):
        return [a for a in get_args(annotation) if _is_model(a)]
    return []


def _walk(prefix: str, obj: BaseModel):
    """Yield (ENV_NAME, owner, field_name, annotation) for every field reachable from ``obj``."""
    for name, info in obj.__class__.model_fields.items():
        env = f"{ENV_VAR_PREFIX}{prefix}_{name}".upper() if prefix else f"{ENV_VAR_PREFIX}{name}".upper()
        yield env, obj, name, info.annotation
        val = getattr(obj, name)
        if isinstance(val, BaseModel):
            yield from _walk(f"{prefix}_{name}" if prefix else name, val)


def resolve_env_vars(config: Config, environ: dict | None = None) -> None:
    """Apply ``ZERO_BAND_*`` overrides in place; raise on prefixed variables that name nothing."""
    environ = os.environ if environ is None else environ
    fields = list(_walk("", config))
    valid = {e for e, *_ in fields} | RUNTIME_ENV_VARS
    bad = [k for k in environ if k.startswith(ENV_VAR_PREFIX) and k not in valid]
    if bad:
        raise ValueError(f"Found invalid environment variables with {ENV_VAR_PREFIX} prefix: {', '.join(sorted(bad))}\n"
                         "See prime_b200/config.py for the list of valid config variables.")
    for env, owner, name, annotation in fields:
        raw = environ.get(env)
        if raw is None or _submodels(annotation):
            continue
        try:
            tmp = create_model("TempModel", __base__=BaseConfig, **{name: (annotation, ...)})
            setattr(owner, name, getattr(tmp.model_validate({name: raw}), name))
        except Exception as e:  # noqa: BLE001
            raise ValueError(f"Error setting {env}={raw}: {e}") from e
