"""Config system: every shipped TOML parses; CLI grammar; env overrides; validators."""
import glob
import os

import pytest

from prime_b200.config import Compression, Config, load_config, parse_argv, resolve_env_vars

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OURS = sorted(glob.glob(os.path.join(ROOT, "configs", "**", "*.toml"), recursive=True))
_ref_dir = os.environ.get("PRIME_B200_REFERENCE_CONFIGS", "")  # optional: a checkout of the reference configs
REF = sorted(glob.glob(os.path.join(_ref_dir, "**", "*.toml"), recursive=True)) if _ref_dir else []


@pytest.mark.parametrize("path", OURS + REF)
def test_config_files_parse(path):
    cfg = Config(**parse_argv([f"@{path}"]))
    assert cfg is not None


def test_expected_config_set_present():
    rel = {os.path.relpath(p, os.path.join(ROOT, "configs")) for p in OURS}
    for need in ["debug/normal.toml", "debug/diloco.toml", "150M/H100.toml", "150M/B200.toml", "10B/H100.toml", "10B/H100_cooldown.toml",
                 "1B/H100.toml", "7B_diloco/H100.toml", "70M/H100.toml", "13B/H100.toml", "test.toml"]:
        assert need in rel


def test_cli_grammar(tmp_path):
    f = tmp_path / "c.toml"
    f.write_text('name_model = "debugmodel"\n[train]\nmicro_bs = 8\n[optim]\nbatch_size = 16\n')
    cfg = load_config([f"@{f}", "--train.micro_bs", "4", "--train.ac_ckpt", "--no-data.sequence_packing", "--diloco.inner_steps", "5",
                       "--diloco.compression", "uint8", "--optim.optim.lr=1e-3", "--train.attn_fn", "math"], env=False)
    assert cfg.train.micro_bs == 4 and cfg.train.ac_ckpt is True and cfg.data.sequence_packing is False
    assert cfg.diloco.inner_steps == 5 and cfg.diloco.compression == Compression.UINT8
    assert cfg.optim.optim.lr == 1e-3 and cfg.optim.batch_size == 16 and cfg.train.attn_fn == "math"
    cfg = load_config([f"@{f}", "--train.ac_ckpt", "2"], env=False)
    assert cfg.train.ac_ckpt == 2
    cfg = load_config([f"@{f}", "--optim.optim.precondition_frequency", "1"], env=False)
    assert cfg.optim.optim.type == "soap"


def test_unknown_keys_rejected(tmp_path):
    with pytest.raises(Exception):
        load_config(["--train.micro_bs", "1", "--train.not_a_key", "3"], env=False)
    with pytest.raises(Exception):
        Config(**{"train": {"micro_bs": 1}, "bogus": 1})


def test_validators():
    with pytest.raises(Exception):
        Config(train={"micro_bs": 1}, ckpt={"path": "/tmp/x"})           # path without interval
    with pytest.raises(Exception):
        Config(train={"micro_bs": 1}, ckpt={"path": "/tmp/x", "interval": 7}, diloco={"inner_steps": 5})
    with pytest.raises(Exception):
        Config(train={"micro_bs": 1}, ckpt={"live_recovery_rank_src": 0})
    with pytest.raises(Exception):
        Config(train={"micro_bs": 1}, ckpt={"remote_data_load": True})
    Config(train={"micro_bs": 1}, ckpt={"path": "/tmp/x", "interval": 10}, diloco={"inner_steps": 5})


def test_env_overrides():
    cfg = Config(train={"micro_bs": 1}, diloco={"inner_steps": 5})
    resolve_env_vars(cfg, {"ZERO_BAND_TRAIN_MICRO_BS": "16", "ZERO_BAND_DILOCO_OUTER_LR": "0.5", "ZERO_BAND_LOG_LEVEL": "DEBUG",
                           "ZERO_BAND_OPTIM_OPTIM_LR": "1e-5", "ZERO_BAND_EDM_HEARTBEAT_INTERVAL_SECONDS": "1", "HOME": "/x"})
    assert cfg.train.micro_bs == 16 and cfg.diloco.outer_lr == 0.5 and cfg.log_level == "DEBUG" and cfg.optim.optim.lr == 1e-5
    with pytest.raises(ValueError):
        resolve_env_vars(cfg, {"ZERO_BAND_NOT_A_FIELD": "1"})
    with pytest.raises(ValueError):
        resolve_env_vars(cfg, {"ZERO_BAND_TRAIN_MICRO_BS": "abc"})
