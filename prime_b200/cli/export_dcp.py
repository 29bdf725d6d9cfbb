"""Convert a distributed checkpoint written by this framework into a HuggingFace Llama folder:
``config.json``, sharded ``safetensors`` (or ``.pt``) weights with an index, generation config and,
when available offline, the tokenizer (reference: scripts/export_dcp.py:32-228).

    python -m prime_b200.cli.export_dcp @configs/10B/B200.toml --ckpt.resume /data/10B/step_100 \
        --ckpt.path /data/10B_hf [--save_format safetensors --torch_dtype bfloat16]

Key map and the Q/K row permutation are those of the reference: weights are stored in the
interleaved (re, im) RoPE pairing, HF expects rotate-half, so each head's even rows go to the top
half and odd rows to the bottom half. The head size comes from the model (the reference hard-codes
128).
"""
from __future__ import annotations

import json
import math
import os
import sys
from pathlib import Path
from typing import Literal

import torch

from ..config import Config, parse_argv
from ..models.llama import ModelArgs, get_model_args


class ExportConfig(Config):
    save_format: Literal["pt", "safetensors"] = "safetensors"
    torch_dtype: Literal["float32", "bfloat16"] = "float32"
    with_debug_automap: bool = False
    vocab_size: int | None = None


_KEY_MAP = [("tok_embeddings", "embed_tokens"), ("attention.wq", "self_attn.q_proj"), ("attention.wk", "self_attn.k_proj"),
            ("attention.wv", "self_attn.v_proj"), ("attention.wo", "self_attn.o_proj"), ("attention_norm", "input_layernorm"),
            ("feed_forward.w3", "mlp.up_proj"), ("feed_forward.w2", "mlp.down_proj"), ("feed_forward.w1", "mlp.gate_proj"),
            ("ffn_norm", "post_attention_layernorm"), ("output.weight", "lm_head.weight")]


def remap_keys_llama(k: str) -> str:
    """Framework parameter name -> HuggingFace Llama parameter name."""
    out = k
    for a, b in _KEY_MAP:
        out = out.replace(a, b)
    return out if "output.weight" in k else "model." + out


def convert_config_to_hf(args: ModelArgs, type_model: str = "llama3", with_debug_automap: bool = False) -> dict:
    cfg = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": args.dim, "num_hidden_layers": args.n_layers,
        "num_attention_heads": args.n_heads, "num_key_value_heads": args.kv_heads, "vocab_size": args.vocab_size,
        "intermediate_size": args.hidden_dim, "rms_norm_eps": args.norm_eps, "rope_theta": float(args.rope_theta),
        "max_position_embeddings": args.max_seq_len, "hidden_act": "silu", "tie_word_embeddings": False, "attention_bias": False,
        "mlp_bias": False, "rope_scaling": {"original_max_position_embeddings": 8192, "rope_type": "default"},
    }
    if type_model == "llama2":
        cfg["bos_token_id"], cfg["eos_token_id"] = [1], [2]
    else:
        cfg["bos_token_id"], cfg["eos_token_id"] = [128000], [128001, 128008, 128009]
    if with_debug_automap:
        cfg["auto_map"] = {"AutoConfig": "PrimeIntellect/prime-llama-debug--configuration_llama.LlamaConfig",
                           "AutoModelForCausalLM": "PrimeIntellect/prime-llama-debug--modeling_llama.LlamaForCausalLM"}
    return cfg


@torch.no_grad()
def convert_qk_from_complex_to_rotate_half(weight: torch.Tensor, head_dim: int) -> torch.Tensor:
    """Per head: rows [0,2,4,...] then rows [1,3,5,...] (interleaved pairs -> rotate-half)."""
    n_heads = weight.size(0) // head_dim
    w = weight.view(n_heads, head_dim // 2, 2, -1)
    return torch.cat([w[:, :, 0], w[:, :, 1]], dim=1).reshape(weight.shape).contiguous()


def load_full_state_dict(ckpt_dir: str) -> dict[str, torch.Tensor]:
    """All ``model.*`` tensors of a DCP checkpoint, assembled on the host (no process group needed)."""
    from torch.distributed.checkpoint import FileSystemReader
    from torch.distributed.checkpoint.metadata import TensorStorageMetadata
    from torch.distributed.checkpoint.state_dict_loader import _load_state_dict
    from torch.distributed.checkpoint.default_planner import _EmptyStateDictLoadPlanner
    reader = FileSystemReader(ckpt_dir)
    meta = reader.read_metadata()
    keys = [k for k, v in meta.state_dict_metadata.items() if k.startswith("model.") and isinstance(v, TensorStorageMetadata)]
    sd: dict = {}
    _load_state_dict(sd, storage_reader=reader, planner=_EmptyStateDictLoadPlanner(keys=set(keys)), no_dist=True)
    flat = {}

    def walk(prefix, obj):
        if isinstance(obj, dict):
            for k, v in obj.items():
                walk(f"{prefix}.{k}" if prefix else k, v)
        else:
            flat[prefix] = obj
    walk("", sd)
    return {k[len("model."):]: v for k, v in flat.items() if k.startswith("model.")}


def export(config: ExportConfig, argv_vocab: int | None = None) -> Path:
    save_path = Path(config.ckpt.path)
    save_path.mkdir(parents=True, exist_ok=True)
    vocab = config.vocab_size or argv_vocab
    state = load_full_state_dict(config.ckpt.resume)
    if vocab is None:
        vocab = state["tok_embeddings.weight"].shape[0]
    args = get_model_args(config.type_model, config.name_model, vocab, config.data.seq_length)
    state.pop("freqs_cis", None)
    dtype = torch.bfloat16 if config.torch_dtype == "bfloat16" else torch.float32
    out = {}
    for k, v in state.items():
        v = v.to(dtype)
        if k.endswith("attention.wq.weight") or k.endswith("attention.wk.weight"):
            v = convert_qk_from_complex_to_rotate_half(v, args.head_dim)
        out[remap_keys_llama(k)] = v.contiguous()
    with open(save_path / "config.json", "w") as f:
        json.dump(dict(convert_config_to_hf(args, config.type_model, config.with_debug_automap), torch_dtype=config.torch_dtype), f, indent=2)
    with open(save_path / "generation_config.json", "w") as f:
        json.dump({"_from_model_config": True, "max_length": 100, "num_return_sequences": 1}, f, indent=2)
    # shard at ~4 GB
    shards, cur, cur_bytes, limit = [], {}, 0, 4 << 30
    for k in sorted(out):
        nbytes = out[k].numel() * out[k].element_size()
        if cur and cur_bytes + nbytes > limit:
            shards.append(cur)
            cur, cur_bytes = {}, 0
        cur[k] = out[k]
        cur_bytes += nbytes
    if cur:
        shards.append(cur)
    ext = "safetensors" if config.save_format == "safetensors" else "pt"
    index = {"metadata": {"total_size": sum(t.numel() * t.element_size() for t in out.values())}, "weight_map": {}}
    for i, sh in enumerate(shards):
        name = f"model-{i + 1:05d}-of-{len(shards):05d}.{ext}"
        if ext == "safetensors":
            from safetensors.torch import save_file
            save_file(sh, str(save_path / name), metadata={"format": "pt"})
        else:
            torch.save(sh, save_path / name)
        for k in sh:
            index["weight_map"][k] = name
    with open(save_path / f"model.{ext}.index.json", "w") as f:
        json.dump(index, f, indent=2)
    try:
        from transformers import AutoTokenizer
        name = {"llama2": "mistralai/Mistral-7B-v0.1", "llama3": "meta-llama/Meta-Llama-3-8B"}[config.type_model]
        AutoTokenizer.from_pretrained(name, use_fast=True, local_files_only=True).save_pretrained(save_path)
    except Exception:  # noqa: BLE001  offline: weights and config are still complete
        pass
    return save_path


def main(argv: list[str] | None = None) -> None:
    config = ExportConfig(**parse_argv(argv))
    assert config.ckpt.resume is not None and config.ckpt.path is not None, "need --ckpt.resume <dcp dir> and --ckpt.path <output dir>"
    print(export(config))


if __name__ == "__main__":
    main()
