"""Checkpoint → HuggingFace conversion CLI.

    python -m verl_b200.model_merger merge --backend fsdp --local_dir ckpt/global_step_1/actor --target_dir out/hf
    python -m verl_b200.model_merger test  --backend fsdp --local_dir ... --test_hf_dir reference/hf

Parity target: ``verl/model_merger/base_model_merger.py:34-191`` (argument surface, merge/test operations, bf16 cast,
tokenizer/config copy, value-head handling).
"""

from __future__ import annotations

import argparse
import os
import shutil
from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from typing import Optional

import torch

__all__ = ["ModelMergerConfig", "BaseModelMerger", "parse_args", "generate_config_from_args"]


def parse_args(argv=None):
    parser = argparse.ArgumentParser(description="verl_b200 model merger")
    sub = parser.add_subparsers(dest="operation", required=True, help="merge or test")
    base = argparse.ArgumentParser(add_help=False)
    base.add_argument("--backend", type=str, required=True, choices=["fsdp", "megatron"], help="engine that wrote the checkpoint")
    base.add_argument("--local_dir", type=str, default=None, help="directory with the rank shard files")
    base.add_argument("--tie-word-embedding", action="store_true", help="model ties input and output embeddings (megatron only)")
    base.add_argument("--trust-remote-code", action="store_true")
    base.add_argument("--is-value-model", action="store_true", help="checkpoint is a value model (megatron only)")
    base.add_argument("--use_cpu_initialization", action="store_true")
    m = sub.add_parser("merge", parents=[base], help="merge shards and save in HuggingFace format")
    m.add_argument("--target_dir", default="tmp", type=str, help="output directory")
    m.add_argument("--hf_upload_path", default=None, type=str, help="HuggingFace repo to upload to (needs network)")
    m.add_argument("--private", action="store_true")
    t = sub.add_parser("test", parents=[base], help="compare merged weights with a HuggingFace directory")
    t.add_argument("--test_hf_dir", type=str, required=True)
    return parser.parse_args(argv)


@dataclass
class ModelMergerConfig:
    operation: str
    backend: str
    target_dir: Optional[str] = "tmp"
    hf_upload_path: Optional[str] = None
    private: bool = False
    test_hf_dir: Optional[str] = None
    tie_word_embedding: bool = False
    trust_remote_code: bool = False
    is_value_model: bool = False
    local_dir: Optional[str] = None
    hf_model_config_path: Optional[str] = None
    hf_upload: bool = field(init=False)
    use_cpu_initialization: bool = False

    def __post_init__(self):
        self.hf_upload = self.operation == "merge" and bool(self.hf_upload_path)
        if self.operation == "test":
            self.target_dir = None
            self.hf_upload_path = None
            self.private = False


def generate_config_from_args(args) -> ModelMergerConfig:
    common = dict(operation=args.operation, backend=args.backend, tie_word_embedding=args.tie_word_embedding,
                  trust_remote_code=args.trust_remote_code, is_value_model=args.is_value_model, local_dir=args.local_dir,
                  hf_model_config_path=os.path.join(args.local_dir, "model", "huggingface") if args.backend == "megatron" else os.path.join(args.local_dir, "huggingface"), use_cpu_initialization=args.use_cpu_initialization)
    if args.operation == "merge":
        cfg = ModelMergerConfig(**common, target_dir=args.target_dir, hf_upload_path=args.hf_upload_path, private=args.private, test_hf_dir=None)
        os.makedirs(cfg.target_dir, exist_ok=True)
        return cfg
    if args.operation == "test":
        return ModelMergerConfig(**common, test_hf_dir=args.test_hf_dir, target_dir=None, hf_upload_path=None, private=False)
    raise NotImplementedError(f"Unknown operation: {args.operation}")


class BaseModelMerger(ABC):
    def __init__(self, config: ModelMergerConfig):
        self.config = config
        self.hf_model_config_path = config.hf_model_config_path
        from verl_b200.models.config import ModelConfig

        self.model_config = ModelConfig.from_pretrained(self.hf_model_config_path)

    def save_hf_model_and_tokenizer(self, state_dict: dict[str, torch.Tensor]):
        from verl_b200.models.hf_io import save_hf_weights

        out = self.config.target_dir
        os.makedirs(out, exist_ok=True)
        save_hf_weights(state_dict.items(), out, dtype=torch.bfloat16)
        for fn in os.listdir(self.hf_model_config_path):
            src = os.path.join(self.hf_model_config_path, fn)
            if os.path.isfile(src) and not fn.endswith(".safetensors") and fn != "model.safetensors.index.json":
                shutil.copy(src, os.path.join(out, fn))
        print(f"Saved HuggingFace model to {out}")

    def upload_to_huggingface(self):
        raise RuntimeError("uploading needs network access and the huggingface_hub client; copy the target_dir manually")

    def _validate_against_hf(self, state_dict: dict[str, torch.Tensor]):
        from verl_b200.models.hf_io import iter_safetensors

        ref = dict(iter_safetensors(self.config.test_hf_dir))
        missing = set(ref) - set(state_dict)
        extra = set(state_dict) - set(ref)
        assert not missing, f"keys missing from the merged checkpoint: {sorted(missing)[:5]}"
        assert not extra, f"unexpected keys in the merged checkpoint: {sorted(extra)[:5]}"
        for k, v in ref.items():
            got = state_dict[k]
            assert got.shape == v.shape, f"shape mismatch for {k}: {tuple(got.shape)} vs {tuple(v.shape)}"
            torch.testing.assert_close(got.to(torch.bfloat16).float(), v.to(torch.bfloat16).float(), atol=1e-6, rtol=1e-6)
        print("Merged checkpoint matches the HuggingFace directory.")

    @abstractmethod
    def merge_and_save(self): ...

    @abstractmethod
    def cleanup(self): ...
