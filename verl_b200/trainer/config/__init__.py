"""Typed views of the trainer-level sections (``algorithm``, ``trainer``, ``data``, checkpoint contents). Reference:
``verl/trainer/config/{algorithm,config}.py``."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from verl_b200.base_config import BaseConfig

__all__ = ["CheckpointConfig", "KLControlConfig", "FilterGroupsConfig", "PFPPOConfig", "RolloutCorrectionConfig", "AlgoConfig", "HybridRolloutSwitchConfig",
           "TrainerConfig", "DataConfig"]


def _sub(cls):
    return field(default_factory=cls, metadata={"cls": cls})


@dataclass
class CheckpointConfig(BaseConfig):
    """What a checkpoint holds (``model`` | ``optimizer`` | ``extra`` | ``hf_model``) and whether the files are written by a background thread."""

    save_contents: list = field(default_factory=lambda: ["model", "optimizer", "extra"])
    load_contents: list = field(default_factory=lambda: ["model", "optimizer", "extra"])
    async_save: bool = False
    # flat_v1: this engine's per-rank slice of the flat buffer; dtensor: {HF name: DTensor dim-0 shard}, the reference's payload
    model_format: str = 'flat_v1'
    strict: bool = True

    def __post_init__(self):
        ok = {"model", "optimizer", "extra", "hf_model"}
        for name in ("save_contents", "load_contents"):
            bad = set(getattr(self, name) or []) - ok
            if bad:
                raise ValueError(f"checkpoint.{name}: unknown entries {sorted(bad)}")


@dataclass
class KLControlConfig(BaseConfig):
    type: str = "fixed"
    kl_coef: float = 0.001
    horizon: int = 10000
    target_kl: float = 0.1

    def __post_init__(self):
        if self.type not in ("fixed", "adaptive"):
            raise ValueError(f"kl_ctrl.type must be fixed or adaptive, got {self.type!r}")


@dataclass
class PFPPOConfig(BaseConfig):
    reweight_method: str = "pow"
    weight_pow: float = 2.0


@dataclass
class FilterGroupsConfig(BaseConfig):
    enable: bool = False
    metric: Any = None
    max_num_gen_batches: int = 0
    max_inflight_gen_batches: int = 1


@dataclass
class RolloutCorrectionConfig(BaseConfig):
    rollout_is: Any = None
    rollout_is_threshold: float = 2.0
    rollout_is_batch_normalize: bool = False
    rollout_rs: Any = None
    rollout_rs_threshold: Any = None
    rollout_rs_threshold_lower: Any = None
    rollout_token_veto_threshold: Any = None
    bypass_mode: bool = False
    loss_type: str = 'ppo_clip'
    score_centering: bool = False

    def __post_init__(self):
        mode = self.rollout_is
        if mode is not None and mode is not False and str(mode) not in ("token", "sequence", "geometric", "True", "true"):
            raise ValueError(f"rollout_is must be token, sequence or geometric, got {mode!r}")
        if self.loss_type not in ("ppo_clip", "reinforce"):
            raise ValueError(f"rollout_correction.loss_type must be ppo_clip or reinforce, got {self.loss_type!r}")


@dataclass
class AlgoConfig(BaseConfig):
    gamma: float = 1.0
    lam: float = 1.0
    adv_estimator: str = 'gae'
    norm_adv_by_std_in_grpo: bool = True
    use_kl_in_reward: bool = False
    kl_penalty: str = 'kl'
    use_pf_ppo: bool = False
    pf_ppo: PFPPOConfig = _sub(PFPPOConfig)
    kl_ctrl: KLControlConfig = _sub(KLControlConfig)
    rollout_correction: RolloutCorrectionConfig = _sub(RolloutCorrectionConfig)
    filter_groups: FilterGroupsConfig = _sub(FilterGroupsConfig)


@dataclass
class HybridRolloutSwitchConfig(BaseConfig):
    """Lending of trainer GPUs to the rollout pool in the separate-async trainer: switch when the rollout backlog ratio
    passes ``switch_threshold_ratio``; with ``adaptive_switch_threshold`` the threshold moves up after a switch that did not pay."""

    enable_switch: bool = False
    switch_threshold_ratio: float = 0.4
    adaptive_switch_threshold: bool = True
    switch_threshold_step_up: float = 0.05
    switch_threshold_step_down: float = 0.03
    switch_threshold_release_steps: int = 2
    switch_cost_window_size: int = 3
    # name of a registered dynamic-schedule policy (default / fixed_ratio / static_fully_async / a custom one) that replaces
    # the built-in threshold logic; null keeps the built-in one
    policy: Any = None
    policy_kwargs: dict = field(default_factory=dict)


@dataclass
class TrainerConfig(BaseConfig):
    use_v1: bool = False
    trainer_mode: str = 'sync'
    balance_batch: bool = True
    total_epochs: int = 30
    total_training_steps: Any = None
    project_name: str = 'verl_b200_examples'
    experiment_name: str = 'gsm8k'
    logger: list = field(default_factory=lambda: ['console'])
    log_val_generations: int = 0
    rollout_data_dir: Any = None
    validation_data_dir: Any = None
    nnodes: int = 1
    n_gpus_per_node: int = 8
    save_freq: int = -1
    esi_redundant_time: int = 0
    resume_mode: str = 'auto'
    resume_from_path: Any = None
    checkpoint_callback_class: Any = None
    val_before_train: bool = True
    val_only: bool = False
    test_freq: int = -1
    critic_warmup: int = 0
    default_hdfs_dir: Any = None
    del_local_ckpt_after_load: bool = False
    default_local_dir: str = 'checkpoints/${trainer.project_name}/${trainer.experiment_name}'
    max_actor_ckpt_to_keep: Any = None
    max_critic_ckpt_to_keep: Any = None
    moe_lb_metrics_interval: int = 0
    ray_wait_register_center_timeout: int = 300
    device: str = 'cuda'
    worker_backend: str = 'spmd'
    v1: dict = field(default_factory=dict)


@dataclass
class DataConfig(BaseConfig):
    tokenizer: Any = None
    use_shm: bool = False
    train_files: Any = None
    val_files: Any = None
    train_max_samples: int = -1
    val_max_samples: int = -1
    prompt_key: str = 'prompt'
    reward_fn_key: str = 'data_source'
    max_prompt_length: int = 512
    max_response_length: int = 512
    train_batch_size: int = 1024
    gen_batch_size: Any = None
    val_batch_size: Any = None
    tool_config_path: Any = None
    function_tool_path: Any = None
    return_raw_input_ids: bool = False
    return_raw_chat: bool = True
    return_full_prompt: bool = False
    return_multi_modal_inputs: bool = True
    shuffle: bool = True
    validation_shuffle: bool = False
    seed: int = 42
    dataloader_num_workers: int = 0
    filter_overlong_prompts: bool = False
    filter_overlong_prompts_workers: int = 1
    truncation: str = 'error'
    image_key: str = 'images'
    video_key: str = 'videos'
    audio_key: str = 'audios'
    image_patch_size: int = 14
    vision: Any = None
    image_min_pixels: Any = None
    image_max_pixels: Any = None
    video_min_pixels: Any = None
    video_max_pixels: Any = None
    video_nframes: Any = None
    video_fps: Any = None
    trust_remote_code: bool = False
    custom_cls: dict = field(default_factory=lambda: {'path': None, 'name': None})
    apply_chat_template_kwargs: dict = field(default_factory=lambda: {})
    mm_processor_kwargs: dict = field(default_factory=lambda: {})
    eos_token_id: Any = None
    synthetic: dict = field(default_factory=lambda: {'enable': False, 'num_prompts': 4096, 'min_prompt_length': 16, 'max_prompt_length': 32, 'id_low': 10, 'id_high': 2048})
