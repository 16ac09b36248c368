"""Offline command-line tools: random checkpoint creation, evaluation of a generations file, config printing."""

import pandas as pd
import torch

from verl_b200.models.config import ModelConfig
from verl_b200.models.hf_io import load_hf_weights
from verl_b200.models.transformer import DecoderLM


def test_init_random_model_roundtrip(tmp_path):
    from verl_b200.scripts.init_random_model import main

    main(["--preset", "tiny-qwen2", "--num-layers", "1", "--dtype", "float32", "--out", str(tmp_path / "m")])
    cfg = ModelConfig.from_pretrained(str(tmp_path / "m"))
    assert cfg.num_hidden_layers == 1 and cfg.hidden_size == 128
    m = DecoderLM(cfg, dtype=torch.float32, init=False)
    load_hf_weights(m, str(tmp_path / "m"))
    assert torch.isfinite(m.embed_tokens).all()


def test_main_eval_scores_generations(tmp_path):
    from verl_b200.trainer.main_eval import main

    df = pd.DataFrame({"prompt": ["q1", "q2"], "responses": [["a #### 5", "b #### 6"], ["#### 7", "#### 7"]], "data_source": ["gsm8k", "gsm8k"],
                       "reward_model": [{"ground_truth": "5"}, {"ground_truth": "7"}]})
    df.to_parquet(tmp_path / "gen.parquet")
    assert main([f"data.path={tmp_path}/gen.parquet"]) == {"test_score/gsm8k": 0.75}
    f = tmp_path / "r.py"
    f.write_text("def my_score(data_source, solution_str, ground_truth, extra_info=None):\n    return 1.0 if '7' in solution_str else 0.0\n")
    assert main([f"data.path={tmp_path}/gen.parquet", f"custom_reward_function.path={f}", "custom_reward_function.name=my_score"]) == {"test_score/gsm8k": 0.5}


def test_print_cfg(capsys):
    from verl_b200.scripts.print_cfg import main

    main(["data.train_batch_size=12"])
    assert "train_batch_size: 12" in capsys.readouterr().out


def test_main_ppo_dispatches_v1_trainers(tmp_path):
    """``trainer.use_v1=true trainer.trainer_mode=sync`` runs the v1 sync trainer from the same entry point."""
    import json
    import os

    from tests.test_trainer_e2e_on_cpu import OV
    from verl_b200.trainer.main_ppo import main

    logf = tmp_path / "v1.jsonl"
    os.environ["VERL_FILE_LOGGER_PATH"] = str(logf)
    try:
        tr = main([o for o in OV if not o.startswith("trainer.logger")] +
                  ["trainer.logger=[file]", "trainer.total_training_steps=1", f"trainer.default_local_dir={tmp_path}/ckpt", "trainer.resume_mode=disable",
                   "trainer.use_v1=true", "trainer.trainer_mode=sync", "actor_rollout_ref.rollout.mode=async", "actor_rollout_ref.rollout.free_cache_engine=false"])
    finally:
        os.environ.pop("VERL_FILE_LOGGER_PATH", None)
    assert type(tr).__name__ == "PPOTrainerSync"
    rows = [json.loads(x)["data"] for x in logf.read_text().splitlines()]
    assert len(rows) == 1 and "replay/staleness_max" in rows[0]
