import json

from verl_b200.trainer.sft_trainer import main as sft_main


def test_sft_loss_goes_down_on_repeated_data(tmp_path, monkeypatch):
    logf = tmp_path / "sft.jsonl"
    monkeypatch.setenv("VERL_FILE_LOGGER_PATH", str(logf))
    sft_main(["data.synthetic.enable=true", "data.synthetic.num_samples=8", "data.train_batch_size=8", "data.micro_batch_size_per_gpu=4",
              "data.max_prompt_length=8", "data.max_response_length=8", "model.preset=tiny-qwen2", "optim.lr=3e-3", "optim.lr_warmup_steps_ratio=0.0",
              "optim.lr_scheduler_type=constant", "trainer.total_epochs=12", "trainer.logger=[file]", f"trainer.default_local_dir={tmp_path}/ck",
              "trainer.device=cpu", "trainer.save_freq=6"])
    rows = [json.loads(x)["data"] for x in logf.read_text().splitlines()]
    assert len(rows) == 12 and rows[-1]["train/loss"] < rows[0]["train/loss"] - 0.5
    assert (tmp_path / "ck" / "global_step_12" / "model_world_size_1_rank_0.pt").exists()
