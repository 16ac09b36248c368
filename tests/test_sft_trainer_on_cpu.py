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


def test_sft_on_conversations_with_images(tmp_path, monkeypatch):
    """``data.multiturn.enable``: conversations (one of them with an image) through the SFT trainer with a vision-language preset;
    only assistant tokens carry loss, and it goes down."""
    import io

    import numpy as np
    import pandas as pd
    from PIL import Image

    buf = io.BytesIO()
    Image.fromarray(np.random.default_rng(0).integers(0, 255, (16, 16, 3), dtype=np.uint8)).save(buf, format="PNG")
    rows = []
    for i in range(4):
        rows.append({"messages": [{"role": "user", "content": ("<image> " if i % 2 == 0 else "") + f"say {i}"}, {"role": "assistant", "content": f"number {i}"},
                                  {"role": "user", "content": "again"}, {"role": "assistant", "content": f"number {i}"}],
                     "images": [{"bytes": buf.getvalue()}] if i % 2 == 0 else []})
    f = tmp_path / "conv.parquet"
    pd.DataFrame(rows).to_parquet(f)
    logf = tmp_path / "sft.jsonl"
    monkeypatch.setenv("VERL_FILE_LOGGER_PATH", str(logf))
    sft_main([f"data.train_files={f}", "data.multiturn.enable=true", "data.multiturn.max_length=128", "data.multiturn.image_min_pixels=64",
              "data.multiturn.image_max_pixels=256", "data.train_batch_size=4", "data.micro_batch_size_per_gpu=2", "model.preset=tiny-qwen2-vl",
              "optim.lr=3e-3", "optim.lr_warmup_steps_ratio=0.0", "optim.lr_scheduler_type=constant", "trainer.total_epochs=10", "trainer.logger=[file]",
              f"trainer.default_local_dir={tmp_path}/ck", "trainer.device=cpu"])
    rows = [json.loads(x)["data"] for x in logf.read_text().splitlines()]
    assert len(rows) == 10 and rows[-1]["train/loss"] < rows[0]["train/loss"] - 0.5


def test_sft_resume_continues_with_the_batches_an_uninterrupted_run_sees(tmp_path, monkeypatch):
    """Stop after step 3 (mid-epoch), restart from the step folder: steps 4-6 see the same batches, so the same losses, as one 6-step run;
    the tracker names the newest step and retention keeps one folder."""
    import pytest

    from verl_b200.utils.checkpoint.checkpoint_handler import CheckpointHandler, SkipFirst, extract_step

    def run(tag, ck, steps, extra=()):
        logf = tmp_path / f"{tag}.jsonl"
        monkeypatch.setenv("VERL_FILE_LOGGER_PATH", str(logf))
        sft_main(["data.synthetic.enable=true", "data.synthetic.num_samples=16", "data.train_batch_size=4", "data.micro_batch_size_per_gpu=4",
                  "data.max_prompt_length=8", "data.max_response_length=8", "model.preset=tiny-qwen2", "optim.lr=1e-3", "optim.lr_warmup_steps_ratio=0.0",
                  "optim.lr_scheduler_type=constant", "trainer.total_epochs=4", f"trainer.total_training_steps={steps}", "trainer.logger=[file]",
                  f"trainer.default_local_dir={ck}", "trainer.device=cpu", "trainer.save_freq=3", "trainer.max_ckpt_to_keep=1", *extra])
        return [json.loads(x) for x in logf.read_text().splitlines()]

    whole = run("whole", tmp_path / "a", 6)
    first = run("first", tmp_path / "b", 3)
    assert (tmp_path / "b" / "latest_checkpointed_iteration.txt").read_text() == "3"
    second = run("second", tmp_path / "b", 6)
    assert [r["step"] for r in second] == [4, 5, 6]
    for a, b in zip(whole[3:], second):
        assert a["data"]["train/loss"] == pytest.approx(b["data"]["train/loss"], rel=1e-5)
    assert [r["data"]["train/loss"] for r in whole[:3]] == pytest.approx([r["data"]["train/loss"] for r in first], rel=1e-5)
    assert sorted(p.name for p in (tmp_path / "b").iterdir() if p.is_dir()) == ["global_step_6"]
    assert (tmp_path / "b" / "latest_checkpointed_iteration.txt").read_text() == "6"
    # resume_mode=disable starts from scratch in a folder that holds checkpoints; resume_path needs a step folder
    fresh = run("fresh", tmp_path / "b", 1, ["trainer.resume_mode=disable"])
    assert [r["step"] for r in fresh] == [1]
    with pytest.raises(ValueError, match="global_step_N"):
        CheckpointHandler(None, default_local_dir=str(tmp_path / "b"), resume_mode="resume_path", resume_from_path=str(tmp_path)).resume_path()
    assert extract_step("/x/global_step_12/actor") == 12 and extract_step("/x/y") is None
    s = SkipFirst(range(10), 4)
    assert list(s) == [4, 5, 6, 7, 8, 9] and list(s) == list(range(10))


def test_controller_driven_sft_over_two_workers_trains_saves_and_resumes(tmp_path, monkeypatch):
    """The driver owns the data; two worker processes (gloo) hold the data-parallel engine. The loss goes down, a checkpoint with the data
    position lands on disk, and a second driver resumes from it instead of starting over."""
    from verl_b200.trainer.sft_trainer_controller import main as controller_main

    def run(tag, steps):
        logf = tmp_path / f"{tag}.jsonl"
        monkeypatch.setenv("VERL_FILE_LOGGER_PATH", str(logf))
        controller_main(["data.synthetic.enable=true", "data.synthetic.num_samples=8", "data.train_batch_size=8", "data.micro_batch_size_per_gpu=4",
                         "data.max_prompt_length=8", "data.max_response_length=8", "model.preset=tiny-qwen2", "optim.lr=3e-3",
                         "optim.lr_warmup_steps_ratio=0.0", "optim.lr_scheduler_type=constant", "trainer.total_epochs=20",
                         f"trainer.total_training_steps={steps}", "trainer.logger=[file]", f"trainer.default_local_dir={tmp_path}/ck",
                         "trainer.device=cpu", "trainer.save_freq=4", "trainer.n_gpus_per_node=2", "trainer.nnodes=1"])
        return [json.loads(x) for x in logf.read_text().splitlines()]

    rows = run("a", 8)
    assert [r["step"] for r in rows] == list(range(1, 9))
    assert rows[-1]["data"]["train/loss"] < rows[0]["data"]["train/loss"] - 0.3
    ck = tmp_path / "ck"
    assert (ck / "latest_checkpointed_iteration.txt").read_text() == "8"
    assert (ck / "global_step_8" / "data.pt").exists() and (ck / "global_step_8" / "model_world_size_2_rank_1.pt").exists()
    more = run("b", 10)
    assert [r["step"] for r in more] == [9, 10]
    assert more[0]["data"]["train/loss"] < rows[0]["data"]["train/loss"] - 0.3   # continued from the trained weights
