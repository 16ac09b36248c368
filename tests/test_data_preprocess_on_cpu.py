"""Dataset preparation scripts: raw rows in, training parquet out, readable by the RL dataset and scored by the matching scorer."""

import json
import os
import subprocess
import sys

import pandas as pd

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPTS = os.path.join(REPO, "examples", "data_preprocess")


def _run(script, raw_dir, out_dir, *extra):
    env = dict(os.environ, PYTHONPATH=REPO + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, os.path.join(SCRIPTS, script), "--local_dataset_path", str(raw_dir), "--local_save_dir", str(out_dir), *extra],
                       env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


def _write(path, rows):
    with open(path, "w") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")


def test_gsm8k_family_and_math(tmp_path):
    from verl_b200.utils.reward_score import default_compute_score

    raw = tmp_path / "raw_gsm8k"
    raw.mkdir()
    rows = [{"question": f"What is {i} + {i}?", "answer": f"We add.\n#### {2 * i:,}"} for i in (3, 700, 1234)]
    _write(raw / "train.jsonl", rows)
    _write(raw / "test.jsonl", rows[:1])
    _run("gsm8k.py", raw, tmp_path / "gsm8k")
    df = pd.read_parquet(tmp_path / "gsm8k" / "train.parquet")
    assert len(df) == 3 and df.iloc[2]["reward_model"]["ground_truth"] == "2468" and df.iloc[0]["data_source"] == "openai/gsm8k"
    assert df.iloc[0]["prompt"][0]["role"] == "user" and df.iloc[1]["extra_info"]["index"] == 1
    assert default_compute_score("openai/gsm8k", "so #### 2468", df.iloc[2]["reward_model"]["ground_truth"]) == 1.0
    _run("gsm8k_multiturn_w_tool.py", raw, tmp_path / "tool", "--max_rows", "2")
    dt = pd.read_parquet(tmp_path / "tool" / "train.parquet")
    assert len(dt) == 2 and dt.iloc[0]["prompt"][0]["role"] == "system"
    assert dt.iloc[1]["extra_info"]["tools_kwargs"]["calc_gsm8k_reward"]["create_kwargs"]["ground_truth"] == "1400"
    _run("gsm8k_multiturn_sft.py", raw, tmp_path / "sft")
    ds = pd.read_parquet(tmp_path / "sft" / "test.parquet")
    assert [m["role"] for m in ds.iloc[0]["messages"]] == ["user", "assistant"]
    # the RL dataset reads the result
    from verl_b200.utils.dataset.rl_dataset import RLHFDataset
    from verl_b200.utils.tokenizer import ByteChatTokenizer

    d = RLHFDataset(str(tmp_path / "gsm8k" / "train.parquet"), ByteChatTokenizer(), {"max_prompt_length": 256, "prompt_key": "prompt"})
    item = d[0]
    assert item["input_ids"].shape[-1] == 256 and "reward_model" in item and item["data_source"] == "openai/gsm8k"

    rawm = tmp_path / "raw_math"
    rawm.mkdir()
    mrows = [{"problem": "Compute $1+1$.", "solution": "It is $\\boxed{2}$."}, {"problem": "No box here.", "solution": "nothing"}]
    _write(rawm / "train.jsonl", mrows)
    _write(rawm / "test.jsonl", mrows)
    _run("math_dataset.py", rawm, tmp_path / "math")
    dm = pd.read_parquet(tmp_path / "math" / "train.parquet")
    assert len(dm) == 1 and dm.iloc[0]["reward_model"]["ground_truth"] == "2"           # the row without a boxed answer is dropped


def test_search_and_hellaswag_rows(tmp_path):
    raw = tmp_path / "raw_nq"
    raw.mkdir()
    _write(raw / "train.jsonl", [{"question": " who wrote it? ", "golden_answers": ["A. Author", "Author"], "data_source": "nq"}])
    _write(raw / "test.jsonl", [{"question": "where?", "golden_answers": ["there"], "data_source": "hotpotqa"}])
    _run("preprocess_search_r1_dataset.py", raw, tmp_path / "search")
    d = pd.read_parquet(tmp_path / "search" / "test.parquet")
    assert d.iloc[0]["data_source"] == "searchR1_hotpotqa" and list(d.iloc[0]["reward_model"]["ground_truth"]["target"]) == ["there"]
    assert d.iloc[0]["extra_info"]["tools_kwargs"]["search"]["create_kwargs"]["question"] == "where?"
    rawh = tmp_path / "raw_hs"
    rawh.mkdir()
    ex = {"activity_label": "Cooking", "ctx_a": "A person [header] stirs.", "ctx_b": "then", "endings": ["a", "b", "c", "d"], "label": "2"}
    _write(rawh / "train.jsonl", [ex])
    _write(rawh / "validation.jsonl", [ex, dict(ex, label="")])
    _run("hellaswag.py", rawh, tmp_path / "hs")
    h = pd.read_parquet(tmp_path / "hs" / "test.parquet")
    assert len(h) == 1 and h.iloc[0]["reward_model"]["ground_truth"] == "c" and h.iloc[0]["reward_model"]["style"] == "model"
