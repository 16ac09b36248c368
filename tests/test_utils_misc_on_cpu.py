"""Small utilities: containers, padding templates, trace/skip helpers, group statistics, score centering."""

import json
import os

import numpy as np
import torch

from verl_b200.protocol import DataProto


def test_py_functional_and_net_and_dtypes(tmp_path):
    from verl_b200.utils.fs import copy_to_local, is_non_local, md5_encode
    from verl_b200.utils.net_utils import format_host_port, get_free_port, is_ipv4, is_ipv6
    from verl_b200.utils.py_functional import DynamicEnum, append_to_dict, temp_env_var, timeout_limit
    from verl_b200.utils.torch_dtypes import PrecisionType

    d = {}
    append_to_dict(d, {"a": 1}, "x/")
    append_to_dict(d, {"a": 2}, "x/")
    assert d == {"x/a": [1, 2]}
    with temp_env_var("VB_T", "1"):
        assert os.environ["VB_T"] == "1"
    assert "VB_T" not in os.environ

    class Est(DynamicEnum):
        pass

    Est.register("gae")
    Est.register("grpo")
    assert Est.GRPO.value == 1 and Est.from_name("gae") is Est.GAE and "GAE" in Est and len(list(Est)) == 2
    with timeout_limit(5):
        pass
    assert is_ipv4("127.0.0.1") and is_ipv6("::1") and format_host_port("::1", 80) == "[::1]:80" and get_free_port() > 0
    assert PrecisionType.to_dtype("bf16") is torch.bfloat16 and PrecisionType.to_str(torch.float32) == "fp32"
    f = tmp_path / "a.txt"
    f.write_text("x")
    assert copy_to_local(str(f)) == str(f) and not is_non_local(str(f)) and len(md5_encode("a")) == 32


def test_unpad_pad_roundtrip_with_grad():
    from verl_b200.utils.attention_utils import pad_input, unpad_input

    x = torch.randn(3, 5, 4, requires_grad=True)
    mask = torch.tensor([[1, 1, 0, 0, 0], [1, 1, 1, 1, 1], [0, 1, 1, 0, 0]])
    flat, idx, cu, mx, lens = unpad_input(x, mask)
    assert flat.shape == (9, 4) and cu.tolist() == [0, 2, 7, 9] and mx == 5
    back = pad_input(flat, idx, 3, 5)
    assert torch.equal(back * mask[..., None], back) and torch.allclose(back[mask.bool()], x[mask.bool()])
    back.sum().backward()
    assert torch.equal(x.grad, mask[..., None].expand_as(x).float())


def test_tensordict_utils_and_padding_templates():
    from verl_b200.trainer.ppo.padding_utils import remove_padding_samples, upsample_batch_to_divisible_size
    from verl_b200.utils.tensordict_utils import assign_non_tensor, get_non_tensor_data, get_tensordict, index_select_tensor_dict, to_padded

    data = get_tensordict({"input_ids": torch.arange(12).reshape(3, 4), "ragged": [torch.arange(2), torch.arange(3), torch.arange(1)]},
                          {"names": ["a", "b", "c"], "temperature": 0.7})
    assert len(data) == 3 and data.meta_info["temperature"] == 0.7 and data.non_tensor_batch["names"][1] == "b"
    assert to_padded(data.batch["ragged"], pad_value=-1).tolist() == [[0, 1, -1], [0, 1, 2], [0, -1, -1]]
    assign_non_tensor(data, uid=["u0", "u1", "u2"], step=3)
    assert get_non_tensor_data(data, "step") == 3 and index_select_tensor_dict(data, [2, 0]).non_tensor_batch["uid"].tolist() == ["u2", "u0"]
    b = DataProto.from_dict(tensors={"input_ids": torch.ones(5, 6, dtype=torch.int64), "attention_mask": torch.ones(5, 6, dtype=torch.int64),
                                     "responses": torch.ones(5, 2, dtype=torch.int64), "response_mask": torch.ones(5, 2, dtype=torch.int64),
                                     "advantages": torch.ones(5, 2)}, non_tensors={"uid": ["a"] * 5})
    out, pad = upsample_batch_to_divisible_size(b, 4)
    assert len(out) == 8 and pad == 3 and out.batch["response_mask"][5:].sum() == 0 and out.batch["attention_mask"][5:].sum() == 3
    assert out.batch["advantages"][5:].abs().sum() == 0 and len(remove_padding_samples(out)) == 5


def test_trace_skip_and_tracker(tmp_path):
    from verl_b200.utils.rollout_skip import SkipManager
    from verl_b200.utils.rollout_trace import RolloutTraceConfig, TrajectoryTracker, rollout_trace_attr, rollout_trace_op

    class S:
        @rollout_trace_op
        def gen(self, ids, k=1):
            return {"out": [i + k for i in ids]}

    RolloutTraceConfig.init("p", "e", "jsonl", path=str(tmp_path / "t.jsonl"))
    with rollout_trace_attr(sample_index=3, step=1):
        S().gen([1, 2], k=2)
    RolloutTraceConfig.reset()
    rec = json.loads((tmp_path / "t.jsonl").read_text().splitlines()[0])
    assert rec["attrs"]["sample_index"] == 3 and rec["output"] == {"out": [3, 4]} and rec["inputs"] == {"ids": [1, 2], "k": 2}
    calls = []

    def gen(p):
        calls.append(1)
        return DataProto.from_dict(tensors={"r": p.batch["x"] + 1})

    sm = SkipManager(True, str(tmp_path / "dump"), max_dump_step=1)
    p = DataProto.from_dict(tensors={"x": torch.zeros(2, 1)}, meta_info={"global_steps": 1})
    a, b = sm.wrap(gen)(p), sm.wrap(gen)(p)
    assert len(calls) == 1 and torch.equal(a.batch["r"], b.batch["r"]) and sm.hits == 1
    tr = TrajectoryTracker(str(tmp_path / "traj"))
    tr.track("logp", torch.ones(3))
    path = tr.dump(1)
    assert TrajectoryTracker.compare(torch.load(path), {"logp": torch.ones(3)})["logp"]["close"]


def test_group_mean_std_and_score_centering():
    from verl_b200.trainer.ppo.score_centering import (pad_rollout_topk, score_centering_correction, score_centering_weight_fn,
                                                       topk_log_probs_from_hidden, topk_log_probs_from_logits)
    from verl_b200.utils.groupwise import as_torch_index, group_mean_std

    g = as_torch_index(np.array(["a", "b", "a", "c"], dtype=object))
    mean, std, cnt = group_mean_std(torch.tensor([1.0, 5.0, 3.0, 7.0]), g)
    assert g.tolist() == [0, 1, 0, 2] and mean.tolist() == [2.0, 0.0, 0.0] and abs(float(std[0]) - 2 ** 0.5) < 1e-6 and std[1] == 1
    torch.manual_seed(0)
    logits = torch.randn(10, 50, requires_grad=True)
    ids = torch.topk(logits.detach() + 0.3 * torch.randn(10, 50), 5).indices
    lp = topk_log_probs_from_logits(logits, ids, chunk_size=4)
    ref = torch.log_softmax(logits, -1).gather(-1, ids)
    assert torch.allclose(lp, ref, atol=1e-6)
    gref = torch.autograd.grad(ref.sum() * 2, logits)[0]
    gl = torch.autograd.grad(lp.sum() * 2, logits)[0]
    assert torch.allclose(gl, gref, atol=1e-6)
    h, w = torch.randn(10, 16, requires_grad=True), torch.randn(50, 16)
    assert torch.allclose(topk_log_probs_from_hidden(h, w, ids, chunk_size=3), torch.log_softmax(h @ w.t(), -1).gather(-1, ids), atol=1e-5)
    # when sampler == trainer and no IS weight, the coefficients q - rho*p vanish: no correction and no gradient
    corr, qm, pm = score_centering_correction(lp, lp.detach(), score_centering_weight_fn(None))
    assert corr.abs().max() < 1e-5 and torch.allclose(qm, pm)
    # full-vocabulary head: the gradient equals that of sum_j sg[q_j - p_j] log p_j
    all_ids = torch.arange(50).expand(10, 50)
    q = torch.log_softmax(torch.randn(10, 50), -1)
    lp_all = topk_log_probs_from_logits(logits, all_ids)
    w_tis = score_centering_weight_fn("token", 2.0)
    corr, _, _ = score_centering_correction(lp_all, q, w_tis)
    assert corr.shape == (10,) and torch.isfinite(corr).all()
    ids2, lps2 = pad_rollout_topk(torch.ones(3, 4, dtype=torch.int64), torch.zeros(3, 4), prompt_length=5)
    assert ids2.shape == (8, 4) and (ids2[4:7] == 1).all() and (lps2[:4] < 0).all()
    assert score_centering_weight_fn("token", "0.5_2.0")(torch.tensor([0.1, 1.0, 3.0])).tolist() == [0.0, 1.0, 0.0]


def test_naive_rollout_matches_engine_greedy_and_engine_aliases():
    from verl_b200.models.config import PRESETS
    from verl_b200.models.transformer import DecoderLM
    from verl_b200.workers.engine.base import EngineRegistry
    from verl_b200.workers.rollout.engine import InferenceEngine, SamplingParams
    from verl_b200.workers.rollout.naive import NaiveRollout

    model = DecoderLM(PRESETS["tiny-qwen2"], dtype=torch.float32, seed=5)
    prompts = [[11, 12, 13, 14, 15], [21, 22, 23]]
    P = 6
    ids = torch.zeros(2, P, dtype=torch.int64)
    att = torch.zeros(2, P, dtype=torch.int64)
    for i, p in enumerate(prompts):
        ids[i, P - len(p):] = torch.tensor(p)
        att[i, P - len(p):] = 1
    out = NaiveRollout(model, response_length=6, do_sample=False).generate_sequences(
        DataProto.from_dict(tensors={"input_ids": ids, "attention_mask": att}, meta_info={"do_sample": False}))
    want = InferenceEngine(model, max_num_seqs=4, max_model_len=64, num_blocks=16).generate(prompts, SamplingParams(temperature=0.0, max_tokens=6))
    for i, w in enumerate(want):
        assert out.batch["responses"][i].tolist() == w.token_ids
        assert torch.allclose(out.batch["rollout_log_probs"][i], torch.tensor(w.log_probs), atol=1e-4)
    eng = EngineRegistry.new("language_model", "veomni", PRESETS["tiny-qwen2"], {"seed": 1}, None, {})
    assert type(eng).__name__ == "FSDPEngine"
    assert type(EngineRegistry.new("language_model", "mindspeed", PRESETS["tiny-qwen2"], {"seed": 1}, None, {})).__name__ == "MegatronEngine"
    from verl_b200.utils.transformers_compat import drop_tied_weight_keys, is_transformers_version_in_range

    assert is_transformers_version_in_range("4.0") and "lm_head.weight" not in drop_tied_weight_keys({"lm_head.weight": 1, "a": 2}, True)


def test_tool_call_dialects():
    """Every chat-template family's function-call syntax parses to (name, JSON arguments) and is cut out of the content."""
    import json

    from verl_b200.experimental.agent_loop.tool_parser import get_tool_parser as g

    cases = {
        "glm": ('hi<tool_call>get_weather<arg_key>city</arg_key><arg_value>Paris</arg_value><arg_key>days</arg_key><arg_value>3</arg_value></tool_call>',
                "hi", [("get_weather", {"city": "Paris", "days": 3})]),
        "seed": ('<seed:tool_call><function=f><parameter=a>[1,2]</parameter></function></seed:tool_call>ok', "ok", [("f", {"a": [1, 2]})]),
        "minimax": ('<minimax:tool_call><invoke name="s"><parameter name="q">x y</parameter></invoke><invoke name="t"></invoke></minimax:tool_call>',
                    "", [("s", {"q": "x y"}), ("t", {})]),
        "kimi": ('a<|tool_calls_section_begin|><|tool_call_begin|>functions.calc:0<|tool_call_argument_begin|>{"x": 1}<|tool_call_end|><|tool_calls_section_end|>',
                 "a", [("calc", {"x": 1})]),
        "deepseek_v4": ('<｜DSML｜tool_calls>\n<｜DSML｜invoke name="f">\n<｜DSML｜parameter name="k" string="true">5</｜DSML｜parameter>\n'
                        '<｜DSML｜parameter name="n" string="false">5</｜DSML｜parameter>\n</｜DSML｜invoke>\n</｜DSML｜tool_calls>', "", [("f", {"k": "5", "n": 5})]),
        "gemma4": ('<|tool_call>call:lookup{q:<|"|>a, b<|"|>,n:3,ok:true,r:1.5}<tool_call|>', "", [("lookup", {"q": "a, b", "n": 3, "ok": True, "r": 1.5})]),
        "qwen3_coder": ('<tool_call>\n<function=run>\n<parameter=cmd>\nls -l\n</parameter>\n</function>\n</tool_call>', "", [("run", {"cmd": "ls -l"})]),
        "hermes": ('x<tool_call>{"name": "a", "arguments": {"b": 1}}</tool_call><tool_call>not json</tool_call>', "x", [("a", {"b": 1})]),
    }
    for name, (text, content, want) in cases.items():
        got_text, calls = g(name).extract_tool_calls(text)
        assert got_text.strip() == content, name
        assert [(c.name, json.loads(c.arguments)) for c in calls] == want, (name, calls)

    class Tok:
        def convert_tokens_to_ids(self, t):
            return {"<|observation|>": 7, "<tool_call|>": 9}.get(t, -1)

    assert g("glm", Tok()).stop_token_ids == [7] and g("gemma4", Tok()).stop_token_ids == [9] and g("kimi", Tok()).stop_token_ids == []
    assert g("hermes", Tok()).stop_token_ids == []


def test_continuous_token_builder_and_template_checker():
    """Token-level continuation of a multi-turn conversation equals a single render; a template that rewrites earlier turns is
    reported; generation cut before the end-of-turn token gets the turn closed."""
    from verl_b200.scripts.chat_template_checker import main as checker_main
    from verl_b200.utils.continuous_token import MOCK_TRAJECTORIES, ContinuousTokenBuilder, check_append_only
    from verl_b200.utils.tokenizer import ByteChatTokenizer

    tok = ByteChatTokenizer()
    rep = check_append_only(tok)
    assert all(r["builder"] and r["raw_prefix"] for r in rep.values()) and rep["parallel_tools"]["boundaries"] == 2
    assert checker_main([]) == 0
    b = ContinuousTokenBuilder(tok)
    msgs = MOCK_TRAJECTORIES["tool_call"]
    prompt = b.initial_prompt(msgs[:1])
    gen = tok.encode(msgs[1]["content"]) + [tok.eos_token_id]
    merged = b.merge_context_tokens(prompt + gen, msgs[2:3])
    assert merged == tok.apply_chat_template(msgs[:3], add_generation_prompt=True, tokenize=True)
    cut = b.merge_context_tokens(prompt + gen[:-1], msgs[2:3])          # length-limited generation: the turn is closed first
    assert cut == merged

    class Rewriting(ByteChatTokenizer):
        """Renders only the LAST assistant turn in full (earlier ones are shortened) — not append-only."""

        def apply_chat_template(self, messages, **kw):
            msgs = [dict(m) for m in messages]
            last = max((i for i, m in enumerate(msgs) if m["role"] == "assistant"), default=-1)
            for i, m in enumerate(msgs):
                if m["role"] == "assistant" and i != last:
                    m["content"] = "…"
            return super().apply_chat_template(msgs, **kw)

    rep = check_append_only(Rewriting())
    # the raw template is not append-only, yet every boundary still merges correctly: the prefix keeps the sampled tokens
    assert not rep["system_multi_turn"]["raw_prefix"] and rep["parallel_tools"]["builder"]

    class Unstable(ByteChatTokenizer):
        """Quotes the conversation's first message in every tool message — the synthetic context renders it differently."""

        def apply_chat_template(self, messages, **kw):
            msgs = [dict(m) for m in messages]
            for m in msgs:
                if m["role"] == "tool":
                    m["content"] = f"[{str(msgs[0]['content'])[:4]}] " + str(m["content"])
            return super().apply_chat_template(msgs, **kw)

    assert not check_append_only(Unstable())["tool_call"]["builder"]


def test_flops_counter_architecture_families():
    """Per-architecture FLOPs: dense formula by hand, MoE counts active experts only, sliding-window layers cost less than
    full ones, MLA / hybrid / vision-language families resolve and scale linearly with the token count."""
    from verl_b200.models.config import PRESETS
    from verl_b200.utils.flops_counter import FlopsCounter, arch_cost, get_device_flops

    c = PRESETS["qwen2.5-7b"]
    fc = FlopsCounter(c)
    lens = [1000, 2000]
    h, L, I, V = 3584, 28, 18944, 152064
    n_w = L * (h * (28 * 128 + 2 * 4 * 128) + 28 * 128 * h + 3 * h * I) + 2 * V * h
    want = 6 * n_w * 3000 + 12 * (1000**2 + 2000**2) * 128 * 28 * L
    got, peak = fc.estimate_flops(lens, 2.0)
    assert abs(got * 2.0 * 1e12 - want) / want < 1e-9 and peak == get_device_flops("T")
    assert get_device_flops("T", "NVIDIA B200") == 2250.0 and get_device_flops("T", "NVIDIA GB200") == 2500.0

    moe = PRESETS["qwen3-30b-a3b"]
    dense_like = arch_cost(moe).flops([4096])
    all_experts = 6 * 4096 * moe.num_hidden_layers * 3 * moe.hidden_size * moe.moe_intermediate_size * (moe.num_experts - moe.num_experts_per_tok)
    assert dense_like < all_experts                        # active experts only: far below the all-expert count

    gem = dict(model_type="gemma3_text", hidden_size=1024, num_attention_heads=8, num_key_value_heads=4, head_dim=128, num_hidden_layers=12,
               intermediate_size=4096, vocab_size=32000, sliding_window=512, sliding_window_pattern=6)
    full = dict(gem, sliding_window=None)
    assert arch_cost(gem).flops([8192]) < arch_cost(full).flops([8192])
    assert arch_cost(gem).flops([256]) == arch_cost(full).flops([256])       # shorter than the window: identical

    dsv3 = dict(model_type="deepseek_v3", hidden_size=1024, num_attention_heads=8, num_hidden_layers=6, first_k_dense_replace=2, intermediate_size=4096,
                moe_intermediate_size=512, n_routed_experts=32, num_experts_per_tok=4, n_shared_experts=1, q_lora_rank=256, kv_lora_rank=128,
                qk_nope_head_dim=64, qk_rope_head_dim=32, v_head_dim=64, vocab_size=32000)
    q35 = dict(model_type="qwen3_5", hidden_size=1024, num_attention_heads=8, num_key_value_heads=2, head_dim=128, num_hidden_layers=8,
               intermediate_size=4096, vocab_size=32000, full_attention_interval=4, linear_num_key_heads=4, linear_key_head_dim=64,
               linear_num_value_heads=8, linear_value_head_dim=64, linear_conv_kernel_dim=4)
    oss = dict(model_type="gpt_oss", hidden_size=1024, num_attention_heads=8, num_key_value_heads=2, head_dim=64, num_hidden_layers=4,
               intermediate_size=1024, num_local_experts=8, num_experts_per_tok=2, vocab_size=32000, sliding_window=128)
    for cfg in (dsv3, q35, oss, dict(gem, model_type="apertus")):
        cost = arch_cost(cfg)
        a, b = cost.flops([512]), cost.flops([512, 512])
        assert a > 0 and abs(b - 2 * a) / b < 1e-12
    assert sum(1 for _, s in arch_cost(q35).attn_layers if s is not None) == 2      # every fourth layer is full attention

    vl = PRESETS["tiny-qwen2-vl"]
    cost = arch_cost(dict(model_type="qwen2_vl", vision_config=vl.vision, text_config=None, **{k: getattr(vl, k) for k in
                     ("hidden_size", "num_attention_heads", "num_key_value_heads", "num_hidden_layers", "intermediate_size", "vocab_size")}))
    assert cost.flops([64], images_seqlens=[16]) > cost.flops([64])


def test_tracking_backends_with_stand_in_sdks(monkeypatch, tmp_path):
    """swanlab / clearml / trackio / rl_insight adapters against stand-in modules: what is initialised, what is logged, how
    metric names are mapped."""
    import sys
    import types

    from verl_b200.utils.tracking import RLInsightLogger, Tracking

    calls = []
    swan = types.ModuleType("swanlab")
    swan.init = lambda **kw: calls.append(("swan.init", kw["project"], kw["experiment_name"], kw["mode"]))
    swan.login = lambda key: calls.append(("swan.login", key))
    swan.log = lambda data, step=None: calls.append(("swan.log", dict(data), step))
    swan.finish = lambda: calls.append(("swan.finish",))
    tio = types.ModuleType("trackio")
    tio.init = lambda **kw: calls.append(("trackio.init", kw["project"], kw["name"]))
    tio.log = lambda data, step=None: calls.append(("trackio.log", dict(data), step))
    tio.finish = lambda: calls.append(("trackio.finish",))

    class _Lg:
        def report_scalar(self, title, series, value, iteration):
            calls.append(("clearml.scalar", title, series, value, iteration))

    class _Task:
        @staticmethod
        def init(**kw):
            calls.append(("clearml.init", kw["project_name"], kw["task_name"]))
            return _Task()

        def connect_configuration(self, cfg, name):
            calls.append(("clearml.cfg", name))

        def get_logger(self):
            return _Lg()

        def close(self):
            calls.append(("clearml.close",))

    cml = types.ModuleType("clearml")
    cml.Task = _Task
    rli = types.ModuleType("rl_insight")
    rli.init = lambda **kw: calls.append(("rli.init", kw["project"], kw["config"]))
    rli.metric_gauge = lambda name, v: calls.append(("rli.gauge", name, v))
    rli.finish = lambda: calls.append(("rli.finish",))
    for name, mod in (("swanlab", swan), ("trackio", tio), ("clearml", cml), ("rl_insight", rli)):
        monkeypatch.setitem(sys.modules, name, mod)
    monkeypatch.setenv("SWANLAB_MODE", "local")
    monkeypatch.setenv("VERL_RL_INSIGHT_ENABLE", "1")
    RLInsightLogger._module, RLInsightLogger._started = None, False
    tr = Tracking("proj", "exp", ["swanlab", "clearml", "trackio", "rl_insight"], config={"trainer": {"rl_insight": {"port": 1}}})
    tr.log({"actor/pg_loss": 0.5, "note": "text"}, step=3)
    assert ("swan.init", "proj", "exp", "local") in calls and ("trackio.init", "proj", "exp") in calls and ("clearml.init", "proj", "exp") in calls
    assert ("rli.init", "proj", {"port": 1}) in calls and ("rli.gauge", "actor_pg_loss", 0.5) in calls
    assert ("clearml.scalar", "actor", "pg_loss", 0.5, 3) in calls
    assert ("trackio.log", {"actor/pg_loss": 0.5, "note": "text"}, 3) in calls
    assert not any(c[0] == "rli.gauge" and c[1] == "note" for c in calls)
    monkeypatch.setenv("VERL_RL_INSIGHT_ENABLE", "0")
    n = len(calls)
    RLInsightLogger.log({"x": 1.0}, 1)                  # opted out: nothing happens
    with RLInsightLogger.trace_state("rollout"):
        pass
    assert len(calls) == n
    RLInsightLogger._module, RLInsightLogger._started = None, False


def test_nsys_wrapping_and_precision_debugger(tmp_path):
    import json
    import os

    import torch

    from verl_b200.utils.profiler.config import ProfilerConfig
    from verl_b200.utils.profiler.nsys import nsys_command_prefix, relocate_results, wrap_worker_command
    from verl_b200.utils.profiler.precision_debugger import PrecisionDebugger, compare_dumps
    from verl_b200.utils.profiler.profile import DistProfiler

    cmd = nsys_command_prefix({"trace": "cuda,nvtx", "kill": None, "cuda-memory-usage": False}, "/tmp/out/rep", discrete=True)
    assert cmd[:2] == ["nsys", "profile"] and "--trace=cuda,nvtx" in cmd and "--capture-range=cudaProfilerApi" in cmd
    assert "--capture-range-end=repeat" in cmd and "--cuda-memory-usage=false" in cmd and not any(c.startswith("--kill") for c in cmd)
    assert cmd[-2:] == ["-o", "/tmp/out/rep"]
    full = wrap_worker_command(["python", "-m", "x"], None, str(tmp_path / "prof"), role="actor", rank=3)
    assert full[-3:] == ["python", "-m", "x"] and "actor_rank3_" in full[full.index("-o") + 1]
    src = tmp_path / "raylogs"
    src.mkdir()
    (src / "worker_process_4242.nsys-rep").write_text("x")
    (src / "worker_process_4242.1.nsys-rep").write_text("y")
    (src / "worker_process_9.nsys-rep").write_text("other process")
    moved = relocate_results(str(tmp_path / "dst"), str(src), pid=4242, role="ref")
    assert len(moved) == 2 and all(os.path.basename(m).startswith("ref_") for m in moved) and (src / "worker_process_9.nsys-rep").exists()
    assert relocate_results(str(tmp_path / "dst"), str(src), pid=4242) == [] and relocate_results(None, str(src)) == []

    def run(scale, out):
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 4))
        prof = DistProfiler(0, ProfilerConfig(tool="precision_debugger", enable=True, all_ranks=True, save_path=str(out),
                                              tool_config={"stages": ["actor_update"]}))
        prof.start(stage="actor_update", model=model, step=7)
        x = torch.ones(2, 8)
        with torch.no_grad():
            model[2].weight.mul_(scale)
        model(x).sum().backward()
        prof.stop()
        prof.start(stage="ref_compute_log_prob", model=model)     # not among the configured stages: records nothing
        model(x)
        prof.stop()
        return os.path.join(out, "precision_rank0.jsonl")

    a, b, c = run(1.0, tmp_path / "a"), run(1.0, tmp_path / "b"), run(1.5, tmp_path / "c")
    rows = [json.loads(x) for x in open(a)]
    assert {r["module"] for r in rows if r["kind"] == "forward"} == {"0", "1", "2"} and all(r["step"] == 7 and r["stage"] == "actor_update" for r in rows)
    assert {r["module"] for r in rows if r["kind"] == "grad"} == {"0.weight", "0.bias", "2.weight", "2.bias"}
    assert compare_dumps(a, b) is None
    diff = compare_dumps(a, c)
    assert diff is not None and diff["a"]["module"] == "2"          # the first module whose output changes
    import pytest as _pt
    with _pt.raises(ValueError):
        PrecisionDebugger(0, str(tmp_path), stages=["nope"])
