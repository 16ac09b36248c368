import logging

from verl_b200.utils.logger import DecoratorLoggerBase, LocalLogger, log_with_rank, print_rank_0, print_with_rank
from verl_b200.utils.logging_utils import configure_verl_logging, log_to_file


def test_rank_gated_printing_and_decorator_base(capsys, caplog):
    print_rank_0("hello")
    print_with_rank("a", rank=1)
    print_with_rank("b", rank=1, log_only_rank_0=True)
    out = capsys.readouterr().out
    assert "hello" in out and "[Rank 1] a" in out and "b" not in out
    d = DecoratorLoggerBase("actor", rank=1, log_only_rank_0=False)
    d.logging_function("mem 1GB")
    assert "actor mem 1GB" in capsys.readouterr().out
    lg = logging.getLogger("t_dec")
    with caplog.at_level(logging.DEBUG, logger="t_dec"):
        DecoratorLoggerBase("critic", logger=lg, rank=0).logging_function("x")
        DecoratorLoggerBase("critic", logger=lg, rank=3).logging_function("hidden")
        log_with_rank("y", 2, lg)
    assert "critic x" in caplog.text and "hidden" not in caplog.text and "[Rank 2] y" in caplog.text
    LocalLogger().log({"a": 1.0}, step=3)
    assert "step:3" in capsys.readouterr().out


def test_package_logger_is_isolated_from_the_root_logger(monkeypatch, tmp_path, capsys):
    monkeypatch.setenv("VERL_LOGGING_LEVEL", "warning")
    lg = configure_verl_logging()
    assert lg.level == logging.WARNING and not lg.propagate and len(lg.handlers) == 1
    logging.getLogger().setLevel(logging.CRITICAL)
    lg.warning("still visible")
    assert "still visible" in capsys.readouterr().err
    (tmp_path / "logs").mkdir()
    log_to_file("line", directory=str(tmp_path / "logs"))
    assert (tmp_path / "logs" / "log_0").read_text() == "line\n"


def test_trajectory_tracker_dumps_a_snapshot_in_the_background(tmp_path, monkeypatch):
    import torch

    from verl_b200.utils.debug.trajectory_tracker import dump_data, get_trajectory_tracker

    x = torch.arange(4.0)
    assert dump_data({"obs": x}, "off") is None and not list(tmp_path.iterdir())
    monkeypatch.setenv("VERL_ENABLE_TRACKER", "1")
    monkeypatch.setenv("VERL_TRACKER_HDFS_DIR", str(tmp_path / "dumps"))
    dump_data({"obs": x}, "step1_obs")
    x.add_(100)   # the dump holds the values at the time of the call
    files = get_trajectory_tracker().wait()
    assert files == [str(tmp_path / "dumps" / "step1_obs.pt")]
    assert torch.equal(torch.load(files[0])["obs"], torch.arange(4.0))


def test_worker_runtime_env_fills_only_what_the_shell_left_open():
    from verl_b200.trainer.constants_ppo import NVTX_INJECTION_ENV, get_worker_runtime_env

    env = get_worker_runtime_env(None, environ={"NCCL_DEBUG": "INFO"})["env_vars"]
    assert "NCCL_DEBUG" not in env and env["TOKENIZERS_PARALLELISM"] == "true"
    cfg = {"global_profiler": {"tool": "torch"}, "trainer": {"disable_nvls": True, "runtime_env": {"env_vars": {"MY_FLAG": 3, "NCCL_DEBUG": "TRACE"}}}}
    env = get_worker_runtime_env(cfg, environ={})["env_vars"]
    assert env["NCCL_NVLS_ENABLE"] == "0" and env["MY_FLAG"] == "3" and env["NCCL_DEBUG"] == "TRACE" and NVTX_INJECTION_ENV in env
    assert "NCCL_NVLS_ENABLE" not in get_worker_runtime_env({"trainer": {}}, environ={})["env_vars"]
