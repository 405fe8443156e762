import datetime
import json
import os

from levanter_b200.infra import cli_helpers, launch
from levanter_b200.main.clean_old_checkpoints import checkpoints_to_delete


def test_torchrun_and_docker_commands():
    cmd = cli_helpers.make_torchrun_command("levanter_b200.main.train_lm", ["--config_path", "x.yaml"], nproc_per_node=8)
    assert cmd[:3] == ["python", "-m", "torch.distributed.run"] and "--nproc-per-node=8" in cmd and cmd[-3:] == ["levanter_b200.main.train_lm", "--config_path", "x.yaml"]
    assert "127.0.0.1" in cmd
    d = cli_helpers.make_docker_run_command("img", cmd, env={"A": "1"}, mounts={"/x": "/y"})
    assert d[:2] == ["docker", "run"] and "A=1" in d and "/x:/y" in d and d[d.index("img") + 1] == "python"


def test_launch_dry_run(monkeypatch, tmp_path, capsys):
    monkeypatch.chdir(tmp_path)
    (tmp_path / ".levanter.yaml").write_text("launch: {nproc_per_node: 2}\nenv: {FOO: bar}\n")
    for k in list(os.environ):
        if k.startswith("SLURM_"):
            monkeypatch.delenv(k)
    assert launch.main(["--dry-run", "--", "levanter_b200.main.train_lm", "--config_path", "c.yaml"]) == 0
    err = capsys.readouterr().err
    assert "--nproc-per-node=2" in err and "levanter_b200.main.train_lm" in err


def test_clean_old_checkpoints_keeps_newest_and_newest_thousand(tmp_path):
    old = datetime.datetime.now() - datetime.timedelta(days=3)
    for step in (500, 1000, 1500, 2000, 2300):
        d = tmp_path / f"step-{step}"
        d.mkdir()
        (d / "metadata.json").write_text(json.dumps({"step": step, "timestamp": old.isoformat()}))
    (tmp_path / "step-2400").mkdir()  # incomplete: no metadata, never touched
    doomed = sorted(os.path.basename(p) for p in checkpoints_to_delete(str(tmp_path), min_age_days=1.0))
    assert doomed == ["step-1000", "step-1500", "step-500"]
    assert checkpoints_to_delete(str(tmp_path), min_age_days=10.0) == []
