import datetime
import json
import os

import pytest

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


def test_a_command_is_rerun_until_it_succeeds(tmp_path):
    import sys

    from levanter_b200.infra.resumable import run_command_resumable

    counter = tmp_path / "count"
    counter.write_text("0")
    script = f"import sys; p = {str(counter)!r}; n = int(open(p).read()) + 1; open(p, 'w').write(str(n)); sys.exit(0 if n >= 3 else 1)"
    retries = []
    rc = run_command_resumable([sys.executable, "-c", script], max_retries_failure=5, backoff_seconds=0, on_retry=lambda kind, n, e: retries.append((kind, n)))
    assert rc == 0 and counter.read_text() == "3" and [n for _, n in retries] == [1, 2]
    counter.write_text("-100")
    import subprocess

    with pytest.raises(subprocess.CalledProcessError):
        run_command_resumable([sys.executable, "-c", script], max_retries_failure=1, backoff_seconds=0)
    assert counter.read_text() == "-98"  # the first try and one retry
