"""Weights & Biases tracker (src/levanter/tracker/wandb.py:35-236).  Only process 0 logs online; other processes run
``offline`` and share the run id and group; the git SHA and a pip freeze are attached to the run."""
from __future__ import annotations

import logging
import os
import tempfile
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Union

from .helpers import generate_pip_freeze, infer_experiment_git_root
from .tracker import Tracker, TrackerConfig

logger = logging.getLogger(__name__)


class WandbTracker(Tracker):
    name = "wandb"

    def __init__(self, run):
        import wandb

        self.run = run if run is not None else (wandb.run or wandb.init())
        self._last_warning_step = -500

    def log_hyperparameters(self, hparams: Dict[str, Any]):
        self.run.config.update(hparams, allow_val_change=True)

    def log(self, metrics, *, step, commit=None):
        if step is None and not commit:
            step = self.run.step
        if step is not None and step < self.run.step:
            if step - self._last_warning_step > 500:
                logger.warning(f"Step {step} is less than the current step {self.run.step}. Cowardly refusing to log metrics.")
                self._last_warning_step = step
            return
        self.run.log({k: _convert(v) for k, v in metrics.items()}, step=step, commit=commit)

    def log_summary(self, metrics):
        self.run.summary.update(metrics)

    def log_artifact(self, artifact_path, *, name=None, type=None):
        self.run.log_artifact(str(artifact_path), name=name, type=type)

    def finish(self):
        self.run.finish()


def _convert(v):
    from .histogram import Histogram

    if isinstance(v, Histogram):
        import wandb

        counts, limits = v.to_numpy_histogram()
        return wandb.Histogram(np_histogram=(counts.tolist(), limits.tolist()))
    return v


def is_wandb_available() -> bool:
    try:
        import wandb  # noqa: F401

        return True
    except ImportError:
        return False


@TrackerConfig.register_subclass("wandb")
@dataclass
class WandbConfig(TrackerConfig):
    entity: Optional[str] = None
    project: Optional[str] = "levanter"
    name: Optional[str] = None
    tags: List[str] = field(default_factory=list)
    id: Optional[str] = None
    group: Optional[str] = None
    mode: Optional[str] = None
    resume: Optional[Union[bool, str]] = "allow"
    save_code: Union[bool, str] = True
    save_xla_dumps: bool = False

    def init(self, run_id: Optional[str]) -> Tracker:
        import wandb

        if run_id is not None and self.id is not None and run_id != self.id:
            logger.warning(f"Both trainer's id {run_id} and WandB's id {self.id} are set. WandB will use the id set in its own config.")
        wid = self.id if self.id is not None else run_id
        hparams = {}
        git_settings = self._git_settings()
        if "git_commit" in git_settings:
            hparams["git_commit"] = git_settings["git_commit"]
        rank = int(os.environ.get("RANK", "0"))
        mode = self.mode
        if rank != 0 and mode is None:
            mode = "offline"
        if mode is None and os.environ.get("WANDB_API_KEY") is None and os.environ.get("WANDB_MODE") is None:
            # no credentials and no explicit mode: stay usable on machines without network access
            mode = "offline"
        code_dir = None
        if isinstance(self.save_code, str):
            code_dir = self.save_code
        elif self.save_code:
            code_dir = infer_experiment_git_root() or "."
        run = wandb.init(entity=self.entity, project=self.project, name=self.name, tags=self.tags, id=wid, group=self.group,
                         resume=self.resume, mode=mode, config=hparams, settings=git_settings or None, allow_val_change=True)
        if code_dir is not None and rank == 0:
            try:
                run.log_code(code_dir)
            except Exception:
                logger.debug("could not log code", exc_info=True)
        if rank == 0:
            try:
                with tempfile.TemporaryDirectory() as tmpdir:
                    req = os.path.join(tmpdir, "requirements.txt")
                    with open(req, "w") as f:
                        f.write(generate_pip_freeze())
                    if wandb.run is not None:
                        wandb.run.log_artifact(req, name="requirements.txt", type="requirements")
            except Exception:
                logger.debug("could not log pip freeze", exc_info=True)
        return WandbTracker(run)

    def _git_settings(self):
        other = {}
        root = infer_experiment_git_root()
        if root:
            other["code_dir"] = root
            other["git_root"] = root
            try:
                import subprocess

                sha = subprocess.check_output(["git", "rev-parse", "HEAD"], cwd=root, text=True, stderr=subprocess.DEVNULL).strip()
                other["git_commit"] = sha
            except Exception:
                pass
        return other
