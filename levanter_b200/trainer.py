"""Trainer: configuration, the training step, hooks, and the step loop (src/levanter/trainer.py).

The reference compiles ``_train_step`` into one XLA executable (:552-580).  Here a step is an explicit sequence on CUDA
streams: for each micro-batch ``loss_fn`` forward/backward (weight gradients land in the engine's fp32 accumulator
from the GEMM epilogues), then the sharded engine reduces gradients, clips, runs the optimizer on the owned slices and
republishes compute-dtype weights.  Loss reduction follows the reference: each micro-batch loss is a masked mean and
micro-batches are averaged with equal weight (src/levanter/grad_accum.py:133-134)."""
from __future__ import annotations

import contextlib
import copy
import logging
import os
import random
import string
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, Iterator, List, Mapping, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist
import torch.nn as nn

from . import tracker as trk
from .callbacks._core import Callback, JitCallback, LambdaCallback, StepInfo
from .checkpoint import CheckpointerConfig, load_checkpoint_or_initialize
from .config import Policy
from .distributed import DistributedConfig, RayConfig, broadcast_one_to_all
from .grad_accum import microbatch_slices
from .optim.config import OptimizerConfig, ParamInfo
from .optim.model_averaging import ModelAveragingConfig
from .optim.transforms import GradientTransformation
from .parallel.engine import ShardedEngine
from .parallel.mesh import DeviceMesh, local_device
from .parallel.tp import TensorParallel
from .quantization import QuantizationConfig
from .schedule import BatchSchedule, IntSchedule, ScheduleStep, distinct_values, value_at_step
from .tracker import TrackerConfig
from .tracker.wandb import WandbConfig
from .trainer_state import TrainerState, make_training_key
from .utils.logging import LoadingTimeTrackerIterator, init_logging

from .utils.watchdog import PeerFailure, WatchdogConfig  # noqa: E402

logger = logging.getLogger(__name__)
DEFAULT_JAX_CONFIG: Dict[str, Any] = {"jax_threefry_partitionable": True, "jax_softmax_custom_jvp": True}


@dataclass
class WatchConfig:
    """Norm / histogram logging of grads, params, updates, optimizer state (src/levanter/callbacks/watch.py:24-60)."""

    watch_targets: Union[str, List[str]] = field(default_factory=lambda: ["grads", "params"])
    include_norms: bool = True
    include_per_parameter_norms: bool = True
    include_histograms: bool = False
    split_scan_layers: bool = True
    interval: int = 10

    @property
    def is_enabled(self) -> bool:
        return len(self.watch_targets) > 0 and self.interval > 0 and (self.include_norms or self.include_histograms)

    def build(self):
        from .callbacks.watch import WatchCallback

        return WatchCallback(self)


@dataclass
class _Hook:
    fn: Callback
    every: int


@dataclass
class _JitHook:
    fn: JitCallback
    every: int


class TrainerHooks:
    """Host hooks and in-step hooks, each with a period (src/levanter/trainer.py:89-141)."""

    def __init__(self):
        self.hooks: List[_Hook] = []
        self.stateful_hooks: List[_JitHook] = []

    def run_hooks(self, info: StepInfo, force: bool = False):
        for h in self.hooks:
            if force or info.step % h.every == 0:
                h.fn.on_step(info, force=force)

    def run_jit_hooks_outside_step(self, info: StepInfo, cb_infos: Sequence[Any], force: bool = False):
        for h, cb in zip(self.stateful_hooks, cb_infos):
            if cb is not None and (force or info.step % h.every == 0):
                h.fn.on_step(info, cb)

    def run_jit_hooks(self, state, grads, step: int, force: bool = False) -> List[Any]:
        return [h.fn.inside_step(state, grads) if (force or step % h.every == 0) else None for h in self.stateful_hooks]

    def add_hook(self, fn=None, *, every: int = 1):
        def decorator(f):
            if isinstance(f, Callback):
                self.hooks.append(_Hook(f, every))
            elif isinstance(f, JitCallback):
                self.stateful_hooks.append(_JitHook(f, every))
            else:
                self.hooks.append(_Hook(LambdaCallback(f), every))
            return f

        if fn is None:
            return decorator
        return decorator(fn)


def _round_to_nearest_multiple(x: int, multiple: int) -> int:
    return ((x + multiple - 1) // multiple) * multiple


@dataclass
class TrainerConfig:
    """All trainer keys of the reference (src/levanter/trainer.py:644-737).  JAX-specific keys (``jax_config``,
    ``log_jaxprs``, ``log_xla_hlo``, ``jax_compilation_cache_dir``, ``ray``) are accepted so the same YAML files load."""

    seed: int = 0
    mp: Policy = field(default_factory=lambda: Policy.parse("f32"))
    quantization: Optional[QuantizationConfig] = None
    model_averaging: Optional[ModelAveragingConfig] = None

    wandb: Optional[WandbConfig] = None
    log_dir: Path = Path("logs/")
    id: Optional[str] = None

    tracker: Union[TrackerConfig, Tuple[TrackerConfig, ...], List[TrackerConfig]] = field(default_factory=WandbConfig)
    watch: WatchConfig = field(default_factory=WatchConfig)

    profiler: bool = False
    profiler_start_step: int = 5
    profiler_num_steps: int = 100
    profiler_perfetto_link: bool = False

    log_jaxprs: bool = True
    log_xla_hlo: bool = True

    crash_on_nan: bool = True
    crash_on_inf: bool = True

    batch_axis: str = "batch"
    fsdp_axis: Union[None, str, List[str]] = "embed"
    tensor_parallel_axes: Optional[List[str]] = None
    axis_resources: Dict[str, Any] = field(default_factory=dict)
    parameter_axis_resources: Dict[str, Any] = field(default_factory=dict)

    replica_ici_axis_size: int = 1
    model_axis_size: int = 1
    replica_dcn_axis_size: int = 1

    train_batch_size: Union[int, List[ScheduleStep]] = 512
    per_device_parallelism: int = -1
    per_device_eval_parallelism: int = -1
    allow_nondivisible_batch_size: bool = False

    num_train_steps: int = 400_000
    steps_per_eval: int = 1_000
    max_eval_batches: Optional[int] = None

    checkpointer: CheckpointerConfig = field(default_factory=CheckpointerConfig)
    load_checkpoint: Optional[bool] = None
    load_checkpoint_path: Optional[str] = None
    initialize_from: Optional[str] = None
    allow_partial_checkpoint: bool = False

    jax_config: Dict[str, Any] = field(default_factory=lambda: copy.deepcopy(DEFAULT_JAX_CONFIG))
    jax_compilation_cache_dir: Optional[str] = None

    distributed: DistributedConfig = field(default_factory=DistributedConfig)
    ray: RayConfig = field(default_factory=RayConfig)

    require_accelerator: Optional[bool] = None
    shutdown_at_exit: Union[bool, float] = False

    # knobs of this framework's engine
    watchdog: WatchdogConfig = field(default_factory=WatchdogConfig)
    """host-side failure detection: heartbeat files and a check between steps (off by default)"""
    shard_optimizer: bool = True
    grad_reduce_dtype: str = "float32"
    use_fused_optimizer: Optional[bool] = None
    zero_stage: int = 3
    """3: layer weights exist only as 1/W slices per rank and are gathered layer by layer, weight gradients are
    reduce-scattered as they are produced (needs >1 data rank, a sharded optimizer and bf16 compute; otherwise the engine
    falls back to 1).  1: weights and the fp32 gradient accumulator are whole on every rank, only fp32 master weights and
    optimizer moments are sliced."""
    comm: Optional[str] = None
    """data-parallel collectives: ``multimem`` (NVSwitch multicast loads/stores from the library's own kernels), ``p2p``
    (plain peer loads/stores) or ``nccl``; unset: ``LEVANTER_B200_COMM`` or ``multimem``"""
    tp_comm: Optional[str] = None
    """tensor-parallel all-reduce: ``peer`` (own kernels over symmetric memory) or ``nccl``"""
    ep_comm: Optional[str] = None
    """expert-parallel token exchange: ``peer`` or ``nccl`` (all-to-all)"""
    kernel_wait_limit: float = 2.0
    """seconds after which a device-side wait for a peer gives up (the step loop then raises ``KernelStatusError``); set it
    above the largest host-side skew between ranks"""

    def __post_init__(self):
        if self.wandb is not None:
            import warnings

            warnings.warn("wandb is deprecated. use tracker with type wandb instead", DeprecationWarning)
            self.tracker = self.wandb
        self._mesh: Optional[DeviceMesh] = None

    # -- derived sizes (src/levanter/trainer.py:757-844) ---------------------------------------------------------
    @property
    def num_devices(self) -> int:
        return dist.get_world_size() if (dist.is_available() and dist.is_initialized()) else 1

    @property
    def replica_axis_size(self) -> int:
        return self.replica_dcn_axis_size * self.replica_ici_axis_size

    @property
    def data_axis_size(self) -> int:
        """Number of distinct data shards: devices / model_axis_size (replicas x FSDP shards)."""
        return max(self.num_devices // self.model_axis_size, 1)

    @property
    def fsdp_axis_size(self) -> int:
        return max(self.num_devices // (self.model_axis_size * self.replica_axis_size), 1)

    @property
    def device_mesh(self) -> DeviceMesh:
        if self._mesh is None:
            self._mesh = DeviceMesh(self.replica_axis_size, self.fsdp_axis_size, self.model_axis_size)
        return self._mesh

    @property
    def batch_schedule(self) -> BatchSchedule:
        return BatchSchedule(self.train_batch_size)

    def batch_size_at_step(self, step: int) -> int:
        return value_at_step(self.train_batch_size, step)

    @property
    def microbatch_size(self) -> Optional[int]:
        if self.per_device_parallelism < 0:
            return None
        return self.per_device_parallelism * self.data_axis_size

    @property
    def eval_batch_size(self) -> int:
        return self.per_device_eval_parallelism * self.data_axis_size

    @property
    def run_id(self) -> str:
        assert self.id is not None, "run id is not set yet; call initialize() first"
        return self.id

    @property
    def compute_axis_mapping(self) -> Dict[str, Any]:
        """Logical -> mesh axis map for activations: batch over (replica, data), TP axes over model
        (src/levanter/trainer.py:846-860)."""
        m: Dict[str, Any] = dict(self.axis_resources)
        for ax in self.tensor_parallel_axes or []:
            m[ax] = "model"
        m[self.batch_axis] = ("replica", "data")
        return m

    @property
    def parameter_axis_mapping(self) -> Dict[str, Any]:
        """Logical -> mesh axis map for parameters and optimizer state: compute map + FSDP axis over data (:862-875)."""
        m = dict(self.compute_axis_mapping)
        fsdp = self.fsdp_axis
        if isinstance(fsdp, str):
            m[fsdp] = "data"
        elif isinstance(fsdp, list):
            for ax in fsdp:
                m[ax] = "data"
        m.update(self.parameter_axis_resources)
        return m

    # -- initialisation ------------------------------------------------------------------------------------------
    def initialize(self, all_config=None):
        """Process-level set-up: distributed init, validation, run id, logging, tracker."""
        self.distributed.initialize()
        self.ray.initialize()
        if self.require_accelerator and not torch.cuda.is_available():
            raise RuntimeError("require_accelerator is set but no CUDA device is available")
        self._validate_and_set_defaults()
        self._maybe_set_id()
        init_logging(self.log_dir, self.run_id)
        t = self._make_tracker()
        trk.set_global_tracker(t) if trk.tracker_fns._global_tracker is None else setattr(trk.tracker_fns, "_global_tracker", t)
        if all_config is not None:
            trk.log_configuration(all_config)
        return t

    def _make_tracker(self):
        cfg = self.tracker
        if isinstance(cfg, (list, tuple)):
            return trk.CompositeTracker([c.init(self.run_id) for c in cfg])
        return cfg.init(self.run_id)

    def _maybe_set_id(self):
        """Run id: from config, else a random 8-character id chosen by process 0 and broadcast
        (src/levanter/trainer.py:884-907)."""
        if self.id is None:
            env_id = os.environ.get("WANDB_RUN_ID") or os.environ.get("RUN_ID")
            if env_id:
                self.id = env_id
            else:
                rnd = random.Random(int.from_bytes(os.urandom(8), "little"))
                gen = "".join(rnd.choice(string.ascii_lowercase + string.digits) for _ in range(8))
                self.id = broadcast_one_to_all(gen)
            logger.info(f"Setting run id to {self.id}")

    def _apply_comm_choices(self):
        """Hand the collective choices to the engine, tensor-parallel and expert-parallel layers (they read environment
        variables, so entry points that build those objects without a trainer config still work).  A run with failure
        detection switched on must not use the multicast (``multimem``) paths: a rank that dies while its memory is bound to
        a multicast object takes its peers' GPUs with it, whereas plain peer accesses and NCCL fail on their own rank only."""
        for key, val in (("LEVANTER_B200_COMM", self.comm), ("LEVANTER_B200_TP_COMM", self.tp_comm), ("LEVANTER_B200_EP_COMM", self.ep_comm)):
            if val is not None:
                os.environ[key] = str(val).lower()
        if self.watchdog.enabled:
            chosen = os.environ.get("LEVANTER_B200_COMM")
            if chosen is None:
                os.environ["LEVANTER_B200_COMM"] = "p2p"
            elif chosen.lower() == "multimem":
                raise ValueError("watchdog.enabled needs comm: p2p or nccl (multicast mappings do not survive the loss of a rank)")
        if torch.cuda.is_available():
            from .ops import lib

            lib.set_wait_limit(self.kernel_wait_limit)

    def _validate_and_set_defaults(self):
        n = self.num_devices
        self._apply_comm_choices()
        if n % self.model_axis_size != 0:
            raise ValueError(f"num_devices ({n}) is not divisible by model_axis_size ({self.model_axis_size})")
        if self.train_batch_size == -1 and self.per_device_parallelism == -1:
            raise ValueError("either train_batch_size or per_device_parallelism must be specified (not -1)")
        if self.per_device_parallelism == -1:
            if isinstance(self.train_batch_size, int):
                self.per_device_parallelism = max(self.train_batch_size // self.data_axis_size, 1)
            else:
                logger.info("per_device_parallelism is not set and train_batch_size is a schedule; not microbatching")
        if self.train_batch_size == -1:
            self.train_batch_size = self.per_device_parallelism * self.data_axis_size
        if self.per_device_parallelism != -1 and not self.allow_nondivisible_batch_size:
            mb = self.per_device_parallelism * self.data_axis_size
            if isinstance(self.train_batch_size, int):
                if self.train_batch_size % mb != 0:
                    raise ValueError(f"train_batch_size ({self.train_batch_size}) must be divisible by per_device_parallelism * "
                                     f"data_axis_size ({self.per_device_parallelism}, {self.data_axis_size})")
            else:
                for phase in self.train_batch_size:
                    if phase.value % mb != 0:
                        raise ValueError(f"At step {phase.start}, train_batch_size ({phase.value}) must be divisible by "
                                         f"per_device_parallelism * data_axis_size ({self.per_device_parallelism}, {self.data_axis_size})")
        if self.per_device_eval_parallelism == -1:
            if self.per_device_parallelism == -1:
                tbs = max(distinct_values(self.train_batch_size))
                self.per_device_eval_parallelism = _round_to_nearest_multiple(tbs, self.data_axis_size) // self.data_axis_size
            else:
                self.per_device_eval_parallelism = self.per_device_parallelism
        if self.replica_dcn_axis_size == -1:
            self.replica_dcn_axis_size = 1


LossFn = Callable[..., torch.Tensor]


class Trainer:
    """Owns the loop.  ``loss_fn(model, batch, **kw) -> scalar`` (default: next-token loss of an ``LmExample``)."""

    def __init__(self, config: TrainerConfig, optimizer: Union[GradientTransformation, OptimizerConfig],
                 loss_fn: Optional[LossFn] = None, *, add_default_hooks: bool = True):
        self.hooks = TrainerHooks()
        self.config = config
        if isinstance(optimizer, OptimizerConfig):
            self.optimizer_config: Optional[OptimizerConfig] = optimizer
            self.optimizer: Optional[GradientTransformation] = None
        else:
            self.optimizer_config = None
            self.optimizer = optimizer
        if loss_fn is None:
            from .models.lm_model import compute_next_token_loss

            loss_fn = compute_next_token_loss
        self.loss_fn = loss_fn
        self._raw_loss_fn = loss_fn
        if isinstance(config.tracker, (list, tuple)):
            self.tracker = None
        self.tracker = None
        self._add_default_hooks = add_default_hooks
        self._cmanagers: List[Any] = []
        self._checkpointer = None
        self.device = local_device()
        self._pending_jit_metrics: Dict[str, Any] = {}

    # -- context -------------------------------------------------------------------------------------------------
    @property
    def mp(self) -> Policy:
        return self.config.mp

    @property
    def run_id(self) -> str:
        return self.config.run_id

    @property
    def num_train_steps(self) -> int:
        return self.config.num_train_steps

    @property
    def device_mesh(self) -> DeviceMesh:
        return self.config.device_mesh

    @property
    def tensor_parallel(self) -> Optional[TensorParallel]:
        return TensorParallel.from_mesh(self.device_mesh)

    @property
    def parameter_axis_mapping(self):
        return self.config.parameter_axis_mapping

    @property
    def compute_axis_mapping(self):
        return self.config.compute_axis_mapping

    @property
    def checkpointer(self):
        if self._checkpointer is None:
            self._checkpointer = self.config.checkpointer.create(self.run_id)
        return self._checkpointer

    def __enter__(self):
        if self.config.id is None:
            self.config._maybe_set_id()
        if trk.tracker_fns._global_tracker is None:
            self.tracker = self.config._make_tracker()
            cm = trk.current_tracker(self.tracker)
            cm.__enter__()
            self._cmanagers.append(cm)
        else:
            self.tracker = trk.tracker_fns._global_tracker
        return self

    def __exit__(self, *exc):
        for cm in reversed(self._cmanagers):
            cm.__exit__(*exc)
        self._cmanagers = []
        if self._checkpointer is not None:
            self._checkpointer.wait_until_finished()

    # -- hooks ---------------------------------------------------------------------------------------------------
    def add_hook(self, fn=None, *, every: int = 1):
        return self.hooks.add_hook(fn, every=every)

    def add_eval_hook(self, eval_dataset, name: Optional[str] = None):
        from . import callbacks

        loader = self.data_loader(eval_dataset, self.config.eval_batch_size)
        if eval_dataset:
            self.add_hook(callbacks.compute_validation_loss(self.loss_fn, loader, max_batches=self.config.max_eval_batches,
                                                            name=name, device=self.device), every=self.config.steps_per_eval)

    def _install_default_hooks(self):
        from . import callbacks

        self.add_hook(callbacks.pbar_logger(total=self.config.num_train_steps), every=1)
        self.add_hook(callbacks.log_step_info(self.config.num_train_steps), every=1)
        if self.config.profiler:
            self.add_hook(callbacks.profile(str(self.config.log_dir / self.run_id / "profiler"), self.config.profiler_start_step,
                                            self.config.profiler_num_steps, self.config.profiler_perfetto_link), every=1)
        self.add_hook(self.checkpointer.on_step, every=1)
        if self.config.watch.is_enabled:
            self.add_hook(self.config.watch.build(), every=self.config.watch.interval)

    # -- state ---------------------------------------------------------------------------------------------------
    def initial_state(self, training_key: Union[int, torch.Tensor], model: Optional[nn.Module] = None,
                      model_init: Optional[Callable[[], nn.Module]] = None, *,
                      is_trainable: Optional[Callable[[str], bool]] = None) -> TrainerState:
        """Build (or load) the training state.  Exactly one of ``model`` / ``model_init`` is given.  If a checkpoint is
        found under ``load_checkpoint_path`` (per ``load_checkpoint``) it is restored on top of the fresh state
        (src/levanter/trainer.py:295-368)."""
        if (model is None) == (model_init is None):
            raise ValueError("only one of model and model_init should be specified")
        if model is None:
            model = model_init()
        cfg = self.config
        model = model.to(self.device)
        if cfg.quantization is not None:
            from .quantization import quantize_linear_layers

            model = quantize_linear_layers(model, cfg.quantization)
        mesh = self.device_mesh if cfg.num_devices > 1 else None
        needs_full = self.optimizer_config is not None and getattr(self.optimizer_config, "needs_full_tensors", False)
        engine = ShardedEngine(model, cfg.mp, mesh, device=self.device,
                               shard_optimizer=cfg.shard_optimizer and not needs_full,
                               grad_reduce_dtype=Policy.parse(cfg.grad_reduce_dtype).param_dtype, is_trainable=is_trainable,
                               zero_stage=cfg.zero_stage)
        info = ParamInfo(model)
        if self.optimizer is None:
            self.optimizer = self.optimizer_config.build(cfg.num_train_steps, info)
        engine.set_optimizer(self.optimizer, optimizer_config=self.optimizer_config, num_train_steps=cfg.num_train_steps,
                             use_fused=cfg.use_fused_optimizer)
        key = make_training_key(training_key) if isinstance(training_key, int) else training_key
        avg = cfg.model_averaging.create(engine.master_tree()) if cfg.model_averaging is not None else None
        state = TrainerState(step=0, model=model, engine=engine, training_key=key, mp=cfg.mp, model_averaging=avg,
                             is_trainable=is_trainable)
        state = load_checkpoint_or_initialize(state, self.checkpoint_path, force_load=cfg.load_checkpoint,
                                              allow_partial=cfg.allow_partial_checkpoint, initialize_from=cfg.initialize_from)
        return state

    @property
    def checkpoint_path(self) -> str:
        """Where this run looks for a checkpoint to resume from: ``load_checkpoint_path`` or the checkpointer's run directory."""
        return self.config.load_checkpoint_path or self.config.checkpointer.expanded_path(self.run_id)

    def write_artifact(self, name: str, artifact, type: Optional[str] = None) -> str:
        """Write ``artifact`` (text or bytes) to ``<log_dir>/<run id>/artifacts/<name>`` and hand the file to the tracker
        (src/levanter/trainer.py:600-615).  A name ending in ``.gz`` / ``.zst`` is compressed on the way."""
        import fsspec

        directory = os.path.join(str(self.config.log_dir), self.run_id, "artifacts")
        os.makedirs(directory, exist_ok=True)
        path = os.path.join(directory, name)
        with fsspec.open(path, "w" if isinstance(artifact, str) else "wb", compression="infer") as f:
            f.write(artifact)
        trk.current_tracker().log_artifact(path, name=name, type=type)
        return path

    # -- data ----------------------------------------------------------------------------------------------------
    def data_loader(self, dataset, batch=None, **kw):
        from .data.loader import DataLoader

        if batch is None:
            batch = self.config.batch_schedule
        return DataLoader(dataset, batch, mesh=self.device_mesh if self.config.num_devices > 1 else None,
                          allow_nondivisible_batch_size=self.config.allow_nondivisible_batch_size, **kw)

    # -- the step ------------------------------------------------------------------------------------------------
    def _microbatches(self, batch, step: int) -> List[Any]:
        cfg = self.config
        n_local = _batch_len(batch)
        if cfg.per_device_parallelism is None or cfg.per_device_parallelism < 0:
            return [batch]
        # the global micro-batch is per_device_parallelism * data_axis_size examples: per_device_parallelism per rank
        return [_batch_slice(batch, a, b) for a, b in microbatch_slices(n_local, cfg.per_device_parallelism)]

    def device_step(self, state: TrainerState, batch, **batch_kwargs):
        """The device part of a step: forward/backward over the micro-batches, gradient reduction, optimizer update,
        weight republication.  Returns ``(loss, jit_metrics, hook_infos)`` with the loss still on the device (no
        host synchronisation happens here)."""
        model, engine = state.model, state.engine
        model.train()
        seed = state.next_key()
        batch = _to_device(batch, self.device)
        micro = self._microbatches(batch, state.step)
        n_micro = len(micro)
        loss_acc = torch.zeros((), dtype=torch.float32, device=self.device)
        with trk.defer_tracker_for_jit() as jit_metrics:
            needs_rng = _has_active_dropout(model)
            for i, mb in enumerate(micro):
                with (_seeded(seed + i, self.device) if needs_rng else contextlib.nullcontext()):
                    loss = self.loss_fn(model, mb, **batch_kwargs)
                loss = loss.mean() if loss.dim() > 0 else loss
                (loss / n_micro).backward()
                loss_acc += loss.detach().float() / n_micro
            cb_infos = None
            if self.hooks.stateful_hooks:
                engine.collect_grads()
                cb_infos = self.hooks.run_jit_hooks(state, engine, state.step)
                engine.capture_updates = any(c is not None and h.fn.wants_updates for h, c in zip(self.hooks.stateful_hooks, cb_infos))
            extra = {}
            if getattr(self.optimizer_config, "needs_objective", False):
                extra["obj_fn"] = self._batch_objective(model, micro, batch_kwargs)
            if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                # before the optimizer sees it: a wrapper that judges the step by its loss (skip-step) must reach the same
                # verdict on every rank, so it gets the loss of the whole batch, not of this rank's part
                dist.all_reduce(loss_acc, op=dist.ReduceOp.AVG)
            engine.step(loss=loss_acc, **extra)
            if cb_infos is not None and engine.last_updates is not None:
                cb_infos = [h.fn.after_update(state, engine, c) if (c is not None and h.fn.wants_updates) else c
                            for h, c in zip(self.hooks.stateful_hooks, cb_infos)]
                engine.last_updates = None
            if state.model_averaging is not None:
                state.model_averaging.update(engine.master_tree(), state.step)
            if engine.fused_adam is not None:
                trk.jit_log({"optim/learning_rate": engine.fused_adam.learning_rate})
            else:
                trk.helpers.log_optimizer_hyperparams(engine.opt_state, "optim")
            if engine.last_grad_norm is not None:
                trk.jit_log({"grad/norm/total": engine.last_grad_norm})
        state.step += 1
        return loss_acc, jit_metrics, cb_infos

    def _batch_objective(self, model: nn.Module, micro: List[Any], batch_kwargs) -> Callable[[Dict[str, torch.Tensor]], torch.Tensor]:
        """``params -> loss of this step's batch`` for optimizers that differentiate the objective themselves (Sophia's
        Hutchinson estimate; the reference builds the same closure, src/levanter/trainer.py:561-568).  The parameters of the
        tree (master dtype, full tensors) are cast to the compute dtype and substituted into the model; the pass runs on the
        differentiable PyTorch statements of the ops, because it is differentiated twice."""
        from torch.nn.utils.stateless import _reparametrize_module

        from .ops import lib

        cd = self.config.mp.compute_dtype
        loss_fn = self.loss_fn

        def obj_fn(params: Dict[str, torch.Tensor]) -> torch.Tensor:
            cast = {k: (v.to(cd) if v.is_floating_point() else v) for k, v in params.items() if v is not None}
            total = None
            with lib.reference_ops(), _reparametrize_module(model, cast, tie_weights=True):
                for mb in micro:
                    loss = loss_fn(model, mb, **batch_kwargs)
                    loss = loss.mean() if loss.dim() > 0 else loss
                    total = loss if total is None else total + loss
            return total / len(micro)

        return obj_fn

    def train_step(self, state: TrainerState, batch, **batch_kwargs) -> StepInfo:
        """One optimizer step on ``batch`` (this rank's shard of the global batch, in pinned host memory or on the
        device), followed by the host part: loss read-back, NaN/Inf checks, hooks and metric logging."""
        t0 = time.perf_counter()
        loss_acc, jit_metrics, cb_infos = self.device_step(state, batch, **batch_kwargs)
        loss_val = loss_acc.item()  # device -> host: the one synchronisation per step
        if self.device.type == "cuda":
            from .ops import lib

            lib.check_status()  # a bounded wait that ran out left wrong values behind: stop here, not many steps later
        if self.config.crash_on_nan and loss_val != loss_val:
            raise RuntimeError("Loss is NaN")
        if self.config.crash_on_inf and loss_val in (float("inf"), float("-inf")):
            raise RuntimeError("Loss is Inf")
        info = StepInfo(state, loss_val, time.perf_counter() - t0)
        with trk.helpers.capture_time() as hook_time:
            self.hooks.run_hooks(info)
            if cb_infos is not None:
                self.hooks.run_jit_hooks_outside_step(info, cb_infos)
        metrics = dict(jit_metrics)
        metrics["throughput/hook_time"] = hook_time()
        trk.log(metrics, step=info.step)
        return info

    def training_steps(self, state: TrainerState, train_loader: Iterable) -> Iterator[StepInfo]:
        """Generator over steps until ``num_train_steps`` (src/levanter/trainer.py:415-433)."""
        iter_data = LoadingTimeTrackerIterator(iter(train_loader))
        watchdog = self._start_watchdog()
        try:
            while int(state.step) < self.num_train_steps:
                with trk.helpers.capture_time() as loading_time:
                    try:
                        example = next(iter_data)
                    except StopIteration:
                        logger.info("Reached end of training data loader")
                        break
                if watchdog is not None:
                    watchdog.raise_if_failed()  # before anything is launched that would wait for a missing peer
                info = self.train_step(state, example)
                if watchdog is not None:
                    watchdog.beat(info.step)
                trk.log({"throughput/loading_time": loading_time()}, step=info.step)
                yield info
        except BaseException as e:
            if watchdog is not None and not isinstance(e, (GeneratorExit, PeerFailure)):
                watchdog.mark_failed(f"{type(e).__name__}: {e}")
            raise
        finally:
            if watchdog is not None:
                watchdog.stop()

    def _start_watchdog(self):
        import torch.distributed as dist

        rank = dist.get_rank() if (dist.is_available() and dist.is_initialized()) else 0
        world = dist.get_world_size() if (dist.is_available() and dist.is_initialized()) else 1
        wd = self.config.watchdog.build(rank, world, str(self.config.log_dir / self.run_id / "heartbeats"))
        return wd.start() if wd is not None else None

    def train(self, state: TrainerState, train_loader: Iterable) -> StepInfo:
        if self._add_default_hooks:
            self._install_default_hooks()
            self._add_default_hooks = False
        info = None
        for info in self.training_steps(state, train_loader):
            pass
        if info is not None:
            self.hooks.run_hooks(info, force=True)
            self.checkpointer.wait_until_finished()
        return info


def initialize(config) -> None:
    """``levanter_b200.initialize(config)``: process-level set-up from a config that has a ``trainer`` field, or from a
    ``TrainerConfig`` (src/levanter/trainer.py:974-983)."""
    trainer_config = config.trainer if hasattr(config, "trainer") else config
    trainer_config.initialize(config)


# ---------------------------------------------------------------------------------------------------- batch helpers
def _batch_len(batch) -> int:
    if hasattr(batch, "tokens"):
        return batch.tokens.shape[0]
    if isinstance(batch, torch.Tensor):
        return batch.shape[0]
    if isinstance(batch, (tuple, list)):
        return _batch_len(batch[0])
    if isinstance(batch, dict):
        return _batch_len(next(iter(batch.values())))
    if hasattr(batch, "batch_size"):
        return batch.batch_size
    raise TypeError(f"cannot determine the batch size of {type(batch)}")


def _batch_slice(batch, a: int, b: int):
    if hasattr(batch, "slice"):
        return batch.slice(a, b)
    if isinstance(batch, torch.Tensor):
        return batch[a:b]
    if isinstance(batch, tuple):
        return tuple(_batch_slice(x, a, b) for x in batch)
    if isinstance(batch, list):
        return [_batch_slice(x, a, b) for x in batch]
    if isinstance(batch, dict):
        return {k: _batch_slice(v, a, b) for k, v in batch.items()}
    return batch


def _to_device(batch, device):
    if hasattr(batch, "to") and not isinstance(batch, torch.Tensor):
        return batch.to(device, non_blocking=True)
    if isinstance(batch, torch.Tensor):
        return batch.to(device, non_blocking=True)
    if isinstance(batch, tuple):
        return tuple(_to_device(x, device) for x in batch)
    if isinstance(batch, list):
        return [_to_device(x, device) for x in batch]
    if isinstance(batch, dict):
        return {k: _to_device(v, device) for k, v in batch.items()}
    return batch


def _has_active_dropout(model: nn.Module) -> bool:
    cached = getattr(model, "_lvb_has_dropout", None)
    if cached is None:
        cached = any(getattr(m, "p", 0.0) > 0.0 for m in model.modules() if type(m).__name__ == "Dropout")
        try:
            model._lvb_has_dropout = cached
        except Exception:
            pass
    return cached


@contextlib.contextmanager
def _seeded(seed: int, device):
    """Deterministic RNG stream for one micro-batch (dropout); the ambient RNG state is restored afterwards."""
    devs = [device] if torch.device(device).type == "cuda" else []
    with torch.random.fork_rng(devices=devs):
        torch.manual_seed(seed)
        yield
