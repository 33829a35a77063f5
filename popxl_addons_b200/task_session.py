"""`TaskSession`: a session that knows the named streams and the named state of a training / inference task and can
checkpoint and restore that state.

Checkpoint layout (compatible with popxl_addons/task_session.py:128-283):
  <dir>/model/<dotted.name>.npz   one file per state variable; the array inside is stored under the same name.
                                   Variables backed by a numpy memmap are copied as `<dotted.name>.npy` instead.
  <dir>/dataloader.bin             written by `dataloader.save(path)` when a dataloader is attached
  <dir>/session_info.json          the `session_state` dict (always contains "steps")
Arrays have the variables' host shapes: a leading replica-group axis when groups differ, and replica-sharded
variables re-assembled to their full shape. In a multi-process run every rank takes part in gathering, rank 0 writes.
"""
import glob
import json
import logging
import os
import shutil
import tempfile
from collections import deque
from typing import Any, Dict, Mapping, Optional, Union

import numpy as np

from . import xl
from .named_tensors import NamedTensorData, NamedTensors
from .streams import InputStreams, OutputStreams
from .variable_factory import open_variable_file
from .utils import timer

try:  # optional
    import wandb  # type: ignore
except Exception:  # pragma: no cover
    wandb = None

__all__ = ["TaskSession", "write_variables_pb", "initialise_memmap_dir_from_checkpoint"]

logger = logging.getLogger(__name__)
_WANDB_PREFIX = "wandb://"


def write_variables_pb(session: xl.Session, weights: Mapping[xl.Tensor, np.ndarray]):
    """Write many variables with a progress bar."""
    try:
        from tqdm import tqdm

        items = tqdm(list(weights.items()), desc="Writing variables")
    except Exception:  # pragma: no cover
        items = list(weights.items())
    for var, data in items:
        session.write_variable_data(var, data)


def _rank() -> int:
    return int(os.environ.get("RANK", "0"))


class TaskSession(xl.Session):
    def __init__(self, inputs: Union[InputStreams, Any], outputs: Union[OutputStreams, Any], state: NamedTensors,
                 max_checkpoints: int = 1, *args, **kwargs):
        """`inputs` / `outputs`: the task's host streams; `state`: every variable that makes up a checkpoint.
        Remaining arguments go to `Session(ir, device_desc)`."""
        with timer("Session creation"):
            super().__init__(*args, **kwargs)
        self.inputs = inputs if isinstance(inputs, InputStreams) else InputStreams.from_streams(
            {getattr(s, "name", str(i)): s for i, s in enumerate(inputs)})
        self.outputs = outputs if isinstance(outputs, OutputStreams) else OutputStreams.from_streams(
            {getattr(s, "name", str(i)): s for i, s in enumerate(outputs)})
        self.state = state
        self.session_state: Dict[str, Any] = {"steps": 0}
        self.max_checkpoints = max_checkpoints
        self._saved = deque()
        self._dataloader = None

    # -- dataloader -----------------------------------------------------------------------------------------
    @property
    def dataloader(self):
        return self._dataloader

    @dataloader.setter
    def dataloader(self, dl):
        if not (hasattr(dl, "save") and hasattr(dl, "resume")):
            raise ValueError("The dataloader must provide `save(path)` and `resume(path)` to be checkpointed")
        self._dataloader = dl

    def add_session_state_info(self, info: Dict):
        """Extra JSON-serialisable entries stored in `session_info.json`."""
        if "steps" in info:
            raise ValueError("`steps` is maintained by the session")
        self.session_state.update(info)

    # -- state access -----------------------------------------------------------------------------------------
    def _owned_state(self) -> Dict[str, Any]:
        """State variables this process holds: all of them, unless replicas span several processes (pipeline
        stages), in which case every process holds the variables of its device slot."""
        return {k: v for k, v in self.state.to_dict().items() if self.owns(v)}

    def _is_writer(self) -> bool:
        """Whether this process writes checkpoint files: the process(es) of replica 0 (one per device slot)."""
        if self.slot is None:
            return _rank() == 0
        return self.comm.rank == 0

    def get_named_tensors_data(self) -> NamedTensorData:
        named = self._owned_state()
        data = self.get_tensors_data(list(named.values()))
        return NamedTensorData.from_dict({k: data[t] for k, t in named.items()})

    def load_from_session(self, src: "TaskSession", report_missing: str = "none"):
        """Copy the state of another session into this one, matching variables by name."""
        self._load_named(src.get_named_tensors_data().to_dict(), report_missing)

    def wandb_histogram(self, name: str, step: int, data: np.ndarray):
        if wandb is None or wandb.run is None:
            return
        data = np.asarray(data, dtype=np.float32).reshape(-1)
        finite = data[np.isfinite(data)]
        # key names as in popxl_addons/task_session.py:115-121, so dashboards built for one read the other
        wandb.log({f"{name}:histogram": wandb.Histogram(finite), f"{name}:not_finite": int(data.size - finite.size)},
                  step=step)

    def wandb_variable_histograms(self, step: int = 0):
        for name, data in self.get_named_tensors_data().to_dict().items():
            self.wandb_histogram(name, step, np.asarray(data, dtype=np.float32))

    # -- checkpoints ------------------------------------------------------------------------------------------
    def save_checkpoint(self, checkpoint_dir: str):
        """Write a checkpoint. `wandb://<name>` uploads it as a W&B artifact instead of keeping a directory.
        At most `max_checkpoints` directories written by this session are kept (oldest removed first).
        Collective when the session spans several processes: every rank must call it."""
        with timer("Fetching state for checkpoint", log_to_wandb=False):
            data = self.get_named_tensors_data().to_dict()  # collective: all ranks
        writer = self._is_writer()
        with timer("Saving checkpoint", log_to_wandb=False):
            if checkpoint_dir.startswith(_WANDB_PREFIX):
                if not writer:
                    return
                if wandb is None:
                    raise RuntimeError("wandb is not installed")
                name = checkpoint_dir[len(_WANDB_PREFIX):]
                with tempfile.TemporaryDirectory() as tmp:
                    self._write_model_files(tmp, data)
                    self._write_completion_marker(tmp)
                    # the artifact type popxl_addons/task_session.py:152,197 saves and looks up
                    artifact = wandb.Artifact(name=name, type="checkpoints")
                    artifact.add_dir(tmp)
                    wandb.log_artifact(artifact)
                return
            if writer:
                self._write_model_files(checkpoint_dir, data)
            if self.slot is not None:
                # one writer per device slot: `session_info.json` marks the checkpoint as complete, so it may only
                # appear (and an older checkpoint may only go) once every slot's files are on disk
                self.comm.barrier()
            if _rank() == 0:
                self._write_completion_marker(checkpoint_dir)
                self._saved.append(checkpoint_dir)
                while self.max_checkpoints and len(self._saved) > self.max_checkpoints:
                    old = self._saved.popleft()
                    if os.path.isdir(old) and os.path.abspath(old) != os.path.abspath(checkpoint_dir):
                        logger.info("Removing old checkpoint %s", old)
                        shutil.rmtree(old, ignore_errors=True)
            if self.slot is not None:
                self.comm.barrier()  # the checkpoint is complete when any process returns

    def _write_model_files(self, checkpoint_dir: str, data: Dict[str, np.ndarray]):
        model_dir = os.path.join(checkpoint_dir, "model")
        os.makedirs(model_dir, exist_ok=True)
        named = self.state.to_dict()
        for name, array in data.items():
            init = self.ir.initial_values.get(named[name])
            if isinstance(init, np.memmap) and getattr(init, "filename", None):
                # memmap-backed variables keep their file name and raw layout (as in the reference, which copies the
                # memmap file), so the file can be put back into a memmap directory and mapped again
                np.ascontiguousarray(np.asarray(array), dtype=init.dtype).tofile(
                    os.path.join(model_dir, os.path.basename(str(init.filename))))
            else:
                np.savez(os.path.join(model_dir, f"{name}.npz"), **{name: array})

    def _write_completion_marker(self, checkpoint_dir: str):
        """The files a checkpoint has once; `session_info.json` comes last and appears atomically: a directory that
        has it is a complete checkpoint (`parallel.elastic.latest_checkpoint` relies on that)."""
        os.makedirs(checkpoint_dir, exist_ok=True)
        if self._dataloader is not None:
            self._dataloader.save(os.path.join(checkpoint_dir, "dataloader.bin"))
        tmp = os.path.join(checkpoint_dir, f".session_info.json.tmp{os.getpid()}")
        with open(tmp, "w") as f:
            json.dump(self.session_state, f)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, os.path.join(checkpoint_dir, "session_info.json"))

    def load_checkpoint(self, checkpoint_dir: str, report_missing: str = "warn", skip_memmap: bool = False):
        """Restore state from a checkpoint directory (or `wandb://artifact`). `report_missing`: what to do when the
        checkpoint and the session's state disagree on the set of variables: `none`, `warn` or `error`."""
        with timer("Loading checkpoint", log_to_wandb=False):
            if checkpoint_dir.startswith(_WANDB_PREFIX):
                if wandb is None:
                    raise RuntimeError("wandb is not installed")
                artifact = wandb.use_artifact(checkpoint_dir[len(_WANDB_PREFIX):], type="checkpoints")
                checkpoint_dir = artifact.download()
            self._read_checkpoint(checkpoint_dir, report_missing, skip_memmap)

    def _read_checkpoint(self, checkpoint_dir: str, report_missing: str, skip_memmap: bool):
        model_dir = os.path.join(checkpoint_dir, "model")
        if not os.path.isdir(model_dir):
            raise FileNotFoundError(f"No `model` directory in checkpoint {checkpoint_dir}")
        loaded: Dict[str, np.ndarray] = {}
        for path in sorted(glob.glob(os.path.join(model_dir, "*.npz"))):
            name = os.path.basename(path)[:-4]
            with np.load(path, allow_pickle=True) as z:
                loaded[name] = z[name] if name in z.files else z[z.files[0]]
        if not skip_memmap:
            # files of memmap-backed variables are named after the variable's memmap file
            by_file = {}
            for key, var in self.state.to_dict().items():
                mm = getattr(var, "_memmap_arr", None)
                fname = os.path.basename(str(mm.filename)) if mm is not None and getattr(mm, "filename", None) else None
                by_file[fname or f"{key}.npy"] = (key, var)
            for path in sorted(glob.glob(os.path.join(model_dir, "*.npy"))):
                if os.path.basename(path) in by_file:
                    key, var = by_file[os.path.basename(path)]
                    loaded[key] = open_variable_file(path, var.dtype.as_numpy(), var.shape_on_host, "r")
                else:
                    loaded[os.path.basename(path)[:-4]] = np.load(path, mmap_mode="r")
        self._load_named(loaded, report_missing)
        dl_path = os.path.join(checkpoint_dir, "dataloader.bin")
        if self._dataloader is not None and os.path.exists(dl_path):
            self._dataloader.resume(dl_path)
        info_path = os.path.join(checkpoint_dir, "session_info.json")
        if os.path.exists(info_path):
            with open(info_path) as f:
                self.session_state = json.load(f)
        else:
            logger.warning("No session_info.json in %s: starting from step 0", checkpoint_dir)
            self.session_state = {"steps": 0}
        self.session_state.setdefault("steps", 0)

    def _load_named(self, loaded: Mapping[str, np.ndarray], report_missing: str):
        if report_missing not in ("none", "warn", "error"):
            raise ValueError(f"report_missing must be one of none, warn, error. Not: {report_missing}")
        named = self._owned_state()
        missing = sorted(set(named) - set(loaded))
        extra = sorted(set(loaded) - set(self.state.to_dict()))
        if (missing or extra) and report_missing != "none":
            msg = ""
            if missing:
                msg += f"Variables of the session that are not in the loaded state: {missing}. "
            if extra:
                msg += f"Entries of the loaded state that match no variable of the session: {extra}."
            if report_missing == "error":
                raise ValueError(msg)
            logger.warning(msg)
        self.write_variables_data({named[k]: np.asarray(v) for k, v in loaded.items() if k in named})

    # -- running ----------------------------------------------------------------------------------------------
    def run(self, inputs: Optional[Mapping] = None, downcast_inputs: bool = True, fetch: bool = True):
        self.session_state["steps"] += 1
        return super().run(inputs or {}, downcast_inputs, fetch)


def initialise_memmap_dir_from_checkpoint(checkpoint_dir: str, memmap_dir: str):
    """Copy the `.npy` files of a checkpoint into `memmap_dir`, ready for `factories.init(memmap_dir=...)`."""
    os.makedirs(memmap_dir, exist_ok=True)
    for path in glob.glob(os.path.join(checkpoint_dir, "model", "*.npy")):
        shutil.copy(path, os.path.join(memmap_dir, os.path.basename(path)))
