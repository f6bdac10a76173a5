"""The training pipeline operator around a trainer - epochs, callbacks, evaluation, best / step / final checkpoints,
interruption - and the curriculum and multi-task operators (reference tools/train/pipeline.py:103-690).

Interruption: the reference's SIGINT handler sleeps for a second INSIDE the handler and raises from it
(pipeline.py:515-540), so the exception lands wherever the main thread happens to be - in the middle of an optimizer
step, or of a collective that the other ranks are still in.  Here the handler only records the press; the loop looks at
the record BETWEEN steps, so a stop always leaves a finished step behind (no rank abandons a collective, the final
checkpoint is consistent).  One press asks for a full stop, a second press within ``double_press_window`` seconds turns
it into "skip the current dataset"."""
from __future__ import annotations

import signal
import threading
import time
from datetime import datetime
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, List, Optional, Union

import torch

from ..utils.opsc import PiscesLxOperatorInterface
from .train_config import PiscesLxTrainingConfig


class PiscesLxTrainingInterruption(Exception):
    SKIP_DATASET = "skip_dataset"
    FULL_STOP = "full_stop"

    def __init__(self, mode: str = "full_stop", message: str = ""):
        self.mode, self.message = mode, message
        super().__init__(message or f"Training interrupted: {mode}")

    @classmethod
    def skip_current_dataset(cls, reason: str = "") -> "PiscesLxTrainingInterruption":
        return cls(cls.SKIP_DATASET, reason)

    @classmethod
    def stop_all(cls, reason: str = "") -> "PiscesLxTrainingInterruption":
        return cls(cls.FULL_STOP, reason)


class _InterruptState:
    """Presses of the interrupt key, recorded by the handler and read by the loop."""

    def __init__(self, double_press_window: float = 1.0, clock: Callable[[], float] = time.monotonic):
        self.window, self.clock = double_press_window, clock
        self.presses: List[float] = []

    def press(self) -> None:
        self.presses.append(self.clock())

    def handler(self, signum: int, frame: Any) -> None:
        self.press()

    def pending(self) -> Optional[str]:
        """None, or the mode asked for.  A single press only counts once the window for a second one has passed (or at
        once when ``window`` is 0)."""
        if not self.presses:
            return None
        if len(self.presses) >= 2 and self.presses[-1] - self.presses[-2] <= self.window:
            return PiscesLxTrainingInterruption.SKIP_DATASET
        if self.clock() - self.presses[-1] >= self.window:
            return PiscesLxTrainingInterruption.FULL_STOP
        return None

    def clear(self) -> None:
        self.presses.clear()


class PiscesLxTrainingPipelineOperator(PiscesLxOperatorInterface):
    """``PiscesLxTrainingPipelineOperator(config, trainer).fit(train_batches, val_batches, epochs)``.  ``trainer`` needs
    ``train_step(batch) -> {"loss", "grad_norm", "throughput", ...}``, ``global_step`` and ``model``; ``save_checkpoint(path,
    metadata=)`` and ``load_checkpoint(path)`` are used when it has them, ``engine.checkpoint`` otherwise.

    Callback stages: training_start, epoch_start, batch_end, checkpoint_saved, evaluation_start, evaluation_end, epoch_end,
    training_end.  A callback is ``callback(stage, **kwargs)``; one that raises is reported in ``callback_errors`` and
    does not stop the run."""

    name = "training_pipeline_operator"

    def __init__(self, config: Optional[Union[PiscesLxTrainingConfig, Dict[str, Any], str]] = None, trainer: Any = None,
                 install_signal_handler: bool = True):
        self.train_config = self._normalize_train_config(config)
        self.trainer = trainer
        self.callbacks: List[Callable] = []
        self.callback_errors: List[str] = []
        self.interrupts = _InterruptState()
        self.install_signal_handler = install_signal_handler
        self._evals_without_gain = 0

    @staticmethod
    def _normalize_train_config(config: Any) -> PiscesLxTrainingConfig:
        if config is None:
            return PiscesLxTrainingConfig()
        if isinstance(config, PiscesLxTrainingConfig):
            return config
        if isinstance(config, dict):
            return PiscesLxTrainingConfig.from_dict(config)
        if isinstance(config, (str, Path)):
            import yaml
            return PiscesLxTrainingConfig.from_dict(yaml.safe_load(Path(config).read_text()) or {})
        params = getattr(config, "parameters", None)
        if isinstance(params, dict):
            return PiscesLxTrainingConfig.from_dict(params)
        raise TypeError(f"cannot make a training configuration from {type(config).__name__}")

    # -- callbacks -----------------------------------------------------------------------------------------------------------------
    def add_callback(self, callback: Callable) -> None:
        if callback not in self.callbacks:
            self.callbacks.append(callback)

    def remove_callback(self, callback: Callable) -> None:
        if callback in self.callbacks:
            self.callbacks.remove(callback)

    def execute_callbacks(self, stage: str, **kwargs: Any) -> None:
        for cb in list(self.callbacks):
            try:
                cb(stage, **kwargs)
            except PiscesLxTrainingInterruption:
                raise
            except Exception as e:
                self.callback_errors.append(f"{stage}: {type(e).__name__}: {e}")

    # -- checkpoints ----------------------------------------------------------------------------------------------------------------
    def _save(self, path: Path, metadata: Optional[Dict[str, Any]] = None) -> str:
        path.parent.mkdir(parents=True, exist_ok=True)
        if hasattr(self.trainer, "save_checkpoint"):
            self.trainer.save_checkpoint(str(path), metadata=metadata)
        else:
            from .checkpoint import save_checkpoint
            save_checkpoint(self.trainer, str(path), metadata=metadata)
        self.execute_callbacks("checkpoint_saved", path=str(path), global_step=self.trainer.global_step)
        return str(path)

    def _check_interrupt(self) -> None:
        mode = self.interrupts.pending()
        if mode is not None:
            self.interrupts.clear()
            raise PiscesLxTrainingInterruption(mode, "requested from the keyboard")

    # -- loops ---------------------------------------------------------------------------------------------------------------------
    def train_epoch(self, dataloader: Iterable, epoch: int) -> Dict[str, float]:
        cfg, tr = self.train_config, self.trainer
        out = Path(cfg.resolved_output_dir())
        tot = {"loss": 0.0, "grad_norm": 0.0, "throughput": 0.0}
        n = 0
        last_saved = last_eval = -1
        self.execute_callbacks("epoch_start", epoch=epoch)
        for batch_idx, batch in enumerate(dataloader):
            res = tr.train_step(batch)
            n += 1
            for k in tot:
                tot[k] += float(res.get(k) or 0.0)
            self.execute_callbacks("batch_end", batch_idx=batch_idx, step_result=res)
            step = int(tr.global_step)
            if step > 0 and cfg.save_steps > 0 and step % cfg.save_steps == 0 and step != last_saved:
                self._save(out / f"checkpoint_step_{step}.pt")
                last_saved = step
            if step > 0 and cfg.eval_steps > 0 and step % cfg.eval_steps == 0 and step != last_eval:
                last_eval = step
                self.execute_callbacks("evaluation_start", global_step=step)
            if cfg.max_steps > 0 and step >= cfg.max_steps:                            # a budget of optimizer steps, not of epochs
                break
            self._check_interrupt()
        stats = {"epoch": epoch, "total_loss": tot["loss"], "batch_count": n, "avg_loss": tot["loss"] / max(n, 1),
                 "avg_grad_norm": tot["grad_norm"] / max(n, 1), "avg_throughput": tot["throughput"] / max(n, 1)}
        self.execute_callbacks("epoch_end", epoch_stats=stats)
        return stats

    @torch.no_grad()
    def evaluate(self, dataloader: Iterable, metrics: Optional[List[str]] = None) -> Dict[str, float]:
        """Mean loss, perplexity and (with ``"accuracy"`` in ``metrics``) next-token accuracy over the labelled positions;
        the sums stay on the device until the end."""
        model = self.trainer.model
        was = model.training
        model.eval()
        dev = next(model.parameters()).device
        want_acc = metrics is not None and "accuracy" in metrics
        loss_sum, n, hit, cnt = torch.zeros((), device=dev), 0, torch.zeros((), device=dev), torch.zeros((), device=dev)
        for batch in dataloader:
            ids = batch["input_ids"].to(dev)
            labels = batch.get("labels", batch["input_ids"]).to(dev)
            out = model(input_ids=ids, labels=labels, return_logits=True) if want_acc else model(input_ids=ids, labels=labels)
            loss = out["loss"] if isinstance(out, dict) else out.loss
            loss_sum += loss.float()
            n += 1
            if want_acc:
                h, c = self._compute_accuracy(out, labels)
                hit += h
                cnt += c
        model.train(was)
        mean = float(loss_sum / max(n, 1))
        res = {"eval_loss": mean, "eval_perplexity": float(torch.exp(torch.tensor(min(mean, 30.0)))), "eval_batches": n}
        if want_acc:
            res["eval_accuracy"] = float(hit / cnt.clamp_min(1))
        self.execute_callbacks("evaluation_end", eval_stats=res)
        return res

    @staticmethod
    def _compute_accuracy(outputs: Any, labels: torch.Tensor):
        lg = outputs["logits"] if isinstance(outputs, dict) else outputs.logits
        pred, tgt = lg[:, :-1].argmax(-1), labels[:, 1:]
        m = tgt != -100
        return ((pred == tgt) & m).sum().float(), m.sum().float()

    def fit(self, train_dataloader: Iterable, val_dataloader: Optional[Iterable] = None, epochs: int = 1, resume_from: Optional[str] = None) -> Dict[str, Any]:
        cfg, tr = self.train_config, self.trainer
        out = Path(cfg.resolved_output_dir())
        self.interrupts.clear()
        old = None
        if self.install_signal_handler and threading.current_thread() is threading.main_thread():
            old = signal.signal(signal.SIGINT, self.interrupts.handler)
        if resume_from:
            if hasattr(tr, "load_checkpoint"):
                tr.load_checkpoint(resume_from)
            else:
                from .checkpoint import load_checkpoint
                load_checkpoint(tr, resume_from)
        hist: Dict[str, Any] = {"epochs": [], "evaluations": [], "best_checkpoint": None, "training_start_time": datetime.now().isoformat()}
        self.execute_callbacks("training_start", total_epochs=epochs, max_steps=cfg.max_steps)
        try:
            for epoch in range(epochs):
                hist["epochs"].append(self.train_epoch(train_dataloader, epoch))
                if val_dataloader is not None:
                    ev = self.evaluate(val_dataloader)
                    hist["evaluations"].append(ev)
                    if ev["eval_loss"] < getattr(tr, "best_metric", float("inf")):
                        tr.best_metric = ev["eval_loss"]
                        hist["best_checkpoint"] = self._save(out / "best_model.pt", {"is_best": True})
                        self._evals_without_gain = 0
                    else:
                        self._evals_without_gain += 1
                        if cfg.early_stopping_patience and self._evals_without_gain >= cfg.early_stopping_patience:
                            hist["early_stopped"] = True
                            break
                if cfg.max_steps > 0 and tr.global_step >= cfg.max_steps:
                    break
        except PiscesLxTrainingInterruption as e:
            hist["interrupted"], hist["interruption_type"] = True, e.mode
            raise
        except KeyboardInterrupt:
            hist["interrupted"], hist["interruption_type"] = True, "keyboard"
            raise
        finally:
            if old is not None:
                signal.signal(signal.SIGINT, old)
            hist["final_checkpoint"] = self._save(out / "final_model.pt", {"is_final": True})
            hist["training_end_time"] = datetime.now().isoformat()
            self.last_history = hist
            self.execute_callbacks("training_end", training_history=hist)
        return hist

    def fit_datasets(self, dataloaders: Dict[str, Iterable], val_dataloader: Optional[Iterable] = None, epochs: int = 1) -> Dict[str, Any]:
        """One ``fit`` per named dataset in turn; "skip the current dataset" moves on to the next one, a full stop ends all."""
        out: Dict[str, Any] = {"datasets": {}, "skipped": []}
        for name, dl in dataloaders.items():
            try:
                out["datasets"][name] = self.fit(dl, val_dataloader, epochs)
            except PiscesLxTrainingInterruption as e:
                out["datasets"][name] = getattr(self, "last_history", {})
                if e.mode == PiscesLxTrainingInterruption.SKIP_DATASET:
                    out["skipped"].append(name)
                    continue
                out["stopped_at"] = name
                break
            if self.train_config.max_steps > 0 and self.trainer.global_step >= self.train_config.max_steps:
                break
        return out

    # -- operator front --------------------------------------------------------------------------------------------------------------
    def transform(self, data: Dict[str, Any]) -> Dict[str, Any]:
        return data

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return self.trainer is not None and inputs.get("train_dataloader") is not None

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        return self.fit(inputs["train_dataloader"], inputs.get("val_dataloader"), int(inputs.get("epochs", 1)), inputs.get("resume_from"))


class PiscesLxCurriculumLearningOperator(PiscesLxOperatorInterface):
    """Stages of rising difficulty.  ``difficulty_schedule`` is a list of stage dictionaries (``name``, ``dataloader_args``,
    optional ``min_steps`` / ``max_steps`` / ``target_loss``).  A stage ends when its loss has PLATEAUED - the relative gain
    over the last ``patience`` reports is under ``min_improvement`` - or reached ``target_loss``, or ``max_steps`` passed;
    never before ``min_steps``.  (The reference advances while the loss is still FALLING by 2 % a report, pipeline.py:
    587-610, i.e. it leaves a stage exactly when the stage is still teaching.)"""

    name = "curriculum_learning_operator"

    def __init__(self, config: Any = None, difficulty_schedule: Optional[List[Dict[str, Any]]] = None, min_improvement: float = 0.02):
        if difficulty_schedule is None and config is not None:
            params = config if isinstance(config, dict) else (getattr(config, "parameters", {}) or {})
            difficulty_schedule = params.get("difficulty_schedule")
            min_improvement = params.get("min_improvement", min_improvement)
        self.difficulty_schedule = list(difficulty_schedule or [])
        self.min_improvement = min_improvement
        self.current_stage = 0
        self.stage_metrics: List[Dict[str, float]] = []
        self.stage_steps = 0
        self.history: List[Dict[str, Any]] = []

    def transform(self, data: Dict[str, Any]) -> Dict[str, Any]:
        return data

    @property
    def stage_config(self) -> Dict[str, Any]:
        return self.difficulty_schedule[self.current_stage] if self.difficulty_schedule else {}

    @property
    def is_last_stage(self) -> bool:
        return self.current_stage >= len(self.difficulty_schedule) - 1

    def get_current_dataloader(self, base_dataloader_factory: Callable) -> Any:
        return base_dataloader_factory(**self.stage_config.get("dataloader_args", {}))

    def should_advance_stage(self, current_metrics: Dict[str, float], patience: int = 3) -> bool:
        self.stage_metrics.append(dict(current_metrics))
        self.stage_steps += int(current_metrics.get("steps", 1))
        if self.is_last_stage:
            return False
        st = self.stage_config
        if self.stage_steps < int(st.get("min_steps", 0)):
            return False
        if "max_steps" in st and self.stage_steps >= int(st["max_steps"]):
            return True
        loss = current_metrics.get("loss")
        if loss is not None and "target_loss" in st and loss <= float(st["target_loss"]):
            return True
        if len(self.stage_metrics) < patience + 1:
            return False
        recent = [m["loss"] for m in self.stage_metrics[-(patience + 1):] if "loss" in m]
        if len(recent) < patience + 1:
            return False
        gain = (recent[0] - min(recent[1:])) / max(abs(recent[0]), 1e-12)
        return gain < self.min_improvement

    def advance_stage(self) -> bool:
        if self.is_last_stage:
            return False
        self.history.append({"stage": self.current_stage, "name": self.stage_config.get("name"), "steps": self.stage_steps,
                             "final_loss": next((m["loss"] for m in reversed(self.stage_metrics) if "loss" in m), None)})
        self.current_stage += 1
        self.stage_metrics, self.stage_steps = [], 0
        return True

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return "metrics" in inputs

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        advanced = self.should_advance_stage(inputs["metrics"], int(inputs.get("patience", 3))) and self.advance_stage()
        return {"advanced": bool(advanced), "current_stage": self.current_stage, "stage": self.stage_config, "history": list(self.history)}

    def state_dict(self) -> Dict[str, Any]:
        return {"current_stage": self.current_stage, "stage_metrics": list(self.stage_metrics), "stage_steps": self.stage_steps, "history": list(self.history)}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.current_stage, self.stage_metrics = int(sd["current_stage"]), list(sd.get("stage_metrics", []))
        self.stage_steps, self.history = int(sd.get("stage_steps", 0)), list(sd.get("history", []))


class PiscesLxMultiTaskTrainingOperator(PiscesLxOperatorInterface):
    """Weighted sum of the tasks' losses.  The per-task values are kept as detached tensors and only turned into numbers
    when ``get_task_metrics`` is asked (the reference calls ``.item()`` on every task's loss in every step, pipeline.py:
    667).  For weights LEARNED from the tasks' uncertainty see ``optim.multitask_modality``."""

    name = "multi_task_training_operator"

    def __init__(self, config: Any = None, task_weights: Optional[Dict[str, float]] = None, normalize: bool = False):
        if task_weights is None and config is not None:
            params = config if isinstance(config, dict) else (getattr(config, "parameters", {}) or {})
            task_weights = params.get("task_weights")
        self.task_weights = dict(task_weights or {})
        self.normalize = normalize
        self._last: Dict[str, torch.Tensor] = {}

    def transform(self, data: Dict[str, Any]) -> Dict[str, Any]:
        return data

    def compute_multi_task_loss(self, task_outputs: Dict[str, Any]) -> torch.Tensor:
        total, wsum = None, 0.0
        self._last = {}
        for task, out in task_outputs.items():
            loss = out.get("loss") if isinstance(out, dict) else getattr(out, "loss", out if isinstance(out, torch.Tensor) else None)
            if loss is None:
                continue
            w = float(self.task_weights.get(task, 1.0))
            term = loss * w
            total = term if total is None else total + term
            wsum += w
            self._last[task] = term.detach()
        if total is None:
            raise ValueError("no task produced a loss")
        return total / wsum if (self.normalize and wsum > 0) else total

    def get_task_metrics(self) -> Dict[str, float]:
        if not self._last:
            return {}
        vals = torch.stack([v.float().reshape(()) for v in self._last.values()]).tolist()      # one read for all tasks
        return dict(zip(self._last.keys(), vals))

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return isinstance(inputs.get("task_outputs"), dict)

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        return {"loss": self.compute_multi_task_loss(inputs["task_outputs"])}
