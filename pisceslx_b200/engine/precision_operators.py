"""Low-precision and sharded training as configured operators (reference opss/train/fp8.py:67-630,
opss/optim/fp4.py:91-800, opss/train/fsdp.py:59-440).

The numerics live in ``quant/fp8.py`` (block-scaled and MX e4m3 / e5m2 linears, delayed scaling) and ``quant/fp4.py`` (E2M1
quantiser, straight-through linear, packed-weight trainer); these operators convert a model's linears to them and run
the loop.  On a B200 the FP8 linear of choice is the MX form (``YvFP8GemmLinear``: one power-of-two scale per 32 elements
applied by the tensor cores themselves, no amax history and no rescaling pass); the block-scaled ``YvFP8Linear`` is the
portable form and the one a host run uses.

The reference's FP8 operator needs NVIDIA's transformer-engine package and refuses to run without it (fp8.py:246-262);
nothing here depends on it."""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from ..utils.opsc import PiscesLxOperatorInterface
from .stage_operators import PiscesLxSFTDataset, _batches, _lr_at, _to_device, causal_lm_loss

SKIP_DEFAULT = ("lm_head", "embed", "router", "gate")


def _replace_linears(model: nn.Module, make: Callable[[nn.Linear, str], Optional[nn.Module]], skip: Sequence[str] = SKIP_DEFAULT) -> List[str]:
    done: List[str] = []
    for name, mod in list(model.named_modules()):
        for child_name, child in list(mod.named_children()):
            full = f"{name}.{child_name}" if name else child_name
            if type(child) is nn.Linear and not any(s in full for s in skip):
                new = make(child, full)
                if new is not None:
                    setattr(mod, child_name, new)
                    done.append(full)
    return done


# ---- FP8 ------------------------------------------------------------------------------------------------------------------------
@dataclass
class PiscesLxFP8TrainingConfig:
    fp8_format: str = "hybrid"                    # e4m3 forward, e5m2 gradients ("e4m3": both e4m3)
    amax_history_len: int = 1024
    amax_compute_algo: str = "max"
    scaling: str = "auto"                         # "mx" | "delayed" | "block" | "auto" (mx on a GPU when shapes allow, else block)
    coat_enabled: bool = True
    coat_amax_epsilon: float = 1e-3
    coat_scale_factor: float = 1.0
    mixed_grain_activation: bool = True
    per_tensor_threshold: int = 1024
    per_group_size: int = 128
    model_path: str = ".pisceslx/ckpt"
    output_dir: str = ".pisceslx/ckpt"
    train_data: str = "./data/train.jsonl"
    batch_size: int = 32
    micro_batch_size: int = 1
    gradient_accumulation_steps: int = 4
    learning_rate: float = 1e-5
    max_steps: int = 100000
    max_grad_norm: float = 1.0
    warmup_steps: int = 1000
    min_lr_ratio: float = 0.1
    weight_decay: float = 0.1
    adam_beta: Tuple[float, float] = (0.9, 0.999)
    adam_eps: float = 1e-8
    use_fused_adamw: bool = False
    checkpoint_interval: int = 5000
    checkpoint_dir: str = ".pisceslx/ckpt"
    save_optimizer_state: bool = True
    load_optimizer_state: bool = False
    resume_from: Optional[str] = None
    max_seq_length: int = 2048
    log_interval: int = 10
    seed: int = 0
    skip_modules: Tuple[str, ...] = SKIP_DEFAULT

    def __post_init__(self) -> None:
        self.max_grad_norm = float(self.max_grad_norm)           # the reference declares this field as a string ("1.0")
        if self.fp8_format not in ("hybrid", "e4m3"):
            raise ValueError(f"unknown fp8_format {self.fp8_format}")
        if self.scaling not in ("auto", "mx", "delayed", "block"):
            raise ValueError(f"unknown scaling {self.scaling}")


class PiscesLxFP8TextDataset(PiscesLxSFTDataset):
    """``.jsonl`` records or plain text for the low-precision operators (the reference's fp8 ``PiscesLxTextDataset``,
    fp8.py:152-220; the data-module class of that name is ``data.datamodule.PiscesLxTextDataset``)."""

    def __init__(self, file_path: str, tokenizer: Any = None, max_length: int = 2048):
        p = Path(file_path)
        if p.suffix in (".txt", ".md"):
            recs = [{"text": t} for t in p.read_text(encoding="utf-8").split("\n\n") if t.strip()]
            super().__init__(recs, tokenizer, max_length)
        else:
            super().__init__(file_path, tokenizer, max_length)


class PiscesLxFP8TrainingOperator(PiscesLxOperatorInterface):
    """``execute({"model", "config", "train_dataset" | "train_records" | config.train_data, "tokenizer"?, "optimizer"?})``:
    converts the model's linears to fp8 linears (``convert``), then trains."""

    name = "fp8_training"

    def __init__(self) -> None:
        self.hardware = self._check_hardware()

    @staticmethod
    def _check_hardware() -> Dict[str, Any]:
        """What the device can do; no requirement is enforced here - the block-scaled form runs anywhere."""
        if not torch.cuda.is_available():
            return {"cuda": False, "fp8_tensor_cores": False, "mx_block_scaling": False}
        major, minor = torch.cuda.get_device_capability()
        return {"cuda": True, "capability": f"{major}.{minor}", "fp8_tensor_cores": (major, minor) >= (8, 9), "mx_block_scaling": major >= 10}

    def _create_fp8_recipe(self, config: PiscesLxFP8TrainingConfig) -> Dict[str, Any]:
        scaling = config.scaling
        if scaling == "auto":
            scaling = "mx" if self.hardware.get("mx_block_scaling") else "block"
        return {"forward": "e4m3", "backward": "e5m2" if config.fp8_format == "hybrid" else "e4m3", "scaling": scaling,
                "amax_history_len": config.amax_history_len, "amax_compute_algo": config.amax_compute_algo}

    def convert(self, model: nn.Module, config: PiscesLxFP8TrainingConfig) -> List[str]:
        from ..quant.fp8 import YvFP8GemmLinear, YvFP8Linear
        recipe = self._create_fp8_recipe(config)

        def make(lin: nn.Linear, name: str) -> Optional[nn.Module]:
            if config.mixed_grain_activation and lin.weight.numel() < config.per_tensor_threshold:
                return None                                                            # tiny layers stay in the compute dtype
            dev = lin.weight.device
            if recipe["scaling"] in ("mx", "delayed") and dev.type == "cuda" and lin.bias is None and lin.in_features % 16 == 0 and lin.out_features % 16 == 0:
                new = YvFP8GemmLinear(lin.in_features, lin.out_features, dev, min(config.amax_history_len, 1024),
                                      "auto" if recipe["scaling"] == "mx" else "delayed")
                with torch.no_grad():
                    new.weight.copy_(lin.weight)
                return new
            new = YvFP8Linear(lin.in_features, lin.out_features, lin.bias is not None, lin.weight.dtype).to(dev)
            with torch.no_grad():
                new.weight.copy_(lin.weight)
                if lin.bias is not None:
                    new.bias.copy_(lin.bias)
            return new
        done = _replace_linears(model, make, config.skip_modules)
        if config.coat_enabled:
            self._apply_coat_scaling(model, config)
        return done

    def _apply_coat_scaling(self, model: nn.Module, config: PiscesLxFP8TrainingConfig) -> int:
        """Dynamic-range expansion of stored optimizer-side values needs no module change here; what the model side of it
        asks for is that no converted weight has a block whose largest magnitude is under ``coat_amax_epsilon`` of the
        tensor's (such a block would land in e4m3's subnormals): those weights are counted and reported."""
        from ..quant.fp8 import YvFP8Linear
        flagged = 0
        for m in model.modules():
            if isinstance(m, YvFP8Linear):
                w = m.weight.detach().float()
                C = (w.shape[1] // config.per_group_size) * config.per_group_size
                if C:
                    amax = w[:, :C].reshape(w.shape[0], -1, config.per_group_size).abs().amax(-1)
                    flagged += int((amax < config.coat_amax_epsilon * amax.max()).sum())
        self.coat_flagged_blocks = flagged
        return flagged

    def _create_optimizer(self, model: nn.Module, config: PiscesLxFP8TrainingConfig) -> torch.optim.Optimizer:
        decay = [p for n, p in model.named_parameters() if p.requires_grad and p.dim() >= 2]
        rest = [p for n, p in model.named_parameters() if p.requires_grad and p.dim() < 2]
        groups = [g for g in ({"params": decay, "weight_decay": config.weight_decay}, {"params": rest, "weight_decay": 0.0}) if g["params"]]
        if config.use_fused_adamw:
            from ..optim import YvFusedAdamW
            return YvFusedAdamW(groups, lr=config.learning_rate, betas=tuple(config.adam_beta), eps=config.adam_eps)
        return torch.optim.AdamW(groups, lr=config.learning_rate, betas=tuple(config.adam_beta), eps=config.adam_eps)

    @staticmethod
    def _save_checkpoint(path: Path, model: nn.Module, optimizer: torch.optim.Optimizer, step: int, save_optimizer: bool = True) -> str:
        path.parent.mkdir(parents=True, exist_ok=True)
        tmp = path.with_suffix(".tmp")
        torch.save({"model_state_dict": model.state_dict(), "optimizer_state_dict": optimizer.state_dict() if save_optimizer else None, "global_step": step}, tmp)
        tmp.replace(path)
        return str(path)

    @staticmethod
    def _load_checkpoint(path: str, model: nn.Module, optimizer: Optional[torch.optim.Optimizer], load_optimizer: bool = False) -> int:
        d = torch.load(path, map_location="cpu", weights_only=False)
        model.load_state_dict(d["model_state_dict"])
        if load_optimizer and optimizer is not None and d.get("optimizer_state_dict") is not None:
            optimizer.load_state_dict(d["optimizer_state_dict"])
        return int(d.get("global_step", 0))

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return isinstance(inputs.get("model"), nn.Module)

    def _dataset(self, inputs: Dict[str, Any], cfg: Any) -> Any:
        if inputs.get("train_dataset") is not None:
            return inputs["train_dataset"]
        if inputs.get("train_records") is not None:
            return PiscesLxSFTDataset(inputs["train_records"], inputs.get("tokenizer"), cfg.max_seq_length)
        if Path(cfg.train_data).exists():
            return PiscesLxFP8TextDataset(cfg.train_data, inputs.get("tokenizer"), cfg.max_seq_length)
        raise ValueError(f"no training data: give train_dataset / train_records or a file at {cfg.train_data}")

    def _train(self, model: nn.Module, opt: torch.optim.Optimizer, ds: Any, cfg: Any, start: int = 0, after_step: Optional[Callable[[int], None]] = None) -> Dict[str, Any]:
        device = next(model.parameters()).device
        params = [p for p in model.parameters() if p.requires_grad]
        stream = _batches(ds, cfg.micro_batch_size, getattr(ds, "collate"), cfg.seed)
        model.train()
        hist: List[Dict[str, float]] = []
        window, n, saved = torch.zeros((), device=device), 0, []
        t0 = time.time()
        for step in range(start, cfg.max_steps):
            lr = _lr_at(step, cfg.learning_rate, cfg.warmup_steps, cfg.max_steps, getattr(cfg, "min_lr_ratio", 0.1))
            for g in opt.param_groups:
                g["lr"] = lr
            opt.zero_grad(set_to_none=True)
            for _ in range(cfg.gradient_accumulation_steps):
                batch = _to_device(next(stream), device)
                loss = causal_lm_loss(model, batch)
                (loss / cfg.gradient_accumulation_steps).backward()
                window += loss.detach().float()
                n += 1
            if cfg.max_grad_norm > 0:
                torch.nn.utils.clip_grad_norm_(params, cfg.max_grad_norm)
            opt.step()
            if after_step is not None:
                after_step(step + 1)
            done = step + 1
            if done % max(getattr(cfg, "log_interval", 10), 1) == 0 or done == cfg.max_steps:
                hist.append({"step": done, "loss": float(window / max(n, 1)), "lr": lr})
                window.zero_()
                n = 0
            if cfg.checkpoint_interval > 0 and done % cfg.checkpoint_interval == 0:
                saved.append(self._save_checkpoint(Path(cfg.checkpoint_dir) / f"{self.name}_step_{done}.pt", model, opt, done, getattr(cfg, "save_optimizer_state", True)))
        return {"steps": cfg.max_steps - start, "history": hist, "final_loss": hist[-1]["loss"] if hist else None, "first_loss": hist[0]["loss"] if hist else None,
                "checkpoints": saved, "seconds": time.time() - t0}

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        model: nn.Module = inputs["model"]
        cfg: PiscesLxFP8TrainingConfig = inputs.get("config") or PiscesLxFP8TrainingConfig()
        converted = self.convert(model, cfg) if inputs.get("convert", True) else []
        opt = inputs.get("optimizer") or self._create_optimizer(model, cfg)
        start = self._load_checkpoint(cfg.resume_from, model, opt, cfg.load_optimizer_state) if cfg.resume_from else 0
        out = self._train(model, opt, self._dataset(inputs, cfg), cfg, start)
        return {**out, "converted_layers": converted, "recipe": self._create_fp8_recipe(cfg), "hardware": self.hardware,
                "coat_flagged_blocks": getattr(self, "coat_flagged_blocks", 0), "model": model}


class PiscesLxFP8Operator(PiscesLxFP8TrainingOperator):
    name = "fp8"


# ---- FP4 ------------------------------------------------------------------------------------------------------------------------
@dataclass
class PiscesLxFP4Config:
    name: str = "fp4"
    block_size: int = 16
    stochastic_rounding: bool = True
    master_weights_dtype: str = "fp32"
    gradient_accumulation_dtype: str = "fp16"
    amax_history_length: int = 256
    use_dynamic_scaling: bool = True
    scale_update_interval: int = 100
    activation_dtype: str = "fp8"
    weight_dtype: str = "fp4"
    gradient_dtype: str = "fp8"
    compute_dtype: str = "bf16"
    enable_gradient_checkpointing: bool = True
    model_path: str = ".pisceslx/ckpt"
    output_dir: str = ".pisceslx/ckpt"
    train_data: str = "./data/train.jsonl"
    batch_size: int = 32
    micro_batch_size: int = 1
    gradient_accumulation_steps: int = 4
    learning_rate: float = 1e-5
    max_steps: int = 100000
    max_grad_norm: float = 1.0
    warmup_steps: int = 1000
    min_lr_ratio: float = 0.1
    weight_decay: float = 0.1
    checkpoint_interval: int = 5000
    checkpoint_dir: str = ".pisceslx/ckpt"
    save_optimizer_state: bool = True
    max_seq_length: int = 2048
    log_interval: int = 10
    seed: int = 0
    storage: str = "master"                       # "master": fp32 master + fp4 forward (straight-through); "packed": weights stored as 4-bit codes
    skip_modules: Tuple[str, ...] = SKIP_DEFAULT

    def __post_init__(self) -> None:
        if self.block_size not in (16, 32, 64, 128):
            raise ValueError("block_size must be 16, 32, 64 or 128")
        if self.storage not in ("master", "packed"):
            raise ValueError(f"unknown storage {self.storage}")
        if self.master_weights_dtype not in ("fp32", "bf16"):
            raise ValueError("master weights are fp32 or bf16")


class PiscesLxFP4Operator(PiscesLxFP8TrainingOperator):
    """Weights in E2M1 with a scale per ``block_size`` elements.  ``storage="master"`` keeps fp32 master weights and
    quantises in the forward pass with a straight-through gradient; ``storage="packed"`` stores the weights themselves as
    packed 4-bit codes and applies every update with stochastic rounding (``quant.fp4.PiscesLxQuartetTrainer``).
    Gradients can be rounded to e5m2 stochastically before the optimizer sees them (``gradient_dtype="fp8"``)."""

    name = "fp4"

    def convert(self, model: nn.Module, config: PiscesLxFP4Config) -> List[str]:      # type: ignore[override]
        from ..quant.fp4 import PiscesLxFP4Linear

        def make(lin: nn.Linear, name: str) -> Optional[nn.Module]:
            if lin.bias is not None:
                return None
            new = PiscesLxFP4Linear(lin.in_features, lin.out_features, config.block_size, config.stochastic_rounding).to(lin.weight.device)
            with torch.no_grad():
                new.weight.copy_(lin.weight.float())
            return new
        return _replace_linears(model, make, config.skip_modules)

    @staticmethod
    def _stochastic_round_to_fp8(tensor: torch.Tensor, generator: Optional[torch.Generator] = None) -> torch.Tensor:
        """Unbiased rounding to e5m2 (per-tensor scale to the format's range): the value moves to one of its two neighbours on
        the e5m2 grid with probabilities proportional to the distances, so that the expectation is the value itself."""
        x = tensor.float()
        amax = x.abs().amax().clamp_min(1e-30)
        s = 57344.0 / amax
        y = x * s
        e = torch.floor(torch.log2(y.abs().clamp_min(2.0 ** -14))).clamp_min(-14.0)                    # binade; below 2^-14 the grid is the subnormal one
        step = torch.exp2(e - 2.0)                                                                     # two mantissa bits
        mag_lo = torch.floor(y.abs() / step) * step
        lo, hi = torch.sign(y) * mag_lo, torch.sign(y) * (mag_lo + step)
        frac = ((y.abs() - mag_lo) / step).clamp(0, 1)
        u = torch.rand(y.shape, generator=generator).to(y.device) if generator is not None else torch.rand_like(y)
        return (torch.where(u < frac, hi, lo) / s).to(tensor.dtype)

    def _quantize_gradients_to_fp8(self, model: nn.Module, generator: Optional[torch.Generator] = None) -> int:
        n = 0
        for p in model.parameters():
            if p.grad is not None and p.grad.dim() >= 2:
                p.grad.copy_(self._stochastic_round_to_fp8(p.grad, generator))
                n += 1
        return n

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        model: nn.Module = inputs["model"]
        cfg: PiscesLxFP4Config = inputs.get("config") or PiscesLxFP4Config()
        ds = self._dataset(inputs, cfg)
        if cfg.storage == "packed":
            from ..quant.fp4 import PiscesLxQuartetTrainer
            qt = PiscesLxQuartetTrainer(model, cfg.block_size, tuple(cfg.skip_modules))
            rest = [p for n, p in model.named_parameters() if p.requires_grad and "weight_shadow" not in n]
            opt = inputs.get("optimizer") or (torch.optim.AdamW(rest, lr=cfg.learning_rate, weight_decay=0.0) if rest else torch.optim.SGD([nn.Parameter(torch.zeros(1))], lr=0.0))
            out = self._train(model, opt, ds, cfg, 0, after_step=lambda s: qt.step(opt.param_groups[0]["lr"]))
            return {**out, "storage": "packed", "compression_ratio": qt.get_compression_ratio(), "model": model}
        converted = self.convert(model, cfg) if inputs.get("convert", True) else []
        opt = inputs.get("optimizer") or torch.optim.AdamW([p for p in model.parameters() if p.requires_grad], lr=cfg.learning_rate, weight_decay=cfg.weight_decay)
        if cfg.gradient_dtype == "fp8":
            inner = opt.step
            gen = torch.Generator().manual_seed(cfg.seed)

            def step_with_rounding(*a: Any, **k: Any):
                self._quantize_gradients_to_fp8(model, gen)
                return inner(*a, **k)
            opt.step = step_with_rounding                                              # type: ignore[method-assign]
        out = self._train(model, opt, ds, cfg)
        return {**out, "storage": "master", "converted_layers": converted, "model": model}

    def save_checkpoint(self, path: str, model: nn.Module, optimizer: torch.optim.Optimizer, step: int = 0) -> str:
        return self._save_checkpoint(Path(path), model, optimizer, step)

    def load_checkpoint(self, path: str, model: nn.Module, optimizer: Optional[torch.optim.Optimizer] = None) -> int:
        return self._load_checkpoint(path, model, optimizer, optimizer is not None)


class PiscesLxFP4Trainer:
    """``PiscesLxFP4Trainer(model, config).train(records_or_dataset, tokenizer)``."""

    def __init__(self, model: nn.Module, config: Optional[PiscesLxFP4Config] = None, optimizer: Optional[torch.optim.Optimizer] = None):
        self.model, self.config, self.optimizer, self.operator = model, config or PiscesLxFP4Config(), optimizer, PiscesLxFP4Operator()
        self.history: List[Dict[str, float]] = []

    def train(self, data: Any, tokenizer: Any = None, save_dir: Optional[str] = None) -> Dict[str, Any]:
        key = "train_records" if isinstance(data, (list, tuple)) else "train_dataset"
        res = self.operator.execute({"model": self.model, "config": self.config, key: data, "tokenizer": tokenizer, "optimizer": self.optimizer})
        if not res.is_success():
            raise RuntimeError(f"fp4 training failed: {res.error}")
        self.history = res.output["history"]
        if save_dir:
            self._save_checkpoint(save_dir)
        return res.output

    def _save_checkpoint(self, save_dir: str) -> str:
        p = Path(save_dir) / "fp4_model.pt"
        p.parent.mkdir(parents=True, exist_ok=True)
        torch.save({"model_state_dict": self.model.state_dict(), "config": self.config.__dict__}, p)
        return str(p)

    def load_checkpoint(self, path: str) -> None:
        self.model.load_state_dict(torch.load(path, map_location="cpu", weights_only=False)["model_state_dict"])


# ---- sharded training --------------------------------------------------------------------------------------------------------
@dataclass
class PiscesLxFSDPTrainingConfig:
    model_path: str = ".pisceslx/ckpt"
    output_dir: str = ".pisceslx/ckpt"
    train_data: str = "./data/train.jsonl"
    val_data: str = "./data/val.jsonl"
    sharding_strategy: str = "ZERO3"              # ZERO2, ZERO3, SHARD_GRAD_OP
    backward_prefetch: str = "BACKWARD_PRE"       # BACKWARD_PRE, BACKWARD_POST, NO_PREFETCH
    forward_prefetch: bool = False
    limit_all_gathers: bool = True
    param_dtype: str = "bf16"
    reduce_dtype: str = "fp32"
    buffer_dtype: str = "fp32"
    cpu_offload: bool = False
    activation_checkpointing: bool = True
    gradient_checkpointing: bool = True
    batch_size: int = 4
    micro_batch_size: int = 1
    gradient_accumulation_steps: int = 4
    learning_rate: float = 1e-5
    warmup_steps: int = 500
    max_steps: int = 10000
    max_grad_norm: float = 1.0
    world_size: int = 8
    local_rank: int = 0
    master_port: int = 29500
    checkpoint_interval: int = 1000
    save_total_limit: int = 3
    max_seq_length: int = 4096
    optimizer: str = "adamw"

    def get_sharding_strategy(self) -> str:
        """This runtime's sharding mode: ``full_shard`` (parameters, gradients and optimizer state by owner; units per block
        gathered ahead of use) for ZERO3 / FULL_SHARD / HYBRID_SHARD, ``zero1``-style owner-sharded state otherwise."""
        s = self.sharding_strategy.upper()
        if s in ("ZERO3", "FULL_SHARD", "HYBRID_SHARD"):
            return "full_shard"
        if s in ("ZERO2", "SHARD_GRAD_OP", "ZERO1", "NO_SHARD"):
            return "zero1"
        raise ValueError(f"unknown sharding strategy {self.sharding_strategy}")

    def get_backward_prefetch(self) -> int:
        """How many units ahead the next all-gather is issued in backward: 1 before the current unit's gradient computation,
        0 after it (or none)."""
        p = self.backward_prefetch.upper()
        if p not in ("BACKWARD_PRE", "BACKWARD_POST", "NO_PREFETCH"):
            raise ValueError(f"unknown backward_prefetch {self.backward_prefetch}")
        return 1 if p == "BACKWARD_PRE" else 0

    def to_trainer_config(self):
        from .trainer import YvTrainerConfig
        return YvTrainerConfig(micro_batch_size=self.micro_batch_size, optimizer=self.optimizer, lr=self.learning_rate, warmup_steps=self.warmup_steps,
                               max_steps=self.max_steps, clip_grad_norm=self.max_grad_norm, save_steps=self.checkpoint_interval, output_dir=self.output_dir,
                               sharding=self.get_sharding_strategy(), state_dtype="fp32" if self.reduce_dtype == "fp32" else "bf16",
                               recompute_policy="auto" if (self.activation_checkpointing or self.gradient_checkpointing) else "config")


class PiscesLxFSDPDataset(PiscesLxSFTDataset):
    def __init__(self, data_path: Any, tokenizer: Any = None, max_length: int = 4096):
        super().__init__(data_path, tokenizer, max_length)


class PiscesLxFSDPTrainingOperator(PiscesLxOperatorInterface):
    """Sharded data-parallel training through this framework's trainer (``engine.trainer.YvTrainer`` with
    ``sharding="full_shard"`` and the given parallel state); one process per GPU, started by ``torchrun``.  With a single
    process it runs the same loop without sharding, which is what the host tests exercise."""

    name = "fsdp_training"

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return isinstance(inputs.get("model"), nn.Module)

    @staticmethod
    def _setup_distributed(config: PiscesLxFSDPTrainingConfig) -> Dict[str, int]:
        import os
        import torch.distributed as dist
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world > 1 and not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", str(config.master_port))
            dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo")
        return {"world_size": world, "rank": int(os.environ.get("RANK", "0")), "local_rank": int(os.environ.get("LOCAL_RANK", str(config.local_rank)))}

    @staticmethod
    def _collect_sharding_info(model: nn.Module, config: PiscesLxFSDPTrainingConfig, world: int) -> Dict[str, Any]:
        total = sum(p.numel() for p in model.parameters())
        mode = config.get_sharding_strategy()
        per_rank = total // world if mode == "full_shard" else total
        bytes_param = {"bf16": 2, "fp16": 2, "fp32": 4, "fp8": 1}.get(config.param_dtype, 2)
        return {"sharding": mode, "world_size": world, "total_parameters": total, "parameters_per_rank": per_rank,
                "parameter_bytes_per_rank": per_rank * bytes_param, "optimizer_state_bytes_per_rank": 2 * 4 * total // world,
                "backward_prefetch_units": config.get_backward_prefetch(), "forward_prefetch": config.forward_prefetch}

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        from .trainer import YvTrainer
        model = inputs["model"]
        cfg: PiscesLxFSDPTrainingConfig = inputs.get("config") or PiscesLxFSDPTrainingConfig()
        dist_info = self._setup_distributed(cfg) if inputs.get("init_distributed", False) else {"world_size": 1, "rank": 0, "local_rank": 0}
        tc = cfg.to_trainer_config()
        if dist_info["world_size"] == 1:
            tc.sharding = "zero1"
        tc.save_steps = tc.save_steps if inputs.get("save_checkpoints", False) else 0
        trainer = inputs.get("trainer") or YvTrainer(model, tc, parallel=inputs.get("parallel"))
        ds = inputs.get("train_dataset")
        if ds is None:
            src = inputs.get("train_records", cfg.train_data)
            ds = PiscesLxFSDPDataset(src, inputs.get("tokenizer"), cfg.max_seq_length)
        per_step = cfg.micro_batch_size * cfg.gradient_accumulation_steps
        stream = _batches(ds, per_step, ds.collate, 0, True, dist_info["rank"], dist_info["world_size"])
        hist = []
        for _ in range(cfg.max_steps):
            r = trainer.train_step(next(stream))
            hist.append({"step": r["global_step"], "loss": r["loss"], "lr": r["learning_rate"]})
        return {"steps": cfg.max_steps, "history": hist, "final_loss": hist[-1]["loss"] if hist else None, "first_loss": hist[0]["loss"] if hist else None,
                "sharding_info": self._collect_sharding_info(model, cfg, dist_info["world_size"]), "distributed": dist_info, "trainer": trainer}
