"""Configured training-stage operators: supervised fine-tuning and direct preference optimisation as whole runs, and
the step-level DPO / PPO operators with their configurations (reference opss/train/sft.py:67-960, dpo.py:98-900,
pref_align.py:48-420).

``engine/alignment.py`` and ``engine/rl.py`` hold the objectives and the step-wise trainers; this module is the layer a
user of the reference's stage operators calls: a configuration, a dataset that reads the usual record layouts, and an
operator whose ``execute`` runs warm-up, accumulation, clipping, evaluation and checkpoints.

Choices made for the device:
* a preference pair is ONE forward of 2 B rows (chosen rows then rejected rows), for the policy and again for the frozen
  reference, instead of four forwards of B rows: twice the rows per launch and half the launches;
* batches are padded to a multiple of 64 tokens, so that the sequence extent of every GEMM and attention tile is aligned
  and the number of distinct shapes (graph captures, allocator bins) stays small;
* running statistics are accumulated on the device and read once per ``log_interval`` - the reference reads the loss,
  both rewards and the accuracy with ``.item()`` for every sample (pref_align.py:176-181), four stream synchronisations a
  sample;
* sequence log-probabilities are masked sums; the reference subtracts 1e9 at padded positions before summing
  (pref_align.py:213-214), which makes the log-probability of any padded row about -1e9 x the padding."""
from __future__ import annotations

import copy
import json
import math
import os
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple, Union

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.data import Dataset

from ..utils.opsc import PiscesLxOperatorInterface
from .checkpoint_operator import PiscesLxCheckpointConfig, PiscesLxCheckpointOperator

PAD_MULTIPLE = 64


# ---- records ------------------------------------------------------------------------------------------------------------------
def read_records(data_path: Union[str, os.PathLike]) -> List[Dict[str, Any]]:
    """``.jsonl`` (one object a line), ``.json`` (a list, or an object with ``data`` / ``train``) or a folder of those."""
    p = Path(data_path)
    if p.is_dir():
        out: List[Dict[str, Any]] = []
        for f in sorted(p.rglob("*")):
            if f.suffix in (".json", ".jsonl"):
                out += read_records(f)
        return out
    if not p.exists():
        raise FileNotFoundError(f"no data at {p}")
    text = p.read_text(encoding="utf-8")
    if p.suffix == ".jsonl":
        return [json.loads(l) for l in text.splitlines() if l.strip()]
    d = json.loads(text)
    if isinstance(d, dict):
        d = d.get("data") or d.get("train") or [d]
    return list(d)


def split_prompt_response(sample: Dict[str, Any], chat: Optional[Callable[[List[Dict[str, str]]], str]] = None) -> Tuple[str, str]:
    """(prompt, response) of a record in one of the usual layouts: instruction / input / output, prompt / response (or
    completion), question / answer, messages or conversations (the last assistant turn is the response), or text only."""
    if "messages" in sample or "conversations" in sample:
        msgs = [{"role": m.get("role", m.get("from", "user")), "content": m.get("content", m.get("value", ""))}
                for m in (sample.get("messages") or sample.get("conversations"))]
        last = max((i for i, m in enumerate(msgs) if m["role"] in ("assistant", "gpt")), default=None)
        if last is None:
            return "", "\n".join(m["content"] for m in msgs)
        head = msgs[:last]
        prompt = chat(head) if chat is not None else "".join(f"<|{m['role']}|>\n{m['content']}\n" for m in head) + "<|assistant|>\n"
        return prompt, msgs[last]["content"]
    if "instruction" in sample:
        inp = sample.get("input", "")
        prompt = f"### Instruction:\n{sample['instruction']}\n\n" + (f"### Input:\n{inp}\n\n" if inp else "") + "### Response:\n"
        return prompt, str(sample.get("output", sample.get("response", "")))
    for pk, rk in (("prompt", "response"), ("prompt", "completion"), ("question", "answer"), ("input", "output")):
        if pk in sample and rk in sample:
            return str(sample[pk]), str(sample[rk])
    return "", str(sample.get("text", ""))


def _pad_to(rows: Sequence[Sequence[int]], value: int, multiple: int = PAD_MULTIPLE) -> torch.Tensor:
    n = max(len(r) for r in rows)
    n = ((n + multiple - 1) // multiple) * multiple
    out = torch.full((len(rows), n), value, dtype=torch.long)
    for i, r in enumerate(rows):
        out[i, :len(r)] = torch.as_tensor(r, dtype=torch.long)
    return out


def _model_logits(model: Any, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor]) -> torch.Tensor:
    try:
        out = model(input_ids=input_ids, attention_mask=attention_mask)
    except TypeError:
        out = model(input_ids)
    if isinstance(out, torch.Tensor):
        return out
    lg = out.get("logits") if isinstance(out, dict) else getattr(out, "logits", None)
    if lg is None:
        raise ValueError("Model outputs must contain 'logits' for log-prob computation")
    return lg


def masked_sequence_logps(model: Any, input_ids: torch.Tensor, labels: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                          ignore_index: int = -100) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(sum of the token log-probabilities of the labelled positions [B], the per-token values [B, T-1], their mask)."""
    lg = _model_logits(model, input_ids, attention_mask)[:, :-1].float()
    tgt = labels[:, 1:]
    mask = tgt != ignore_index
    lp = torch.log_softmax(lg, -1).gather(-1, tgt.clamp_min(0).unsqueeze(-1)).squeeze(-1) * mask
    return lp.sum(-1), lp, mask


def _lr_at(step: int, base: float, warmup: int, total: int, min_ratio: float) -> float:
    if step < warmup:
        return base * (step + 1) / max(warmup, 1)
    p = min((step - warmup) / max(total - warmup, 1), 1.0)
    return base * (min_ratio + (1 - min_ratio) * 0.5 * (1 + math.cos(math.pi * p)))


def _autocast(cfg: Any, device: torch.device):
    dt = torch.bfloat16 if getattr(cfg, "use_bf16", False) else (torch.float16 if getattr(cfg, "use_fp16", False) else None)
    if dt is None or device.type != "cuda":
        return torch.autocast(device_type=device.type, enabled=False)
    return torch.autocast(device_type="cuda", dtype=dt)


def _batches(dataset: Dataset, batch_size: int, collate: Callable, seed: int, shuffle: bool = True, rank: int = 0, world: int = 1) -> Iterator[Dict[str, torch.Tensor]]:
    """Endless stream of collated batches; every epoch reshuffles with seed + epoch, ranks take strided parts."""
    n, epoch = len(dataset), 0
    if n == 0:
        raise ValueError("empty dataset")
    while True:
        g = torch.Generator().manual_seed(seed + epoch)
        order = torch.randperm(n, generator=g).tolist() if shuffle else list(range(n))
        order = order[rank::world] or order
        for i in range(0, len(order), batch_size):
            yield collate([dataset[j] for j in order[i:i + batch_size]])
        epoch += 1


def _to_device(batch: Dict[str, torch.Tensor], device: torch.device) -> Dict[str, torch.Tensor]:
    if device.type == "cuda":
        return {k: (v.pin_memory().to(device, non_blocking=True) if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}
    return batch


# ---- SFT ------------------------------------------------------------------------------------------------------------------------
@dataclass
class PiscesLxSFTTrainingConfig:
    model_path: str = ".pisceslx/ckpt"
    output_dir: str = ".pisceslx/ckpt"
    train_data: str = "./data/train.jsonl"
    val_data: str = "./data/val.jsonl"
    batch_size: int = 4
    micro_batch_size: int = 1
    gradient_accumulation_steps: int = 4
    learning_rate: float = 1e-5
    min_lr_ratio: float = 0.1
    warmup_steps: int = 500
    max_steps: int = 10000
    max_grad_norm: float = 1.0
    weight_decay: float = 0.0
    use_fp16: bool = False
    use_bf16: bool = True
    use_fp8: bool = False
    fp8_amax_history_length: int = 1024
    fp8_amax_compute_algo: str = "max"
    use_gradient_checkpointing: bool = True
    checkpoint_interval: int = 1000
    eval_interval: int = 500
    log_interval: int = 10
    save_total_limit: int = 3
    local_rank: int = 0
    world_size: int = 1
    master_port: int = 29500
    max_seq_length: int = 4096
    ignore_index: int = -100
    seed: int = 0
    use_memsep_training: bool = False
    memsep_phase_1_steps: int = 5000
    memsep_phase_2_steps: int = 2000
    memsep_gate_target: float = 0.5
    memsep_freeze_backbone_phase2: bool = True
    memsep_freeze_router_phase1: bool = True
    memsep_reason_data_path: str = ""
    memsep_mem_data_path: str = ""
    memsep_alignment_weight: float = 0.1
    memsep_gate_schedule: str = "sigmoid"
    memsep_gate_warmup_steps: int = 500

    def __post_init__(self) -> None:
        if self.use_fp16 and self.use_bf16:
            self.use_bf16 = False
        if self.micro_batch_size < 1 or self.gradient_accumulation_steps < 1:
            raise ValueError("micro_batch_size and gradient_accumulation_steps must be at least 1")


class PiscesLxSFTDataset(Dataset):
    """Records (a path or a list) -> ``input_ids`` / ``attention_mask`` / ``labels`` with the prompt tokens excluded from the
    loss.  A sample longer than ``max_seq_length`` loses the BEGINNING of its prompt, not its response."""

    def __init__(self, data: Union[str, os.PathLike, Sequence[Dict[str, Any]]], tokenizer: Any = None, max_seq_length: int = 4096,
                 ignore_index: int = -100):
        self.records = read_records(data) if isinstance(data, (str, os.PathLike)) else list(data)
        if tokenizer is None:
            from ..models.tokenizer import YvTokenizer
            tokenizer = YvTokenizer.instance()
        self.tok, self.max_seq_length, self.ignore_index = tokenizer, max_seq_length, ignore_index
        self.pad_id = int(getattr(tokenizer, "pad_token_id", 0) or 0)
        self._chat = getattr(tokenizer, "apply_chat_template", None)

    def __len__(self) -> int:
        return len(self.records)

    def _encode(self, text: str, eos: bool = False) -> List[int]:
        try:
            return list(self.tok.encode(text, add_eos=eos))
        except TypeError:
            ids = list(self.tok.encode(text))
            return ids + [int(self.tok.eos_token_id)] if eos and getattr(self.tok, "eos_token_id", None) is not None else ids

    def _format_sample(self, sample: Dict[str, Any]) -> str:
        p, r = split_prompt_response(sample, self._chat)
        return p + r

    def __getitem__(self, idx: int) -> Dict[str, torch.Tensor]:
        prompt, response = split_prompt_response(self.records[idx], self._chat)
        p, r = (self._encode(prompt) if prompt else []), self._encode(response, eos=True)
        r = r[: self.max_seq_length]
        p = p[max(0, len(p) - (self.max_seq_length - len(r))):] if len(p) + len(r) > self.max_seq_length else p
        ids = torch.tensor(p + r, dtype=torch.long)
        labels = ids.clone()
        labels[: len(p)] = self.ignore_index
        return {"input_ids": ids, "attention_mask": torch.ones_like(ids), "labels": labels}

    def collate(self, samples: List[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
        return {"input_ids": _pad_to([s["input_ids"] for s in samples], self.pad_id),
                "attention_mask": _pad_to([s["attention_mask"] for s in samples], 0),
                "labels": _pad_to([s["labels"] for s in samples], self.ignore_index)}


def causal_lm_loss(model: Any, batch: Dict[str, torch.Tensor], ignore_index: int = -100) -> torch.Tensor:
    """The model's own loss when it computes one from ``labels`` (our models fuse the head and the loss), else shifted
    cross-entropy over its logits."""
    try:
        out = model(input_ids=batch["input_ids"], labels=batch["labels"])
        loss = out.get("loss") if isinstance(out, dict) else getattr(out, "loss", None)
        if loss is not None:
            return loss
        lg = out.get("logits") if isinstance(out, dict) else getattr(out, "logits", out)
    except TypeError:
        lg = _model_logits(model, batch["input_ids"], batch.get("attention_mask"))
    return F.cross_entropy(lg[:, :-1].float().reshape(-1, lg.shape[-1]), batch["labels"][:, 1:].reshape(-1), ignore_index=ignore_index)


class PiscesLxSFTTrainingOperator(PiscesLxOperatorInterface):
    """``execute({"model", "config", "train_dataset" | "train_records" | config.train_data, ...})``.  Optional inputs:
    ``val_dataset`` / ``val_records``, ``tokenizer``, ``optimizer`` (AdamW over the trainable parameters otherwise),
    ``scheduler`` (an object with ``step()``; warm-up + cosine to ``min_lr_ratio`` otherwise), ``memsep_trainer`` (its
    ``pre_step`` runs before every optimizer step and its memory loss is added), ``callback(step, logs)``."""

    name = "sft_training"

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return inputs.get("model") is not None

    @staticmethod
    def _dataset(inputs: Dict[str, Any], key: str, path: str, cfg: PiscesLxSFTTrainingConfig) -> Optional[Dataset]:
        if inputs.get(f"{key}_dataset") is not None:
            return inputs[f"{key}_dataset"]
        if inputs.get(f"{key}_records") is not None:
            return PiscesLxSFTDataset(inputs[f"{key}_records"], inputs.get("tokenizer"), cfg.max_seq_length, cfg.ignore_index)
        if path and os.path.exists(path):
            return PiscesLxSFTDataset(path, inputs.get("tokenizer"), cfg.max_seq_length, cfg.ignore_index)
        return None

    @torch.no_grad()
    def _evaluate(self, model: Any, dataset: Dataset, cfg: PiscesLxSFTTrainingConfig, device: torch.device, max_batches: int = 50) -> float:
        was = model.training
        model.eval()
        collate = getattr(dataset, "collate", None) or (lambda b: torch.utils.data.default_collate(b))
        tot, n = torch.zeros((), device=device), 0
        for i in range(0, min(len(dataset), max_batches * cfg.micro_batch_size), cfg.micro_batch_size):
            batch = _to_device(collate([dataset[j] for j in range(i, min(i + cfg.micro_batch_size, len(dataset)))]), device)
            with _autocast(cfg, device):
                tot += causal_lm_loss(model, batch, cfg.ignore_index).float()
            n += 1
        model.train(was)
        return float(tot / max(n, 1))

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        model: nn.Module = inputs["model"]
        cfg: PiscesLxSFTTrainingConfig = inputs.get("config") or PiscesLxSFTTrainingConfig()
        train = self._dataset(inputs, "train", cfg.train_data, cfg)
        if train is None:
            raise ValueError(f"no training data: give train_dataset / train_records or a file at {cfg.train_data}")
        val = self._dataset(inputs, "val", cfg.val_data, cfg)
        device = next(model.parameters()).device
        if cfg.use_gradient_checkpointing and hasattr(model, "gradient_checkpointing_enable"):
            model.gradient_checkpointing_enable()
        params = [p for p in model.parameters() if p.requires_grad]
        opt = inputs.get("optimizer") or torch.optim.AdamW(params, lr=cfg.learning_rate, weight_decay=cfg.weight_decay)
        sched, memsep, callback = inputs.get("scheduler"), inputs.get("memsep_trainer"), inputs.get("callback")
        scaler = torch.amp.GradScaler("cuda", enabled=cfg.use_fp16 and device.type == "cuda")
        ckpt = None
        if cfg.checkpoint_interval > 0 and inputs.get("save_checkpoints", True):
            ckpt = PiscesLxCheckpointOperator(PiscesLxCheckpointConfig(save_dir=cfg.output_dir, prefix="sft_step", interval=cfg.checkpoint_interval,
                                                                       max_to_keep=cfg.save_total_limit, save_best=val is not None, best_metric="eval_loss"))
        collate = getattr(train, "collate", None) or (lambda b: torch.utils.data.default_collate(b))
        stream = _batches(train, cfg.micro_batch_size, collate, cfg.seed, True, cfg.local_rank if cfg.world_size > 1 else 0, max(cfg.world_size, 1))
        model.train()
        history: List[Dict[str, float]] = []
        window, window_n, tokens = torch.zeros((), device=device), 0, 0
        eval_loss, saved, t0 = None, [], time.time()
        for step in range(cfg.max_steps):
            lr = _lr_at(step, cfg.learning_rate, cfg.warmup_steps, cfg.max_steps, cfg.min_lr_ratio)
            if sched is None:
                for g in opt.param_groups:
                    g["lr"] = lr * g.get("lr_scale", 1.0)
            opt.zero_grad(set_to_none=True)
            for _ in range(cfg.gradient_accumulation_steps):
                batch = _to_device(next(stream), device)
                with _autocast(cfg, device):
                    loss = causal_lm_loss(model, batch, cfg.ignore_index)
                    if memsep is not None and hasattr(memsep, "compute_memory_loss"):
                        loss = loss + cfg.memsep_alignment_weight * memsep.compute_memory_loss(getattr(model, "last_knowledge_ctx", None))
                scaler.scale(loss / cfg.gradient_accumulation_steps).backward()
                window += loss.detach().float()
                window_n += 1
                tokens += int(batch["input_ids"].numel())
            if memsep is not None and hasattr(memsep, "pre_step"):
                memsep.pre_step()
            scaler.unscale_(opt)
            gn = torch.nn.utils.clip_grad_norm_(params, cfg.max_grad_norm) if cfg.max_grad_norm > 0 else None
            scaler.step(opt)
            scaler.update()
            if sched is not None:
                sched.step()
            done = step + 1
            if done % max(cfg.log_interval, 1) == 0 or done == cfg.max_steps:
                logs = {"step": done, "loss": float(window / max(window_n, 1)), "lr": opt.param_groups[0]["lr"],
                        "grad_norm": float(gn) if gn is not None else 0.0, "tokens": tokens}
                window.zero_()
                window_n = 0
                history.append(logs)
                if callback is not None:
                    callback(done, logs)
            if val is not None and cfg.eval_interval > 0 and (done % cfg.eval_interval == 0 or done == cfg.max_steps):
                eval_loss = self._evaluate(model, val, cfg, device)
                history.append({"step": done, "eval_loss": eval_loss})
            if ckpt is not None and (done % cfg.checkpoint_interval == 0 or done == cfg.max_steps):
                metrics = {"loss": history[-1].get("loss", 0.0) if history else 0.0}
                if eval_loss is not None:
                    metrics["eval_loss"] = eval_loss
                saved.append(ckpt.save(model=model, optimizer=opt, global_step=done, metrics=metrics)["path"])
        if ckpt is not None:
            ckpt.shutdown()
        train_losses = [h["loss"] for h in history if "loss" in h]
        return {"steps": cfg.max_steps, "final_loss": train_losses[-1] if train_losses else None, "first_loss": train_losses[0] if train_losses else None,
                "eval_loss": eval_loss, "history": history, "checkpoints": saved, "tokens": tokens, "seconds": time.time() - t0,
                "model": model}


# ---- DPO ------------------------------------------------------------------------------------------------------------------------
@dataclass
class PiscesLxDPOTrainingConfig:
    model_path: str = ".pisceslx/ckpt"
    ref_model_path: str = ".pisceslx/ckpt"
    output_dir: str = ".pisceslx/ckpt"
    train_data: str = "./data/preferences.jsonl"
    val_data: str = "./data/val_preferences.jsonl"
    batch_size: int = 4
    micro_batch_size: int = 1
    gradient_accumulation_steps: int = 4
    learning_rate: float = 5e-7
    min_lr_ratio: float = 0.1
    warmup_steps: int = 100
    max_steps: int = 2000
    max_grad_norm: float = 1.0
    weight_decay: float = 0.0
    beta: float = 0.1
    label_smoothing: float = 0.0
    loss_type: str = "sigmoid"
    reference_free: bool = False
    use_fp16: bool = False
    use_bf16: bool = True
    use_fp8: bool = False
    use_gradient_checkpointing: bool = True
    checkpoint_interval: int = 500
    eval_interval: int = 250
    log_interval: int = 10
    save_total_limit: int = 3
    local_rank: int = 0
    world_size: int = 1
    master_port: int = 29501
    max_prompt_length: int = 1024
    max_response_length: int = 1024
    seed: int = 0

    def __post_init__(self) -> None:
        if self.use_fp16 and self.use_bf16:
            self.use_bf16 = False
        if self.loss_type not in ("sigmoid", "hinge", "ipo"):
            raise ValueError(f"Unknown loss type: {self.loss_type}")


@dataclass
class PiscesLxGRMConfig:
    grm_model_path: str = ""
    grm_learning_rate: float = 1e-6
    grm_hidden_size: int = 4096
    grm_num_layers: int = 2
    grm_use_implicit_reward: bool = True


@dataclass
class PiscesLxDPOConfig:
    name: str = "dpo"
    beta: float = 0.1
    label_smoothing: float = 0.0
    loss_type: str = "sigmoid"
    reference_free: bool = False
    max_length: int = 512
    max_grad_norm: float = 1.0


@dataclass
class PiscesLxPPOConfig:
    name: str = "ppo"
    learning_rate: float = 1e-5
    ppo_epochs: int = 4
    num_mini_batches: int = 1
    mini_batch_size: int = 64
    clip_range: float = 0.2
    clip_range_value: float = 0.2
    entropy_coef: float = 0.01
    value_loss_coef: float = 0.5
    gamma: float = 1.0
    lam: float = 0.95
    kl_target: float = 0.01
    kl_early_stopping: bool = True
    use_reference_model: bool = True
    ref_model_alpha: float = 0.5
    max_grad_norm: float = 1.0


@dataclass
class PiscesLxKTOConfig:
    name: str = "kto"
    kl_weight: float = 0.1
    desirability_weight: float = 1.0
    use_empirical_likelihood: bool = True
    focal_loss_gamma: float = 2.0


@dataclass
class PiscesLxBCOConfig:
    name: str = "bco"
    positive_weight: float = 1.0
    negative_weight: float = 1.0
    use_focal_loss: bool = False
    focal_gamma: float = 2.0


class PiscesLxDPODataset(Dataset):
    """Preference records ``{"prompt", "chosen", "rejected"}`` (also ``question`` / ``chosen_response`` ...) -> token rows
    with the prompt masked out of the labels.  The prompt keeps its END when it is longer than ``max_prompt_length``."""

    def __init__(self, data: Union[str, os.PathLike, Sequence[Dict[str, Any]]], tokenizer: Any = None, max_prompt_length: int = 1024,
                 max_response_length: int = 1024, ignore_index: int = -100):
        self.records = read_records(data) if isinstance(data, (str, os.PathLike)) else list(data)
        if tokenizer is None:
            from ..models.tokenizer import YvTokenizer
            tokenizer = YvTokenizer.instance()
        self.tok, self.max_p, self.max_r, self.ignore_index = tokenizer, max_prompt_length, max_response_length, ignore_index
        self.pad_id = int(getattr(tokenizer, "pad_token_id", 0) or 0)

    def __len__(self) -> int:
        return len(self.records)

    def _enc(self, text: str, eos: bool = False) -> List[int]:
        try:
            return list(self.tok.encode(text, add_eos=eos))
        except TypeError:
            ids = list(self.tok.encode(text))
            return ids + [int(self.tok.eos_token_id)] if eos and getattr(self.tok, "eos_token_id", None) is not None else ids

    def __getitem__(self, idx: int) -> Dict[str, torch.Tensor]:
        r = self.records[idx]
        prompt = r.get("prompt", r.get("question", r.get("instruction", "")))
        chosen = r.get("chosen", r.get("chosen_response", r.get("preferred", "")))
        rejected = r.get("rejected", r.get("rejected_response", r.get("dispreferred", "")))
        p = self._enc(str(prompt))[-self.max_p:]
        out: Dict[str, torch.Tensor] = {}
        for name, text in (("chosen", chosen), ("rejected", rejected)):
            a = self._enc(str(text), eos=True)[: self.max_r]
            ids = torch.tensor(p + a, dtype=torch.long)
            lab = ids.clone()
            lab[: len(p)] = self.ignore_index
            out[f"{name}_input_ids"], out[f"{name}_attention_mask"], out[f"{name}_labels"] = ids, torch.ones_like(ids), lab
        return out

    def collate(self, samples: List[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
        """Chosen rows then rejected rows in ONE tensor of 2 B rows."""
        ids = [s["chosen_input_ids"] for s in samples] + [s["rejected_input_ids"] for s in samples]
        lab = [s["chosen_labels"] for s in samples] + [s["rejected_labels"] for s in samples]
        return {"input_ids": _pad_to(ids, self.pad_id), "attention_mask": _pad_to([torch.ones_like(i) for i in ids], 0),
                "labels": _pad_to(lab, self.ignore_index)}


def preference_loss(pi_chosen: torch.Tensor, pi_rejected: torch.Tensor, ref_chosen: torch.Tensor, ref_rejected: torch.Tensor, beta: float = 0.1,
                    loss_type: str = "sigmoid", label_smoothing: float = 0.0) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
    """sigmoid (DPO, with conservative label smoothing), hinge (SLiC) or ipo; statistics are detached tensors."""
    h = (pi_chosen - pi_rejected) - (ref_chosen - ref_rejected)
    if loss_type == "sigmoid":
        loss = -(1 - label_smoothing) * F.logsigmoid(beta * h) - label_smoothing * F.logsigmoid(-beta * h)
    elif loss_type == "hinge":
        loss = F.relu(1.0 - beta * h)
    elif loss_type == "ipo":
        loss = (h - 1.0 / (2.0 * beta)).pow(2)
    else:
        raise ValueError(f"Unknown loss type: {loss_type}")
    rc, rr = beta * (pi_chosen - ref_chosen).detach(), beta * (pi_rejected - ref_rejected).detach()
    return loss.mean(), {"chosen_reward": rc.mean(), "rejected_reward": rr.mean(), "accuracy": (rc > rr).float().mean(), "margin": (rc - rr).mean()}


def paired_logps(model: Any, batch: Dict[str, torch.Tensor], ignore_index: int = -100) -> Tuple[torch.Tensor, torch.Tensor]:
    lp, _, _ = masked_sequence_logps(model, batch["input_ids"], batch["labels"], batch.get("attention_mask"), ignore_index)
    b = lp.shape[0] // 2
    return lp[:b], lp[b:]


class PiscesLxDPOLoggingCallback:
    """Keeps the logged dictionaries and prints one line per log (to ``sink``, ``print`` by default; None for silence)."""

    def __init__(self, log_every: int = 1, sink: Optional[Callable[[str], None]] = print):
        self.log_every, self.sink, self.records = max(log_every, 1), sink, []

    def __call__(self, step: int, logs: Dict[str, float]) -> None:
        self.records.append(dict(logs, step=step))
        if self.sink is not None and len(self.records) % self.log_every == 0:
            self.sink(f"[dpo] step {step} " + " ".join(f"{k}={v:.4g}" for k, v in logs.items() if isinstance(v, (int, float)) and k != "step"))

    on_log = __call__

    def summary(self) -> Dict[str, float]:
        if not self.records:
            return {}
        keys = [k for k, v in self.records[-1].items() if isinstance(v, (int, float))]
        return {k: self.records[-1][k] for k in keys}


class PiscesLxDPOTrainingOperator(PiscesLxOperatorInterface):
    """The whole preference stage: ``execute({"model", "ref_model"?, "config", "train_dataset" | "train_records" | path})``.
    Without a reference model a frozen copy of the policy is made at the start (``reference_free`` skips the reference)."""

    name = "dpo_training"

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return inputs.get("model") is not None

    @staticmethod
    def _dataset(inputs: Dict[str, Any], key: str, path: str, cfg: PiscesLxDPOTrainingConfig) -> Optional[Dataset]:
        if inputs.get(f"{key}_dataset") is not None:
            return inputs[f"{key}_dataset"]
        src = inputs.get(f"{key}_records")
        if src is None and path and os.path.exists(path):
            src = path
        return None if src is None else PiscesLxDPODataset(src, inputs.get("tokenizer"), cfg.max_prompt_length, cfg.max_response_length)

    def _loss(self, model: Any, ref: Any, batch: Dict[str, torch.Tensor], cfg: PiscesLxDPOTrainingConfig) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
        pc, pr = paired_logps(model, batch)
        if ref is None or cfg.reference_free:
            rc, rr = torch.zeros_like(pc), torch.zeros_like(pr)
        else:
            with torch.no_grad():
                rc, rr = paired_logps(ref, batch)
        return preference_loss(pc, pr, rc, rr, cfg.beta, cfg.loss_type, cfg.label_smoothing)

    @torch.no_grad()
    def _evaluate(self, model: Any, ref: Any, dataset: Dataset, cfg: PiscesLxDPOTrainingConfig, device: torch.device, max_batches: int = 50) -> Dict[str, float]:
        was = model.training
        model.eval()
        agg, n = None, 0
        for i in range(0, min(len(dataset), max_batches * cfg.micro_batch_size), cfg.micro_batch_size):
            batch = _to_device(dataset.collate([dataset[j] for j in range(i, min(i + cfg.micro_batch_size, len(dataset)))]), device)
            with _autocast(cfg, device):
                loss, st = self._loss(model, ref, batch, cfg)
            vec = torch.stack([loss.float(), st["accuracy"], st["margin"]])
            agg = vec if agg is None else agg + vec
            n += 1
        model.train(was)
        a = (agg / max(n, 1)).tolist() if agg is not None else [0.0, 0.0, 0.0]
        return {"eval_loss": a[0], "eval_accuracy": a[1], "eval_margin": a[2]}

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        model: nn.Module = inputs["model"]
        cfg: PiscesLxDPOTrainingConfig = inputs.get("config") or PiscesLxDPOTrainingConfig()
        train = self._dataset(inputs, "train", cfg.train_data, cfg)
        if train is None:
            raise ValueError(f"no preference data: give train_dataset / train_records or a file at {cfg.train_data}")
        val = self._dataset(inputs, "val", cfg.val_data, cfg)
        device = next(model.parameters()).device
        ref = inputs.get("ref_model", inputs.get("reference_model"))
        if ref is None and not cfg.reference_free:
            ref = copy.deepcopy(model)
        if ref is not None:
            ref.eval().requires_grad_(False)
        params = [p for p in model.parameters() if p.requires_grad]
        opt = inputs.get("optimizer") or torch.optim.AdamW(params, lr=cfg.learning_rate, weight_decay=cfg.weight_decay)
        callback = inputs.get("callback")
        ckpt = None
        if cfg.checkpoint_interval > 0 and inputs.get("save_checkpoints", True):
            ckpt = PiscesLxCheckpointOperator(PiscesLxCheckpointConfig(save_dir=cfg.output_dir, prefix="dpo_step", interval=cfg.checkpoint_interval,
                                                                       max_to_keep=cfg.save_total_limit))
        stream = _batches(train, cfg.micro_batch_size, train.collate, cfg.seed, True, cfg.local_rank if cfg.world_size > 1 else 0, max(cfg.world_size, 1))
        model.train()
        history: List[Dict[str, float]] = []
        window, window_n, evals, saved = torch.zeros(5, device=device), 0, {}, []
        for step in range(cfg.max_steps):
            lr = _lr_at(step, cfg.learning_rate, cfg.warmup_steps, cfg.max_steps, cfg.min_lr_ratio)
            for g in opt.param_groups:
                g["lr"] = lr
            opt.zero_grad(set_to_none=True)
            for _ in range(cfg.gradient_accumulation_steps):
                batch = _to_device(next(stream), device)
                with _autocast(cfg, device):
                    loss, st = self._loss(model, ref, batch, cfg)
                (loss / cfg.gradient_accumulation_steps).backward()
                window += torch.stack([loss.detach().float(), st["chosen_reward"], st["rejected_reward"], st["accuracy"], st["margin"]])
                window_n += 1
            if cfg.max_grad_norm > 0:
                torch.nn.utils.clip_grad_norm_(params, cfg.max_grad_norm)
            opt.step()
            done = step + 1
            if done % max(cfg.log_interval, 1) == 0 or done == cfg.max_steps:
                w = (window / max(window_n, 1)).tolist()
                logs = {"step": done, "loss": w[0], "chosen_reward": w[1], "rejected_reward": w[2], "accuracy": w[3], "margin": w[4], "lr": lr}
                window.zero_()
                window_n = 0
                history.append(logs)
                if callback is not None:
                    callback(done, logs)
            if val is not None and cfg.eval_interval > 0 and (done % cfg.eval_interval == 0 or done == cfg.max_steps):
                evals = self._evaluate(model, ref, val, cfg, device)
                history.append(dict(evals, step=done))
            if ckpt is not None and (done % cfg.checkpoint_interval == 0 or done == cfg.max_steps):
                saved.append(ckpt.save(model=model, optimizer=opt, global_step=done, metrics={"loss": history[-1].get("loss", 0.0)})["path"])
        if ckpt is not None:
            ckpt.shutdown()
        logs = [h for h in history if "loss" in h]
        return {"steps": cfg.max_steps, "final_loss": logs[-1]["loss"] if logs else None, "accuracy": logs[-1]["accuracy"] if logs else None,
                "margin": logs[-1]["margin"] if logs else None, "history": history, "checkpoints": saved, "model": model, **evals}


class PiscesLxDPOOperator(PiscesLxOperatorInterface):
    """One pass over a list of preference samples (``chosen_input_ids`` / ``rejected_input_ids`` with their masks, and
    optionally ``chosen_labels`` / ``rejected_labels`` to keep the prompt out of the sums); with an optimizer every sample
    is a step.  Returns the means over the samples."""

    name = "dpo"

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return inputs.get("model") is not None and bool(inputs.get("preference_data"))

    @staticmethod
    def _compute_logps(model: Any, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor], labels: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        if labels is None:
            labels = input_ids if attention_mask is None else input_ids.masked_fill(attention_mask == 0, -100)
        s, per_token, _ = masked_sequence_logps(model, input_ids, labels, attention_mask)
        return s, per_token

    @staticmethod
    def _compute_dpo_loss(chosen_logps, rejected_logps, ref_chosen_logps, ref_rejected_logps, config: PiscesLxDPOConfig):
        loss, st = preference_loss(chosen_logps, rejected_logps, ref_chosen_logps, ref_rejected_logps, config.beta, config.loss_type, config.label_smoothing)
        return loss, st["chosen_reward"], st["rejected_reward"]

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        model, ref = inputs["model"], inputs.get("reference_model")
        cfg: PiscesLxDPOConfig = inputs.get("config") or PiscesLxDPOConfig()
        opt = inputs.get("optimizer")
        model.train()
        if ref is not None:
            ref.eval()
        agg, n = None, 0
        for s in inputs["preference_data"]:
            ch, rj = s.get("chosen_input_ids"), s.get("rejected_input_ids")
            if ch is None or rj is None:
                continue
            pc, _ = self._compute_logps(model, ch, s.get("chosen_attention_mask"), s.get("chosen_labels"))
            pr, _ = self._compute_logps(model, rj, s.get("rejected_attention_mask"), s.get("rejected_labels"))
            if ref is not None and not cfg.reference_free:
                with torch.no_grad():
                    rc, _ = self._compute_logps(ref, ch, s.get("chosen_attention_mask"), s.get("chosen_labels"))
                    rr, _ = self._compute_logps(ref, rj, s.get("rejected_attention_mask"), s.get("rejected_labels"))
            else:
                rc, rr = torch.zeros_like(pc), torch.zeros_like(pr)
            loss, st = preference_loss(pc, pr, rc, rr, cfg.beta, cfg.loss_type, cfg.label_smoothing)
            if opt is not None:
                opt.zero_grad(set_to_none=True)
                loss.backward()
                torch.nn.utils.clip_grad_norm_(model.parameters(), cfg.max_grad_norm)
                opt.step()
            vec = torch.stack([loss.detach().float(), st["chosen_reward"], st["rejected_reward"], st["accuracy"]])
            agg = vec if agg is None else agg + vec
            n += 1
        if agg is None:
            raise ValueError("no usable preference sample (chosen_input_ids and rejected_input_ids are required)")
        a = (agg / n).tolist()                                                         # the one read of the pass
        return {"loss": a[0], "mean_chosen_reward": a[1], "mean_rejected_reward": a[2], "accuracy": a[3], "samples": n}


class PiscesLxPPOStepOperator(PiscesLxOperatorInterface):
    """PPO from a configuration: builds ``engine.rl.PiscesLxPPOOperator`` (rollout, GAE, clipped policy and value updates,
    adaptive KL) from ``PiscesLxPPOConfig`` and runs ``steps`` updates over ``prompts`` [B, P]."""

    name = "ppo"

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return inputs.get("model") is not None and inputs.get("prompts") is not None and callable(inputs.get("reward_fn"))

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        from .rl import PiscesLxPPOOperator, YvAdaptiveKLController
        cfg: PiscesLxPPOConfig = inputs.get("config") or PiscesLxPPOConfig()
        model = inputs["model"]
        opt = inputs.get("optimizer") or torch.optim.AdamW([p for p in model.parameters() if p.requires_grad], lr=cfg.learning_rate)
        ppo = inputs.get("ppo") or PiscesLxPPOOperator(
            model, opt, inputs["reward_fn"], ref_model=inputs.get("reference_model") if cfg.use_reference_model else model,
            clip=cfg.clip_range, vf_coef=cfg.value_loss_coef, gamma=cfg.gamma, lam=cfg.lam, ppo_epochs=cfg.ppo_epochs,
            max_new_tokens=int(inputs.get("max_new_tokens", 16)), kl=YvAdaptiveKLController(target=cfg.kl_target),
            eos_token_id=inputs.get("eos_token_id"))
        stats = [ppo.step(inputs["prompts"]) for _ in range(int(inputs.get("steps", 1)))]
        return {"ppo": ppo, "history": stats, **stats[-1]}


class PiscesLxDPOOperators:
    """Constructors by name (the reference's facade, dpo.py:1404-1440)."""

    @staticmethod
    def create_training_operator() -> PiscesLxDPOTrainingOperator:
        return PiscesLxDPOTrainingOperator()

    @staticmethod
    def create_config(**kw: Any) -> PiscesLxDPOTrainingConfig:
        return PiscesLxDPOTrainingConfig(**kw)

    @staticmethod
    def create_dataset(data: Any, tokenizer: Any = None, **kw: Any) -> PiscesLxDPODataset:
        return PiscesLxDPODataset(data, tokenizer, **kw)

    @staticmethod
    def create_opd_trainer(*a: Any, **kw: Any):
        from .operators import PiscesLxOPDTrainer
        return PiscesLxOPDTrainer(*a, **kw)

    @staticmethod
    def create_reward_model(*a: Any, **kw: Any):
        from .rl import PiscesLxGenerativeRewardModel
        return PiscesLxGenerativeRewardModel(*a, **kw)
