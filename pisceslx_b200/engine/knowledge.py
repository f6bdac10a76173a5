"""Knowledge store and the Subconscious trainer (reference opss/knowledge/builder.py ``PiscesLxKnowledgeBuilder``:
encoder trained with NT-Xent, FAISS IVF-PQ index, memory-mapped payloads; opss/subconscious_trainer.py
``PiscesLxSubconsciousTrainer`` three phases: router pre-training -> policy-gradient refinement -> self-play).

FAISS is not assumed: the IVF-PQ index (coarse k-means cells, product-quantised residuals, asymmetric distance
tables) is implemented on tensors, so the same code indexes on the CPU or the GPU; the PQ codebooks it learns are the
layout ``YvPQKnowledgeField`` consumes ([C, N, D/C] codebooks + int codes per entry)."""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F


def nt_xent(z1: torch.Tensor, z2: torch.Tensor, temperature: float = 0.07) -> torch.Tensor:
    """Normalised-temperature cross entropy over a batch of positive pairs (z1[i], z2[i])."""
    z = F.normalize(torch.cat([z1, z2]).float(), dim=1)
    sim = z @ z.t() / temperature
    n = z1.shape[0]
    sim = sim.masked_fill(torch.eye(2 * n, dtype=torch.bool, device=z.device), float("-inf"))
    target = torch.cat([torch.arange(n, 2 * n), torch.arange(0, n)]).to(z.device)
    return F.cross_entropy(sim, target)


def kmeans(x: torch.Tensor, k: int, iters: int = 15, seed: int = 0) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(seed)
    cent = x[torch.randperm(x.shape[0], generator=g)[:k].to(x.device)].clone().float()
    for _ in range(iters):
        a = torch.cdist(x.float(), cent).argmin(1)
        for j in range(k):
            m = a == j
            if m.any():
                cent[j] = x[m].float().mean(0)
    return cent


class PiscesLxIVFPQIndex:
    """Inverted file over ``n_list`` coarse cells; residuals product-quantised into ``m`` sub-vectors of
    ``2**nbits`` centroids each."""

    def __init__(self, dim: int, n_list: int = 16, m: int = 8, nbits: int = 6):
        assert dim % m == 0
        self.dim, self.n_list, self.m, self.ks = dim, n_list, m, 2 ** nbits
        self.coarse: Optional[torch.Tensor] = None
        self.codebooks: Optional[torch.Tensor] = None          # [m, ks, dim/m]
        self.codes: Optional[torch.Tensor] = None              # [N, m] int16
        self.cells: Optional[torch.Tensor] = None              # [N]
        self.ids: Optional[torch.Tensor] = None

    def train(self, x: torch.Tensor, seed: int = 0) -> None:
        self.coarse = kmeans(x, self.n_list, seed=seed)
        res = x.float() - self.coarse[torch.cdist(x.float(), self.coarse).argmin(1)]
        sub = res.view(res.shape[0], self.m, -1)
        self.codebooks = torch.stack([kmeans(sub[:, j], min(self.ks, sub.shape[0]), seed=seed + j + 1)
                                      for j in range(self.m)])

    def _encode(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        cells = torch.cdist(x.float(), self.coarse).argmin(1)
        res = (x.float() - self.coarse[cells]).view(x.shape[0], self.m, -1)
        codes = torch.stack([torch.cdist(res[:, j], self.codebooks[j]).argmin(1) for j in range(self.m)], 1)
        return cells, codes.to(torch.int16)

    def add(self, x: torch.Tensor, ids: Optional[torch.Tensor] = None) -> None:
        cells, codes = self._encode(x)
        ids = ids if ids is not None else torch.arange(x.shape[0]) + (0 if self.ids is None else self.ids.numel())
        cat = lambda a, b: b if a is None else torch.cat([a, b])
        self.cells, self.codes, self.ids = cat(self.cells, cells), cat(self.codes, codes), cat(self.ids, ids.to(cells.device))

    def search(self, q: torch.Tensor, k: int = 5, n_probe: int = 4) -> Tuple[torch.Tensor, torch.Tensor]:
        """Asymmetric distance: query residual against PQ centroids (one [m, ks] table per probed cell)."""
        out_d, out_i = [], []
        for qi in q.float():
            probe = torch.cdist(qi[None], self.coarse)[0].topk(min(n_probe, self.n_list), largest=False).indices
            ds, ii = [], []
            for c in probe:
                members = (self.cells == c).nonzero(as_tuple=True)[0]
                if members.numel() == 0:
                    continue
                res = (qi - self.coarse[c]).view(self.m, 1, -1)
                table = (res - self.codebooks).pow(2).sum(-1)                          # [m, ks]
                codes = self.codes[members].long()
                ds.append(table.gather(1, codes.t()).sum(0))
                ii.append(self.ids[members])
            if not ds:
                out_d.append(torch.full((k,), float("inf"))); out_i.append(torch.full((k,), -1)); continue
            d, i = torch.cat(ds), torch.cat(ii)
            top = d.topk(min(k, d.numel()), largest=False)
            pad = k - top.indices.numel()
            out_d.append(F.pad(top.values, (0, pad), value=float("inf")))
            out_i.append(F.pad(i[top.indices], (0, pad), value=-1))
        return torch.stack(out_d), torch.stack(out_i)


class PiscesLxKnowledgeBuilder:
    """Encodes texts, trains the index, and writes a memory-mapped store (vectors.f32, payload offsets, meta.json)."""

    def __init__(self, encode: Callable[[List[str]], torch.Tensor], dim: int, n_list: int = 16, m: int = 8):
        self.encode, self.index = encode, PiscesLxIVFPQIndex(dim, n_list, m)
        self.payloads: List[str] = []

    def build(self, texts: List[str]) -> None:
        vecs = F.normalize(self.encode(texts).float(), dim=1)
        self.index.train(vecs)
        self.index.add(vecs)
        self.payloads = list(texts)
        self._vecs = vecs

    def query(self, text: str, k: int = 3) -> List[Tuple[str, float]]:
        d, i = self.index.search(F.normalize(self.encode([text]).float(), dim=1), k)
        return [(self.payloads[int(j)], float(dist)) for dist, j in zip(d[0], i[0]) if int(j) >= 0]

    def save(self, directory: str) -> None:
        os.makedirs(directory, exist_ok=True)
        mm = np.memmap(os.path.join(directory, "vectors.f32"), dtype=np.float32, mode="w+", shape=tuple(self._vecs.shape))
        mm[:] = self._vecs.cpu().numpy()
        mm.flush()
        with open(os.path.join(directory, "payloads.jsonl"), "w") as f:
            for p in self.payloads:
                f.write(json.dumps(p) + "\n")
        torch.save({"coarse": self.index.coarse, "codebooks": self.index.codebooks, "codes": self.index.codes,
                    "cells": self.index.cells, "ids": self.index.ids}, os.path.join(directory, "index.pt"))
        json.dump({"shape": list(self._vecs.shape), "m": self.index.m, "n_list": self.index.n_list},
                  open(os.path.join(directory, "meta.json"), "w"))

    @staticmethod
    def load_vectors(directory: str) -> np.memmap:
        meta = json.load(open(os.path.join(directory, "meta.json")))
        return np.memmap(os.path.join(directory, "vectors.f32"), dtype=np.float32, mode="r", shape=tuple(meta["shape"]))

    def to_pq_field(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """(codebooks [C, ks, D/C], codes [N, C]) in the layout of the Subconscious PQ knowledge field."""
        return self.index.codebooks, self.index.codes.long()


class PiscesLxSubconsciousTrainer:
    """Three phases over a model that owns a ``subconscious`` system:
    1. router pre-training: cross entropy of the knowledge router against given block labels;
    2. policy refinement: REINFORCE on the router's sampled choice with the LM loss improvement as reward;
    3. self-play: the model's own continuations become the next round's inputs (reward = -loss on them)."""

    def __init__(self, model: Any, router: torch.nn.Module, lr: float = 1e-3):
        """``router``: the knowledge router (``YvKnowledgeRouter`` or any module mapping pooled hidden states
        [B, H] to scores over knowledge entries); its parameters are what the three phases train."""
        self.model, self.router = model, router
        self.params = [p for p in router.parameters() if p.requires_grad]
        self.opt = torch.optim.AdamW(self.params, lr=lr)
        self.phase_log: List[Dict[str, float]] = []

    def _router_logits(self, ids: torch.Tensor) -> torch.Tensor:
        with torch.no_grad():
            h = self.model.model.embed_tokens(ids, None).float().mean(1)
        return self.router(h)

    def phase1_router_pretrain(self, ids: torch.Tensor, block_labels: torch.Tensor, steps: int = 10) -> float:
        loss = torch.zeros(())
        for _ in range(steps):
            loss = F.cross_entropy(self._router_logits(ids), block_labels)
            self.opt.zero_grad(); loss.backward(); self.opt.step()
        self.phase_log.append({"phase": 1, "loss": float(loss)})
        return float(loss)

    def phase2_policy(self, ids: torch.Tensor, steps: int = 5) -> float:
        base = float(self.model(input_ids=ids, labels=ids)["loss"].detach())
        r = 0.0
        for _ in range(steps):
            logits = self._router_logits(ids)
            dist = torch.distributions.Categorical(logits=logits)
            a = dist.sample()
            with torch.no_grad():
                r = base - float(self.model(input_ids=ids, labels=ids)["loss"])
            loss = -(dist.log_prob(a) * r).mean() - 0.01 * dist.entropy().mean()
            self.opt.zero_grad(); loss.backward(); self.opt.step()
        self.phase_log.append({"phase": 2, "reward": r})
        return r

    def phase3_self_play(self, ids: torch.Tensor, rounds: int = 2, new_tokens: int = 8) -> float:
        loss_v = 0.0
        for _ in range(rounds):
            with torch.no_grad():
                ids, _ = self.model.generate(ids, max_new_tokens=new_tokens, eos_token_id=-1)
            self.phase2_policy(ids, steps=1)              # the model's own continuation is the next round's input
            with torch.no_grad():
                loss_v = float(self.model(input_ids=ids, labels=ids)["loss"])
        self.phase_log.append({"phase": 3, "loss": loss_v})
        return loss_v
