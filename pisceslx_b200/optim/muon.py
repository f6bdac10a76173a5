"""Muon (orthogonalised momentum) + AdamW hybrid optimizer.

What it keeps from the reference's ``PiscesLxMuon`` (utils/muon.py:84-278): momentum 0.95 with optional
Nesterov, a 10-step quintic Newton-Schulz schedule with coefficients (3.4445, -4.7750, 2.0315) x 8 then
(2, -1.5, 0.5) x 2 run on the Gram matrix of the short side, RMS rescale to ``gamma * sqrt(max(n, m))``,
decoupled weight decay ``p * (1 - lr * wd)``, AdamW (betas 0.9/0.95) for everything that is not a 2-D
hidden weight (embeddings, LM head, norms, biases, router).

What differs on purpose: the reference iterates the polynomial on the Gram matrix itself and multiplies the
result into G once (utils/muon.py:258-271), which does not equalise singular values; here every step
updates X (``A = X X^T; X <- aX + (bA + cA^2) X``), the standard Newton-Schulz orthogonalisation, still with
all GEMMs on the short side.  Stacked parameters (``[E, n, m]`` expert weights, fused QKV / gate-up rows)
are split into the matrices the reference holds as separate parameters and orthogonalised as one batch
through the batched tcgen05 GEMM.

Two gradient intakes:
  * ``step()`` reads ``p.grad`` (plain training loop, gradient accumulation in ``.grad``);
  * ``attach_backward_hooks()`` folds each gradient into its momentum buffer (Muon) or applies AdamW the
    moment autograd has accumulated it and frees ``p.grad`` - parameters, momentum and one layer of
    gradients are then all that is resident, which is what lets the 40 B-parameter model train on one GPU.
    In this mode Muon's momentum doubles as the accumulator, so Nesterov look-ahead is not available.
"""
from __future__ import annotations

import math
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from ..ops import kernels, reference as ref, status_word

NS_COEFFS = ref.MUON_NS_COEFFS
Q8_BLOCK = 128            # elements per scale of the int8 momentum (the reference's Ink optimizer keeps block-quantised
                          # int8 / int4 moments too, opss/optim/ink/optimizer.py:84-638)


def dequantize_q8(q: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """int8 values + per-128-element scales -> dense tensor of ``q``'s shape."""
    if q.is_cuda and dtype == torch.bfloat16:
        out = torch.empty(q.shape, dtype=torch.bfloat16, device=q.device)
        kernels().dequant_q8(q, scale, out)
        return out
    return (q.view(-1, Q8_BLOCK).float() * scale.view(-1, 1)).view(q.shape).to(dtype)


def fold_q8_reference(q: torch.Tensor, scale: torch.Tensor, grad: torch.Tensor, mu: float, gscale: float, first: bool,
                      generator: Optional[torch.Generator] = None) -> None:
    """PyTorch form of the quantised momentum fold (CPU path and oracle of the kernel's arithmetic): de-quantise,
    ``m = (mu * m if first else m) + gscale * g``, new per-block scale ``max|m| / 127``, stochastic rounding."""
    m = q.view(-1, Q8_BLOCK).float() * scale.view(-1, 1)
    if first:
        m = m * mu
    m = m + grad.reshape(-1, Q8_BLOCK).float() * gscale
    amax = m.abs().amax(dim=1)
    ns = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    u = torch.rand(m.shape, generator=generator, device=m.device)
    t = torch.floor(m / ns.view(-1, 1) + u).clamp_(-127, 127)
    q.copy_(t.to(torch.int8).view(q.shape))
    scale.copy_(ns)


def split_spec_for(name: str, p: torch.Tensor, cfg=None) -> Optional[List[Tuple[int, int]]]:
    """Row ranges of the matrices fused into one parameter (None = the whole matrix is one)."""
    if cfg is None:
        return None
    d = cfg.head_dim
    if name.endswith("qkv_proj"):
        heads = p.shape[0] // d                              # local heads (q + k + v) of this tensor-parallel shard
        hk = heads * cfg.n_kv_head // (cfg.n_head + 2 * cfg.n_kv_head)
        hq = heads - 2 * hk
        return [(0, hq * d), (hq * d, (hq + hk) * d), ((hq + hk) * d, (hq + 2 * hk) * d)]
    return None


def _matrix_view(name: str, p: torch.Tensor) -> torch.Tensor:
    """View a (possibly stacked / fused) parameter as a batch of the matrices Muon orthogonalises."""
    if p.dim() == 3:
        if name.endswith("experts_w13"):                  # [E, 2F, H]: gate rows then up rows
            E, twoF, H = p.shape
            return p.view(E * 2, twoF // 2, H)
        return p
    if name.endswith("shared_w13"):                       # [S*2Fs, H]: per expert gate rows then up rows
        return p
    return p.unsqueeze(0)


def newton_schulz_batched(x: torch.Tensor, coeffs: Sequence[Tuple[float, float, float]] = NS_COEFFS,
                          eps: float = 1e-7) -> torch.Tensor:
    """Orthogonalise a batch ``x [G, n, m]`` (bf16, CUDA) in place of the reference's per-tensor Python loop.
    Returns a new tensor; GEMMs run on the short side."""
    if not x.is_cuda:
        return ref.newton_schulz(x, coeffs, eps).to(x.dtype)
    K = kernels()
    st = status_word(x.device)
    G, n, m = x.shape
    X = x.to(torch.bfloat16).contiguous().clone()
    norms = torch.empty(G, dtype=torch.float32, device=x.device)
    K.frob_normalize(X, norms, eps)
    short = min(n, m)
    usable = (n % 128 == 0 and m % 64 == 0) if n <= m else (m % 128 == 0 and n % 128 == 0)
    if not usable:
        return ref.newton_schulz(X.float() * 1.0, coeffs, eps).to(x.dtype)
    A = torch.empty(G, short, short, dtype=torch.bfloat16, device=x.device)
    A2 = torch.empty_like(A)
    Y = torch.empty_like(X)
    # X <- (aI + bA + cA^2) X with A = X X^T: the polynomial is formed on the small Gram matrix, so every
    # iteration is three GEMMs and one pass over [G, n, n]; the big operand is only ever read and written by GEMMs.
    # A and the polynomial are symmetric: those two products compute the tiles on or above the diagonal only and
    # mirror them (about 0.6 of the tiles at n = 1408 with 128 x 256 tiles)
    fused_poly = short % 128 == 0 and short % 64 == 0

    def poly(a: float, b: float, c: float) -> None:
        """A2 <- aI + bA + cA^2; in the epilogue of the A A product when the shape allows, else a separate pass."""
        if fused_poly:
            K.gemm_batched_affine(A, A, A, A2, a, b, c, st, True)        # symmetric: upper tiles + mirrored stores
        else:
            K.gemm_batched(A, A, A2, False, False, False, 0, st, True)   # A2 = A A^T = A^2 (A symmetric)
            K.ns_poly(A, A2, A2, a, b, c)

    for a, b, c in coeffs:
        if n <= m:
            K.gemm_batched(X, X, A, False, False, False, 0, st, True)    # A = X X^T        [n,n], symmetric
            poly(a, b, c)                                                # B = aI + bA + cA^2
            K.gemm_batched(A2, X, Y, False, True, False, 0, st)          # Y = B X          [n,m]
        else:
            K.gemm_batched(X, X, A, True, True, False, 0, st, True)      # A = X^T X        [m,m], symmetric
            poly(a, b, c)
            K.gemm_batched(X, A2, Y, False, False, False, 0, st)         # Y = X B^T = X B  [n,m]
        X, Y = Y, X
    return X


class YvMuon(torch.optim.Optimizer):
    """Hybrid Muon / AdamW.  ``named_params``: iterable of (name, parameter)."""

    def __init__(self, named_params: Iterable[Tuple[str, torch.nn.Parameter]], lr: float = 2e-4,
                 momentum: float = 0.95, nesterov: bool = True, ns_steps: int = 10, gamma: float = 0.18,
                 weight_decay: float = 0.1, adamw_lr: Optional[float] = None, adamw_betas=(0.9, 0.95),
                 adamw_eps: float = 1e-8, adamw_weight_decay: Optional[float] = None,
                 state_dtype: Optional[torch.dtype] = None, cfg=None):
        named = [(n, p) for n, p in named_params if p.requires_grad]
        muon, adam = [], []
        self._names: Dict[int, str] = {}
        for n, p in named:
            self._names[id(p)] = n
            (muon if self.is_muon_param(n, p) else adam).append(p)
        groups = [
            dict(params=muon, use_muon=True, lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps,
                 gamma=gamma, weight_decay=weight_decay),
            dict(params=adam, use_muon=False, lr=adamw_lr if adamw_lr is not None else lr, betas=adamw_betas,
                 eps=adamw_eps, weight_decay=weight_decay if adamw_weight_decay is None else adamw_weight_decay),
        ]
        super().__init__([g for g in groups if g["params"]], {})
        self.state_dtype = state_dtype
        self.cfg = cfg
        self._hooks: List[Any] = []
        self._streaming = False
        self._micro = 0
        self._grad_scale = 1.0
        self._step_count = 0
        self.sq_norm: Optional[torch.Tensor] = None       # running sum of squared gradient norms (device scalar)

    @staticmethod
    def is_muon_param(name: str, p: torch.Tensor) -> bool:
        """2-D hidden weights go to Muon; embeddings, LM head, norms, biases and the router stay on AdamW
        (reference factory, utils/muon.py:41-83)."""
        if p.dim() < 2:
            return False
        low = name.lower()
        return not any(k in low for k in ("embed", "lm_head", "norm", "bias", "router", "gate.weight", "mtp_heads",
                                          "codebook", "pos_emb"))

    # ------------------------------------------------------------------------------------------------
    def _state_for(self, p: torch.Tensor, group: Dict[str, Any]) -> Dict[str, Any]:
        st = self.state[p]
        if not st:
            dt = self.state_dtype or p.dtype
            if group["use_muon"]:
                if dt == torch.int8 and p.numel() % Q8_BLOCK == 0:
                    # block-quantised momentum: int8 values + one fp32 scale per 128 consecutive elements
                    st["momentum_q"] = torch.zeros_like(p, dtype=torch.int8)
                    st["momentum_scale"] = torch.ones(p.numel() // Q8_BLOCK, dtype=torch.float32, device=p.device)
                else:
                    st["momentum_buffer"] = torch.zeros_like(p, dtype=p.dtype if dt == torch.int8 else dt)
            else:
                dt = p.dtype if dt == torch.int8 else dt      # AdamW moments stay in the parameter dtype
                st["adam_step"] = 0
                st["adam_exp_avg"] = torch.zeros_like(p, dtype=dt)
                st["adam_exp_avg_sq"] = torch.zeros_like(p, dtype=dt)
        return st

    def _group_of(self, p: torch.Tensor) -> Dict[str, Any]:
        for g in self.param_groups:
            for q in g["params"]:
                if q is p:
                    return g
        raise KeyError("parameter not owned by this optimizer")

    # ---- Muon pieces --------------------------------------------------------------------------------
    def _fold(self, p: torch.Tensor, grad: torch.Tensor, group: Dict[str, Any], first: bool,
              want_update: bool) -> Optional[torch.Tensor]:
        st = self._state_for(p, group)
        mu = group["momentum"]
        if "momentum_q" in st:
            q, sc = st["momentum_q"], st["momentum_scale"]
            if p.is_cuda and grad.dtype == torch.bfloat16:
                self._q8_calls = getattr(self, "_q8_calls", 0) + 1
                seed = (self._step_count * 1000003 + self._q8_calls * 7919) & 0x7FFFFFFF
                kernels().momentum_fold_q8(q, sc, grad.contiguous(), mu, self._grad_scale, first, seed)
            else:
                fold_q8_reference(q, sc, grad, mu, self._grad_scale, first)
            if not want_update:
                return None
            m = dequantize_q8(q, sc, p.dtype)
            return (grad.to(p.dtype) * self._grad_scale).add(m, alpha=mu) if group["nesterov"] else m
        buf = st["momentum_buffer"]
        if p.is_cuda and buf.dtype == torch.bfloat16 and grad.dtype == torch.bfloat16:
            out = torch.empty_like(buf) if want_update else None
            kernels().momentum_fold(buf, grad.contiguous(), out, mu, self._grad_scale, bool(group["nesterov"]), first)
            return out
        g = grad.to(buf.dtype) * self._grad_scale
        if first:
            buf.mul_(mu)
        buf.add_(g)
        if not want_update:
            return None
        return g.add(buf, alpha=mu) if group["nesterov"] else buf.clone()

    def _apply_muon(self, p: torch.Tensor, update: torch.Tensor, group: Dict[str, Any]) -> None:
        name = self._names.get(id(p), "")
        mats = _matrix_view(name, update)
        rows = None
        if name.endswith("shared_w13") and self.cfg is not None:
            S = self.cfg.moe_shared_experts
            mats = update.view(S * 2, update.shape[0] // (S * 2), update.shape[1])
        elif name.endswith("qkv_proj") and self.cfg is not None:
            rows = split_spec_for(name, p, self.cfg)
        lr, wd, gamma = group["lr"], group["weight_decay"], group["gamma"]
        coeffs = NS_COEFFS[: group["ns_steps"]] if group["ns_steps"] <= len(NS_COEFFS) else NS_COEFFS
        if rows is None:
            O = newton_schulz_batched(mats, coeffs)
            n, m = mats.shape[-2], mats.shape[-1]
            # an orthogonalised n x m matrix has Frobenius norm sqrt(min(n,m)); rescale to gamma*sqrt(max(n,m))
            scale = gamma * math.sqrt(max(n, m)) / math.sqrt(min(n, m))
            O = O.reshape(p.shape)
            self._apply(p, O, lr, wd, scale)
        else:
            for lo, hi in rows:
                O = newton_schulz_batched(update[lo:hi].unsqueeze(0), coeffs).squeeze(0)
                n, m = hi - lo, update.shape[1]
                scale = gamma * math.sqrt(max(n, m)) / math.sqrt(min(n, m))
                self._apply(p[lo:hi], O, lr, wd, scale)

    @staticmethod
    def _apply(p: torch.Tensor, O: torch.Tensor, lr: float, wd: float, scale: float) -> None:
        if p.is_cuda and p.dtype == torch.bfloat16 and p.is_contiguous():
            kernels().muon_apply(p.data, O.to(torch.bfloat16).contiguous(), lr, wd, scale)
        else:
            p.data.mul_(1 - lr * wd).add_(O.to(p.dtype), alpha=-lr * scale)

    # ---- AdamW piece ----------------------------------------------------------------------------------
    def _apply_adamw(self, p: torch.Tensor, grad: torch.Tensor, group: Dict[str, Any]) -> None:
        st = self._state_for(p, group)
        st["adam_step"] += 1
        b1, b2 = group["betas"]
        if p.is_cuda:
            kernels().adamw(p.data, grad.contiguous(), st["adam_exp_avg"], st["adam_exp_avg_sq"], group["lr"], b1, b2,
                            group["eps"], group["weight_decay"], st["adam_step"], self._grad_scale)
        else:
            ref.adamw_step(p.data, grad.to(p.dtype) * self._grad_scale, st["adam_exp_avg"], st["adam_exp_avg_sq"],
                           group["lr"], b1, b2, group["eps"], group["weight_decay"], st["adam_step"])

    # ---- plain mode ------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, closure: Optional[Callable[[], torch.Tensor]] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._step_count += 1
        if self._streaming:
            self._finish_streaming_step()
            return loss
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                if group["use_muon"]:
                    upd = self._fold(p, p.grad, group, True, True)
                    self._apply_muon(p, upd, group)
                else:
                    self._apply_adamw(p, p.grad, group)
        return loss

    # ---- streaming (optimizer-in-backward) mode ------------------------------------------------------------
    def attach_backward_hooks(self, track_grad_norm: bool = False) -> None:
        """Consume gradients as autograd produces them.  Call ``begin_micro_batch(i, n)`` before each
        backward and ``step()`` after the last one."""
        self._streaming = True
        self._track_norm = track_grad_norm
        for group in self.param_groups:
            if group["use_muon"]:
                group["nesterov"] = False
            for p in group["params"]:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(group)))

    def detach_backward_hooks(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []
        self._streaming = False

    def begin_micro_batch(self, index: int, total: int) -> None:
        self._micro, self._micro_total = index, total
        self._grad_scale = 1.0 / total
        if index == 0 and getattr(self, "_track_norm", False):
            dev = self.param_groups[0]["params"][0].device
            self.sq_norm = torch.zeros(1, dtype=torch.float32, device=dev)

    def set_external_grad_params(self, ids) -> None:
        """Parameters whose gradients are reduced across data-parallel ranks first (``parallel.zero``): their
        backward hooks leave ``p.grad`` alone and the reduced gradient arrives through ``consume_external_grad``."""
        self._external = set(ids)

    @torch.no_grad()
    def consume_external_grad(self, p: torch.Tensor, grad: torch.Tensor) -> None:
        group = self._group_of(p)
        keep = self._grad_scale
        self._grad_scale = 1.0                              # already averaged by the synchronizer
        try:
            if group["use_muon"]:
                if self._streaming:
                    self._fold(p, grad, group, True, False)
                else:
                    p.grad = grad
            else:
                if self._streaming:
                    self._apply_adamw(p, grad, group)
                else:
                    p.grad = grad
        finally:
            self._grad_scale = keep

    def _make_hook(self, group: Dict[str, Any]):
        def hook(p: torch.Tensor) -> None:
            g = p.grad
            if g is None or id(p) in getattr(self, "_external", ()):
                return
            with torch.no_grad():
                if getattr(self, "_track_norm", False) and self.sq_norm is not None and g.is_cuda:
                    kernels().sumsq(g.contiguous(), self.sq_norm)
                if group["use_muon"]:
                    self._fold(p, g, group, self._micro == 0, False)
                else:
                    st = self._state_for(p, group)
                    acc = st.get("grad_acc")
                    if self._micro_total == 1:
                        self._apply_adamw(p, g, group)
                    else:
                        if acc is None:
                            st["grad_acc"] = g.detach().clone()
                        else:
                            acc.add_(g)
            p.grad = None
        return hook

    @torch.no_grad()
    def _finish_streaming_step(self) -> None:
        for group in self.param_groups:
            for p in group["params"]:
                st = self.state.get(p)
                if not st:
                    continue
                if group["use_muon"]:
                    if "momentum_q" in st:
                        self._apply_muon(p, dequantize_q8(st["momentum_q"], st["momentum_scale"], p.dtype), group)
                    else:
                        self._apply_muon(p, st["momentum_buffer"], group)
                elif st.get("grad_acc") is not None:
                    self._apply_adamw(p, st.pop("grad_acc"), group)
        self._grad_scale = 1.0

    def zero_grad(self, set_to_none: bool = True) -> None:  # type: ignore[override]
        super().zero_grad(set_to_none=set_to_none)
