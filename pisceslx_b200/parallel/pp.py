"""Pipeline parallelism: stages exchange activations and activation gradients with NCCL point-to-point calls.

The reference's "pipeline schedules" reorder forward / backward of micro-batches on one rank and never send
anything between stages (opss/train/parallel_3d.py:526-644).  Here a stage owns a contiguous slice of layers
(``YvModel`` builds only layers ``[layer_lo, layer_hi)``; the first stage owns the embedding, the last the final norm
and the LM head) and the schedules below move real tensors:

  * ``gpipe``  all forwards, then all backwards;
  * ``1f1b``   warm-up forwards, then one forward / one backward alternation, then the cool-down backwards, which
               bounds the number of live micro-batch activations by the pipeline depth.

The activation receive of micro-batch i+1 is posted before micro-batch i computes (``irecv`` runs on the
communicator's own stream), so the transfer from the previous stage overlaps with this stage's compute; sends are
asynchronous and are only waited for at the end of the step.  In 1F1B the previous stage always sends micro-batch
i+1 before it waits for a gradient that depends on this stage having consumed it, so the early receive cannot
deadlock.  Send / recv stays on NCCL by design.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist


class YvPipelineStage:
    def __init__(self, model: Any, parallel: Any, hidden_size: int, dtype: torch.dtype):
        self.model, self.par, self.hidden, self.dtype = model, parallel, hidden_size, dtype
        self.first, self.last = parallel.pp_rank == 0, parallel.pp_rank == parallel.pp_size - 1
        self.device = parallel.device

    # ---- p2p ------------------------------------------------------------------------------------------
    def _irecv(self, shape: Tuple[int, ...], src: int):
        buf = torch.empty(shape, dtype=self.dtype, device=self.device)
        return buf, dist.irecv(buf, src=src)

    def _isend(self, t: torch.Tensor, dst: int):
        return dist.isend(t.contiguous(), dst=dst)

    # ---- one micro-batch ---------------------------------------------------------------------------------
    def forward_micro(self, batch: Dict[str, torch.Tensor], recv: Optional[Tuple[torch.Tensor, Any]]):
        hidden_in = None
        if not self.first:
            buf, req = recv
            req.wait()
            hidden_in = buf.requires_grad_(True)
        out = self.model(input_ids=batch["input_ids"] if self.first else None, labels=batch.get("labels") if self.last else None,
                         hidden_in=hidden_in, return_logits=False, return_hidden=not self.last)
        if self.last:
            return hidden_in, out["loss"], None
        h = out["hidden_states"]
        send = self._isend(h.detach(), self.par.pp_next)
        return hidden_in, h, send

    def backward_micro(self, hidden_in: Optional[torch.Tensor], out: torch.Tensor, grad_recv, scale: float):
        if self.last:
            (out * scale).backward()
        else:
            buf, req = grad_recv
            req.wait()
            out.backward(buf)
        if not self.first:
            return self._isend(hidden_in.grad, self.par.pp_prev)
        return None

    # ---- schedules -------------------------------------------------------------------------------------------
    def run(self, micro_batches: List[Dict[str, torch.Tensor]], schedule: str = "1f1b") -> Optional[torch.Tensor]:
        """Forward + backward of all micro-batches; returns the mean loss on the last stage."""
        n = len(micro_batches)
        B, S = micro_batches[0]["input_ids"].shape
        shape = (B, S, self.hidden)
        scale = 1.0 / n
        warm = n if schedule == "gpipe" else min(self.par.pp_size - self.par.pp_rank - 1, n)
        live: List[Tuple[Optional[torch.Tensor], torch.Tensor]] = []
        sends: List[Any] = []
        losses: List[torch.Tensor] = []
        fwd_i = bwd_i = 0
        # activation receive posted one micro-batch ahead of the compute that consumes it
        pending = None if (self.first or n == 0) else self._irecv(shape, self.par.pp_prev)
        self.prefetched_receives = 0

        def do_forward():
            nonlocal fwd_i, pending
            recv = pending
            pending = None
            if not self.first and fwd_i + 1 < n:
                pending = self._irecv(shape, self.par.pp_prev)
                self.prefetched_receives += 1
            hin, out, send = self.forward_micro(micro_batches[fwd_i], recv)
            if send is not None:
                sends.append(send)
            if self.last:
                losses.append(out.detach())
            live.append((hin, out))
            fwd_i += 1

        def do_backward():
            nonlocal bwd_i
            hin, out = live.pop(0)
            grecv = None if self.last else self._irecv(shape, self.par.pp_next)
            s = self.backward_micro(hin, out, grecv, scale)
            if s is not None:
                sends.append(s)
            bwd_i += 1

        for _ in range(warm):
            do_forward()
        while fwd_i < n:
            do_forward()
            do_backward()
        while bwd_i < n:
            do_backward()
        for s in sends:
            s.wait()
        if self.last:
            return torch.stack(losses).mean()
        return None
