"""Per-kernel device time of one decode step of the serving engine.

    python -m pisceslx_b200.serve.profile_decode --batch 64 --prompt-len 2048 --steps 5

Builds the model (``--model yv_7b_moe`` or ``tiny``), admits ``--batch`` requests of ``--prompt-len`` random tokens,
warms up, then records ``--steps`` eager decode steps with the PyTorch profiler (CUDA activities only) and prints
the kernels sorted by device time per step.  The eager step is profiled because a graph replay shows up as one
launch; the kernels are the same."""
from __future__ import annotations

import argparse

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="yv_7b_moe", choices=["yv_7b_moe", "tiny"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--top", type=int, default=30)
    a = ap.parse_args()

    from torch.profiler import ProfilerActivity, profile

    from .. import YvConfig
    from ..models import build_model
    from .engine import YvEngineConfig, YvInferenceEngine

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = YvConfig.yv_7b_moe() if a.model == "yv_7b_moe" else YvConfig.tiny_text_moe()
    model = build_model(cfg, device=dev, dtype=torch.bfloat16, seed=0).eval()
    per_seq = (a.prompt_len + 64 + a.steps + 63) // 64 + 1
    eng = YvInferenceEngine(model, cfg=YvEngineConfig(max_num_seqs=a.batch, num_blocks=per_seq * a.batch + 8, block_size=64,
                                                      eos_token_id=-1, use_cuda_graphs=False))
    g = torch.Generator().manual_seed(0)
    for _ in range(a.batch):
        eng.add_request(torch.randint(0, cfg.vocab_size, (a.prompt_len,), generator=g).tolist(), max_new_tokens=a.steps + 16)
    for _ in range(5):
        eng.step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(a.steps):
            eng.step()
        torch.cuda.synchronize()
    rows = [(e.key, e.self_device_time_total / 1e3 / a.steps, e.count / a.steps) for e in prof.key_averages()
            if e.self_device_time_total > 0]
    rows.sort(key=lambda r: -r[1])
    total = sum(r[1] for r in rows)
    print(f"device ms per decode step: {total:.3f}  (batch {a.batch}, context {a.prompt_len}, {a.model})")
    for k, ms, c in rows[: a.top]:
        print(f"{ms:9.3f} ms {100 * ms / total:5.1f}% {c:7.1f}  {k[:110]}")


if __name__ == "__main__":
    main()
