"""Serving benchmark of the Yv 7B-class MoE: decode tokens/s at a fixed batch and p50 time-to-first-token, through the
continuous-batching engine (the call a user of the server makes).

    python bench_serve.py --batch 64 --prompt-len 2048 --new-tokens 512                       (one GPU)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29551 \
        bench_serve.py --gpus 8 --prompt-len 32768 --new-tokens 512 --batch 64 --probe-len 131072

With ``--gpus N > 1`` every rank runs the same engine over the layout "tensor-parallel attention x expert-parallel
experts on the same N GPUs" (``init_parallel(tp=N, ep_over_tp=True)``): heads and the KV cache are sharded N ways, every
GPU holds 1/N of the routed experts, token rows are sharded between the layers.  ``--probe-len L`` adds a batch-1
prefill of an L-token prompt (time to first token of the long-context probe).

The reference serves one request at a time from a Python block pool (tools/infer/core.py:1106-1144,
model/utils/cache.py:807-835); its documents give targets only (>= 35 tok/s decode, TTFT <= 200 ms under 128 prompt
tokens, on a T4).  Two measurements are printed as one JSON line:

* ``ttft_p50_ms_unloaded``: one request at a time (prompt copied from pinned host memory, prefill, first token
  read back), median over ``--ttft-samples`` requests after warm-up;
* ``decode_tokens_per_s``: ``--batch`` requests admitted together, every one generating ``--new-tokens`` tokens;
  the timed region is the decode phase only (device events around it, every step's tokens read back to the host
  as the engine does), tokens / time.

Weights are random-init bf16 of the full architecture; prompts are uniform-random token ids."""
from __future__ import annotations

import argparse
import json
import statistics
import time

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--new-tokens", type=int, default=512)
    ap.add_argument("--ttft-prompt-len", type=int, default=128)
    ap.add_argument("--ttft-samples", type=int, default=8)
    ap.add_argument("--block-size", type=int, default=64)
    ap.add_argument("--model", default="yv_7b_moe")
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (result is then not a benchmark)")
    ap.add_argument("--no-graphs", action="store_true", help="decode through the eager step instead of CUDA graph replay")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--probe-len", type=int, default=0, help="also time a batch-1 prefill of this many tokens")
    ap.add_argument("--no-fused-comm", action="store_true")
    args = ap.parse_args()
    import os
    world = int(os.environ.get("WORLD_SIZE", "1"))

    from pisceslx_b200 import YvConfig
    from pisceslx_b200.models import build_model
    from pisceslx_b200.ops import check_status
    from pisceslx_b200.serve.engine import YvEngineConfig, YvInferenceEngine

    par = None
    if world > 1:
        from pisceslx_b200.ops import load_extension
        from pisceslx_b200.parallel.state import init_parallel
        load_extension()
        par = init_parallel(tp=world, ep_over_tp=True)
        dev = par.device
    else:
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
    cfg = YvConfig.yv_7b_moe() if args.model == "yv_7b_moe" else YvConfig.tiny_text_moe()
    if args.layers:
        cfg.n_layer = args.layers
    cfg.fused_comm = not args.no_fused_comm
    if world > 1:
        cfg.tensor_parallel, cfg.expert_parallel = world, world
    model = build_model(cfg, device=dev, dtype=torch.bfloat16, parallel=par, seed=0).eval()
    per_seq = (max(args.prompt_len, args.ttft_prompt_len) + args.new_tokens + args.block_size - 1) // args.block_size + 1
    probe_blocks = (args.probe_len + args.block_size - 1) // args.block_size + 2 if args.probe_len else 0
    eng = YvInferenceEngine(model, cfg=YvEngineConfig(max_num_seqs=args.batch,
                                                      num_blocks=max(per_seq * args.batch + 8, probe_blocks),
                                                      block_size=args.block_size, eos_token_id=-1,
                                                      max_model_len=max(131072, args.probe_len + 64),
                                                      use_cuda_graphs=not args.no_graphs and world == 1))
    gen = torch.Generator().manual_seed(0)

    def prompt(n: int):
        return torch.randint(0, cfg.vocab_size, (n,), generator=gen).pin_memory().tolist()

    # ---- unloaded TTFT ---------------------------------------------------------------------------------------
    ttft = []
    for i in range(args.ttft_samples + 3):
        r = eng.add_request(prompt(args.ttft_prompt_len), max_new_tokens=1)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.step()                                          # prefill + first token (read back inside)
        torch.cuda.synchronize()
        if i >= 3:
            ttft.append((time.perf_counter() - t0) * 1e3)
        eng.run_until_done()
    # prefill throughput at the long prompt
    prefill_s = 0.0
    for i in range(3):                                      # first pass loads the kernels of this shape
        r = eng.add_request(prompt(args.prompt_len), max_new_tokens=1)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.run_until_done()
        torch.cuda.synchronize()
        prefill_s = time.perf_counter() - t0

    # ---- long-context probe: batch 1, one prefill --------------------------------------------------------------
    probe_ms = None
    if args.probe_len:
        r = eng.add_request(prompt(args.probe_len), max_new_tokens=1)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.run_until_done()
        torch.cuda.synchronize()
        probe_ms = (time.perf_counter() - t0) * 1e3
        assert r.finished and r.finish_reason == "length", r.finish_reason

    # ---- batched decode ----------------------------------------------------------------------------------------
    reqs = [eng.add_request(prompt(args.prompt_len), max_new_tokens=args.new_tokens) for _ in range(args.batch)]
    t_admit = time.perf_counter()
    eng.step()                                              # admits + prefills every request, then one decode step
    for _ in range(3):
        eng.step()                                          # warm-up decode steps
    torch.cuda.synchronize()
    done0 = sum(len(q.output_ids) for q in reqs)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    steps = 0
    while eng.has_work():
        eng.step()
        steps += 1
    e1.record()
    torch.cuda.synchronize()
    check_status(dev)
    dec_ms = e0.elapsed_time(e1)
    toks = sum(len(q.output_ids) for q in reqs) - done0
    loaded = sorted(q.ttft * 1e3 for q in reqs)
    out = {
        "metric": "decode tokens/sec Yv-7B MoE", "value": toks / (dec_ms / 1e3), "unit": "tokens/s", "n_gpus": world,
        "higher_is_better": True, "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init weights",
        "decode_tokens_per_s": toks / (dec_ms / 1e3), "decode_ms_per_step": dec_ms / max(steps, 1), "decode_steps": steps,
        "ttft_p50_ms_unloaded": statistics.median(ttft), "ttft_prompt_len": args.ttft_prompt_len,
        "ttft_p50_ms_batch_admitted_together": loaded[len(loaded) // 2],
        "prefill_tokens_per_s": args.prompt_len / prefill_s,
        "config": {"model": "Yv 7B-class text MoE: 32L h4096 32q/8kv hd128, 64 experts ffn1408 top6 + 2 shared ffn2816, "
                            "vocab 154856" if not args.layers and args.model == "yv_7b_moe" else f"{args.model} layers={cfg.n_layer}",
                   "batch": args.batch, "prompt_len": args.prompt_len, "new_tokens": args.new_tokens,
                   "kv_block": args.block_size,
                   "parallelism": "tp1" if world == 1 else f"tp{world} attention x ep{world} experts on the same GPUs",
                   "fused_comm": bool(cfg.fused_comm) if world > 1 else None},
        "long_context_probe": {"prompt_len": args.probe_len, "ttft_ms": probe_ms} if args.probe_len else None,
        "max_memory_gb": torch.cuda.max_memory_allocated() / 1e9,
        "decode_graphs": eng.graph.stats(),
    }
    if world == 1 or par.rank == 0:
        print(json.dumps(out))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
