"""Vision + text training step (the multimodal benchmark configuration): the 7B-class MoE language model with a
YvVisionEncoder (ViT, 24 layers, width 1024, 16 heads, patch 14, all images of a micro-batch packed into one token
stream), 4 synthetic 1024 x 1024 images per sample fused by YvDynamicModalFusion (cross-modal attention read-out)
into prefix tokens ahead of 2048 uniform-random text tokens, trained with the text next-token loss.

    python bench_multimodal.py --layers 8 --samples 4 --steps 2 --warmup 3

Prints one JSON line: samples/s and tokens/s (text tokens + vision patch tokens) of the whole step through the public
trainer API, timed with CUDA events after warm-up, inputs staged from pinned host memory every step.  ``--layers`` below
32 is a reduced-depth run and is labelled as such (the full model plus the vision tower needs the 8-GPU layout)."""
from __future__ import annotations

import argparse
import json
import os

VOCAB = 154856


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8, help="language-model layers (32 = the named configuration)")
    ap.add_argument("--samples", type=int, default=4, help="samples per optimizer step")
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--images", type=int, default=4)
    ap.add_argument("--image-size", type=int, default=1024)
    ap.add_argument("--text-len", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    import torch

    from pisceslx_b200 import YvConfig
    from pisceslx_b200.engine.trainer import YvTrainer, YvTrainerConfig
    from pisceslx_b200.models import build_model
    from pisceslx_b200.models.multimodal.fusion import attach_multimodal
    from pisceslx_b200.ops import check_status, load_extension
    from pisceslx_b200.parallel.state import init_parallel

    load_extension()
    par = init_parallel()
    dev = par.device
    cfg = YvConfig.yv_7b_moe(vocab_size=VOCAB, n_layer=a.layers)
    cfg.vision_hidden_size, cfg.vision_n_layer, cfg.vision_n_head, cfg.image_patch = 1024, 24, 16, 14
    cfg.use_gradient_checkpointing = True
    model = build_model(cfg, dev, torch.bfloat16, seed=1234)
    attach_multimodal(model, vision=True)
    n_vit = sum(p.numel() for p in model.model.vision_encoder.parameters())
    n_fuse = sum(p.numel() for p in model.model.modal_fusion.parameters())
    tcfg = YvTrainerConfig(micro_batch_size=a.micro_batch, optimizer="muon", lr=2e-4, weight_decay=0.1, warmup_steps=10,
                           max_steps=10_000, streaming_optimizer=True, clip_grad_norm=0.0, log_steps=1,
                           track_grad_norm=False, recompute_policy="auto", state_dtype="int8")
    trainer = YvTrainer(model, tcfg)
    g = torch.Generator().manual_seed(7)
    grid = a.image_size // 14
    batches = []
    for _ in range(2):
        ids = torch.randint(0, VOCAB, (a.samples, a.text_len), generator=g, dtype=torch.int64).pin_memory()
        img = torch.randn(a.samples, a.images, 3, a.image_size, a.image_size, generator=g).to(torch.bfloat16).pin_memory()
        batches.append({"input_ids": ids, "labels": ids, "images": img})

    def run(n):
        last = None
        for i in range(n):
            last = trainer.train_step(batches[i % 2])
        return last

    run(a.warmup)
    while trainer.recompute_planner is not None and trainer.recompute_planner.stage < 3:
        run(1)
    check_status()
    trainer.h2d_bytes = trainer.d2h_bytes = 0
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    last = run(a.steps)
    e1.record()
    torch.cuda.synchronize(dev)
    check_status()
    ms = e0.elapsed_time(e1) / a.steps
    vis_tokens = a.images * (grid * grid + 1)
    print(json.dumps({
        "metric": "multimodal train samples/s (vision + text)", "value": a.samples / (ms / 1e3), "unit": "samples/s",
        "tokens_per_s": a.samples * (a.text_len + vis_tokens) / (ms / 1e3), "ms_per_step": ms, "n_gpus": 1,
        "steps": a.steps, "warmup": a.warmup, "dtype": "bf16", "data": "synthetic N(0,1) pixels and uniform-random token ids, random-init weights",
        "config": {"language_model": f"Yv 7B-class MoE, {a.layers} of 32 layers" + ("" if a.layers == 32 else " [reduced depth]"),
                   "vision": f"ViT 24 x 1024 x 16 heads, patch 14, {a.images} images of {a.image_size}^2 per sample = "
                             f"{vis_tokens} vision tokens, packed per micro-batch ({n_vit / 1e6:.0f} M parameters)",
                   "fusion": f"YvDynamicModalFusion: {cfg.native_fusion_num_layers} blocks at width {cfg.hidden_size} + "
                             f"YvCrossModalAttention read-out to {cfg.native_fusion_output_tokens} prefix tokens "
                             f"({n_fuse / 1e6:.0f} M parameters)",
                   "text_len": a.text_len, "samples_per_step": a.samples, "micro_batch": a.micro_batch,
                   "optimizer": "Muon(2-D)+AdamW, int8 Muon momentum"},
        "e2e": {"h2d_bytes_per_step": trainer.h2d_bytes // a.steps, "d2h_bytes_per_step": trainer.d2h_bytes // a.steps},
        "loss": last["loss"], "max_memory_gb": torch.cuda.max_memory_allocated(dev) / 1e9}))


if __name__ == "__main__":
    main()
