"""CPU tests of the engine subsystems: optimizers and schedules, checkpoint / resume contract, run store and recovery,
data pipeline, quantisation, alignment losses, speculative decoding, serving engine, CLI."""
import json
import math
import os
import subprocess
import sys
import time

import pytest
import torch

from pisceslx_b200 import YvConfig
from pisceslx_b200.models import build_model

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def tiny(**kw):
    cfg = YvConfig.tiny_text_moe(vocab_size=512)
    cfg.n_layer = 2
    for k, v in kw.items():
        setattr(cfg, k, v)
    return cfg


# ------------------------------------------------------------------------------------------------ optim
def test_newton_schulz_orthogonalises():
    from pisceslx_b200.ops.reference import newton_schulz
    torch.manual_seed(0)
    for shape in [(32, 64), (64, 32), (48, 48)]:
        g = torch.randn(*shape)
        o = newton_schulz(g)
        s = torch.linalg.svdvals(o)
        assert s.max() < 1.3 and s.min() > 0.5, (shape, s.min(), s.max())
        # same singular vectors: O^T G is (nearly) symmetric positive
        u, _, vh = torch.linalg.svd(g, full_matrices=False)
        assert torch.allclose(o, u @ torch.diag(s) @ vh, atol=1e-3)


def test_muon_int8_momentum_cpu_path_and_state_dict():
    """The quantised-momentum option on CPU (PyTorch fold): state is int8 + per-128 scales, survives a state-dict
    round trip, and a few steps move the weights like the bf16-state optimizer does."""
    from pisceslx_b200.optim.muon import YvMuon, dequantize_q8
    torch.manual_seed(0)
    w0 = torch.randn(128, 256)
    outs = {}
    for name, sd in (("q8", torch.int8), ("fp32", None)):
        p = torch.nn.Parameter(w0.clone())
        opt = YvMuon([("layer.w", p)], lr=1e-2, state_dtype=sd, nesterov=False)
        g = torch.Generator().manual_seed(1)
        for _ in range(3):
            p.grad = torch.randn(128, 256, generator=g)
            opt.step()
        outs[name] = (p.detach().clone(), opt)
    st = outs["q8"][1].state_dict()["state"][0]
    assert st["momentum_q"].dtype == torch.int8 and st["momentum_scale"].numel() == 128 * 256 // 128
    ref_m = outs["fp32"][1].state_dict()["state"][0]["momentum_buffer"]
    got_m = dequantize_q8(st["momentum_q"], st["momentum_scale"], torch.float32)
    assert (got_m - ref_m).norm() / ref_m.norm() < 2e-2
    assert (outs["q8"][0] - outs["fp32"][0]).norm() / (outs["fp32"][0] - w0).norm() < 0.1
    # tensors whose size is not a multiple of 128 keep a dense momentum
    p = torch.nn.Parameter(torch.randn(3, 50))
    opt = YvMuon([("odd.w", p)], state_dtype=torch.int8)
    p.grad = torch.randn(3, 50)
    opt.step()
    assert "momentum_buffer" in opt.state[p]


def test_muon_param_split_and_adamw_formula():
    from pisceslx_b200.optim import YvMuon
    from pisceslx_b200.ops.reference import adamw_step
    m = build_model(tiny())
    opt = YvMuon(m.named_parameters(), lr=1e-2, cfg=m.cfg)
    muon = {opt._names[id(p)] for g in opt.param_groups if g["use_muon"] for p in g["params"]}
    adam = {opt._names[id(p)] for g in opt.param_groups if not g["use_muon"] for p in g["params"]}
    assert "model.layers.0.attention.qkv_proj" in muon and "model.layers.0.mlp.experts_w13" in muon
    assert "model.embed.weight" in adam and "lm_head" in adam and "model.norm.weight" in adam
    assert "model.layers.0.mlp.router.gate.weight" in adam
    # AdamW: decay uses the pre-update parameter
    p, g, mm, v = torch.tensor([1.0]), torch.tensor([0.5]), torch.zeros(1), torch.zeros(1)
    adamw_step(p, g, mm, v, 0.1, 0.9, 0.999, 1e-8, 0.1, 1)
    assert abs(float(p) - (1.0 - 0.1 * (1.0 + 0.1 * 1.0))) < 1e-5


def test_lr_schedules():
    from pisceslx_b200.optim import YvLRSchedulerConfig, lr_at
    c = YvLRSchedulerConfig("cosine", 1.0, warmup_steps=10, total_steps=110, min_lr_ratio=0.1)
    assert abs(lr_at(c, 0) - 0.1) < 1e-9 and abs(lr_at(c, 9) - 1.0) < 1e-9
    assert abs(lr_at(c, 110) - 0.1) < 1e-6 and lr_at(c, 60) < 1.0
    for kind in ("linear", "polynomial", "inverse_sqrt", "step", "exponential", "constant"):
        c.scheduler_type = kind
        vals = [lr_at(c, s) for s in range(0, 120, 10)]
        assert all(v > 0 for v in vals)


def test_ink_optimizer_quantised_state_and_progress():
    from pisceslx_b200.optim.ink import PiscesLxInkBlockQuantizer, YvInkOptimizer
    q = PiscesLxInkBlockQuantizer(8, 64)
    x = torch.randn(1000)
    qq, s, shape, n = q.quantize(x)
    assert qq.dtype == torch.int8 and (q.dequantize(qq, s, shape, n) - x).abs().max() < 0.05
    w = torch.nn.Parameter(torch.randn(16, 16))
    opt = YvInkOptimizer([w], lr=0.05, weight_decay=0.0)
    l0 = None
    for _ in range(40):
        loss = (w ** 2).sum()
        l0 = l0 or float(loss)
        opt.zero_grad(); loss.backward(); opt.step()
    assert float((w ** 2).sum()) < 0.5 * l0
    assert opt.state_bytes() < 4 * 2 * w.numel()          # far below two fp32 moments


# ------------------------------------------------------------------------------------------------ checkpoint
def test_checkpoint_layout_resume_and_retention(tmp_path):
    from pisceslx_b200.engine.checkpoint import load_checkpoint, save_checkpoint
    from pisceslx_b200.engine.trainer import YvTrainer, YvTrainerConfig
    m = build_model(tiny())
    tr = YvTrainer(m, YvTrainerConfig(micro_batch_size=2, optimizer="adamw", lr=1e-3, max_steps=50))
    ids = torch.randint(0, 512, (2, 16))
    for _ in range(2):
        tr.train_step({"input_ids": ids, "labels": ids})
    for step in (1, 2, 3, 4, 5):
        save_checkpoint(tr, str(tmp_path / f"checkpoint_step_{step}.pt"))
    kept = sorted(p.name for p in tmp_path.glob("checkpoint_step_*.pt"))
    assert kept == ["checkpoint_step_3.pt", "checkpoint_step_4.pt", "checkpoint_step_5.pt"]
    ck = torch.load(tmp_path / "checkpoint_step_5.pt", weights_only=False)
    for k in ["model_state_dict", "adapter_state_dict", "optimizer_state_dict", "scheduler_state_dict", "global_step",
              "best_metric", "config", "training_stats", "materialized_components", "timestamp"]:
        assert k in ck
    assert "layers.0.mlp.experts.0.gate_proj.weight" in ck["model_state_dict"]
    m2 = build_model(tiny(), seed=9)
    tr2 = YvTrainer(m2, YvTrainerConfig(micro_batch_size=2, optimizer="adamw", lr=1e-3, max_steps=50))
    info = load_checkpoint(tr2, str(tmp_path / "checkpoint_step_5.pt"))
    assert tr2.global_step == 2 and not info["warnings"]
    a = tr.train_step({"input_ids": ids, "labels": ids})["loss"]
    b = tr2.train_step({"input_ids": ids, "labels": ids})["loss"]
    assert abs(a - b) < 1e-5
    # param-group mismatch degrades with a warning instead of failing (resume contract)
    tr3 = YvTrainer(build_model(tiny()), YvTrainerConfig(optimizer="muon", lr=1e-3))
    info3 = load_checkpoint(tr3, str(tmp_path / "checkpoint_step_5.pt"))
    assert info3["warnings"]


def test_checkpoint_verifier(tmp_path):
    from pisceslx_b200.engine.verify import PiscesLxCheckpointVerifier
    cfg = YvConfig.from_yaml(os.path.join(ROOT, "configs/model/0.01B.yaml"))
    cfg.vocab_size = 512
    p = tmp_path / "c.json"
    cfg.to_json(p)
    m = build_model(cfg)
    torch.save({"model_state_dict": m.to_reference_state_dict()}, tmp_path / "m.pt")
    rep = PiscesLxCheckpointVerifier().verify(str(tmp_path / "m.pt"), model_config=str(p), tokens=32)
    assert rep["ok"] and rep["strict_loadable"] and rep["tensors_differing_from_fresh_init"] > 0


# ------------------------------------------------------------------------------------------------ run store / recovery
def test_run_store_control_and_recovery(tmp_path):
    from pisceslx_b200.engine.runstore import (PiscesLxGPUAllocationScheduler, PiscesLxGPUInfo, PiscesLxHeartbeatMonitor,
                                               PiscesLxRunStore, PiscesLxStateFileCorruptedError, PiscesLxTaskQueue,
                                               PiscesLxTaskRecovery, PiscesLxTrainingRunReporter)
    store = PiscesLxRunStore(tmp_path / "runs")
    store.init_run("r1", {"argv": ["x"]})
    assert store.read_state("r1")["status"] == "pending"
    rep = PiscesLxTrainingRunReporter(store, "r1")
    rep({"global_step": 1, "loss": 2.0, "learning_rate": 1e-3})
    assert store.read_jsonl("r1", "metrics.jsonl")[0]["loss"] == 2.0
    store.send_control("r1", "stop")
    rep.poll_control()
    assert rep.stop_requested
    # crash detection: state says running, pid does not exist
    store.update_state("r1", status="running", pid=2 ** 22 + 12345)
    rec = PiscesLxTaskRecovery(store, max_restarts=1)
    assert rec.check_crashed("r1") and rec.restart_task("r1") and not rec.restart_task("r1")
    assert store.read_state("r1")["status"] == "failed"
    # heartbeat staleness
    hb = PiscesLxHeartbeatMonitor(store, "r1", timeout_s=0.05)
    hb.beat()
    assert not hb.is_stale()
    assert hb.is_stale(now=time.time() + 1.0)
    # tampering with state.json is detected
    p = store.run_dir("r1") / "state.json"
    st = json.load(open(p)); st["status"] = "completed"; json.dump(st, open(p, "w"))
    with pytest.raises(PiscesLxStateFileCorruptedError):
        store.read_state("r1")
    # newest checkpoint discovery ignores empty files
    d = tmp_path / "ck"; d.mkdir()
    (d / "checkpoint_step_10.pt").write_bytes(b"x"); (d / "checkpoint_step_20.pt").write_bytes(b"")
    assert PiscesLxTaskRecovery.find_latest_checkpoint(str(d)).step == 10
    q = PiscesLxTaskQueue(); q.submit({"a": 1}, priority=5); q.submit({"a": 2}, priority=1)
    assert q.pop().spec["a"] == 2
    fake = lambda: [PiscesLxGPUInfo(0, 1000, 900, 90), PiscesLxGPUInfo(1, 1000, 10, 0), PiscesLxGPUInfo(2, 1000, 20, 5)]
    sch = PiscesLxGPUAllocationScheduler(fake)
    assert sch.allocate("a", 2) == [1, 2]
    with pytest.raises(RuntimeError):
        sch.allocate("b", 2)


# ------------------------------------------------------------------------------------------------ data
def test_collator_and_dedup(tmp_path):
    from pisceslx_b200.data.cleaning import (PiscesLxDataExactDeduplicator, PiscesLxDataMinHashDeduplicator,
                                             PiscesLxDatasetCleaner)
    from pisceslx_b200.data.datasets import PiscesLxToolsDataTextCollator, SyntheticTokenDataset
    col = PiscesLxToolsDataTextCollator(8)
    b = col([{"input_ids": [5, 6, 7], "prompt_len": 2}, {"input_ids": list(range(10, 22))}])
    assert b["input_ids"].shape == (2, 8) and b["labels"][0].tolist() == [-100, -100, 7, -100, -100, -100, -100, -100]
    assert b["attention_mask"][0].tolist() == [1, 1, 1, 0, 0, 0, 0, 0]
    packed = PiscesLxToolsDataTextCollator(4, pack=True)([{"input_ids": [1, 2, 3]}, {"input_ids": [4, 5, 6]}])
    assert packed["input_ids"].tolist() == [[1, 2, 3, 4], [5, 6, 0, 0]] and packed["labels"][1].tolist() == [5, 6, -100, -100]
    it = iter(SyntheticTokenDataset(100, 16, 3, seed=1))
    assert next(it)["input_ids"].shape == (3, 16)
    base = ("the quick brown fox jumps over the lazy dog while the tensor cores of the accelerator multiply matrices in "
            "low precision and accumulate the products in a wider format held close to the arithmetic units")
    texts = [base, base, base.replace("lazy dog", "lazy cat"), "completely different sentence about paged caches " * 3]
    assert len(list(PiscesLxDataExactDeduplicator().dedup(texts))) == 3
    assert len(list(PiscesLxDataMinHashDeduplicator(threshold=0.7).dedup(texts))) == 2
    assert list(PiscesLxDatasetCleaner(min_chars=5).clean(["ok text here\x00", "!!!!!!!!!!!!!!!!!!!!!!!"])) == ["ok text here"]


# ------------------------------------------------------------------------------------------------ quantisation
def test_fp8_blockwise_and_fp4_and_ptq():
    from pisceslx_b200.quant import (PiscesLxAWQQuantizer, PiscesLxBlockWiseINT4Quantizer, PiscesLxFP4Quantizer,
                                     PiscesLxGPTQQuantizer, PiscesLxSmoothQuantizer, YvFP8Linear, dequantize_fp8_blockwise,
                                     fp8_gemm_reference, quantize_fp8_blockwise)
    torch.manual_seed(0)
    x = torch.randn(40, 300) * torch.logspace(-2, 2, 300)
    q, s = quantize_fp8_blockwise(x, (1, 128))
    assert q.dtype == torch.float8_e4m3fn and s.shape == (40, 3)
    rel = ((dequantize_fp8_blockwise(q, s, (1, 128)) - x).norm() / x.norm()).item()
    assert rel < 0.04
    q2, s2 = quantize_fp8_blockwise(x, (1, 128), pow2_scales=True)
    assert torch.allclose(torch.log2(s2), torch.log2(s2).round())
    w = torch.randn(256, 300) * 0.05
    wq, ws = quantize_fp8_blockwise(w, (128, 128))
    y = fp8_gemm_reference(q, s, wq, ws)
    assert ((y - x @ w.t()).norm() / (x @ w.t()).norm()).item() < 0.06
    lin = YvFP8Linear(64, 32)
    inp = torch.randn(4, 64, requires_grad=True)
    lin(inp).sum().backward()
    assert inp.grad is not None and lin.weight.grad is not None
    f4 = PiscesLxFP4Quantizer(16, stochastic=True, seed=0)
    v = torch.randn(4096)
    est = torch.stack([f4.fake_quant(v) for _ in range(64)]).mean(0)
    assert (est - v).abs().mean() < 0.08                       # stochastic rounding is unbiased
    grid = f4.quantize(v)[0].abs().unique()
    assert set(grid.tolist()) <= {0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0}
    W = torch.randn(32, 128) * 0.1
    X = torch.randn(256, 128) * torch.linspace(0.1, 3.0, 128)
    rtn = PiscesLxBlockWiseINT4Quantizer(64).fake_quant(W)
    gptq = PiscesLxGPTQQuantizer(4, 64).quantize(W, X)
    awq, _ = PiscesLxAWQQuantizer(4, 64).quantize(W, X)
    err = lambda Wq: float(((X @ Wq.t()) - (X @ W.t())).pow(2).mean())
    assert err(gptq) <= err(rtn) * 1.001 and err(awq) <= err(rtn) * 1.001
    Ws, sc = PiscesLxSmoothQuantizer(0.5).apply(W, X)
    assert torch.allclose((X / sc) @ Ws.t(), X @ W.t(), atol=1e-3)


# ------------------------------------------------------------------------------------------------ alignment
def test_alignment_losses():
    from pisceslx_b200.engine import alignment as al
    pc, pr, rc, rr = torch.tensor([-1.0]), torch.tensor([-3.0]), torch.tensor([-2.0]), torch.tensor([-2.0])
    loss, stats = al.dpo_loss(pc, pr, rc, rr, beta=0.5)
    assert abs(float(loss) - (-math.log(1 / (1 + math.exp(-1.0))))) < 1e-6 and float(stats["accuracy"]) == 1.0
    adv = al.group_relative_advantages(torch.tensor([1.0, 0.0, 3.0, 3.0]), 2)
    assert abs(float(adv[0]) + float(adv[1])) < 1e-5 and float(adv[2]) == 0.0
    assert al.dapo_filter_groups(torch.tensor([1.0, 0.0, 3.0, 3.0]), 2).tolist() == [True, True, False, False]
    lp = torch.zeros(2, 3, requires_grad=True)
    l = al.ppo_loss(lp, torch.zeros(2, 3), torch.ones(2, 3), clip=0.2)
    l.backward()
    assert abs(float(l) + 1.0) < 1e-6
    a, r = al.gae(torch.tensor([[0.0, 0.0, 1.0]]), torch.zeros(1, 3), gamma=1.0, lam=1.0)
    assert a[0].tolist() == [1.0, 1.0, 1.0]
    assert al.PiscesLxRLVRVerifier("numeric").reward(" 3.0", "3") == 1.0
    s, t = torch.randn(4, 10), torch.randn(4, 10)
    assert float(al.distill_logits_loss(t, t)) < 1e-6 and float(al.distill_logits_loss(s, t)) > 0
    m = build_model(tiny())
    m.eval()
    ids = torch.randint(0, 512, (1, 8))
    before = m(input_ids=ids).logits.clone()
    al.grow_depth(m, [0])
    assert len(m.model.layers) == 3
    assert torch.allclose(m(input_ids=ids).logits, before, atol=1e-4)        # function preserving
    al.grow_experts(m.model.layers[0].mlp, 12)
    assert m.model.layers[0].mlp.experts_w13.shape[0] == 12 and torch.isfinite(m(input_ids=ids).logits).all()


# ------------------------------------------------------------------------------------------------ generation / serving
def test_speculative_matches_greedy_and_sampler_filters():
    from pisceslx_b200.models.generation import YvSampler, YvSamplingConfig
    from pisceslx_b200.models.speculative import YvSpeculativeConfig, YvSpeculativeDecoder, beam_search
    torch.manual_seed(0)
    m = build_model(tiny())
    m.eval()
    ids = torch.randint(0, 512, (1, 6))
    greedy, _ = m.generate(ids, max_new_tokens=8, eos_token_id=-1)
    spec, stats = YvSpeculativeDecoder(m, YvSpeculativeConfig(draft_length=3)).speculative_generate(ids, 8, eos_token_id=-1)
    assert torch.equal(spec, greedy) and stats["generated_tokens"] >= 8
    # with the target as its own draft model every greedy draft is accepted
    spec2, st2 = YvSpeculativeDecoder(m, YvSpeculativeConfig(draft_length=3), draft_model=m).speculative_generate(ids, 8, eos_token_id=-1)
    assert torch.equal(spec2, greedy) and st2["acceptance_rate"] == 1.0
    assert beam_search(m, ids, num_beams=2, max_new_tokens=3).shape[1] == 9
    logits = torch.tensor([[5.0, 4.0, 1.0, -2.0, -9.0]])
    s = YvSampler(YvSamplingConfig(strategy="top_k", top_k=2, temperature=1.0, seed=0))
    assert set(int(s.sample(logits)) for _ in range(50)) <= {0, 1}
    f = YvSampler(YvSamplingConfig(strategy="top_p", top_p=0.5)).filter(logits)
    assert torch.isfinite(f[0, 0]) and not torch.isfinite(f[0, 2])
    pen = YvSampler.apply_repetition_penalty(logits.clone(), torch.tensor([[0]]), 2.0)
    assert float(pen[0, 0]) == 2.5
    blocked = YvSampler.block_repeated_ngrams(torch.zeros(1, 5), torch.tensor([[1, 2, 1]]), 2)
    assert blocked[0, 2] == float("-inf")


def test_serving_engine_continuous_batching_matches_single_requests():
    from pisceslx_b200.serve.engine import YvEngineConfig, YvInferenceEngine
    torch.manual_seed(1)
    m = build_model(tiny())
    eng = YvInferenceEngine(m, cfg=YvEngineConfig(max_num_seqs=4, num_blocks=64, block_size=16, eos_token_id=-1))
    prompts = [[5, 6, 7, 8], [9, 10], [11, 12, 13, 14, 15, 16, 17], [3]]
    reqs = [eng.add_request(p, max_new_tokens=6) for p in prompts]
    eng.run_until_done()
    for p, r in zip(prompts, reqs):
        ref, _ = m.generate(torch.tensor([p]), max_new_tokens=6, eos_token_id=-1)
        assert r.output_ids == ref[0, len(p):].tolist() and r.finish_reason == "length" and r.ttft is not None
    st = eng.get_stats()
    assert st["tokens_generated"] == 24 and st["free_blocks"] == 64 and st["p50_ttft"] is not None
    assert len(eng.embeddings("hello")) == m.cfg.hidden_size


def test_serving_engine_admission_reserves_worst_case_blocks():
    """A small cache with concurrent long generations: admission counts the blocks that running requests may still
    take, so the allocator never runs dry inside a decode step; requests wait and all finish with exact outputs.
    A request forced in behind the scheduler's back is preempted and resumed, again token for token."""
    from pisceslx_b200.serve.engine import YvEngineConfig, YvInferenceEngine
    torch.manual_seed(1)
    m = build_model(tiny())
    # 8 blocks of 4 tokens: one request needs ceil((3 + 17) / 4) = 5 blocks in the worst case, so two never fit
    eng = YvInferenceEngine(m, cfg=YvEngineConfig(max_num_seqs=4, num_blocks=8, block_size=4, eos_token_id=-1,
                                                  use_cuda_graphs=False))
    prompts = [[5, 6, 7], [9, 10, 11], [11, 12, 13]]
    reqs = [eng.add_request(p, max_new_tokens=17) for p in prompts]
    peak = 0
    while eng.has_work():
        eng.step()
        peak = max(peak, len(eng.running))
        assert eng.cache.alloc.available() >= 0
    assert peak == 1                                       # lazily allocated blocks would have let two in
    for p, r in zip(prompts, reqs):
        ref, _ = m.generate(torch.tensor([p]), max_new_tokens=17, eos_token_id=-1)
        assert r.output_ids == ref[0, len(p):].tolist() and r.finish_reason == "length"
    assert eng.get_stats()["free_blocks"] == 8 and eng.stats["errors"] == 0
    # preemption path: shrink the reservations by hand so that two requests run and the pool runs out mid-way
    reqs = [eng.add_request(p, max_new_tokens=17) for p in prompts[:2]]
    eng._worst_case_blocks = lambda req: 1
    eng.run_until_done()
    assert eng.stats["preemptions"] >= 1
    for p, r in zip(prompts[:2], reqs):
        ref, _ = m.generate(torch.tensor([p]), max_new_tokens=17, eos_token_id=-1)
        assert r.output_ids == ref[0, len(p):].tolist()
    # a request that can never fit is rejected, not queued forever
    big = eng.add_request(list(range(3, 40)), max_new_tokens=8)
    del eng._worst_case_blocks
    eng.run_until_done()
    assert big.finished and big.finish_reason.startswith("error")


def test_openai_server_endpoints():
    from fastapi.testclient import TestClient
    from pisceslx_b200.serve.engine import YvEngineConfig, YvInferenceEngine
    from pisceslx_b200.serve.server import PiscesLxInferService
    cfg = tiny()
    m = build_model(cfg)
    svc = PiscesLxInferService(YvInferenceEngine(m, cfg=YvEngineConfig(num_blocks=64, block_size=16, eos_token_id=-1)))
    with TestClient(svc.build_app()) as c:
        assert c.get("/healthz").json()["status"] == "ok"
        assert c.get("/v1/models").json()["data"][0]["id"] == "yv"
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4}).json()
        assert r["object"] == "chat.completion" and r["usage"]["completion_tokens"] == 4
        r = c.post("/v1/completions", json={"prompt": "abc", "max_tokens": 3}).json()
        assert r["choices"][0]["finish_reason"] == "length"
        with c.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3,
                                                          "stream": True}) as s:
            body = "".join(s.iter_text())
        assert body.count("chat.completion.chunk") == 4 and body.strip().endswith("data: [DONE]")
        assert len(c.post("/v1/embeddings", json={"input": "x"}).json()["data"][0]["embedding"]) == cfg.hidden_size
        assert c.get("/stats").json()["requests"] >= 3
    svc.stop()


def test_server_tools_agents_runs_media_and_model_router(tmp_path, monkeypatch):
    from fastapi.testclient import TestClient
    from pisceslx_b200.engine.runstore import PiscesLxRunStore
    from pisceslx_b200.serve.engine import YvEngineConfig, YvInferenceEngine
    from pisceslx_b200.serve.server import PiscesLxInferService, PiscesLxModelRouter
    m = build_model(tiny())
    svc = PiscesLxInferService(YvInferenceEngine(m, cfg=YvEngineConfig(num_blocks=64, block_size=16, eos_token_id=-1)))
    svc.runs = PiscesLxRunStore(tmp_path / "runs")
    svc.runs.init_run("run-1", {"stage": "pretrain"}, {"step": 3})
    svc.media = {"audio": lambda body: {"samples": len(body.get("input", "")) * 100}}
    app = svc.build_app()
    svc.tools.register("add", "adds two integers", {"a": "int", "b": "int"})(lambda a, b: a + b)
    with TestClient(app) as c:
        assert [t["name"] for t in c.get("/v1/tools/list").json()["data"]] == ["add"]
        assert c.post("/v1/tools/search", json={"query": "integers"}).json()["data"][0]["name"] == "add"
        assert c.post("/v1/tools/execute", json={"name": "add", "arguments": {"a": 2, "b": 5}}).json()["result"] == 7
        assert c.post("/v1/tools/execute", json={"name": "nope"}).status_code == 404
        assert c.post("/v1/tools/execute", json={"name": "add", "arguments": {"a": 1}}).status_code == 400
        assert c.get("/v1/agents/list").json()["data"][0]["id"] == "react"
        r = c.post("/v1/agents/execute", json={"task": "say hi", "max_turns": 1, "max_tokens": 4})
        assert r.status_code == 200 and "result" in r.json()
        assert c.get("/v1/runs").json()["data"] == ["run-1"]
        assert c.get("/v1/runs/run-1").json()["state"]["step"] == 3
        assert c.post("/v1/runs/run-1/control", json={"command": "pause"}).json()["accepted"]
        assert c.post("/v1/runs/run-1/control", json={"command": "explode"}).status_code == 400
        assert c.post("/v1/runs/none/control", json={"command": "stop"}).status_code == 404
        assert c.post("/v1/images/generations", json={"prompt": "a cat"}).status_code == 501
        assert c.post("/v1/audio/speech", json={"input": "hello"}).json()["data"]["samples"] == 500
    svc.stop()
    assert svc.runs.read_jsonl("run-1", "control.jsonl")[-1]["command"] == "pause"
    from pisceslx_b200.serve.server import PiscesLxAgentInterceptor
    script = iter(['I need a sum. <tool_call><name>add</name><arguments>{"a": 40, "b": 2}</arguments></tool_call>',
                   "The answer is 42."])
    seen = []
    icpt = PiscesLxAgentInterceptor(lambda p, n: seen.append(p) or next(script), svc.tools, mode="auto")
    out = icpt.run("what is 40 + 2?")
    assert out["content"] == "The answer is 42." and out["rounds"] == 1 and out["tool_calls"][0]["result"] == 42
    assert '<tool_result name="add">42</tool_result>' in seen[1]
    off = PiscesLxAgentInterceptor(lambda p, n: "<tool_call><name>add</name><arguments>{}</arguments></tool_call>", svc.tools, "off")
    assert off.run("x")["rounds"] == 0
    forced = PiscesLxAgentInterceptor(lambda p, n: seen.append(p) or "done", svc.tools, "forced")
    forced.run("task")
    assert "add(a, b)" in seen[-1]
    router = PiscesLxModelRouter(available=["0.5B", "7B"], default_size="7B")
    assert router.resolve("piscesl1-7b") == {"model_id": "piscesl1-7b", "model_size": "7B", "strategy": "explicit",
                                             "fallback_chain": ["0.5B"]}
    r = router.resolve("671B")
    assert r["strategy"] == "fallback" and r["model_size"] == "7B" and r["fallback_chain"] == ["0.5B"]
    assert router.resolve("whatever")["strategy"] == "auto" and router.load["7B"] == 3
    assert PiscesLxModelRouter.parse_size("yv_0.5b") == "0.5B" and PiscesLxModelRouter.parse_size("1T") == "1T"


# ------------------------------------------------------------------------------------------------ CLI
def test_manage_cli_train_infer_dry_run_and_short_train(tmp_path):
    env = dict(os.environ, PISCESLX_HOME=str(tmp_path / "home"), PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "manage.py"), "train", "--model_size", "0.01B", "--dry_run",
                        "--device", "cpu"], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0 and "trainer" in r.stdout, r.stderr[-2000:]
    cfgp = tmp_path / "m.json"
    c = tiny(); c.to_json(cfgp)
    out = tmp_path / "ck"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "manage.py"), "train", "--model_config", str(cfgp), "--stage",
                        "pretrain_cpu", "--device", "cpu", "--max_steps", "3", "--seq_len", "32", "--batch_size", "2",
                        "--save_steps", "2", "--output_dir", str(out), "--run_id", "t1", "--run_dir", str(tmp_path / "runs")],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    assert (out / "final_model.pt").exists() and (out / "checkpoint_step_2.pt").exists()
    st = json.load(open(tmp_path / "runs" / "t1" / "state.json"))
    assert st["status"] == "completed" and st["global_step"] == 3
    r = subprocess.run([sys.executable, os.path.join(ROOT, "manage.py"), "infer", "--model_config", str(cfgp), "--ckpt",
                        str(out / "final_model.pt"), "--device", "cpu", "--prompt", "hi", "--max_new_tokens", "4"],
                       capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0 and "tokens_per_second" in r.stdout, r.stderr[-2000:]
