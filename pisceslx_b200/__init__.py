"""pisceslx_b200: a Blackwell (sm_100a) native framework for training and serving
Yv-architecture Mixture-of-Experts models.

Layout
------
config      YvConfig (hyper-parameters, YAML/JSON round trip, presets)
models/     Yv model family (text MoE trunk, multimodal encoders, Subconscious field, caches, generation)
ops/        hand-written sm_100a CUDA kernels (``ops/csrc``), their autograd wrappers and fp32 oracles
parallel/   process-group mesh, expert/tensor/data/pipeline/context parallel layers, symmetric peer memory
optim/      AdamW, Muon, Ink, LR schedules, ZeRO-1 sharding
engine/     trainer, checkpointing, run store, profiler, failure detection
serve/      OpenAI-compatible service, continuous batching over the paged KV cache
utils/      logging, paths, seeding, device helpers
"""

__version__ = "0.1.0"

from .config import YvConfig  # noqa: F401
