"""Yv model family."""
from .attention import AttnContext, YvAttention
from .blocks import YvTransformerBlock
from .cache import YvCacheConfig, YvPagedKVCache, cache_for_model
from .generation import YvSampler, YvSamplerFactory, YvSamplingConfig, YvSamplingStrategy, generate
from .model import YvModel, YvModelForCausalLM, YvModelOutput, build_model
from .moe import YvExpert, YvMoEGate, YvSharedExpert, YvStableMoEGate, YvSwiGLUExpert
from .moe_layer import YvDeepSeekMoELayer, YvDynamicMoELayer
from .norms import YvFiLMModulation, YvLayerNorm, YvRMSNorm, YvRotaryEmbedding, YvSpatioTemporalRoPE3D
