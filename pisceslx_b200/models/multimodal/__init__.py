"""Multimodal encoders and fusion."""
from .fusion import YvAudioEncoder, YvCrossModalAttention, YvDynamicModalFusion, attach_multimodal
from .vision import YvPatchEmbed, YvVideoEncoder, YvVisionEncoder, YvViTBlock
from .generator import (YvGenerationBackend, YvGenerationCondition, YvGenerationConfig, YvGenerationModality,
                        YvGenerationResult, YvGenerator, YvGeneratorFactory, YvSelfDevelopedGenerator,
                        YvTextToAudioBackend, YvTextToImageBackend, YvTextToVideoBackend)
