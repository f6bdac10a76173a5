"""Low-precision training and post-training quantisation.

Block-scaled fp8 (E4M3 / E5M2; 1x128 activation blocks, 128x128 weight blocks; power-of-two "ue8m0" scales optional),
fp4 (E2M1, blocks of 16, stochastic rounding, fp32 masters), and PTQ methods (GPTQ, AWQ, SmoothQuant, block-wise INT4,
KV-cache quantisation).  The reference trains fp8 through Transformer-Engine delayed per-tensor scaling
(opss/train/fp8.py:381-399) and "quantises" PTQ tensors by scaling and clamping in the input dtype
(opss/quantize/engine.py:808-1103); here the scales are per block and the values are really rounded to the target
grid.  ``YvFP8Linear`` is numerically the fp8 computation (operands rounded to E4M3 with block scales, fp32
accumulation); its matrix product currently runs on the bf16 tcgen05 GEMM after de-scaling - the ``kind::f8f6f4``
tensor-core variant of the GEMM kernel is the planned replacement and changes no numerics contract.
"""
from .fp8 import (YvFP8Linear, dequantize_fp8_blockwise, fp8_gemm_reference, quantize_fp8_blockwise,
                  PiscesLxFP8QuantizationEngine)
from .fp4 import PiscesLxFP4Linear, PiscesLxFP4Quantizer
from .ptq import (PiscesLxAWQQuantizer, PiscesLxBlockWiseINT4Quantizer, PiscesLxGPTQQuantizer, PiscesLxKVCacheQuantizer,
                  PiscesLxSmoothQuantizer, quantize_model_weights)
