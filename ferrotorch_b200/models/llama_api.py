"""Everything the reference's ``ferrotorch-llama`` crate exports, in one namespace
(``ferrotorch_b200.llama``): configuration, the model classes, generation, speculative decoding,
4-bit loaders, GGUF key mapping, the grammar-masked loop and -- on first use, because it binds the
kernel library -- the inference engine."""
from .generation import *  # noqa: F401,F403
from .generation import GenerationConfig, generate  # noqa: F401
from .llama import LlamaConfig, LlamaDecoderLayer, LlamaForCausalLM, LlamaModel  # noqa: F401
from .llama_compat import *  # noqa: F401,F403
from .spec_decode import (FunctionHandle, LlamaHandle, ModelHandle, SpecSamplingConfig, SpecSamplingOutput,  # noqa: F401
                          residual_distribution, speculative_sample)
from ..serialize.quant_loaders import (dequantize_awq, dequantize_awq_q4, dequantize_gptq, dequantize_gptq_q4,  # noqa: F401
                                       dequantize_hqq, dequantize_hqq_q4_axis1, hqq_q4_axis1_to_dense,
                                       hqq_state_dict_to_dense, to_q4_linear)
from ..serialize.gguf import dequantize_on_device as gpu_dequantize_to_bf16_cudarc  # noqa: F401  (raw blocks on the device -> bf16)
from ..utils import grammar  # noqa: F401
from ..utils.grammar import JsonSchemaProcessor, SchemaLogitsProcessor, TokenMask  # noqa: F401


def __getattr__(name):
    from .. import models

    return getattr(models, name)          # LlamaEngine / LlamaGpuInferencer / GraphedDecoder / ProfiledForwardResult
