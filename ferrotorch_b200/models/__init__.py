"""Model families: Llama (single-GPU, tensor-parallel training, inference engine), ResNet, and the
small zoo (BERT, Whisper encoder, GCN, PPO policy) and the latent-diffusion stack (``diffusion``)."""
from .llama import LlamaConfig, LlamaForCausalLM, LlamaModel  # noqa: F401
from .llama_compat import (AwqQ4, GptqQ4, HqqQ4Axis1, LlamaActivation, LlamaAttention, LlamaGpuLayer, LlamaMLP,  # noqa: F401
                           LayerKvCache, LlamaKvCache, apply_grammar_mask_gpu, gguf_key_to_hf, gguf_to_hf_state_dict,
                           masked_decode_loop)
from .resnet import create_model, list_models, register_model, resnet18, resnet34, resnet50  # noqa: F401


def __getattr__(name):
    """Loaded on first use: the batched, paged, tensor-parallel
    :class:`~ferrotorch_b200.models.engine.LlamaEngine` (binds the kernel library), the continuous-batching
    server of :mod:`~ferrotorch_b200.models.serving` and the reference's single-sequence inference objects (ferrotorch-llama/src/gpu.rs) from
    :mod:`~ferrotorch_b200.models.inferencer`."""
    if name == "LlamaEngine":
        from .engine import LlamaEngine

        return LlamaEngine
    if name in ("LlamaGpuInferencer", "GraphedDecoder", "ProfiledForwardResult"):
        from . import inferencer

        return getattr(inferencer, name)
    if name in ("ModelHandle", "LlamaHandle", "FunctionHandle", "SpecSamplingConfig", "SpecSamplingOutput", "speculative_sample"):
        from . import spec_decode

        return getattr(spec_decode, name)
    if name in ("ContinuousBatcher", "Request", "RequestState", "SamplingParams", "ServingStats"):
        from . import serving

        return getattr(serving, name)
    if name == "KVCache":
        from ..nn.layers import KVCache

        return KVCache
    raise AttributeError(name)
