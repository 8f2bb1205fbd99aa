"""Model families: Llama (single-GPU, tensor-parallel training, inference engine), ResNet, and the
small zoo (BERT, Whisper encoder, GCN, PPO policy) and the latent-diffusion stack (``diffusion``)."""
from .llama import LlamaConfig, LlamaForCausalLM, LlamaModel  # noqa: F401
from .llama_compat import (AwqQ4, GptqQ4, HqqQ4Axis1, LlamaActivation, LlamaAttention, LlamaGpuLayer, LlamaMLP,  # noqa: F401
                           LayerKvCache, LlamaKvCache, ProfiledForwardResult, apply_grammar_mask_gpu, gguf_key_to_hf, gguf_to_hf_state_dict,
                           masked_decode_loop)
from .resnet import create_model, list_models, register_model, resnet18, resnet34, resnet50  # noqa: F401


def __getattr__(name):
    """Names of the reference's GPU inference types (ferrotorch-llama/src/gpu.rs): the batched,
    paged, tensor-parallel :class:`~ferrotorch_b200.models.engine.LlamaEngine` plays both roles --
    ``LlamaGpuInferencer`` and, with ``cuda_graph=True``, ``GraphedDecoder``.  Loaded on first use
    because the engine binds the kernel library."""
    if name in ("LlamaEngine", "LlamaGpuInferencer", "GraphedDecoder"):
        from .engine import LlamaEngine

        return LlamaEngine
    if name in ("ModelHandle", "LlamaHandle", "FunctionHandle", "SpecSamplingConfig", "SpecSamplingOutput", "speculative_sample"):
        from . import spec_decode

        return getattr(spec_decode, name)
    if name == "KVCache":
        from ..nn.layers import KVCache

        return KVCache
    raise AttributeError(name)
