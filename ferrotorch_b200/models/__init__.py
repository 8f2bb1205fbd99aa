"""Model families: Llama (single-GPU, tensor-parallel training, inference engine), ResNet, and the
small zoo (BERT, Whisper encoder, GCN, PPO policy) and the latent-diffusion stack (``diffusion``)."""
from .llama import LlamaConfig, LlamaForCausalLM, LlamaModel  # noqa: F401
from .resnet import create_model, list_models, register_model, resnet18, resnet34, resnet50  # noqa: F401


def __getattr__(name):
    """Names of the reference's GPU inference types (ferrotorch-llama/src/gpu.rs): the batched,
    paged, tensor-parallel :class:`~ferrotorch_b200.models.engine.LlamaEngine` plays both roles --
    ``LlamaGpuInferencer`` and, with ``cuda_graph=True``, ``GraphedDecoder``.  Loaded on first use
    because the engine binds the kernel library."""
    if name in ("LlamaEngine", "LlamaGpuInferencer", "GraphedDecoder"):
        from .engine import LlamaEngine

        return LlamaEngine
    if name in ("LlamaKvCache", "LayerKvCache", "KVCache"):
        from ..nn.layers import KVCache

        return KVCache
    raise AttributeError(name)
