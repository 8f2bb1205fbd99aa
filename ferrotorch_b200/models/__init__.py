"""Model families: Llama (single-GPU, tensor-parallel training, inference engine), ResNet, and the
small zoo (BERT, Whisper encoder, GCN, PPO policy) and the latent-diffusion stack (``diffusion``)."""
from .llama import LlamaConfig, LlamaForCausalLM, LlamaModel  # noqa: F401
from .resnet import create_model, list_models, register_model, resnet18, resnet34, resnet50  # noqa: F401
