"""The reference's portable-GPU crate (``ferrotorch-cubecl``) under its own names, for code written
against it: GGUF block planes and their device expansion (``serialize/gguf_planes.py``), the
automaton token mask (``utils/dfa_mask.py``) and the mask application (``utils/grammar.py``).
The crate's run-time plumbing (``CubeClient``, ``CubeDevice``, ``CubeRuntime``, storage handles,
``upload_f32``) has no counterpart: tensors and ``torch.device`` play those roles."""
from ..serialize.gguf_planes import *  # noqa: F401,F403
from ..serialize.gguf_planes import (GgufBlockKind, dequantize_q4_0_to_gpu, dequantize_q4_1_to_gpu, dequantize_q5_0_to_gpu,  # noqa: F401
                                     dequantize_q5_1_to_gpu, dequantize_q8_0_to_gpu, dequantize_q8_1_to_gpu, expand_planes,
                                     split_blocks, split_q4_0_blocks, split_q4_1_blocks, split_q5_0_blocks, split_q5_1_blocks,
                                     split_q8_0_blocks, split_q8_1_blocks)
from .dfa_mask import DfaMaskInputs, compute_token_mask_dfa, compute_token_mask_dfa_to_gpu, literal_dfa  # noqa: F401
from .grammar import apply_packed_mask_ as apply_token_mask_to_gpu  # noqa: F401

kernel_compute_token_mask_dfa = compute_token_mask_dfa
