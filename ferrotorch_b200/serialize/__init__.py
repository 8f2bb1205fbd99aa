"""Checkpoint formats: SafeTensors, PyTorch .pt, native state dicts, training checkpoints, GGUF."""
from .gguf import (GgmlType, GgufFile, GgufMetadata, GgufTensorInfo, GgufValue, dequantize_gguf_tensor, gguf_key_to_hf,  # noqa: F401
                   gguf_to_hf_state_dict, load_gguf, load_gguf_mmap, load_gguf_state_dict, load_gguf_state_dict_mmap,
                   parse_gguf_bytes, quantize_q4_0, tensor_infos, write_gguf)
from .gguf_planes import (GgufBlockKind, dequantize_q4_0_to_gpu, dequantize_q4_1_to_gpu, dequantize_q5_0_to_gpu,  # noqa: F401
                          dequantize_q5_1_to_gpu, dequantize_q8_0_to_gpu, dequantize_q8_1_to_gpu, expand_planes, split_blocks,
                          split_q4_0_blocks, split_q4_1_blocks, split_q5_0_blocks, split_q5_1_blocks, split_q8_0_blocks,
                          split_q8_1_blocks)
from .state import PickleValue, TrainingCheckpoint  # noqa: F401
from .state import (AsyncCheckpointer, CheckpointFuture, dumps_state_dict, load_checkpoint,  # noqa: F401
                    load_pytorch_state_dict, load_safetensors, load_safetensors_parallel, read_file_parallel, read_safetensors_header, load_safetensors_sharded, load_state_dict,
                    ShardProgress, load_safetensors_auto, load_safetensors_mmap, load_safetensors_sharded_filtered,
                    load_safetensors_sharded_mmap, load_safetensors_sharded_with_progress, validate_checkpoint,
                    load_pytorch_state_dict_mmap, parse_pickle, pickle_imports,
                    loads_state_dict, save_checkpoint, save_reference_checkpoint, save_pytorch, save_safetensors, save_safetensors_sharded,
                    save_state_dict)


from .onnx import (OnnxExportConfig, OnnxExportError, export_from_program, export_ir_graph_to_onnx, export_onnx,  # noqa: F401,E402
                   ir_graph_to_onnx, load_onnx, run_onnx, encode_dim_param, encode_shape_with_dynamic, encode_value_info_dynamic)
