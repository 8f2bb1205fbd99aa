"""Trace-and-fuse JIT: ``trace`` / ``compile`` -> IR -> passes -> generated sm_100a kernels."""
from .codegen import compile_cubin, generate_source, run_fused, run_program_torch  # noqa: F401
from .ir import (IrGraph, Node, OptimizationConfig, constant_fold, dead_code_eliminate, fuse_elementwise,  # noqa: F401
                 optimize, pattern_fuse, plan_memory)
from .module import (Autotuner, CompileConfig, EagerFallback, JitError, TracedModule, apply_fused, compile,  # noqa: F401
                     lower_fx, trace, with_fusion)
from .advanced import (AotGraphPair, AotModule, DimSpec, ExportedProgram, ExportedProgramMetadata, GraphSegment,  # noqa: F401
                       Guard, InputSpec, SegmentedModule, ShapeSignature, SymbolicDim, SymbolicTracedModule,
                       compile_aot, compile_symbolic, decompose_forward_backward, export,
                       patch_reshape_for_symbolic_dims, trace_with_breaks)
from .backends import (BinOpKind, Codegen, CompiledGraph, CpuCodegen, Expr, FusedChain, FusedOp, GpuCodegen,  # noqa: F401,E402
                       InductorBackend, InductorCompileStatus, InductorTarget, InterpreterBackend, LoopIR, MemoryPlan,
                       NativeBackend, ReductionKind, UnaryOpKind, compile_loop_ir_kernel, compile_with_config,
                       estimate_numel_for_inputs, generate_reduction_source, interpret, interpret_multi,
                       interpret_multi_with_captures, is_fusion_enabled, reduce_reference,
                       AotCompiledModule, AutotuneCandidate, AutotuneKey, AutotuneResult, FusionGroup, FusionGroupKind,
                       JitCompiledKernel, TraceResult, autotune, estimate_matmul_dims, export_with_dynamic_shapes,
                       generate_reduction_ptx, generate_reduction_rust, BackendTuneResult, InductorCompileOutcome, MatmulLoops,
                       apply_binary_op_expr, apply_fused_gpu, apply_op_expr, find_fusion_groups, fuse_dag, ir_op_to_binary,
                       ir_op_to_unary, is_binary_elementwise, is_elementwise, is_reduction, is_unary_elementwise, jit_supports,
                       lower_matmul, lower_to_loops)


def script(fn):
    """Decorator form (the reference's ``#[script]`` proc-macro, ferrotorch-jit-script/src/lib.rs):
    compiles on first call with that call's arguments as the example inputs."""
    cache = {}

    def wrapper(*args):
        key = tuple((tuple(a.shape), a.dtype) if hasattr(a, "shape") else a for a in args)
        if key not in cache:
            cache[key] = compile(fn, args)
        return cache[key](*args)

    wrapper.__wrapped__ = fn
    return wrapper
