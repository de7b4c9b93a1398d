"""B200-native FP8 gate/up projection with fused SwiGLU.

    from sol_execbench_b200_kernels_b200 import run
    run(x, scale_x, gate_proj_weight, scale_gate, up_proj_weight, scale_up, output)

`run` keeps the reference submission's entry-point signature
(kernels/179_fp8_mlp_gate_up_projection/kernel.py:398-407).  The arithmetic is
hand-written sm_100a CUDA in libgateup.so (C ABI in include/gateup.h); build it
with `python -m sol_execbench_b200_kernels_b200.build`.  Importing the compute
entry points without the built library raises: there is no fallback path.
"""
from . import workloads  # noqa: F401  (pure torch, no native code)
from .sharded import (GatherBuffers, PeerBarrier, ReduceBuffers, assemble_gathered, gather_columns, mlp_block_sharded,  # noqa: F401
                      mlp_block_sharded_fused, owned_rows,
                      run_sharded, run_sharded_fused, shard_bounds, shard_concat_weights, shard_down_weights,
                      shard_weights)

_NATIVE = ("run", "run_concat", "run_with_plan", "run_gather", "quantize_activation", "blockwise_gemm", "blockwise_gemm_scatter", "reduce_gather", "run_fp8_output", "mlp_block", "select_plan", "last_status",
           "launch_count", "peer_barrier")


def __getattr__(name):
    # the native entry points load libgateup.so on first use and raise if it is missing
    if name in _NATIVE:
        from . import kernel
        return getattr(kernel, name)
    raise AttributeError(name)


__all__ = list(_NATIVE) + ["workloads", "run_sharded", "run_sharded_fused", "GatherBuffers", "shard_bounds",
                           "shard_weights", "shard_concat_weights", "shard_down_weights", "mlp_block_sharded", "mlp_block_sharded_fused", "ReduceBuffers", "owned_rows",
                           "gather_columns", "assemble_gathered", "PeerBarrier"]
