"""Tensor parallelism: shard plan, per-rank weight loader, NCCL and fused in-kernel collectives, the reference-style
group facade, and the multi-process engine."""


def __getattr__(name):
    lazy = {"ShardPlan": ("shard_plan", "ShardPlan"), "make_plan": ("shard_plan", "make_plan"),
            "TPWeightLoader": ("tp_weight_loader", "TPWeightLoader"), "NcclComm": ("comm", "NcclComm"),
            "FusedComm": ("comm", "FusedComm"), "make_comm": ("comm", "make_comm"),
            "TensorParallelGroup": ("tensor_parallel", "TensorParallelGroup"), "TPConfig": ("tensor_parallel", "TPConfig"),
            "tp_launch": ("tensor_parallel", "tp_launch"), "NcclCommunicator": ("tensor_parallel", "NcclCommunicator"),
            "TPEngine": ("tp_engine", "TPEngine"), "TPEngineStats": ("tp_engine", "TPEngineStats")}
    if name in lazy:
        import importlib
        mod, attr = lazy[name]
        return getattr(importlib.import_module(f"{__name__}.{mod}"), attr)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
