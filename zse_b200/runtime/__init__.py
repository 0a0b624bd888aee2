"""Execution layer: model runner (staging, CUDA graphs, pipelined decode), C++ step driver binding, memory plan,
weight streaming and the name-based weight store, graph wrapper, profiler and microbenchmarks.  (The reference's
``orchestrator`` package; ``ZSEEngine`` itself lives in ``zse_b200.engine``.)"""


def __getattr__(name):
    lazy = {"ModelRunner": ("runner", "ModelRunner"), "TPModelRunner": ("runner", "TPModelRunner"),
            "VRAMAllocator": ("vram", "VRAMAllocator"), "VRAMPlan": ("vram", "VRAMPlan"),
            "ScratchBuffers": ("vram", "ScratchBuffers"), "WeightLoader": ("weight_stream", "WeightLoader"),
            "WeightStore": ("weight_stream", "WeightStore"), "GPUWeight": ("weight_stream", "GPUWeight"),
            "CUDAGraphRunner": ("graph", "CUDAGraphRunner"), "NativeStep": ("step_driver", "NativeStep"),
            "FastDecoder": ("step_driver", "FastDecoder"), "KernelProfiler": ("profiler", "KernelProfiler"),
            "AutoTuner": ("profiler", "AutoTuner"), "KernelProfile": ("profiler", "KernelProfile"),
            "TuneResult": ("profiler", "TuneResult"), "ProfileResult": ("profiler", "ProfileResult")}
    if name == "ZSEEngine":
        from ..engine import ZSEEngine
        return ZSEEngine
    if name == "InferenceKernels":
        from ..ops.registry import InferenceKernels
        return InferenceKernels
    if name in lazy:
        import importlib
        mod, attr = lazy[name]
        return getattr(importlib.import_module(f"{__name__}.{mod}"), attr)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
