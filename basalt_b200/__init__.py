"""basalt_b200: a B200-native device path for the Basalt kernel compiler -- BIR to sm_100a PTX
(`Ptx`), a CUDA Driver API launch runtime (`CudaDriver` ...), hand-written comparator kernels,
and 1/2/4/8-GPU sharding -- behind the reference's own Backend and runtime interfaces.

Names are resolved on first use, so `python -m basalt_b200.build` can run before the native
library exists; anything else raises ImportError until it has been built."""
_BACKEND = ("Artifact", "Diag", "EmitOpts", "Ptx", "Support", "roundtrip", "compile_cuda", "compile_triton")
_RUNTIME = ("Communicator", "PeerGroup", "CudaContext", "CudaDriver", "CudaError", "CudaFunction", "CudaModule", "DeviceBuffer", "f32", "f64",
            "i32", "i64", "ptr", "shard_range")
__all__ = list(_BACKEND + _RUNTIME)


def __getattr__(name):
    import importlib
    if name in _BACKEND:
        return getattr(importlib.import_module(".backend", __name__), name)
    if name in _RUNTIME:
        return getattr(importlib.import_module(".runtime", __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
