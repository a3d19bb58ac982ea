"""basalt_b200: a B200-native device path for the Basalt kernel compiler -- BIR to sm_100a PTX
(`Ptx`), a CUDA Driver API launch runtime (`CudaDriver` ...), hand-written comparator kernels,
and 1/2/4/8-GPU sharding -- behind the reference's own Backend and runtime interfaces."""
from .backend import Artifact, Diag, EmitOpts, Ptx, Support, roundtrip
from .runtime import (Communicator, CudaContext, CudaDriver, CudaError, CudaFunction, CudaModule, DeviceBuffer, f32, f64, i32,
                      i64, ptr, shard_range)

__all__ = ["Artifact", "Diag", "EmitOpts", "Ptx", "Support", "roundtrip", "Communicator", "CudaContext", "CudaDriver",
           "CudaError", "CudaFunction", "CudaModule", "DeviceBuffer", "f32", "f64", "i32", "i64", "ptr", "shard_range"]
