"""Helpers for the GPU parity tests: compile BIR through the C-ABI backend, JIT it through the
C-ABI runtime, cache the loaded functions."""
import numpy as np

import basalt_b200 as b

_cache = {}


def emitted(ctx, src: str, kernel: str, opt_level: int = 2) -> b.CudaFunction:
    key = (id(ctx), hash(src), kernel, opt_level)
    if key not in _cache:
        ptx = b.Ptx().emit(src, b.EmitOpts(opt_level=opt_level)).text
        mod = ctx.load_module(ptx)
        _cache[key] = (mod, mod.get_function(kernel))
    return _cache[key][1]


def dev(ctx, array: np.ndarray) -> b.DeviceBuffer:
    return ctx.upload(np.ascontiguousarray(array))


def grid_for(n: int, block: int = 256) -> int:
    return max(1, (n + block - 1) // block)
