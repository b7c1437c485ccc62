"""Launch contract of the reference's backend/driver.py, re-hosted on the C-ABI.

The reference driver (backend/driver.py) gives Triton three things for a compiled kernel: a launcher
class whose instances are called as
    launcher(gridX, gridY, gridZ, stream, function, packed_metadata, launch_metadata,
             launch_enter_hook, launch_exit_hook, *kernel_args)                      (:98-111)
a `utils` object with load_binary / get_device_properties (:68-82), and driver queries
(target, device, stream, benchmarker, :445-535).  This module keeps those shapes.  There is no
compiler behind it: `function` is the name of one of the hand-written sm_100a kernels plus its
constexpr specialisation ("name:KEY=VAL,..."), the role the compiled binary plays in the reference.

Argument marshalling follows TTLauncher.__call__ :134-162 exactly: arguments whose signature type is
"constexpr" are dropped, tensors become device pointers, a TensorDescriptor is flattened to
base, shape..., strides..., padding flag, shape..., strides... (the duplication is the reference's),
other scalars pass through.
"""
from __future__ import annotations

import ctypes
from collections import namedtuple
from dataclasses import dataclass, field

import torch

from . import _lib
from .tensor_descriptor import TensorDescriptor

GPUTarget = namedtuple("GPUTarget", ["backend", "arch", "warp_size"])

# kernels this library implements (the reference's compiled-kernel names)
KERNEL_NAMES = ("add_kernel", "sin_kernel", "mul_add_kernel", "muladd_kernel", "memcpy_kernel", "copy_scalar_kernel", "matmul_kernel_tma", "matmul_kernel_fused", "matmul_kernel",
                "_attn_fwd")


@dataclass
class KernelSource:
    """What the reference launcher reads from `src`: the signature {index: type string} where
    "constexpr" marks compile-time arguments, and the names of the arguments."""
    name: str
    arg_names: tuple
    signature: dict
    constants: dict = field(default_factory=dict)


def pack_metadata(num_warps=1, num_ctas=1, shared=0, cluster_dims=(1, 1, 1)):
    """(num_warps, num_ctas, shared, clusterX, clusterY, clusterZ), backend/compiler.py:77-85."""
    return (num_warps, num_ctas, shared, cluster_dims[0], cluster_dims[1], cluster_dims[2])


def flatten_args(signature: dict, args) -> list:
    """The reference's argument list as (kind, value) pairs; see the module docstring."""
    sig_types = list(signature.values())
    flat = []
    for i, arg in enumerate(args):
        ty = sig_types[i]
        if ty == "constexpr":
            continue
        if isinstance(arg, torch.Tensor):
            flat.append((_lib.ARG_PTR, arg.data_ptr()))
        elif isinstance(arg, TensorDescriptor) or (hasattr(arg, "base") and hasattr(arg, "strides") and hasattr(arg, "block_shape")):
            # this package's descriptor, or any object of the same shape (Triton's own TensorDescriptor)
            dims = [(_lib.ARG_I64, int(d)) for d in arg.shape] + [(_lib.ARG_I64, int(s)) for s in arg.strides]
            flat.append((_lib.ARG_PTR, arg.base.data_ptr()))
            flat.extend(dims)
            flat.append((_lib.ARG_I32, 1 if getattr(arg, "padding", "zero") == "nan" else 0))
            flat.extend(dims)  # shape and strides a second time, as the reference passes them
        elif isinstance(arg, bool):
            flat.append((_lib.ARG_I32, int(arg)))
        elif isinstance(arg, int):
            flat.append((_lib.ARG_I64 if abs(arg) >= 2 ** 31 else _lib.ARG_I32, arg))
        elif isinstance(arg, float):
            flat.append((_lib.ARG_F32, arg))
        else:
            raise TypeError(f"Don't know how to pass argument {i} of type {type(arg).__name__}")
    return flat


def _to_c_args(flat):
    arr = (_lib.Arg * len(flat))()
    for slot, (kind, value) in zip(arr, flat):
        slot.kind = kind
        if kind == _lib.ARG_PTR:
            slot.v.ptr = value
        elif kind == _lib.ARG_I32:
            slot.v.i32 = value
        elif kind == _lib.ARG_I64:
            slot.v.i64 = value
        else:
            slot.v.f32 = value
    return arr


class B200Launcher:
    """Counterpart of TTLauncher (backend/driver.py:85-170)."""

    def __init__(self, src: KernelSource, metadata=None):
        self.src = src
        self.metadata = metadata
        self.signature = {idx: value for idx, value in src.signature.items()}

    def __call__(self, gridX, gridY, gridZ, stream, function, *args):
        kernel_metadata, launch_metadata, launch_enter_hook, launch_exit_hook = args[:4]
        assert len(kernel_metadata) == 6, "packed metadata is (num_warps, num_ctas, shared, clusterX, clusterY, clusterZ)"
        flat = flatten_args(self.signature, args[4:])
        c_args = _to_c_args(flat)
        lib = _lib.load()
        name = function.encode() if isinstance(function, str) else function
        if launch_enter_hook is not None:
            launch_enter_hook(launch_metadata)
        _lib.check(lib.b200k_launch(name, int(gridX), int(gridY), int(gridZ), ctypes.c_void_p(stream or 0), c_args,
                                    len(flat)))
        if launch_exit_hook is not None:
            launch_exit_hook(launch_metadata)


class B200Utils:
    """Counterpart of TTUtils (backend/driver.py:63-82)."""

    def load_binary(self, name, kernel, shared_mem, device_id):
        """Returns (module, function, n_regs, n_spills, n_max_threads) like the reference (:68-74, :203-211).
        The kernels are ahead-of-time compiled into the library, so `kernel` (the binary) is only checked to
        name a kernel this build has; `function` is the name handed to the launcher."""
        base = name.split(":")[0]
        if base not in KERNEL_NAMES:
            raise KeyError(f"no sm_100a kernel named {base!r} in libb200kernels")
        return (_lib.load(), name, 0, 0, 1024)

    def get_device_properties(self, device=0):
        """max_num_regs / max_shared_mem / multiprocessor_count / warpSize, as :76-82."""
        props = _lib.Props()
        _lib.check(_lib.load().b200k_device_props(int(device), ctypes.byref(props)))
        return {"max_num_regs": props.max_num_regs, "max_shared_mem": props.max_shared_mem,
                "multiprocessor_count": props.multiprocessor_count, "warpSize": props.warp_size}


class B200DeviceInterface:
    """Counterpart of TTDeviceInterface (backend/driver.py:390-442) on CUDA events: the object
    triton.testing.do_bench-style harnesses use for Event / elapsed_time / synchronize."""

    Event = staticmethod(lambda enable_timing=True: torch.cuda.Event(enable_timing=enable_timing))

    def synchronize(self):
        torch.cuda.synchronize()


class B200Driver:
    """Counterpart of TTDriver (backend/driver.py:445-535)."""

    launcher_cls = B200Launcher

    def __init__(self):
        self.utils = B200Utils()

    @staticmethod
    def is_active():
        return torch.cuda.is_available()

    def get_current_device(self):
        return torch.cuda.current_device()

    def set_current_device(self, device):
        torch.cuda.set_device(device)

    def get_current_stream(self, device_id=None):
        raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
        if raw is not None:   # the handle without building a Stream object (this sits on every launch)
            return raw(torch.cuda.current_device() if device_id is None else device_id)
        return torch.cuda.current_stream(device_id).cuda_stream

    def get_device_interface(self):
        return B200DeviceInterface()

    def get_current_target(self):
        return GPUTarget("cuda", 100, 32)

    def get_active_torch_device(self):
        return torch.device("cuda", torch.cuda.current_device())

    def map_python_to_cpp_type(self, ty: str) -> str:
        return ty

    def get_benchmarker(self):
        from .benchmarking import do_bench
        return do_bench

    def get_empty_cache_for_benchmark(self):
        # larger than the 126 MB L2 so that zeroing it evicts the working set
        return torch.empty(256 * 1024 * 1024 // 4, dtype=torch.int, device="cuda")

    def clear_cache(self, cache):
        cache.zero_()


active = B200Driver()
