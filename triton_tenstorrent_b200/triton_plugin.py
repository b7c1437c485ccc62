"""Registers this library with an installed Triton as a backend + driver, the way the reference plugs
itself in (backend/compiler.py TTBackend, backend/driver.py TTDriver :445-535), so that the
reference's example files run UNMODIFIED: their `@triton.jit` kernels are traced by Triton's own front
end, and `kernel[grid](...)` reaches `b200k_launch` through the launcher contract
`launcher(gridX, gridY, gridZ, stream, function, packed_metadata, launch_metadata, enter_hook,
exit_hook, *args)` (backend/driver.py:98-111, called from triton/runtime/jit.py).

There is no code generation behind it: the "compiler" stops at Triton IR (which validates the kernel
source and yields the kernel's name) and emits, in place of a binary, the name of the hand-written
sm_100a kernel that implements that example kernel.  The constexpr values the reference bakes into its
compiled binary (BLOCK_SIZE, STAGE, ACTIVATION, the element type) travel in the launch instead: the
launcher receives every bound argument, drops the constexpr ones from the argument list exactly as
TTLauncher does (:134-137), and encodes them in the "name:KEY=VALUE,..." string `b200k_launch` parses.

Like the reference's D2M launcher (backend/driver.py:303-381), a launch accepts HOST tensors: they are
copied to the current device, the kernel runs there, and every tensor argument is copied back into the
caller's storage (the reference writes back what its binary declares as outputs; here the kernel's
output arguments are known by name).  Launches on device tensors are asynchronous on the current stream.

    import triton_tenstorrent_b200.triton_plugin as plugin
    plugin.register()          # before the example file is imported
"""
from __future__ import annotations

import ctypes
import hashlib
import json
import re
from dataclasses import dataclass
from types import ModuleType
from typing import Dict, Tuple

import torch
from triton.backends import Backend, backends
from triton.backends.compiler import BaseBackend, GPUTarget, Language
from triton.backends.driver import DriverBase

from . import _lib
from . import driver as _driver

BACKEND_NAME = "b200"

# example kernel -> names of its arguments the kernel writes (copied back to host tensors after the launch)
_OUTPUT_ARGS = {
    "add_kernel": ("output_ptr",), "sin_kernel": ("output_ptr",), "muladd_kernel": ("output_ptr",),
    "mul_add_kernel": ("output_ptr",), "matmul_kernel_tma": ("c_desc",), "matmul_kernel_fused": ("c_desc",),
    "matmul_kernel": ("c_ptr",), "_attn_fwd": ("M", "desc_o"),
}
_ACTIVATION_CODES = {"": 0, None: 0, "none": 0, "relu": 1, "leaky_relu": 2}


@dataclass(frozen=True)
class B200Options:
    """Counterpart of TTOptions (backend/compiler.py:21-43).  Nothing here changes the generated code (there is
    none); the fields exist because Triton's front end and cache read them."""
    num_warps: int = 4
    num_ctas: int = 1
    num_stages: int = 1
    cluster_dims: tuple = (1, 1, 1)
    debug: bool = False
    arch: str = "sm_100a"
    enable_fp_fusion: bool = True
    backend_name: str = BACKEND_NAME
    sanitize_overflow: bool = True
    instrumentation_mode: str = ""
    allowed_dot_input_precisions: Tuple[str, ...] = ("ieee", "tf32", "tf32x3")
    default_dot_input_precision: str = "ieee"
    supported_fp8_dtypes: Tuple[str, ...] = ()
    deprecated_fp8_dot_operand_dtypes: Tuple[str, ...] = ()
    max_num_imprecise_acc_default: int = 0
    launch_cooperative_grid: bool = False
    launch_pdl: bool = False
    extern_libs: tuple = ()
    maxnreg: int = None
    warp_size: int = 32

    def hash(self):
        key = "_".join(f"{name}-{val}" for name, val in sorted(self.__dict__.items()))
        return hashlib.sha256(key.encode("utf-8")).hexdigest()


class B200Backend(BaseBackend):
    """Counterpart of TTBackend (backend/compiler.py:46-105, :474-502)."""
    binary_ext = "b200k"

    @staticmethod
    def supports_target(target: GPUTarget):
        return target.backend == BACKEND_NAME

    def __init__(self, target: GPUTarget) -> None:
        super().__init__(target)

    def get_target_name(self, options) -> str:
        return BACKEND_NAME

    def parse_options(self, options):
        args = {k: options[k] for k in B200Options.__dataclass_fields__ if k in options and options[k] is not None}
        return B200Options(**args)

    def pack_metadata(self, metadata):
        """(num_warps, num_ctas, shared, clusterX, clusterY, clusterZ), backend/compiler.py:77-85."""
        return _driver.pack_metadata(metadata.num_warps, metadata.num_ctas, metadata.shared, metadata.cluster_dims)

    def get_codegen_implementation(self, options):
        return {"min_dot_size": lambda lhs, rhs: (1, 1, 1)}

    def get_module_map(self) -> Dict[str, ModuleType]:
        return {}

    def load_dialects(self, ctx):
        pass   # the core dialects Triton's front end emits are loaded by Triton itself

    @staticmethod
    def make_ttir(mod, metadata, options):
        """The kernel as Triton IR, inlined and canonicalised: proof that the source is a valid Triton kernel, and
        the place the kernel's name is read from."""
        from triton._C.libtriton import ir, passes
        pm = ir.pass_manager(mod.context)
        passes.common.add_inliner(pm)
        passes.common.add_canonicalizer(pm)
        passes.common.add_symbol_dce(pm)
        pm.run(mod, "make_ttir")
        return mod

    @staticmethod
    def make_binary(src, metadata, options):
        """In place of machine code: which hand-written kernel of libb200kernels implements this Triton kernel."""
        names = re.findall(r"tt\.func\s+public\s+@([A-Za-z_][A-Za-z0-9_]*)", str(src))
        if len(names) != 1:
            raise RuntimeError(f"expected one public kernel in the module, found {names}")
        name = names[0]
        if name not in _driver.KERNEL_NAMES:
            raise NotImplementedError(
                f"libb200kernels has no hand-written sm_100a kernel for '{name}' (this backend runs the example "
                f"kernels {', '.join(_driver.KERNEL_NAMES)}; it does not compile arbitrary Triton code)")
        metadata["name"] = name
        metadata["shared"] = 0
        return json.dumps({"kernel": name, "library": "libb200kernels.so"}).encode()

    def add_stages(self, stages, options, language=Language.TRITON):
        if language != Language.TRITON:
            raise NotImplementedError("only Triton-language kernels are supported")
        stages["ttir"] = lambda src, metadata: self.make_ttir(src, metadata, options)
        stages[self.binary_ext] = lambda src, metadata: self.make_binary(src, metadata, options)

    def hash(self):
        return f"b200k-{_lib.load().b200k_version() if _lib.LIB_PATH.exists() else 0}-{self.target.arch}"


def _base_tensor(arg):
    """The torch tensor behind a tensor or tensor-descriptor argument, or None."""
    if isinstance(arg, torch.Tensor):
        return arg
    base = getattr(arg, "base", None)
    return base if isinstance(base, torch.Tensor) else None


class _DescriptorOnDevice:
    """A tensor descriptor whose base tensor has been replaced by its device copy."""

    def __init__(self, desc, base):
        self.base, self.shape, self.strides = base, list(desc.shape), list(desc.strides)
        self.block_shape, self.padding = list(desc.block_shape), getattr(desc, "padding", "zero")


class B200TritonLauncher:
    """Counterpart of TTLauncher / TTRTLauncher (backend/driver.py:85-170, :303-381) for kernels traced by Triton."""

    def __init__(self, src, metadata):
        self.src = src
        self.metadata = metadata
        self.arg_names = list(src.fn.arg_names) if hasattr(src, "fn") else list(src.arg_names)
        sig = dict(src.signature)
        # {position: type string}, "constexpr" marking compile-time arguments, like TTLauncher.__init__ (:98-101).
        # One difference: Triton also turns a RUNTIME integer argument into a constant when its value is 1 (Z = 1,
        # a stride of 1), and the reference, whose binary has that constant compiled in, drops it from the list.
        # The hand-written kernels take every declared runtime argument, so only arguments DECLARED tl.constexpr
        # are dropped here.
        declared = {}
        for prm in getattr(getattr(src, "fn", None), "params", []) or []:
            declared[prm.name] = bool(prm.is_constexpr)
        self.signature = {}
        for i, name in enumerate(self.arg_names):
            ty = sig.get(name, sig.get(i, "constexpr"))
            if ty == "constexpr" and declared.get(name) is False:
                ty = "i32"
            self.signature[i] = ty

    def _spec(self, name, bound):
        """The constexpr specialisation that the reference compiles into its binary, as KEY=VALUE items."""
        items = []
        for key in ("BLOCK_SIZE", "BLOCK_SIZE_M", "BLOCK_SIZE_N", "BLOCK_M", "STAGE"):
            if key in bound and isinstance(bound[key], (int, bool)):
                items.append(f"{key}={int(bound[key])}")
        tensors = [t for t in (_base_tensor(v) for v in bound.values()) if t is not None]
        dtype = tensors[0].dtype if tensors else None
        if name in ("add_kernel",) and dtype == torch.bfloat16:
            items.append("BF16=1")
        if name in ("matmul_kernel_tma", "matmul_kernel_fused") and dtype == torch.float16:
            items.append("F16=1")
        if name == "matmul_kernel":
            act = bound.get("ACTIVATION", "")
            if act not in _ACTIVATION_CODES:
                raise ValueError(f"matmul_kernel: unknown ACTIVATION {act!r}")
            # the reference kernel addresses its buffers tile-major (examples/matmul/03-matrix-multiplication.py:333-386)
            items += [f"ACTIVATION={_ACTIVATION_CODES[act]}", f"F16={1 if dtype == torch.float16 else 0}", "TILE32=1"]
        if bound.get("FP8_OUTPUT"):
            raise NotImplementedError(f"{name}: FP8 output is not built")
        return ",".join(items)

    def __call__(self, gridX, gridY, gridZ, stream, function, *args):
        kernel_metadata, launch_metadata, launch_enter_hook, launch_exit_hook = args[:4]
        kernel_args = list(args[4:])
        name = function.split(":")[0] if isinstance(function, str) else function.decode().split(":")[0]
        bound = dict(zip(self.arg_names, kernel_args))
        spec = self._spec(name, bound)
        target = f"{name}:{spec}" if spec else name

        # host tensors travel to the current device for the launch and back afterwards (backend/driver.py:350-381)
        device = torch.device("cuda", torch.cuda.current_device())
        staged = {}     # id(host tensor) -> (host tensor, device copy)
        for i, a in enumerate(kernel_args):
            t = _base_tensor(a)
            if t is None or t.is_cuda:
                continue
            if id(t) not in staged:
                staged[id(t)] = (t, t.to(device, non_blocking=True))
            dev = staged[id(t)][1]
            kernel_args[i] = dev if isinstance(a, torch.Tensor) else _DescriptorOnDevice(a, dev)

        flat = _driver.flatten_args(self.signature, kernel_args)
        c_args = _driver._to_c_args(flat)
        lib = _lib.load()
        if launch_enter_hook is not None:
            launch_enter_hook(launch_metadata)
        raw_stream = stream if isinstance(stream, int) else getattr(stream, "cuda_stream", 0)
        if staged:      # the copies above ran on torch's current stream: launch there too
            raw_stream = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.b200k_launch(target.encode(), int(gridX), int(gridY), int(gridZ), ctypes.c_void_p(raw_stream or 0),
                                    c_args, len(flat)))
        if launch_exit_hook is not None:
            launch_exit_hook(launch_metadata)
        if staged:
            outputs = _OUTPUT_ARGS.get(name, ())
            for arg_name in outputs:
                t = _base_tensor(bound.get(arg_name))
                if t is not None and id(t) in staged:
                    host, dev = staged[id(t)]
                    host.copy_(dev)          # synchronises: the reference's launches are synchronous as well
            torch.cuda.current_stream().synchronize()


class B200TritonDriver(_driver.B200Driver, DriverBase):
    """Counterpart of TTDriver (backend/driver.py:445-535) as a real Triton driver."""

    launcher_cls = B200TritonLauncher

    def __init__(self):
        _driver.B200Driver.__init__(self)

    @classmethod
    def is_active(cls):
        return torch.cuda.is_available()

    def get_current_target(self):
        return GPUTarget(BACKEND_NAME, 100, 32)

    def get_device_capability(self, device=None):
        return (10, 0)


def register(activate: bool = True):
    """Adds the backend to Triton's registry and (by default) makes its driver the active one.  Returns the driver."""
    import triton
    backends[BACKEND_NAME] = Backend(compiler=B200Backend, driver=B200TritonDriver)
    drv = B200TritonDriver()
    if activate:
        triton.runtime.driver.set_active(drv)
    return drv


def unregister():
    """Removes the backend from Triton's registry and lets Triton pick its default driver again on next use."""
    import triton
    backends.pop(BACKEND_NAME, None)
    triton.runtime.driver._active = None
