"""The library registered with Triton as a backend + driver (triton_tenstorrent_b200/triton_plugin.py), the way
the reference plugs itself in (backend/compiler.py, backend/driver.py:445-535).

CPU part: the reference's example files are loaded UNMODIFIED from a checkout of the reference (the directory named
by REFERENCE_ROOT, or the default checkout location when it exists), their `@triton.jit` kernels go through Triton's own front end and this backend's
stages, and a recording launcher checks what would reach b200k_launch.  Skipped where no checkout is available.
GPU part: the same path with real launches; a kernel written here stands in where no checkout is available.
"""
import importlib.util
import os
import sys
from pathlib import Path

import pytest
import torch

triton = pytest.importorskip("triton")

import golden_inputs as gi  # noqa: E402
from oracle import cpu_oracle as oracle  # noqa: E402
from triton_tenstorrent_b200 import _lib, driver  # noqa: E402
from triton_tenstorrent_b200 import triton_plugin as plugin  # noqa: E402

REF = Path(os.environ.get("REFERENCE_ROOT", "/root/reference"))
needs_reference = pytest.mark.skipif(not (REF / "examples" / "01-sin-kernel.py").exists(),
                                     reason="no checkout of the reference (set REFERENCE_ROOT)")


def _load(rel: str, name: str):
    """Imports a reference example file as it is (its module-level code runs)."""
    spec = importlib.util.spec_from_file_location(name, REF / rel)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


class _Recorder:
    calls = []

    def __init__(self, src, metadata):
        self.inner = plugin.B200TritonLauncher(src, metadata)

    def __call__(self, gx, gy, gz, stream, function, *args):
        name = function.split(":")[0]
        bound = dict(zip(self.inner.arg_names, args[4:]))
        _Recorder.calls.append(dict(grid=(gx, gy, gz), name=name, spec=self.inner._spec(name, bound),
                                    metadata=args[0], flat=driver.flatten_args(self.inner.signature, args[4:])))


@pytest.fixture
def recording_driver(monkeypatch, tmp_path):
    """The registered driver with every device query and the launcher replaced, so that Triton's JIT, the backend's
    stages and the launcher's marshalling run without a GPU."""
    monkeypatch.setenv("TRITON_CACHE_DIR", str(tmp_path))
    drv = plugin.register()
    monkeypatch.setattr(drv, "get_current_device", lambda: 0)
    monkeypatch.setattr(drv, "get_current_stream", lambda device=None: 0)
    monkeypatch.setattr(drv, "get_active_torch_device", lambda: torch.device("cpu"))
    monkeypatch.setattr(drv, "get_benchmarker", lambda: (lambda fn, quantiles=None, **kw: (fn(), [1.0, 1.0, 1.0])[1]))
    monkeypatch.setattr(drv, "get_empty_cache_for_benchmark", lambda: torch.empty(16))
    monkeypatch.setattr(drv.utils, "get_device_properties", lambda device=0: {
        "max_num_regs": 65536, "max_shared_mem": 232448, "multiprocessor_count": 148, "warpSize": 32})
    monkeypatch.setattr(type(drv), "launcher_cls", _Recorder)
    _Recorder.calls = []
    yield _Recorder.calls
    plugin.unregister()


def test_backend_is_registered_like_the_reference():
    drv = plugin.register(activate=False)
    from triton.backends import backends
    from triton.backends.compiler import BaseBackend
    from triton.backends.driver import DriverBase
    assert issubclass(backends["b200"].compiler, BaseBackend) and issubclass(backends["b200"].driver, DriverBase)
    target = drv.get_current_target()
    assert backends["b200"].compiler.supports_target(target) and target.warp_size == 32
    be = backends["b200"].compiler(target)
    # packed metadata: (num_warps, num_ctas, shared, clusterX, clusterY, clusterZ), backend/compiler.py:77-85
    opts = be.parse_options({"num_warps": 8})
    md = type("MD", (), dict(num_warps=opts.num_warps, num_ctas=1, shared=0, cluster_dims=(1, 1, 1)))
    assert be.pack_metadata(md) == (8, 1, 0, 1, 1, 1)
    stages = {}
    be.add_stages(stages, opts)
    assert list(stages) == ["ttir", "b200k"] and be.binary_ext == "b200k"
    for method in ("launcher_cls", "utils", "get_current_target", "get_device_interface", "get_benchmarker",
                   "get_empty_cache_for_benchmark", "clear_cache", "get_active_torch_device", "get_current_stream"):
        assert hasattr(drv, method), method


@needs_reference
def test_reference_examples_reach_the_launcher_unmodified(recording_driver):
    calls = recording_driver
    # python/tutorials/01-vector-add.py runs add() on 66560 elements at import (:84-90)
    _load("python/tutorials/01-vector-add.py", "ref_vector_add")
    c = calls[-1]
    assert (c["grid"], c["name"], c["spec"]) == ((65, 1, 1), "add_kernel", "BLOCK_SIZE=1024")
    assert [k for k, _ in c["flat"]] == [_lib.ARG_PTR] * 3 + [_lib.ARG_I32] and c["flat"][3][1] == 66560
    assert len(c["metadata"]) == 6
    # examples/01-sin-kernel.py: sin(x) :32-37
    m = _load("examples/01-sin-kernel.py", "ref_sin_kernel")
    m.sin(torch.zeros(98432))
    c = calls[-1]
    assert (c["grid"], c["name"], c["spec"]) == ((97, 1, 1), "sin_kernel", "BLOCK_SIZE=1024")
    assert [k for k, _ in c["flat"]] == [_lib.ARG_PTR] * 2 + [_lib.ARG_I32]
    # examples/matmul_tensor_descriptor/09-persistent-matmul.ttnn.py: matmul_tma(a, b, ws) :146-173 (autotuned, pre-hook)
    m = _load("examples/matmul_tensor_descriptor/09-persistent-matmul.ttnn.py", "ref_persistent_matmul")
    a, b = torch.zeros(96, 160, dtype=torch.bfloat16), torch.zeros(160, 64, dtype=torch.bfloat16)
    m.matmul_tma(a, b, False)
    c = calls[-1]
    assert (c["grid"], c["name"]) == ((6, 1, 1), "matmul_kernel_tma") and "BLOCK_SIZE_M=32" in c["spec"]
    flat = c["flat"]
    assert len(flat) == 3 * 10 + 3                    # three flattened descriptors, then M, N, K
    assert [v for _, v in flat[1:10]] == [96, 160, 160, 1, 0, 96, 160, 160, 1]     # shape, strides, padding, shape, strides
    assert [v for _, v in flat[-3:]] == [96, 64, 160]
    # examples/fused-attn/06-fused-attention.py: _attention.apply(q, k, v, causal, sm_scale, warp_specialize) :224-273
    m = _load("examples/fused-attn/06-fused-attention.py", "ref_fused_attention")
    q = torch.zeros(1, 2, 256, 128, dtype=torch.bfloat16)
    m._attention.apply(q, q, q, True, 0.1, True)
    c = calls[-1]
    assert c["name"] == "_attn_fwd" and "STAGE=3" in c["spec"] and c["grid"][1:] == (2, 1)
    bm = int(c["spec"].split("BLOCK_M=")[1].split(",")[0])
    assert c["grid"][0] == 256 // bm
    assert len(c["flat"]) == 4 + 4 * 10 + 1 and c["flat"][0][0] == _lib.ARG_F32


def test_unknown_kernels_are_rejected_at_compile_time(recording_driver):
    import triton.language as tl

    @triton.jit
    def not_an_example_kernel(x_ptr, n, BLOCK: tl.constexpr):
        offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
        tl.store(x_ptr + offs, tl.load(x_ptr + offs, mask=offs < n) * 2, mask=offs < n)

    with pytest.raises(Exception, match="no hand-written sm_100a kernel"):
        not_an_example_kernel[(1,)](torch.zeros(64), 64, BLOCK=64)


# ------------------------------------------------------------------------------------------------ GPU
@pytest.fixture
def active_driver(tmp_path, monkeypatch):
    monkeypatch.setenv("TRITON_CACHE_DIR", str(tmp_path))
    drv = plugin.register()
    yield drv
    plugin.unregister()


@pytest.mark.gpu
def test_jit_kernel_launches_through_the_registered_driver(active_driver):
    # a kernel written here with the example's name, signature and meaning: traced by Triton, launched as the
    # hand-written sm_100a kernel through b200k_launch; device tensors and host tensors
    import triton.language as tl

    @triton.jit
    def add_kernel(x_ptr, y_ptr, output_ptr, n_elements, BLOCK_SIZE: tl.constexpr):
        offsets = tl.program_id(axis=0) * BLOCK_SIZE + tl.arange(0, BLOCK_SIZE)
        mask = offsets < n_elements
        tl.store(output_ptr + offsets, tl.load(x_ptr + offsets, mask=mask) + tl.load(y_ptr + offsets, mask=mask), mask=mask)

    lib = _lib.load()
    x, y = gi.add_inputs(98432)
    n = x.numel()
    grid = lambda meta: (triton.cdiv(n, meta["BLOCK_SIZE"]),)
    before = lib.b200k_launch_count()
    xd, yd = x.cuda(), y.cuda()
    out = torch.empty_like(xd)
    add_kernel[grid](xd, yd, out, n, BLOCK_SIZE=1024)
    assert torch.equal(out.cpu().view(torch.int32), oracle.add(x, y).view(torch.int32))
    out_host = torch.empty_like(x)
    add_kernel[grid](x, y, out_host, n, BLOCK_SIZE=1024)            # host tensors: staged like the reference's launcher
    assert torch.equal(out_host.view(torch.int32), oracle.add(x, y).view(torch.int32))
    assert lib.b200k_launch_count() - before == 2


@pytest.mark.gpu
@needs_reference
def test_reference_example_files_run_unmodified_on_the_gpu(active_driver, capsys):
    # 01-vector-add.py checks itself at import and prints its verdict (:84-102)
    _load("python/tutorials/01-vector-add.py", "ref_vector_add_gpu")
    assert "PASS" in capsys.readouterr().out
    add = sys.modules["ref_vector_add_gpu"].add
    x, y = gi.add_inputs(98432)
    got = add(x.cuda(), y.cuda()).cpu()
    assert torch.equal(got.view(torch.int32), oracle.add(x, y).view(torch.int32))

    m = _load("examples/01-sin-kernel.py", "ref_sin_kernel_gpu")
    xs = gi.sin_inputs(98432)
    assert oracle.ulp_diff_f32(m.sin(xs), oracle.sin_correctly_rounded(xs)) <= 2            # host tensor in, host out
    m.validate(1024, torch.float32)                                                        # the file's own check

    m = _load("examples/matmul_tensor_descriptor/09-persistent-matmul.ttnn.py", "ref_persistent_matmul_gpu")
    a, b = gi.matmul_inputs(512, 768, 1024)
    got = m.matmul_tma(a.cuda(), b.cuda(), False).cpu()
    assert oracle.rel_frobenius(got.float(), oracle.golden_matmul(a, b).float()) <= 1e-2
    m.validate(128, 128, 128, torch.bfloat16)                                              # host tensors, PCC > 0.97

    m = _load("examples/fused-attn/06-fused-attention.py", "ref_fused_attention_gpu")
    q, k, v = gi.attn_inputs(1, 2, 512, 128)
    for causal in (False, True):
        o = m._attention.apply(q.cuda(), k.cuda(), v.cuda(), causal, 128 ** -0.5, True).cpu()
        ref_o, _ = oracle.attention(q, k, v, causal, 128 ** -0.5)
        assert float((o.float() - ref_o.float()).abs().max()) <= 2e-2
