"""Generates the golden vectors under tests/golden/ by EXECUTING the reference's own kernel sources.

The reference's kernels are Triton `@triton.jit` functions.  This script reads them from a checkout
of kernelize-ai/triton-tenstorrent (its path is taken from the REFERENCE_ROOT environment variable), extracts
the kernel functions by name with `ast` (several example files cannot be imported as a whole: they
query an active Triton driver or launch on a device at import time), writes them to a temporary
module and runs them on CPU tensors with Triton's interpreter (TRITON_INTERPRET=1, triton 3.6).
Two harness-side shims repair bf16 handling of the triton 3.6 interpreter (neither touches a
reference file):
  * `create_dot` multiplies bf16 handles as raw uint16; bf16 operands are widened to fp32 before
    `np.matmul` (products of bf16 values are exact in fp32, accumulation is fp32 as `tl.dot` specifies);
  * `cast_impl` truncates fp32 -> bf16 (it calls its converter without a rounding mode), whereas the
    language's downcast rounds to nearest even (`fp_downcast_rounding="rtne"` is the default of
    `tl.cast` / `.to`), which is also what compiled Triton does; fp32 -> bf16 is routed through
    torch's round-to-nearest-even conversion.
No reference file is modified or copied into this repository; only the resulting output arrays are
stored.

Outputs (small .npz files, a few hundred KB in total):
  add.npz, add_loop.npz, mul_add.npz, sin.npz, matmul.npz, matmul_fused.npz, attention.npz, matmul_tile32.npz
Inputs are regenerated from their seeds by `golden_inputs.py`; each .npz keeps a sha256 of the
input bytes so that a drift of torch's CPU RNG cannot silently invalidate the vectors.

Run:  REFERENCE_ROOT=<checkout of the reference> python tests/golden/make_golden.py [set ...]
      (sets: add add_loop mul_add sin matmul matmul_fused attention matmul_tile32; default all)
"""
from __future__ import annotations

import ast
import importlib.util
import os
import sys
import tempfile
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import golden_inputs as gi  # noqa: E402

if "REFERENCE_ROOT" not in os.environ:
    raise SystemExit("set REFERENCE_ROOT to a checkout of kernelize-ai/triton-tenstorrent")
REF = Path(os.environ["REFERENCE_ROOT"])

KERNEL_SOURCES = {
    # module name -> (reference file, functions to extract in order)
    "ref_add": ("python/tutorials/01-vector-add.py", ["add_kernel"]),
    "ref_add_loop": ("python/tutorials/01-vector-add.loop.py", ["add_kernel"]),
    "ref_sin": ("examples/01-sin-kernel.py", ["sin_kernel"]),
    "ref_muladd": ("python/tutorials/01-vector-mul-add.py", ["muladd_kernel"]),
    "ref_matmul": ("examples/matmul_tensor_descriptor/09-persistent-matmul.ttnn.py", ["matmul_kernel_tma"]),
    "ref_fused": ("python/tutorials/09-matmul-fused.py", ["matmul_kernel_fused"]),
    "ref_attn": ("examples/fused-attn/06-fused-attention.py", ["_attn_fwd_inner", "_maybe_make_tensor_desc", "_attn_fwd"]),
    "ref_mm03": ("examples/matmul/03-matrix-multiplication.py", ["leaky_relu", "matmul_kernel"]),
}

HEADER = "import triton\nimport triton.language as tl\n\n"


def _extract(path: Path, names) -> str:
    """Source text of the named top-level functions, decorators replaced by a bare @triton.jit."""
    text = path.read_text()
    tree = ast.parse(text)
    lines = text.splitlines()
    chunks = []
    for name in names:
        node = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == name)
        body = "\n".join(lines[node.lineno - 1:node.end_lineno])  # from `def` (decorators excluded)
        chunks.append("@triton.jit\n" + body + "\n")
    return HEADER + "\n\n".join(chunks)


def _load_kernels(tmpdir: Path):
    mods = {}
    for mod_name, (rel, names) in KERNEL_SOURCES.items():
        src = _extract(REF / rel, names)
        f = tmpdir / f"{mod_name}.py"
        f.write_text(src)
        spec = importlib.util.spec_from_file_location(mod_name, f)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[mod_name] = mod
        spec.loader.exec_module(mod)
        mods[mod_name] = mod
    return mods


def _patch_interpreter_dot():
    import triton.language as tl
    from triton.runtime import interpreter as interp

    def create_dot(self, a, b, d, input_precision, max_num_imprecise_acc):
        def widen(h):
            if h.dtype.scalar == tl.bfloat16:  # stored as uint16 bit patterns
                return (h.data.astype(np.uint32) << 16).view(np.float32)
            return h.data.astype(np.float32)
        return interp.TensorHandle(np.matmul(widen(a), widen(b), dtype=np.float32) + d.data, d.dtype.scalar)

    interp.InterpreterBuilder.create_dot = create_dot

    orig_cast = interp.InterpreterBuilder.cast_impl

    def cast_impl(self, src, dst_type):
        if src.dtype.scalar == tl.float32 and dst_type.scalar == tl.bfloat16:
            f = torch.from_numpy(np.ascontiguousarray(src.data, dtype=np.float32))
            bits = f.bfloat16().view(torch.int16).numpy().view(np.uint16)  # round to nearest even
            return interp.TensorHandle(bits.reshape(src.data.shape), dst_type.scalar)
        return orig_cast(self, src, dst_type)

    interp.InterpreterBuilder.cast_impl = cast_impl
    for name in ("create_fp_trunc", "create_fp_ext", "create_si_to_fp", "create_ui_to_fp", "create_fp_to_si",
                 "create_fp_to_ui"):
        setattr(interp.InterpreterBuilder, name, lambda self, src, dst_type: self.cast_impl(src, dst_type))


def _bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> uint16 bit patterns (numpy has no bf16)."""
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main():
    from triton.tools.tensor_descriptor import TensorDescriptor
    _patch_interpreter_dot()
    only = set(sys.argv[1:])

    def want(name):
        return not only or name in only

    with tempfile.TemporaryDirectory() as td:
        k = _load_kernels(Path(td))

        if want("add"):
            # ---- add_kernel (python/tutorials/01-vector-add.py:29-54), launch as in add() :75
            out = {}
            for n in gi.ADD_SIZES:
                x, y = gi.add_inputs(n)
                o = torch.empty_like(x)
                k["ref_add"].add_kernel[((n + 1023) // 1024,)](x, y, o, n, BLOCK_SIZE=1024)
                out[f"in_sha_{n}"], out[f"out_{n}"] = np.array(gi.digest(x, y)), o.numpy()
            np.savez_compressed(HERE / "add.npz", **out)

        if want("add_loop"):
            # ---- add_kernel with the row_count loop (python/tutorials/01-vector-add.loop.py:29-66), launched as
            #      add() does (:89).  fp32 only: the interpreter cannot do bf16 arithmetic.  The output starts as a
            #      sentinel so that elements no program owns are visible.
            out = {}
            for (n, programs, row_count) in gi.ADD_LOOP_CASES:
                x, y = gi.add_inputs(n, seed=2)
                o = torch.full_like(x, -7.5)
                k["ref_add_loop"].add_kernel[(programs,)](x, y, o, n, row_count, BLOCK_SIZE=1024)
                tag = f"{n}_{programs}_{row_count}"
                # the op is bit-exact, so a digest of the output pins it as well as the bytes; the full output is
                # kept for the smallest case only
                out[f"in_sha_{tag}"], out[f"out_sha_{tag}"] = np.array(gi.digest(x, y)), np.array(gi.digest(o))
                if n < 40000:
                    out[f"out_{tag}"] = o.numpy()
            np.savez_compressed(HERE / "add_loop.npz", **out)

        if want("mul_add"):
            # ---- muladd_kernel (python/tutorials/01-vector-mul-add.py:29-56), launched as muladd() does (:62-80)
            out = {}
            for n in gi.MUL_ADD_SIZES:
                x, y, z = gi.mul_add_inputs(n)
                o = torch.empty_like(x)
                k["ref_muladd"].muladd_kernel[((n + 1023) // 1024,)](x, y, z, o, n, BLOCK_SIZE=1024)
                out[f"in_sha_{n}"], out[f"out_{n}"] = np.array(gi.digest(x, y, z)), o.numpy()
            np.savez_compressed(HERE / "mul_add.npz", **out)

        if want("sin"):
            # ---- sin_kernel (examples/01-sin-kernel.py:17-29)
            out = {}
            for n in gi.SIN_SIZES:
                x = gi.sin_inputs(n)
                o = torch.empty_like(x)
                k["ref_sin"].sin_kernel[((n + 1023) // 1024,)](x, o, n, BLOCK_SIZE=1024)
                out[f"in_sha_{n}"], out[f"out_{n}"] = np.array(gi.digest(x)), o.numpy()
            np.savez_compressed(HERE / "sin.npz", **out)

        if want("matmul"):
            # ---- matmul_kernel_tma (09-persistent-matmul.ttnn.py:105-143), the reference's 32x32x32 config :77-86
            out = {}
            for (M, N, K) in gi.MATMUL_SHAPES:
                a, b = gi.matmul_inputs(M, N, K)
                c = torch.full((M, N), 7.5, dtype=torch.bfloat16)
                BM = BN = BK = 32
                ad = TensorDescriptor.from_tensor(a, [BM, BK])
                bd = TensorDescriptor.from_tensor(b, [BK, BN])
                cd = TensorDescriptor.from_tensor(c, [BM, BN])
                grid = (((M + BM - 1) // BM) * ((N + BN - 1) // BN),)
                k["ref_matmul"].matmul_kernel_tma[grid](ad, bd, cd, M, N, K, BLOCK_SIZE_M=BM, BLOCK_SIZE_N=BN,
                                                        BLOCK_SIZE_K=BK, GROUP_SIZE_M=1, FP8_OUTPUT=False,
                                                        WARP_SPECIALIZE=False)
                tag = f"{M}x{N}x{K}"
                out[f"in_sha_{tag}"], out[f"c_{tag}"] = np.array(gi.digest(a, b)), _bits(c)
            np.savez_compressed(HERE / "matmul.npz", **out)

        if want("matmul_fused"):
            # ---- matmul_kernel_fused (python/tutorials/09-matmul-fused.py:105-148): bias [M,N] added after the
            #      downcast.  The reference hard-codes float16 as the output type (:115), so these vectors are
            #      generated with fp16 operands exactly as that file runs; they pin the oracle's fp16 mode.
            out = {}
            for (M, N, K) in gi.FUSED_SHAPES:
                a, b, bias = gi.fused_inputs(M, N, K, dtype=torch.float16)
                c = torch.empty((M, N), dtype=torch.float16)
                BM, BN, BK = 64, 64, 256  # the reference's config :74-83
                ad = TensorDescriptor.from_tensor(a, [BM, BK])
                bd = TensorDescriptor.from_tensor(b, [BK, BN])
                cd = TensorDescriptor.from_tensor(c, [BM, BN])
                biasd = TensorDescriptor.from_tensor(bias, [BM, BN])
                grid = (((M + BM - 1) // BM) * ((N + BN - 1) // BN),)
                k["ref_fused"].matmul_kernel_fused[grid](ad, bd, cd, biasd, M, N, K, BLOCK_SIZE_M=BM, BLOCK_SIZE_N=BN,
                                                         BLOCK_SIZE_K=BK, GROUP_SIZE_M=1, FP8_OUTPUT=False,
                                                         WARP_SPECIALIZE=False)
                tag = f"{M}x{N}x{K}"
                out[f"in_sha_{tag}"], out[f"c_{tag}"] = np.array(gi.digest(a, b, bias)), c.numpy()
            np.savez_compressed(HERE / "matmul_fused.npz", **out)

        if want("attention"):
            # ---- _attn_fwd (examples/fused-attn/06-fused-attention.py:143-215), launched as _attention.forward :257-267
            out = {}
            for (Z, H, S, D, causal, BM, BN) in gi.ATTN_CASES:
                q, kk, v = gi.attn_inputs(Z, H, S, D)
                sm_scale = D ** -0.5
                o = torch.empty_like(q)
                M = torch.empty((Z, H, S), dtype=torch.float32)
                y = Z * H * S
                dq = TensorDescriptor(q, shape=[y, D], strides=[D, 1], block_shape=[BM, D])
                dk = TensorDescriptor(kk, shape=[y, D], strides=[D, 1], block_shape=[BN, D])
                dv = TensorDescriptor(v, shape=[y, D], strides=[D, 1], block_shape=[BN, D])
                do = TensorDescriptor(o, shape=[y, D], strides=[D, 1], block_shape=[BM, D])
                grid = ((S + BM - 1) // BM, Z * H, 1)
                k["ref_attn"]._attn_fwd[grid](sm_scale, M, Z, H, dq, dk, dv, do, N_CTX=S, HEAD_DIM=D, BLOCK_M=BM,
                                              BLOCK_N=BN, FP8_OUTPUT=False, STAGE=3 if causal else 1,
                                              warp_specialize=False, IS_HOPPER=False)
                tag = f"{Z}x{H}x{S}x{D}_{'c' if causal else 'n'}_{BM}x{BN}"
                out[f"in_sha_{tag}"] = np.array(gi.digest(q, kk, v))
                out[f"o_{tag}"], out[f"M_{tag}"] = _bits(o), M.numpy()
            np.savez_compressed(HERE / "attention.npz", **out)
        if want("matmul_tile32"):
            # ---- matmul_kernel (examples/matmul/03-matrix-multiplication.py:241-395) on TILE-MAJOR buffers, launched
            #      as matmul() does (:413-420) with the reference's only configuration 32x32x32, GROUP_SIZE_M=1
            #      (:217-222).  The kernel ignores the strides; the stored result is the raw (tile-major) C buffer.
            out = {}
            for (M, N, K, activation) in gi.TILE32_CASES:
                a, b = gi.tile32_inputs(M, N, K)
                at, bt = gi.tilize(a), gi.tilize(b)
                c = torch.full((M, N), 7.5, dtype=torch.float16)
                grid = ((M // 32) * (N // 32),)
                k["ref_mm03"].matmul_kernel[grid](at, bt, c, M, N, K, at.stride(0), at.stride(1), bt.stride(0),
                                                  bt.stride(1), c.stride(0), c.stride(1), BLOCK_SIZE_M=32,
                                                  BLOCK_SIZE_N=32, BLOCK_SIZE_K=32, GROUP_SIZE_M=1,
                                                  ACTIVATION=activation)
                tag = f"{M}x{N}x{K}_{activation or 'none'}"
                out[f"in_sha_{tag}"], out[f"c_{tag}"] = np.array(gi.digest(a, b)), c.numpy()
            np.savez_compressed(HERE / "matmul_tile32.npz", **out)
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
