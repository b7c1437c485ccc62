"""Parity of the CUDA path (called through the C-ABI) with the CPU oracle and with the golden vectors
made from the reference's kernel sources.  Tolerances are the workload's:
  add: bit-exact;  sin: <= 2 ulp;  matmul: relative Frobenius error <= 1e-2;  attention: max-abs <= 2e-2.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

import golden_inputs as gi
from oracle import cpu_oracle as oracle
from triton_tenstorrent_b200 import _lib, kernels, ops
from triton_tenstorrent_b200.tensor_descriptor import TensorDescriptor

pytestmark = pytest.mark.gpu

MATMUL_REL_FRO = 1e-2
ATTN_MAX_ABS = 2e-2
SIN_MAX_ULP = 2


@pytest.fixture(scope="module", autouse=True)
def _device():
    if not torch.cuda.is_available():
        pytest.fail("the -m gpu tests need a CUDA device")
    torch.cuda.set_device(0)
    yield
    torch.cuda.synchronize()
    assert ops.device_status() == 0, "a kernel reported a bounded-wait timeout"


def _bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


def _bits_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    return torch.equal(a.contiguous().view(torch.int32), b.contiguous().view(torch.int32))


# ------------------------------------------------------------------------------------------------ add
@pytest.mark.parametrize("n", gi.ADD_SIZES)
def test_add_golden_bit_exact(golden_dir, n):
    g = np.load(golden_dir / "add.npz")
    x, y = gi.add_inputs(n)
    out = ops.add(x.cuda(), y.cuda()).cpu()
    assert np.array_equal(out.numpy().view(np.uint32), g[f"out_{n}"].view(np.uint32))


@pytest.mark.parametrize("n", [0, 1, 3, 4, 1023, 1025, 4099, 66560, (1 << 20) + 7])
def test_add_oracle_bit_exact_edges(n):
    x, y = gi.add_inputs(n, seed=3)
    got = ops.add(x.cuda(), y.cuda()).cpu()
    assert _bits_equal(got, oracle.add(x, y)) if n else got.numel() == 0


@pytest.mark.parametrize("case", gi.ADD_LOOP_CASES[:3])
def test_add_loop_golden_bit_exact(golden_dir, case):
    # the row_count-loop launch form (python/tutorials/01-vector-add.loop.py:89) against what the reference's
    # kernel source wrote; fp32 through kernels.add_kernel_loop, then the tutorial's bf16 through ops.add_loop
    n, programs, row_count = case
    g = np.load(golden_dir / "add_loop.npz")
    x, y = gi.add_inputs(n, seed=2)
    out = torch.full((n,), -7.5, device="cuda")
    kernels.add_kernel_loop[(programs,)](x.cuda(), y.cuda(), out, n, row_count, BLOCK_SIZE=1024, num_warps=1)
    assert gi.digest(out.cpu()) == str(g[f"out_sha_{n}_{programs}_{row_count}"])
    xb, yb = x.bfloat16(), y.bfloat16()
    got = ops.add_loop(xb.cuda(), yb.cuda()).cpu()
    assert torch.equal(got.view(torch.int16), oracle.add_loop(xb, yb, -(-(-(-n // 1024)) // 130), 130).view(torch.int16))


def test_add_loop_rejects_uncovered_launch():
    # the reference leaves elements that no program owns untouched; this launcher refuses such a grid
    n, programs, row_count = gi.ADD_LOOP_CASES[3]
    x, y = gi.add_inputs(n, seed=2)
    with pytest.raises(_lib.B200KError) as e:
        kernels.add_kernel_loop[(programs,)](x.cuda(), y.cuda(), torch.empty(n, device="cuda"), n, row_count, BLOCK_SIZE=1024)
    assert "does not cover" in str(e.value)


@pytest.mark.parametrize("n", [0, 1, 7, 8, 9, 1023, 4099, 98432, (1 << 20) + 5])
def test_add_bf16_bit_exact(n):
    # bf16 add == exact sum rounded to nearest even, over the whole exponent range and with unaligned views
    g = torch.Generator().manual_seed(9)
    x = (torch.randn(n + 3, generator=g) * torch.exp2(torch.randint(-20, 20, (n + 3,), generator=g).float())).bfloat16()
    y = (torch.randn(n + 3, generator=g) * torch.exp2(torch.randint(-20, 20, (n + 3,), generator=g).float())).bfloat16()
    got = ops.add(x[:n].cuda(), y[:n].cuda()).cpu()
    assert torch.equal(got.view(torch.int16), (x[:n] + y[:n]).view(torch.int16))
    got = ops.add(x.cuda()[3:], y.cuda()[1:n + 1]).cpu()          # 6- and 2-byte offsets: scalar path
    assert torch.equal(got.view(torch.int16), (x[3:] + y[1:n + 1]).view(torch.int16))


def test_add_unaligned_views_and_canaries():
    x, y = gi.add_inputs(5003, seed=5)
    xd, yd = x.cuda(), y.cuda()
    for off in (1, 2, 3):
        got = ops.add(xd[off:], yd[off:]).cpu()           # 4-byte aligned only: scalar path
        assert _bits_equal(got, oracle.add(x[off:], y[off:]))
    # direct C-ABI call into the middle of a canary-filled buffer: nothing outside [0, n) is written
    n = 4097
    buf = torch.full((n + 64,), -7.0, device="cuda")
    lib = _lib.load()
    _lib.check(lib.b200k_add_f32(xd.data_ptr(), yd.data_ptr(), buf[32:].data_ptr(), n, 1024,
                                 torch.cuda.current_stream().cuda_stream))
    host = buf.cpu()
    assert torch.all(host[:32] == -7.0) and torch.all(host[32 + n:] == -7.0)
    assert _bits_equal(host[32:32 + n], oracle.add(x[:n], y[:n]))


def test_add_full_size_property():
    # 2^26 elements: the same bits as an fp32 add done by torch on the device
    n = 1 << 26
    g = torch.Generator(device="cuda").manual_seed(0)
    x, y = torch.rand(n, device="cuda", generator=g), torch.rand(n, device="cuda", generator=g)
    assert torch.equal(ops.add(x, y), x + y)


@pytest.mark.parametrize("n", gi.MUL_ADD_SIZES)
def test_mul_add_golden_bit_exact(golden_dir, n):
    # golden vectors made by running the reference's muladd_kernel (python/tutorials/01-vector-mul-add.py:29-56)
    g = np.load(golden_dir / "mul_add.npz")
    x, y, z = gi.mul_add_inputs(n)
    got = ops.mul_add(x.cuda(), y.cuda(), z.cuda()).cpu()
    assert np.array_equal(got.numpy().view(np.uint32), g[f"out_{n}"].view(np.uint32))


def test_mul_add_oracle_bit_exact():
    x, y = gi.add_inputs(98432, seed=7)
    z = gi.sin_inputs(98432, seed=8)
    got = ops.mul_add(x.cuda(), y.cuda(), z.cuda()).cpu()
    assert _bits_equal(got, oracle.mul_add(x, y, z))


# ------------------------------------------------------------------------------------------------ sin
@pytest.mark.parametrize("n", gi.SIN_SIZES)
def test_sin_golden_within_2ulp(golden_dir, n):
    g = np.load(golden_dir / "sin.npz")
    x = gi.sin_inputs(n)
    got = ops.sin(x.cuda()).cpu()
    assert oracle.ulp_diff_f32(got, torch.from_numpy(g[f"out_{n}"])) <= SIN_MAX_ULP
    assert oracle.ulp_diff_f32(got, oracle.sin(x)) <= SIN_MAX_ULP            # the CPU path's libm sinf
    assert oracle.ulp_diff_f32(got, oracle.sin_correctly_rounded(x)) <= SIN_MAX_ULP


def test_sin_full_size_within_2ulp():
    n = 1 << 26
    x = gi.sin_inputs(n, seed=11)
    got = ops.sin(x.cuda()).cpu()
    assert oracle.ulp_diff_f32(got, oracle.sin_correctly_rounded(x)) <= SIN_MAX_ULP
    assert oracle.pcc(got[: 1 << 20], oracle.sin_correctly_rounded(x[: 1 << 20])) > 0.97   # the reference's own gate


def test_sin_ragged_and_special_values():
    x = torch.tensor([0.0, -0.0, math.pi, -math.pi, 4 * math.pi, -4 * math.pi, 1e-30, 0.5, 100.0, -1234.5, 1e6],
                     dtype=torch.float32)
    got = ops.sin(x.cuda()).cpu()
    ref = oracle.sin_correctly_rounded(x)
    assert oracle.ulp_diff_f32(got, ref) <= SIN_MAX_ULP
    assert math.copysign(1.0, got[1].item()) == -1.0    # sin(-0) = -0


# ------------------------------------------------------------------------------------------------ memcpy (Gluon intro)
@pytest.mark.parametrize("n,xblock", [(1, 64), (40, 64), (500, 64), (98432, 1024), (2 ** 22 + 3, 2048)])
def test_memcpy_bit_exact(n, xblock):
    # memcpy_kernel / memcpy(), python/tutorials/gluon/01-intro.py:84-99 (its own tests: xnumel 40 and 500, XBLOCK 64, atol 0)
    g = torch.Generator(device="cpu").manual_seed(n)
    x = torch.randn(n, generator=g, dtype=torch.float32)
    bits = x.view(torch.int32)
    bits[::7] = torch.tensor(0x7FC12345, dtype=torch.int32)        # NaNs with a payload
    bits[3::11] = torch.tensor(0x7F800001, dtype=torch.int32)      # a signalling NaN: must not be quieted
    if n > 2:
        x[1], x[2] = float("inf"), -0.0
    ref = oracle.memcpy(x, xblock)
    assert torch.equal(ref.view(torch.int32), x.view(torch.int32))
    pad = 64
    buf = torch.full((n + 2 * pad,), -7.0, device="cuda")
    out = buf[pad:pad + n]
    ops.memcpy(x.cuda(), out, xblock)
    torch.cuda.synchronize()
    assert torch.equal(out.cpu().view(torch.int32), ref.view(torch.int32))
    assert bool((buf[:pad] == -7.0).all()) and bool((buf[pad + n:] == -7.0).all())
    # unaligned source and destination (scalar path), through the kernel[grid] surface
    if n > 8:
        xs = x.cuda()
        dst = torch.full((n,), -7.0, device="cuda")
        kernels.memcpy_kernel[((n - 1 + xblock - 1) // xblock,)](xs[1:], dst[1:], n - 1, xblock, num_warps=1)
        torch.cuda.synchronize()
        assert torch.equal(dst[1:].cpu().view(torch.int32), x[1:].view(torch.int32)) and float(dst[0]) == -7.0


def test_copy_scalar_and_full_size():
    x = torch.tensor([42.0], device="cuda")                      # test_copy_scalar of the reference file
    out = torch.empty_like(x)
    kernels.copy_scalar_kernel[(1,)](x, out, num_warps=1)
    assert float(out[0]) == 42.0
    n = 2 ** 26
    big = torch.rand(n, device="cuda")
    got = ops.memcpy(big)
    assert torch.equal(got, big)
    assert ops.device_status() == 0


# ------------------------------------------------------------------------------------------------ matmul
@pytest.mark.parametrize("shape", gi.MATMUL_SHAPES)
def test_matmul_golden(golden_dir, shape):
    M, N, K = shape
    g = np.load(golden_dir / "matmul.npz")
    a, b = gi.matmul_inputs(M, N, K)
    golden = _bf16(g[f"c_{M}x{N}x{K}"])
    got = ops.matmul_tma(a.cuda(), b.cuda(), warp_specialize=True).cpu()
    assert oracle.rel_frobenius(got.float(), golden.float()) <= MATMUL_REL_FRO
    # in fact only summation order differs: at most one bf16 ulp, rarely
    assert float((got.float() - golden.float()).abs().max()) <= float(golden.float().abs().max()) * 2 ** -7
    assert float((got.view(torch.int16) != golden.view(torch.int16)).float().mean()) < 5e-3


@pytest.mark.parametrize("shape", [(128, 128, 64), (512, 384, 640), (200, 264, 136), (1000, 8, 72), (40, 1032, 8),
                                   (1024, 1024, 1024), (129, 257 * 8, 65 * 8)])
def test_matmul_oracle_shapes_and_tails(shape):
    M, N, K = shape
    a, b = gi.matmul_inputs(M, N, K, seed=2)
    ref = oracle.golden_matmul(a, b)
    c = torch.full((M, N), 7.5, dtype=torch.bfloat16, device="cuda")   # the reference pre-fills C with 7.5
    got = ops._matmul_call(a.cuda(), b.cuda(), c=c).cpu()
    assert not torch.any(got == 7.5), "an element of C was left unwritten"
    assert oracle.rel_frobenius(got.float(), ref.float()) <= MATMUL_REL_FRO
    assert oracle.pcc(got.float(), ref.float()) > 0.97


@pytest.mark.parametrize("shape", [(2200, 2312, 520), (2304, 2304, 64), (4096, 1288, 1000)])
def test_matmul_cta_pair_kernel_tails(shape):
    # enough 256 x 256 tiles for the CTA-pair kernel, with M, N and K tails (second CTA of a pair partly or
    # wholly outside M; last tile column partly outside N; K not a multiple of 64)
    M, N, K = shape
    a, b, bias_full = gi.fused_inputs(M, N, K, seed=14)
    c = torch.full((M, N), 7.5, dtype=torch.bfloat16, device="cuda")
    got = ops._matmul_call(a.cuda(), b.cuda(), c=c).cpu()
    ref = oracle.golden_matmul(a, b)
    assert not torch.any(got == 7.5), "an element of C was left unwritten"
    assert oracle.rel_frobenius(got.float(), ref.float()) <= MATMUL_REL_FRO
    got = ops.matmul_tma_fused(a.cuda(), b.cuda(), bias_full.cuda()).cpu()
    assert oracle.rel_frobenius(got.float(), oracle.golden_matmul(a, b, bias=bias_full, mode=2).float()) <= MATMUL_REL_FRO


@pytest.mark.parametrize("shape", [(4096, 4096, 192), (2560, 4096, 320), (4352, 4608, 136)])
def test_matmul_split_last_wave(shape, monkeypatch):
    # tile counts whose last wave fills at most half of the CTA pairs: its tiles are computed as two 256 x 128 halves.
    # Same MMAs over K in the same order, so the result equals the unsplit schedule bit for bit; rows against the oracle.
    M, N, K = shape
    props = torch.cuda.get_device_properties(0)
    pairs = props.multi_processor_count // 2
    tiles = -(-M // 256) * -(-N // 256)
    if not (tiles >= pairs and 0 < tiles % pairs <= pairs // 2):
        pytest.skip("this device's SM count does not give a sparse last wave for the shape")
    a, b = gi.matmul_inputs(M, N, K, seed=71)
    bias = gi.row_bias(N).cuda()
    ad, bd = a.cuda(), b.cuda()
    split = ops.matmul_fused(ad, bd, bias, "relu")
    monkeypatch.setenv("B200K_MATMUL_SPLIT_TAIL", "0")
    whole = ops.matmul_fused(ad, bd, bias, "relu")
    monkeypatch.delenv("B200K_MATMUL_SPLIT_TAIL")
    assert torch.equal(split.view(torch.int16), whole.view(torch.int16))
    rows = torch.tensor([0, 255, 256, M // 2 + 3, M - 257, M - 1])
    ref = oracle.golden_matmul(a[rows], b, bias=bias.cpu(), mode=3, activation="relu")
    assert oracle.rel_frobenius(split[rows.cuda()].cpu().float(), ref.float()) <= MATMUL_REL_FRO


def test_matmul_strided_operands_and_canaries():
    M, N, K = 300, 200, 264
    a, b = gi.matmul_inputs(M, N, K, seed=4)
    abig = torch.zeros(M, K + 24, dtype=torch.bfloat16, device="cuda"); abig[:, :K] = a.cuda()
    bbig = torch.zeros(K, N + 8, dtype=torch.bfloat16, device="cuda"); bbig[:, :N] = b.cuda()
    cbig = torch.full((M + 2, N + 16), -3.0, dtype=torch.bfloat16, device="cuda")
    ops._matmul_call(abig[:, :K], bbig[:, :N], c=cbig[:M, :N])
    host = cbig.cpu()
    assert torch.all(host[M:, :] == -3.0) and torch.all(host[:, N:] == -3.0), "store outside [M,N]"
    ref = oracle.golden_matmul(a, b)
    assert oracle.rel_frobenius(host[:M, :N].float(), ref.float()) <= MATMUL_REL_FRO


def _random_matmul_shapes(n, seed):
    rng = np.random.RandomState(seed)
    return [(int(rng.randint(1, 2000)), 8 * int(rng.randint(1, 260)), 8 * int(rng.randint(1, 130)), int(rng.randint(0, 4)))
            for _ in range(n)]


@pytest.mark.parametrize("M,N,K,mode", _random_matmul_shapes(24, 81))
def test_matmul_random_shapes(M, N, K, mode):
    # seeded random sizes (any M; N and K multiples of 8, the 16-byte row rule of TMA): single-CTA and CTA-pair kernels,
    # whole / half / missing last waves, with each epilogue; C sits between canaries
    a, b, bias_full = gi.fused_inputs(M, N, K, seed=82)
    ad, bd = a.cuda(), b.cuda()
    pad = 1024
    buf = torch.full((M * N + 2 * pad,), 7.5, dtype=torch.bfloat16, device="cuda")
    c = buf[pad:pad + M * N].view(M, N)
    if mode == 0:
        got, ref = ops._matmul_call(ad, bd, c=c), oracle.golden_matmul(a, b)
    elif mode == 1:
        got, ref = ops.matmul(ad, bd, activation="leaky_relu"), oracle.golden_matmul(a, b, mode=0, activation="leaky_relu")
    elif mode == 2:
        bias_row = gi.row_bias(N)
        got, ref = (ops.matmul_fused(ad, bd, bias_row.cuda(), activation="relu"),
                    oracle.golden_matmul(a, b, bias=bias_row, mode=3, activation="relu"))
    else:
        got, ref = ops.matmul_tma_fused(ad, bd, bias_full.cuda(), True), oracle.golden_matmul(a, b, bias=bias_full, mode=2)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    got = got.cpu()
    assert tuple(got.shape) == (M, N)
    denom = float(ref.float().norm())
    assert float((got.float() - ref.float()).norm()) <= MATMUL_REL_FRO * denom + 1e-3
    if mode == 0:
        assert not torch.any(got == 7.5), "an element of C was left unwritten"
        assert bool((buf[:pad] == 7.5).all()) and bool((buf[pad + M * N:] == 7.5).all())


def test_matmul_activation_and_bias_epilogues():
    M, N, K = 384, 320, 256
    a, b, bias_full = gi.fused_inputs(M, N, K, seed=6)
    bias_row = gi.row_bias(N)
    ad, bd = a.cuda(), b.cuda()
    cases = [
        (ops.matmul(ad, bd, activation="leaky_relu"), oracle.golden_matmul(a, b, mode=0, activation="leaky_relu")),
        (ops.matmul(ad, bd, activation="relu"), oracle.golden_matmul(a, b, mode=0, activation="relu")),
        (ops.matmul_fused(ad, bd, bias_row.cuda(), activation="relu"),
         oracle.golden_matmul(a, b, bias=bias_row, mode=3, activation="relu")),
        (ops.matmul_fused(ad, bd, bias_row.cuda(), activation=""), oracle.golden_matmul(a, b, bias=bias_row, mode=3)),
        (ops.matmul_tma_fused(ad, bd, bias_full.cuda(), True), oracle.golden_matmul(a, b, bias=bias_full, mode=2)),
        (ops.matmul_tma_fused(ad, bd, bias_full.cuda(), True, round_before_bias=False),
         oracle.golden_matmul(a, b, bias=bias_full, mode=1)),
    ]
    for got, ref in cases:
        got = got.cpu()
        assert oracle.rel_frobenius(got.float(), ref.float()) <= MATMUL_REL_FRO
        assert float((got.view(torch.int16) != ref.view(torch.int16)).float().mean()) < 1e-2
    relu = cases[2][0].cpu().float()
    assert float(relu.min()) >= 0.0 and float((relu == 0).float().mean()) > 0.2


def test_matmul_fused_tail_bias():
    # N not a multiple of 64 and M not a multiple of 32: the guarded bias paths
    M, N, K = 100, 72, 64
    a, b, bias_full = gi.fused_inputs(M, N, K, seed=9)
    bias_row = gi.row_bias(N)
    got = ops.matmul_fused(a.cuda(), b.cuda(), bias_row.cuda()).cpu()
    assert oracle.rel_frobenius(got.float(), oracle.golden_matmul(a, b, bias=bias_row, mode=3, activation="relu").float()) <= MATMUL_REL_FRO
    got = ops.matmul_tma_fused(a.cuda(), b.cuda(), bias_full.cuda()).cpu()
    assert oracle.rel_frobenius(got.float(), oracle.golden_matmul(a, b, bias=bias_full, mode=2).float()) <= MATMUL_REL_FRO


@pytest.mark.parametrize("S", [4096, 8192, 16384])
def test_matmul_full_size_rows_against_oracle(S):
    # full-size problem on the GPU (all three sizes of the workload definition); the oracle recomputes a sample of
    # rows (whole rows of C, all of B)
    a, b = gi.matmul_inputs(S, S, S, seed=12)
    ad, bd = a.cuda(), b.cuda()
    got = ops.matmul_tma(ad, bd)
    rows = torch.tensor([0, 1, 127, 128, 255, 256, S // 2 + 3, S - 257, S - 129, S - 1] + list(range(1000, 1000 + 22)))
    ref = oracle.golden_matmul(a[rows], b)
    assert oracle.rel_frobenius(got[rows.cuda()].cpu().float(), ref.float()) <= MATMUL_REL_FRO
    # linearity in A: (2A).B == 2 (A.B) exactly (power-of-two scaling commutes with every rounding)
    ad.mul_(2)
    got2 = ops.matmul_tma(ad, bd)
    got.mul_(2)
    assert torch.equal(got2, got)


def test_matmul_fused_workload_shape_sample():
    M, N, K = 16384, 4096, 4096
    a, b = gi.matmul_inputs(M, N, K, seed=13)
    bias = gi.row_bias(N)
    got = ops.matmul_fused(a.cuda(), b.cuda(), bias.cuda(), activation="relu")
    rows = torch.arange(0, M, 512)
    ref = oracle.golden_matmul(a[rows], b, bias=bias, mode=3, activation="relu")
    assert oracle.rel_frobenius(got[rows.cuda()].cpu().float(), ref.float()) <= MATMUL_REL_FRO


# fp16: the reference's fused kernel and its pointer-based example compute in fp16
@pytest.mark.parametrize("shape", gi.FUSED_SHAPES)
def test_matmul_fused_fp16_golden(golden_dir, shape):
    # golden vectors made by running the reference's matmul_kernel_fused (python/tutorials/09-matmul-fused.py:105-148)
    M, N, K = shape
    g = np.load(golden_dir / "matmul_fused.npz")
    a, b, bias = gi.fused_inputs(M, N, K, dtype=torch.float16)
    golden = torch.from_numpy(g[f"c_{M}x{N}x{K}"])
    got = ops.matmul_tma_fused(a.cuda(), b.cuda(), bias.cuda(), True).cpu()       # add after the downcast, like the kernel
    assert got.dtype == torch.float16
    assert oracle.rel_frobenius(got.float(), golden.float()) <= MATMUL_REL_FRO
    diff = (got.float() - golden.float()).abs()
    assert float(diff.max()) <= float(golden.float().abs().max()) * 2 ** -10       # one fp16 ulp of the largest value
    assert float((diff > 0).float().mean()) < 5e-3
    # the same through the kernel[grid] surface with descriptors over fp16 tensors
    ad, bd, biasd = a.cuda(), b.cuda(), bias.cuda()
    c = torch.full((M, N), 7.5, device="cuda", dtype=torch.float16)
    descs = [TensorDescriptor.from_tensor(t, [32, 32]) for t in (ad, bd, c, biasd)]
    mgrid = lambda META: (-(-M // META["BLOCK_SIZE_M"]) * -(-N // META["BLOCK_SIZE_N"]),)
    kernels.matmul_kernel_fused[mgrid](*descs, M, N, K, FP8_OUTPUT=False, WARP_SPECIALIZE=True)
    assert torch.equal(c.cpu().view(torch.int16), got.view(torch.int16))


def test_matmul_fp16_example_shapes_and_activation():
    # the reference's unit test of matmul(a, b): 32x64 . 64x32 fp16, atol 1e-2
    # (examples/matmul/03-matrix-multiplication.py:431-438), plus larger shapes and leaky_relu
    torch.manual_seed(0)
    a = torch.rand((32, 64), dtype=torch.float16) - 0.5
    b = torch.rand((64, 32), dtype=torch.float16) - 0.5
    got = ops.matmul(a.cuda(), b.cuda()).cpu()
    assert got.dtype == torch.float16
    assert torch.allclose(got.float(), oracle.golden_matmul(a, b).float(), atol=1e-2, rtol=0)
    for (M, N, K) in ((512, 384, 640), (2304, 2304, 136)):
        a, b = gi.matmul_inputs(M, N, K, seed=15, dtype=torch.float16)
        for act in ("", "leaky_relu"):
            got = ops.matmul(a.cuda(), b.cuda(), activation=act).cpu()
            ref = oracle.golden_matmul(a, b, mode=0, activation=act)
            assert oracle.rel_frobenius(got.float(), ref.float()) <= MATMUL_REL_FRO
            assert float((got.view(torch.int16) != ref.view(torch.int16)).float().mean()) < 1e-2


@pytest.mark.parametrize("shape", [(128, 128, 64), (640, 384, 200), (2304, 2304, 256)])
def test_matmul_multi_destinations(shape):
    # the epilogue stores every tile into all destinations (here: row blocks of three local "full C" buffers, the
    # layout the multi-GPU all-gather uses); both kernels, tails included; neighbours of the blocks stay untouched
    M, N, K = shape
    a, b = gi.matmul_inputs(M, N, K, seed=31)
    bias = gi.row_bias(N)
    ad, bd = a.cuda(), b.cuda()
    full = [torch.full((3 * M, N), 7.5, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    dests = [f[M:2 * M] for f in full]
    out = ops.matmul_multi(ad, bd, dests[:2], bias=bias.cuda(), activation="relu", remote_ptrs=[dests[2].data_ptr()])
    ref = ops.matmul_fused(ad, bd, bias.cuda(), "relu")
    assert out.data_ptr() == dests[0].data_ptr()
    for f in full:
        assert torch.equal(f[M:2 * M].view(torch.int16), ref.view(torch.int16))
        assert bool((f[:M] == 7.5).all()) and bool((f[2 * M:] == 7.5).all())
    with pytest.raises(ValueError):
        ops.matmul_multi(ad, bd, [])
    with pytest.raises(ValueError):
        ops.matmul_multi(ad, bd, [dests[0], torch.empty((M, N + 8), dtype=torch.bfloat16, device="cuda")[:, :N]])


@pytest.mark.parametrize("case", gi.TILE32_CASES)
def test_matmul_tile32_golden(golden_dir, case):
    # tile-major buffers in, tile-major buffer out, against what the reference's matmul_kernel source wrote
    M, N, K, act = case
    g = np.load(golden_dir / "matmul_tile32.npz")
    a, b = gi.tile32_inputs(M, N, K)
    golden = torch.from_numpy(g[f"c_{M}x{N}x{K}_{act or 'none'}"])
    got = ops.matmul(gi.tilize(a).cuda(), gi.tilize(b).cuda(), activation=act, layout="tile32").cpu()
    assert got.dtype == torch.float16
    assert oracle.rel_frobenius(got.float(), golden.float()) <= MATMUL_REL_FRO
    diff = (got.float() - golden.float()).abs()
    assert float(diff.max()) <= float(golden.float().abs().max()) * 2 ** -9
    assert float((diff > 0).float().mean()) < 1e-2


@pytest.mark.parametrize("shape,dtype", [((32, 32, 32), torch.float16), ((160, 96, 224), torch.float16),
                                          ((384, 640, 416), torch.bfloat16), ((2304, 2304, 160), torch.float16),
                                          ((2560, 4608, 96), torch.bfloat16)])
def test_matmul_tile32_oracle_shapes(shape, dtype):
    # single-CTA kernels (few tiles) and the CTA-pair kernel (>= 74 tiles of 256 x 256), with tile rows / columns that
    # end inside a 128 / 256-wide kernel tile; sentinel-filled C catches unwritten tiles
    M, N, K = shape
    a, b = gi.matmul_inputs(M, N, K, seed=21, dtype=dtype)
    for act in ("", "leaky_relu"):
        c = torch.full((M, N), 7.5, dtype=dtype, device="cuda")
        kernels.matmul_kernel[lambda META: (-(-M // META["BLOCK_SIZE_M"]) * -(-N // META["BLOCK_SIZE_N"]),)](
            gi.tilize(a).cuda(), gi.tilize(b).cuda(), c, M, N, K, K, 1, N, 1, N, 1, ACTIVATION=act, LAYOUT="tile32")
        ref = oracle.matmul_kernel_tile32(gi.tilize(a), gi.tilize(b), act)
        got = c.cpu()
        assert oracle.rel_frobenius(got.float(), ref.float()) <= MATMUL_REL_FRO
        assert float((got.view(torch.int16) != ref.view(torch.int16)).float().mean()) < 2e-2
        # and the logical result equals the row-major path's, bit for bit (same kernel, same shared-memory image)
        row = ops.matmul(a.cuda(), b.cuda(), activation=act).cpu()
        assert torch.equal(ops.untilize(got).view(torch.int16), row.view(torch.int16))


def test_matmul_tile32_full_size_equals_row_major():
    # the workload's full size through the CTA-pair kernel: tile-major in / out equals the row-major result bit for
    # bit (both layouts feed the same MMAs; the row-pair fetch of A only permutes accumulator rows, undone in the epilogue)
    S = 8192
    g = torch.Generator(device="cuda").manual_seed(5)
    a = (torch.randn(S, S, device="cuda", generator=g) / S ** 0.5).bfloat16()
    b = (torch.randn(S, S, device="cuda", generator=g) / S ** 0.5).bfloat16()
    row = ops.matmul(a, b, "leaky_relu")
    tiled = ops.matmul(ops.tilize(a), ops.tilize(b), "leaky_relu", layout="tile32")
    assert torch.equal(ops.untilize(tiled).view(torch.int16), row.view(torch.int16))
    # a sample of rows against the CPU oracle
    rows = torch.tensor([0, 1, 8, 9, 15, 31, 127, 128, 4095, 8191])
    ref = oracle.golden_matmul(a[rows].cpu(), b.cpu(), activation="leaky_relu")
    assert oracle.rel_frobenius(row[rows.cuda()].cpu().float(), ref.float()) <= MATMUL_REL_FRO


def test_matmul_tile32_rejects_bad_arguments():
    t = torch.zeros(64, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        ops.matmul(torch.zeros(48, 64, dtype=torch.float16, device="cuda"), t, layout="tile32")
    with pytest.raises(ValueError):
        ops.matmul(t, t, layout="tile16")
    lib = _lib.load()
    rc = lib.b200k_matmul_tile32(t.data_ptr(), t.data_ptr(), t.data_ptr(), 64, 40, 64, 0, 1, None)
    assert rc == _lib.ERR_INVALID_ARG and "multiples of 32" in _lib.last_error()
    rc = lib.b200k_matmul_tile32(t.data_ptr(), t.data_ptr(), t.data_ptr(), 64, 64, 64, 0, 2, None)
    assert rc == _lib.ERR_INVALID_ARG


def test_matmul_rejects_bad_arguments():
    a = torch.zeros(64, 36, dtype=torch.bfloat16, device="cuda")      # 72-byte rows
    b = torch.zeros(36, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        ops.matmul_tma(a, b)
    with pytest.raises(AssertionError):
        ops.matmul_tma(torch.zeros(64, 32, dtype=torch.bfloat16, device="cuda"), b)   # K mismatch
    lib = _lib.load()
    t = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    rc = lib.b200k_matmul_bf16(t.data_ptr() + 2, t.data_ptr(), t.data_ptr(), 32, 32, 32, 64, 64, 64, None, 0, 0, 0, 0, None)
    assert rc == _lib.ERR_INVALID_ARG and "16-byte aligned" in _lib.last_error()


@pytest.mark.parametrize("D,causal", [(128, True), (64, False)])
def test_attention_multi_destinations(D, causal):
    Z, H, S = 1, 3, 384
    q, k, v = gi.attn_inputs(Z, H, S, D, seed=51)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    rows = Z * H * S
    full = [torch.full((3 * rows, D), 7.5, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    out, m = ops.attention_multi(qd, kd, vd, causal, D ** -0.5, full[0][rows:2 * rows],
                                 remote_ptrs=[f[rows:2 * rows].data_ptr() for f in full[1:]])
    ref_o, ref_m = ops.attention_with_lse(qd, kd, vd, causal, D ** -0.5)
    assert torch.equal(m, ref_m)
    for f in full:
        assert torch.equal(f[rows:2 * rows].view(torch.int16), ref_o.reshape(rows, D).view(torch.int16))
        assert bool((f[:rows] == 7.5).all()) and bool((f[2 * rows:] == 7.5).all())


def test_concurrent_threads_and_streams():
    # the library is re-entrant: host threads with their own streams launch concurrently (tensor-map cache, error
    # strings and the launch counter are shared or thread-local state) and every result equals the serial one
    import threading
    a, b = gi.matmul_inputs(512, 768, 640, seed=61)
    q, k, v = gi.attn_inputs(1, 2, 256, 128, seed=61)
    x, y = gi.add_inputs(1 << 18, seed=61)
    ad, bd, qd, kd, vd, xd, yd = (t.cuda() for t in (a, b, q, k, v, x, y))
    want = (ops.matmul_tma(ad, bd), ops.attention(qd, kd, vd, True, 0.09), ops.add(xd, yd))
    torch.cuda.synchronize()
    errors = []

    def worker(idx):
        try:
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                for _ in range(20):
                    got = (ops.matmul_tma(ad, bd), ops.attention(qd, kd, vd, True, 0.09), ops.add(xd, yd))
                stream.synchronize()
            for g, w in zip(got, want):
                if not _bits_equal(g.float(), w.float()):
                    errors.append(f"thread {idx}: result differs")
            try:
                ops.matmul_tma(ad, bd[:100])          # K mismatch: an error on this thread only
            except AssertionError:
                pass
        except Exception as e:  # noqa: BLE001
            errors.append(f"thread {idx}: {e!r}")

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors


def test_cuda_graph_capture_and_replay():
    # the launch-bound calls (the reference's own add at n = 98432 is one) can be recorded once and replayed: every
    # entry point launches on the caller's stream and neither allocates nor synchronises once the device is warm
    n = 98432
    x, y = gi.add_inputs(n)
    a, b = gi.matmul_inputs(256, 512, 192, seed=41)
    q, k, v = gi.attn_inputs(1, 2, 256, 128, seed=41)
    sx, sy, sa, sb = x.cuda(), y.cuda(), a.cuda(), b.cuda()
    sq, sk, sv = q.cuda(), k.cuda(), v.cuda()
    eager = lambda: (ops.add(sx, sy), ops.sin(sx), ops.matmul(sa, sb, "leaky_relu"), ops.attention(sq, sk, sv, True, 0.1))
    want1 = [t.clone() for t in eager()]                       # also warms every kernel up
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = eager()
    graph.replay()
    torch.cuda.synchronize()
    for got, want in zip(outs, want1):
        assert _bits_equal(got.float(), want.float())
    # new contents in the captured input buffers, replay again
    x2, y2 = gi.add_inputs(n, seed=8)
    a2, b2 = gi.matmul_inputs(256, 512, 192, seed=42)
    q2, k2, v2 = gi.attn_inputs(1, 2, 256, 128, seed=42)
    for dst, src in ((sx, x2), (sy, y2), (sa, a2), (sb, b2), (sq, q2), (sk, k2), (sv, v2)):
        dst.copy_(src)
    graph.replay()
    torch.cuda.synchronize()
    got2 = [t.clone() for t in outs]
    want2 = eager()
    torch.cuda.synchronize()
    for got, want in zip(got2, want2):
        assert _bits_equal(got.float(), want.float())
    assert _bits_equal(got2[0], oracle.add(x2, y2).cuda())


# ------------------------------------------------------------------------------------------------ attention
@pytest.mark.parametrize("case", gi.ATTN_CASES)
def test_attention_golden(golden_dir, case):
    Z, H, S, D, causal, BM, BN = case
    g = np.load(golden_dir / "attention.npz")
    q, k, v = gi.attn_inputs(Z, H, S, D)
    tag = f"{Z}x{H}x{S}x{D}_{'c' if causal else 'n'}_{BM}x{BN}"
    golden_o, golden_m = _bf16(g[f"o_{tag}"]), torch.from_numpy(g[f"M_{tag}"])
    o, m = ops.attention_with_lse(q.cuda(), k.cuda(), v.cuda(), causal, D ** -0.5)
    assert float((o.cpu().float() - golden_o.float()).abs().max()) <= ATTN_MAX_ABS
    assert float((m.cpu() - golden_m).abs().max()) <= 1e-4


@pytest.mark.parametrize("Z,H,S,causal", [(1, 1, 128, False), (1, 1, 128, True), (1, 3, 384, True), (2, 2, 512, False),
                                          (1, 2, 1024, True), (1, 1, 2048, False), (3, 5, 256, True)])
def test_attention_oracle(Z, H, S, causal):
    D = 128
    q, k, v = gi.attn_inputs(Z, H, S, D, seed=21)
    ref_o, ref_m = oracle.attention(q, k, v, causal, D ** -0.5, BLOCK_M=128, BLOCK_N=128)
    o, m = ops.attention_with_lse(q.cuda(), k.cuda(), v.cuda(), causal, D ** -0.5)
    assert float((o.cpu().float() - ref_o.float()).abs().max()) <= ATTN_MAX_ABS
    assert float((m.cpu() - ref_m).abs().max()) <= 1e-4
    assert oracle.pcc(o.cpu().float(), ref_o.float()) > 0.999


def test_attention_scale_and_large_logits():
    # large sm_scale: sharp softmax, exercises the running-maximum updates and the rescale of O
    Z, H, S, D = 1, 2, 512, 128
    q, k, v = gi.attn_inputs(Z, H, S, D, seed=22)
    for causal in (False, True):
        ref_o, ref_m = oracle.attention(q, k, v, causal, 0.5)
        o, m = ops.attention_with_lse(q.cuda(), k.cuda(), v.cuda(), causal, 0.5)
        assert float((o.cpu().float() - ref_o.float()).abs().max()) <= ATTN_MAX_ABS
        assert float((m.cpu() - ref_m).abs().max()) <= 1e-3


@pytest.mark.parametrize("causal", [False, True])
def test_attention_full_size_heads_against_oracle(causal):
    # the full workload on the GPU; the oracle recomputes two (batch, head) pairs
    Z, H, S, D = 4, 32, 4096, 128
    q, k, v = gi.attn_inputs(Z, H, S, D, seed=23)
    o, m = ops.attention_with_lse(q.cuda(), k.cuda(), v.cuda(), causal, D ** -0.5)
    # the first head, one from the middle and the last one (the causal schedule merges the last heads' items)
    for (z, h) in ((0, 0), (1, 17), (3, 31)):
        sl = (slice(z, z + 1), slice(h, h + 1))
        ref_o, ref_m = oracle.attention(q[sl], k[sl], v[sl], causal, D ** -0.5)
        assert float((o[sl].cpu().float() - ref_o.float()).abs().max()) <= ATTN_MAX_ABS
        assert float((m[sl].cpu() - ref_m).abs().max()) <= 1e-4
    # M of EVERY (batch, head) is the base-2 log-sum-exp of the scaled scores: recomputed head by head in fp32 on the GPU
    # (an exact property of the workload, independent of the blockwise order)
    scale = D ** -0.5
    qd, kd = q.cuda(), k.cuda()
    keep = torch.ones(S, S, dtype=torch.bool, device="cuda").tril() if causal else None
    worst = 0.0
    for z in range(Z):
        for h in range(H):
            sc = (qd[z, h].float() @ kd[z, h].float().t()) * scale
            if causal:
                sc = sc.masked_fill(~keep, float("-inf"))
            lse2 = torch.logsumexp(sc, dim=-1) * 1.4426950408889634
            worst = max(worst, float((m[z, h] - lse2).abs().max()))
    assert worst <= 1e-3, f"M differs from logsumexp * log2(e) by {worst}"
    # rows of softmax sum to one: with V = 1 the output is exactly 1 (l normalisation)
    ones = torch.ones_like(v[:1, :2]).cuda()
    o1 = ops.attention(q[:1, :2].cuda(), k[:1, :2].cuda(), ones, causal, D ** -0.5)
    assert float((o1.float() - 1).abs().max()) <= 2 ** -7


@pytest.mark.parametrize("Z,H,S,causal", [(1, 2, 512, False), (1, 3, 1024, True), (2, 2, 2048, True), (1, 5, 1536, False)])
def test_attention_cta_pair_kernel_is_bit_identical(monkeypatch, Z, H, S, causal):
    # the alternative kernel on CTA pairs (cta_group::2, four Q tiles per pair; selected with B200K_ATTN_2CTA=1 for
    # HEAD_DIM 128 and N_CTX a multiple of 512): same arithmetic per row, so the same bits for O and M
    D = 128
    q, k, v = (t.cuda() for t in gi.attn_inputs(Z, H, S, D, seed=29))
    monkeypatch.delenv("B200K_ATTN_2CTA", raising=False)
    o1, m1 = ops.attention_with_lse(q, k, v, causal, D ** -0.5)
    lib = _lib.load()
    before = lib.b200k_launch_count()
    monkeypatch.setenv("B200K_ATTN_2CTA", "1")
    o2, m2 = ops.attention_with_lse(q, k, v, causal, D ** -0.5)
    torch.cuda.synchronize()
    assert lib.b200k_launch_count() - before == 1
    assert torch.equal(o1.view(torch.int16), o2.view(torch.int16)) and torch.equal(m1.view(torch.int32), m2.view(torch.int32))
    assert ops.device_status() == 0


@pytest.mark.parametrize("Z,H,S,D,causal", [(1, 2, 100, 128, False), (2, 3, 100, 128, True), (1, 2, 333, 128, False),
                                            (1, 3, 333, 64, True), (1, 2, 1, 128, True), (1, 1, 129, 256, False),
                                            (2, 2, 200, 32, True), (1, 2, 1000, 128, False), (1, 2, 1000, 128, True)])
def test_attention_ragged_sequence_lengths(Z, H, S, D, causal):
    # N_CTX that is not a multiple of the 128-row tiles: the last tile's rows past N_CTX are not stored and the last
    # block's keys past N_CTX are masked.  O sits between canaries inside one buffer, M likewise.
    q, k, v = gi.attn_inputs(Z, H, S, D, seed=31)
    blk = 1
    for b in (128, 64, 32, 25, 16, 9, 8, 4, 3, 2):       # an oracle block size that divides N_CTX (and <= HEAD_DIM)
        if S % b == 0 and b <= D:
            blk = b
            break
    ref_o, ref_m = oracle.attention(q, k, v, causal, D ** -0.5, BLOCK_M=blk, BLOCK_N=blk)
    lib = _lib.load()
    n = q.numel()
    obuf = torch.full((n + 512,), -7.0, dtype=torch.bfloat16, device="cuda")
    mbuf = torch.full((Z * H * S + 64,), -7.0, dtype=torch.float32, device="cuda")
    o = obuf[256:256 + n].view(Z, H, S, D)
    m = mbuf[32:32 + Z * H * S].view(Z, H, S)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    _lib.check(lib.b200k_attn_fwd_bf16(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), m.data_ptr(), Z, H, S, D,
                                       int(causal), D ** -0.5, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert float((o.cpu().float() - ref_o.float()).abs().max()) <= ATTN_MAX_ABS
    assert float((m.cpu() - ref_m).abs().max()) <= 1e-4
    assert bool((obuf[:256] == -7.0).all()) and bool((obuf[256 + n:] == -7.0).all())
    assert bool((mbuf[:32] == -7.0).all()) and bool((mbuf[32 + Z * H * S:] == -7.0).all())
    assert ops.device_status() == 0


# ------------------------------------------------------------------------------------------------ attention backward
def _d_o(Z, H, S, D, seed=33):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(Z, H, S, D, generator=g, dtype=torch.float32).bfloat16()


def _autograd_truth(q, k, v, d_o, causal, scale):
    """fp32 automatic differentiation of the attention definition, on the GPU."""
    qf, kf, vf = (t.cuda().float().requires_grad_(True) for t in (q, k, v))
    sc = (qf @ kf.transpose(-1, -2)) * scale
    if causal:
        S = q.shape[-2]
        sc = sc.masked_fill(~torch.ones(S, S, dtype=torch.bool, device="cuda").tril(), float("-inf"))
    (torch.softmax(sc, dim=-1) @ vf).backward(d_o.cuda().float())
    return qf.grad, kf.grad, vf.grad


@pytest.mark.parametrize("Z,H,S,causal,D", [(1, 1, 128, False, 128), (1, 1, 128, True, 128), (1, 2, 256, False, 128),
                                            (1, 3, 512, True, 128), (2, 2, 1024, False, 128), (1, 2, 1024, True, 128),
                                            (3, 5, 384, True, 128), (1, 1, 128, True, 64), (2, 3, 512, False, 64),
                                            (1, 4, 1024, True, 64), (3, 5, 384, True, 64),
                                            # N_CTX not a multiple of 128 (3-D tensor maps, zero-filled tails)
                                            (1, 2, 200, False, 128), (2, 3, 333, True, 128), (1, 2, 96, True, 64),
                                            (1, 1, 1000, False, 64), (2, 2, 129, True, 128), (1, 1, 7, False, 128)])
def test_attention_backward_oracle(Z, H, S, causal, D):
    # dq, dk, dv against the CPU oracle (parity unpinned: the reference has no backward) and against fp32 autograd
    scale = D ** -0.5
    q, k, v = gi.attn_inputs(Z, H, S, D, seed=32)
    d_o = _d_o(Z, H, S, D)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    o, m = ops.attention_with_lse(qd, kd, vd, causal, scale)
    lib = _lib.load()
    before = lib.b200k_launch_count()
    dq, dk, dv = ops.attention_backward(qd, kd, vd, o, m, d_o.cuda(), causal, scale)
    torch.cuda.synchronize()
    assert lib.b200k_launch_count() - before == 3            # delta, dK/dV, dQ
    ref = oracle.attention_backward(q, k, v, o.cpu(), d_o, m.cpu(), causal, scale)
    truth = _autograd_truth(q, k, v, d_o, causal, scale)
    for name, got, r, t in zip(("dq", "dk", "dv"), (dq, dk, dv), ref, truth):
        assert not torch.isnan(got.float()).any(), name
        assert oracle.rel_frobenius(got.cpu().float(), r.float()) <= 1e-2, name
        assert float((got.cpu().float() - r.float()).abs().max()) <= 3e-2, name
        assert float((got.float() - t).norm() / t.norm()) <= 1e-2, name
    assert ops.device_status() == 0


def test_attention_backward_through_autograd_and_determinism():
    # ops.attention is differentiable (the reference's _attention function with the backward it lacks); two runs give
    # the same bits (no atomics anywhere)
    Z, H, S, D = 1, 4, 512, 128
    q, k, v = (t.cuda().requires_grad_(True) for t in gi.attn_inputs(Z, H, S, D, seed=34))
    d_o = _d_o(Z, H, S, D).cuda()
    grads = []
    for _ in range(2):
        o = ops.attention(q, k, v, True, D ** -0.5)
        gq, gk, gv = torch.autograd.grad(o, (q, k, v), d_o)
        grads.append((gq, gk, gv))
    for a, b in zip(*grads):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    truth = _autograd_truth(q.detach().cpu(), k.detach().cpu(), v.detach().cpu(), d_o.cpu(), True, D ** -0.5)
    for got, t in zip(grads[0], truth):
        assert float((got.float() - t).norm() / t.norm()) <= 1e-2


@pytest.mark.parametrize("causal", [False, True])
def test_attention_backward_full_size_heads(causal):
    # the full workload on the GPU; three (batch, head) pairs against fp32 autograd
    Z, H, S, D = 4, 32, 4096, 128
    scale = D ** -0.5
    q, k, v = (t.cuda() for t in gi.attn_inputs(Z, H, S, D, seed=35))
    d_o = _d_o(Z, H, S, D).cuda()
    o, m = ops.attention_with_lse(q, k, v, causal, scale)
    dq, dk, dv = ops.attention_backward(q, k, v, o, m, d_o, causal, scale)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    for (z, h) in ((0, 0), (2, 13), (3, 31)):
        sl = (slice(z, z + 1), slice(h, h + 1))
        truth = _autograd_truth(q[sl].cpu(), k[sl].cpu(), v[sl].cpu(), d_o[sl].cpu(), causal, scale)
        for name, got, t in zip(("dq", "dk", "dv"), (dq, dk, dv), truth):
            assert float((got[sl].float() - t).norm() / t.norm()) <= 1e-2, (name, z, h)


@pytest.mark.parametrize("S,D", [(256, 128), (200, 128), (333, 64)])
def test_attention_backward_cabi_writes_only_its_outputs(S, D):
    # straight through the C-ABI with dq, dk, dv inside canary-filled buffers: every element written, nothing around them
    # (the ragged lengths end inside a 128-row block of the last head: the rows past the end must not be stored)
    Z, H = 2, 3
    scale = D ** -0.5
    q, k, v = (t.cuda() for t in gi.attn_inputs(Z, H, S, D, seed=36))
    d_o = _d_o(Z, H, S, D).cuda()
    o, m = ops.attention_with_lse(q, k, v, True, scale)
    pad, n = 2048, q.numel()
    bufs = [torch.full((n + 2 * pad,), -3.0, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    outs = [b[pad:pad + n].view(Z, H, S, D) for b in bufs]
    for t in outs:
        t.fill_(float("nan"))
    delta = torch.empty(Z, H, S, device="cuda")
    lib = _lib.load()
    _lib.check(lib.b200k_attn_bwd_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), m.data_ptr(),
                                       outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), delta.data_ptr(),
                                       Z, H, S, D, 1, scale, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    want = ops.attention_backward(q, k, v, o, m, d_o, True, scale)
    for b, got, w in zip(bufs, outs, want):
        assert not torch.isnan(got.float()).any()
        assert torch.equal(got.view(torch.int16), w.view(torch.int16))
        assert bool((b[:pad] == -3.0).all()) and bool((b[pad + n:] == -3.0).all())
    # delta = rowsum(o * dO) in fp32
    ref_delta = (o.float() * d_o.float()).sum(-1)
    assert float((delta - ref_delta).abs().max()) <= 1e-4 * float(ref_delta.abs().max()) + 1e-5


def test_attention_backward_in_a_cuda_graph():
    # forward + backward recorded once and replayed on new data: neither allocates inside the library nor synchronises
    Z, H, S, D = 1, 2, 384, 128
    scale = D ** -0.5
    q, k, v = (t.cuda() for t in gi.attn_inputs(Z, H, S, D, seed=37))
    d_o = _d_o(Z, H, S, D, seed=38).cuda()

    def step():
        o, m = ops.attention_with_lse(q, k, v, True, scale)
        return ops.attention_backward(q, k, v, o, m, d_o, True, scale)

    want1 = [t.clone() for t in step()]
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = step()
    graph.replay()
    torch.cuda.synchronize()
    for got, want in zip(outs, want1):
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    q2, k2, v2 = gi.attn_inputs(Z, H, S, D, seed=39)
    for dst, src in ((q, q2), (k, k2), (v, v2), (d_o, _d_o(Z, H, S, D, seed=40))):
        dst.copy_(src)
    graph.replay()
    torch.cuda.synchronize()
    got2 = [t.clone() for t in outs]
    want2 = step()
    torch.cuda.synchronize()
    for got, want in zip(got2, want2):
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    assert ops.device_status() == 0


@pytest.mark.parametrize("S,D,causal", [(4096, 128, False), (4096, 64, True), (1000, 128, True)])
def test_attention_backward_repeats_bit_for_bit(S, D, causal):
    # no atomics and no order-dependent reduction anywhere: five runs at the workload's size give the same bits (a race
    # between the score warps and the MMAs over the shared tensor-memory columns would show up here)
    Z, H = 4, 32
    scale = D ** -0.5
    g = torch.Generator(device="cuda").manual_seed(61)
    q, k, v, d_o = (torch.randn(Z, H, S, D, device="cuda", generator=g).bfloat16() for _ in range(4))
    o, m = ops.attention_with_lse(q, k, v, causal, scale)
    first = ops.attention_backward(q, k, v, o, m, d_o, causal, scale)
    for _ in range(4):
        again = ops.attention_backward(q, k, v, o, m, d_o, causal, scale)
        for a, b in zip(first, again):
            assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    for t in first:
        assert bool(torch.isfinite(t.float()).all())
    assert ops.device_status() == 0


def _random_attention_shapes(n, seed, dims):
    rng = np.random.RandomState(seed)
    shapes = []
    for _ in range(n):
        shapes.append((int(rng.randint(1, 3)), int(rng.randint(1, 5)), int(rng.randint(1, 700)), int(rng.choice(dims)),
                       bool(rng.randint(0, 2))))
    return shapes


@pytest.mark.parametrize("Z,H,S,D,causal", _random_attention_shapes(24, 71, (64, 128)))
def test_attention_forward_and_backward_random_shapes(Z, H, S, D, causal):
    # seeded random (Z, H, N_CTX, HEAD_DIM, causal): lengths that end anywhere inside a block, single-block heads, more
    # and fewer items than SMs; forward and backward against the CPU oracle
    scale = D ** -0.5
    q, k, v = gi.attn_inputs(Z, H, S, D, seed=72)
    d_o = _d_o(Z, H, S, D, seed=73)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    o, m = ops.attention_with_lse(qd, kd, vd, causal, scale)
    blk = 1
    for b in (128, 64, 32, 25, 16, 9, 8, 4, 3, 2):       # an oracle block size that divides N_CTX (the reference walks
        if S % b == 0 and b <= D:                        # whole blocks: it has no keys past N_CTX only then)
            blk = b
            break
    ro, rm = oracle.attention(q, k, v, causal, scale, BLOCK_M=blk, BLOCK_N=blk)
    assert float((o.cpu().float() - ro.float()).abs().max()) <= ATTN_MAX_ABS
    assert float((m.cpu() - rm).abs().max()) <= 1e-3
    grads = ops.attention_backward(qd, kd, vd, o, m, d_o.cuda(), causal, scale)
    ref = oracle.attention_backward(q, k, v, o.cpu(), d_o, m.cpu(), causal, scale)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    for name, got, want in zip(("dq", "dk", "dv"), grads, ref):
        assert bool(torch.isfinite(got.float()).all()), name
        diff = (got.cpu().float() - want.float())
        assert float(diff.norm()) <= 1e-2 * float(want.float().norm()) + 1e-3, name
        assert float(diff.abs().max()) <= 3e-2, name


def test_attention_backward_single_key():
    # N_CTX = 1: the softmax of one score is 1 whatever q and k are, so dv = dO and dq = dk = 0 (up to the rounding
    # difference between the MMA's dO.V and the delta kernel's O.dO)
    Z, H, D = 2, 3, 128
    q, k, v = (t.cuda() for t in gi.attn_inputs(Z, H, 1, D, seed=45))
    d_o = _d_o(Z, H, 1, D, seed=46).cuda()
    o, m = ops.attention_with_lse(q, k, v, False, D ** -0.5)
    dq, dk, dv = ops.attention_backward(q, k, v, o, m, d_o, False, D ** -0.5)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(dv.view(torch.int16), d_o.view(torch.int16))
    assert float(dq.float().abs().max()) <= 1e-4 and float(dk.float().abs().max()) <= 1e-4


def test_attention_backward_rejects_unsupported():
    q = torch.zeros(1, 1, 256, 32, dtype=torch.bfloat16, device="cuda")
    m = torch.zeros(1, 1, 256, device="cuda")
    with pytest.raises(NotImplementedError):
        ops.attention_backward(q, q, q, q, m, q, False, 0.1)          # HEAD_DIM 32
    q = torch.zeros(1, 1, 192, 256, dtype=torch.bfloat16, device="cuda")
    m = torch.zeros(1, 1, 192, device="cuda")
    with pytest.raises(NotImplementedError):
        ops.attention_backward(q, q, q, q, m, q, False, 0.1)          # HEAD_DIM 256


def test_attention_rejects_unsupported():
    q48 = torch.zeros(1, 1, 128, 48, dtype=torch.bfloat16, device="cuda")       # not in {16, 32, 64, 128, 256}
    with pytest.raises(AssertionError):
        ops.attention(q48, q48, q48, False, 0.1)
    lib = _lib.load()
    rc = lib.b200k_attn_fwd_bf16(q48.data_ptr(), q48.data_ptr(), q48.data_ptr(), q48.data_ptr(), q48.data_ptr(), 1, 1, 128,
                                 48, 0, 0.1, None)
    assert rc == _lib.ERR_UNSUPPORTED


@pytest.mark.parametrize("Z,H,S,causal", [(1, 2, 128, True), (2, 3, 512, False), (1, 4, 1024, True), (1, 1, 384, False)])
def test_attention_head_dim_64(Z, H, S, causal):
    D = 64
    q, k, v = gi.attn_inputs(Z, H, S, D, seed=24)
    ref_o, ref_m = oracle.attention(q, k, v, causal, D ** -0.5, BLOCK_M=128, BLOCK_N=64)   # BLOCK_N <= HEAD_DIM
    o, m = ops.attention_with_lse(q.cuda(), k.cuda(), v.cuda(), causal, D ** -0.5)
    assert float((o.cpu().float() - ref_o.float()).abs().max()) <= ATTN_MAX_ABS
    assert float((m.cpu() - ref_m).abs().max()) <= 1e-4


@pytest.mark.parametrize("D,Z,H,S,causal", [(16, 1, 2, 128, True), (16, 2, 3, 640, False), (32, 1, 3, 384, True),
                                            (32, 1, 2, 1024, False), (256, 1, 2, 128, True), (256, 1, 3, 384, True),
                                            (256, 2, 2, 512, False)])
def test_attention_other_head_dims(D, Z, H, S, causal):
    # the reference's remaining head dimensions (06-fused-attention.py:233): 16 and 32 (box rows narrower than the
    # swizzle span), 256 (one Q tile per CTA); BLOCK_N <= HEAD_DIM in the oracle as the reference asserts (:158)
    q, k, v = gi.attn_inputs(Z, H, S, D, seed=27)
    ref_o, ref_m = oracle.attention(q, k, v, causal, D ** -0.5, BLOCK_M=128, BLOCK_N=min(D, 128))
    o, m = ops.attention_with_lse(q.cuda(), k.cuda(), v.cuda(), causal, D ** -0.5)
    assert float((o.cpu().float() - ref_o.float()).abs().max()) <= ATTN_MAX_ABS
    assert float((m.cpu() - ref_m).abs().max()) <= 1e-4


# ------------------------------------------------------------------------------------------------ launch surface
def test_kernel_grid_launch_surface():
    n = 98432
    x, y = gi.add_inputs(n)
    xd, yd = x.cuda(), y.cuda()
    out = torch.empty_like(xd)
    grid = lambda meta: ((n + meta["BLOCK_SIZE"] - 1) // meta["BLOCK_SIZE"],)
    kernels.add_kernel[grid](xd, yd, out, n, BLOCK_SIZE=1024)
    assert _bits_equal(out.cpu(), oracle.add(x, y))
    kernels.sin_kernel[grid](xd, out, n, BLOCK_SIZE=1024)
    assert oracle.ulp_diff_f32(out.cpu(), oracle.sin_correctly_rounded(x)) <= SIN_MAX_ULP

    M, N, K = 256, 512, 192
    a, b, bias = gi.fused_inputs(M, N, K, seed=31)
    ad, bd, biasd = a.cuda(), b.cuda(), bias.cuda()
    c = torch.full((M, N), 7.5, device="cuda", dtype=torch.bfloat16)
    descs = [TensorDescriptor.from_tensor(t, [32, 32]) for t in (ad, bd, c)]
    mgrid = lambda META: (-(-M // META["BLOCK_SIZE_M"]) * -(-N // META["BLOCK_SIZE_N"]),)
    kernels.matmul_kernel_tma[mgrid](*descs, M, N, K, FP8_OUTPUT=False, WARP_SPECIALIZE=True)
    assert oracle.rel_frobenius(c.cpu().float(), oracle.golden_matmul(a, b).float()) <= MATMUL_REL_FRO
    kernels.matmul_kernel_fused[mgrid](*descs, TensorDescriptor.from_tensor(biasd, [32, 32]), M, N, K,
                                       FP8_OUTPUT=False, WARP_SPECIALIZE=True)
    assert oracle.rel_frobenius(c.cpu().float(), oracle.golden_matmul(a, b, bias=bias, mode=2).float()) <= MATMUL_REL_FRO

    Z, H, S, D = 1, 2, 256, 128
    q, k, v = gi.attn_inputs(Z, H, S, D, seed=32)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    o = torch.empty_like(qd)
    Mt = torch.empty((Z, H, S), device="cuda", dtype=torch.float32)
    ydim = Z * H * S
    dq, dk, dv, do = (TensorDescriptor(t, shape=[ydim, D], strides=[D, 1], block_shape=[1, 1]) for t in (qd, kd, vd, o))
    agrid = lambda META: (-(-S // META["BLOCK_M"]), Z * H, 1)
    kernels._attn_fwd[agrid](D ** -0.5, Mt, Z, H, dq, dk, dv, do, N_CTX=S, HEAD_DIM=D, FP8_OUTPUT=False, STAGE=3,
                             warp_specialize=True, IS_HOPPER=False)
    ref_o, ref_m = oracle.attention(q, k, v, True, D ** -0.5)
    assert float((o.cpu().float() - ref_o.float()).abs().max()) <= ATTN_MAX_ABS
    assert float((Mt.cpu() - ref_m).abs().max()) <= 1e-4


def test_host_tensor_round_trip():
    # host buffers in, host result out: what the reference's launcher does on every launch
    x, y = gi.add_inputs(98432)
    out = ops.add(x, y)
    assert not out.is_cuda and _bits_equal(out, oracle.add(x, y))
    a, b = gi.matmul_inputs(256, 256, 256)
    c = ops.matmul_tma(a, b, True)
    assert not c.is_cuda and oracle.rel_frobenius(c.float(), oracle.golden_matmul(a, b).float()) <= MATMUL_REL_FRO


def test_host_tensor_pipeline_matches_device_path():
    # large host operands go through the row-block pipeline (upload / multiply / download overlapped);
    # the result must be bit-identical to the plain device path
    M, N, K = 4096 + 384, 1288, 520                      # ragged last block, N and K tails
    a, b = gi.matmul_inputs(M, N, K, seed=41)
    bias = gi.row_bias(N)
    ref = ops.matmul_tma(a.cuda(), b.cuda(), True).cpu()
    got = ops.matmul_tma(a.pin_memory(), b.pin_memory(), True)
    assert not got.is_cuda and torch.equal(got.view(torch.int16), ref.view(torch.int16))
    got2 = ops.matmul_tma(a, b, True, out=torch.empty((M, N), dtype=torch.bfloat16).pin_memory())   # pageable inputs
    assert torch.equal(got2.view(torch.int16), ref.view(torch.int16))
    reff = ops.matmul_fused(a.cuda(), b.cuda(), bias.cuda(), "relu").cpu()
    gotf = ops.matmul_fused(a, b, bias, "relu")
    assert torch.equal(gotf.view(torch.int16), reff.view(torch.int16))
    assert oracle.rel_frobenius(got[:64].float(), oracle.golden_matmul(a[:64], b).float()) <= MATMUL_REL_FRO


def test_bounded_wait_gives_up_and_context_survives():
    # a wait that can never be satisfied runs out of its (tiny) budget: status word set, kernel returns,
    # and the device keeps working
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    assert ops.device_status() == 0
    _lib.check(lib.b200k_selftest_wait_timeout(2_000_000, stream))       # about a millisecond
    code = ctypes.c_uint32(0)
    rc = lib.b200k_device_status(stream, ctypes.byref(code))
    assert rc == _lib.ERR_DEVICE_TIMEOUT and code.value >> 8 == 99 and "site 99" in _lib.last_error()
    assert ops.device_status() == 0                                      # reading the status cleared it
    x, y = gi.add_inputs(4096)
    assert _bits_equal(ops.add(x.cuda(), y.cuda()).cpu(), oracle.add(x, y))
    a, b = gi.matmul_inputs(256, 256, 256)
    assert oracle.rel_frobenius(ops.matmul_tma(a.cuda(), b.cuda()).cpu().float(), oracle.golden_matmul(a, b).float()) <= MATMUL_REL_FRO
    with pytest.raises(_lib.B200KError):
        _lib.check(lib.b200k_selftest_wait_timeout(0, stream))


def test_launch_counter_counts_kernels():
    lib = _lib.load()
    before = lib.b200k_launch_count()
    x = torch.zeros(4096, device="cuda")
    ops.add(x, x)
    assert lib.b200k_launch_count() == before + 1
    props = _lib.Props()
    _lib.check(lib.b200k_device_props(0, ctypes.byref(props)))
    assert props.cc_major == 10 and props.multiprocessor_count >= 100
