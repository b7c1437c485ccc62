"""Host-side mirror of the reference interface: argument flattening, kernel[grid] binding,
descriptors, partition helpers.  No GPU needed (a recording launcher stands in for the C-ABI call)."""
import pytest
import torch

from oracle import cpu_oracle as oracle
from triton_tenstorrent_b200 import _lib, driver, kernels, sharding
from triton_tenstorrent_b200.tensor_descriptor import TensorDescriptor


class FakeCudaTensor(torch.Tensor):
    """A host tensor that claims to be on the GPU, to drive the launch surface without one."""
    @property
    def is_cuda(self):
        return True


def fake(t):
    return t.as_subclass(FakeCudaTensor)


class RecordingLauncher:
    calls = []

    def __init__(self, src, metadata):
        self.signature = dict(src.signature)

    def __call__(self, gx, gy, gz, stream, function, *args):
        RecordingLauncher.calls.append(dict(grid=(gx, gy, gz), function=function, metadata=args[0],
                                            flat=driver.flatten_args(self.signature, args[4:])))


@pytest.fixture
def recording(monkeypatch):
    RecordingLauncher.calls = []
    monkeypatch.setattr(driver.active, "launcher_cls", RecordingLauncher)
    monkeypatch.setattr(driver.active, "get_current_stream", lambda device_id=None: 0)
    for k in (kernels.add_kernel, kernels.add_kernel_loop, kernels.sin_kernel, kernels.matmul_kernel_tma, kernels.matmul_kernel_fused,
              kernels.matmul_kernel, kernels._attn_fwd, kernels.memcpy_kernel, kernels.copy_scalar_kernel):
        monkeypatch.setattr(k, "launcher", None)
    return RecordingLauncher.calls


def test_add_kernel_launch_surface(recording):
    n = 98432
    x, y, out = (fake(torch.zeros(n)) for _ in range(3))
    grid = lambda meta: ((n + meta["BLOCK_SIZE"] - 1) // meta["BLOCK_SIZE"],)
    kernels.add_kernel[grid](x, y, out, n, BLOCK_SIZE=1024)
    call = recording[0]
    assert call["grid"] == (97, 1, 1)                      # 98432 = 96*1024 + 128
    assert call["function"] == "add_kernel:BLOCK_SIZE=1024"
    assert call["metadata"] == (1, 1, 0, 1, 1, 1)          # num_warps, num_ctas, shared, cluster dims
    kinds = [k for k, _ in call["flat"]]
    assert kinds == [_lib.ARG_PTR] * 3 + [_lib.ARG_I32]    # the constexpr BLOCK_SIZE is dropped
    assert call["flat"][3][1] == n
    assert [v for _, v in call["flat"][:3]] == [x.data_ptr(), y.data_ptr(), out.data_ptr()]


def test_memcpy_kernel_launch_surface(recording):
    # memcpy_kernel[grid](input, output, xnumel, XBLOCK, num_warps=1) and copy_scalar_kernel[(1,)](input, output, num_warps=1),
    # python/tutorials/gluon/01-intro.py:96-99 and :60-63
    n = 500
    x, out = fake(torch.zeros(n)), fake(torch.zeros(n))
    kernels.memcpy_kernel[((n + 63) // 64,)](x, out, n, 64, num_warps=1)
    call = recording[0]
    assert call["grid"] == (8, 1, 1) and call["function"] == "memcpy_kernel:XBLOCK=64"
    assert [k for k, _ in call["flat"]] == [_lib.ARG_PTR, _lib.ARG_PTR, _lib.ARG_I32]      # the constexpr XBLOCK is dropped
    assert [v for _, v in call["flat"]] == [x.data_ptr(), out.data_ptr(), n]
    kernels.copy_scalar_kernel[(1,)](x, out, num_warps=1)
    call = recording[1]
    assert call["grid"] == (1, 1, 1) and call["function"] == "copy_scalar_kernel"
    assert [k for k, _ in call["flat"]] == [_lib.ARG_PTR, _lib.ARG_PTR]


def test_add_kernel_loop_launch_surface(recording):
    # add_kernel[grid](x, y, output, n_elements, row_count, BLOCK_SIZE=..., num_warps=1), 01-vector-add.loop.py:89
    n = 300000
    x, y, out = (fake(torch.zeros(n, dtype=torch.bfloat16)) for _ in range(3))
    n_cores, block = 130, 1024
    n_rows = -(-n // block)
    row_count = -(-n_rows // n_cores)
    kernels.add_kernel_loop[lambda meta: (n_cores,)](x, y, out, n, row_count, BLOCK_SIZE=block, num_warps=1)
    call = recording[0]
    assert call["grid"] == (130, 1, 1) and row_count == 3
    assert call["function"] == "add_kernel:BLOCK_SIZE=1024,BF16=1"
    assert [k for k, _ in call["flat"]] == [_lib.ARG_PTR] * 3 + [_lib.ARG_I32] * 2
    assert [v for _, v in call["flat"][3:]] == [n, row_count]
    with pytest.raises(TypeError):
        kernels.add_kernel_loop[(1,)](x, y, fake(torch.zeros(n)), n, row_count, BLOCK_SIZE=block)   # mixed dtypes


def test_descriptor_flattening_matches_reference_order(recording):
    M, N, K = 256, 512, 128
    a, b, c = fake(torch.zeros(M, K, dtype=torch.bfloat16)), fake(torch.zeros(K, N, dtype=torch.bfloat16)), fake(torch.zeros(M, N, dtype=torch.bfloat16))
    descs = [TensorDescriptor.from_tensor(t, [32, 32]) for t in (a, b, c)]
    grid = lambda META: (-(-M // META["BLOCK_SIZE_M"]) * -(-N // META["BLOCK_SIZE_N"]),)
    kernels.matmul_kernel_tma[grid](*descs, M, N, K, FP8_OUTPUT=False, WARP_SPECIALIZE=True)
    call = recording[0]
    assert call["grid"] == (2 * 2, 1, 1)
    flat = call["flat"]
    assert len(flat) == 3 * 10 + 3
    # base, shape.., strides.., padding, shape.., strides..   (backend/driver.py:141-159)
    first = [v for _, v in flat[:10]]
    assert first == [a.data_ptr(), M, K, K, 1, 0, M, K, K, 1]
    assert [v for _, v in flat[-3:]] == [M, N, K]


def test_pointer_matmul_kernel_launch_surface(recording):
    # matmul_kernel[grid](a, b, c, M, N, K, 6 strides, ACTIVATION=...), examples/matmul/03-matrix-multiplication.py:413-420
    M, N, K = 256, 512, 128
    a, b, c = (fake(torch.zeros(s, dtype=torch.float16)) for s in ((M, K), (K, N), (M, N)))
    grid = lambda META: (-(-M // META["BLOCK_SIZE_M"]) * -(-N // META["BLOCK_SIZE_N"]),)
    kernels.matmul_kernel[grid](a, b, c, M, N, K, a.stride(0), a.stride(1), b.stride(0), b.stride(1), c.stride(0),
                                c.stride(1), ACTIVATION="leaky_relu")
    call = recording[0]
    assert call["function"] == "matmul_kernel:BLOCK_SIZE_M=128,BLOCK_SIZE_N=256,ACTIVATION=2,F16=1,TILE32=0"
    assert [k for k, _ in call["flat"]] == [_lib.ARG_PTR] * 3 + [_lib.ARG_I32] * 9   # constexprs are dropped
    assert [v for _, v in call["flat"][3:]] == [M, N, K, K, 1, N, 1, N, 1]
    kernels.matmul_kernel[grid](a, b, c, M, N, K, a.stride(0), a.stride(1), b.stride(0), b.stride(1), c.stride(0),
                                c.stride(1), ACTIVATION="", LAYOUT="tile32")
    assert recording[1]["function"].endswith("ACTIVATION=0,F16=1,TILE32=1")
    with pytest.raises(ValueError):
        kernels.matmul_kernel[grid](a, b, c, M, N, K, K, 1, N, 1, N, 1, ACTIVATION="gelu")
    with pytest.raises(ValueError):
        kernels.matmul_kernel[grid](a, b, c, M, N, K, K, 1, N, 1, N, 1, LAYOUT="tile64")


def test_tilize_round_trip_and_addressing():
    # element (r, c) of the logical matrix sits at ((r/32)*(S/32) + c/32)*1024 + (r%32)*32 + c%32
    # (examples/matmul/03-matrix-multiplication.py:333-344)
    from triton_tenstorrent_b200 import ops
    R, S = 96, 160
    t = torch.arange(R * S, dtype=torch.float32).reshape(R, S)
    tiled = ops.tilize(t)
    flat = tiled.reshape(-1)
    for (r, c) in ((0, 0), (31, 31), (32, 0), (5, 47), (95, 159), (64, 33)):
        off = ((r // 32) * (S // 32) + c // 32) * 1024 + (r % 32) * 32 + c % 32
        assert flat[off] == t[r, c]
    assert torch.equal(ops.untilize(tiled), t)
    assert torch.equal(tiled, oracle.tilize(t))
    with pytest.raises(ValueError):
        ops.tilize(torch.zeros(40, 64))


def test_attention_launch_surface(recording):
    Z, H, S, D = 2, 3, 256, 128
    q = fake(torch.zeros(Z, H, S, D, dtype=torch.bfloat16))
    Mt = fake(torch.zeros(Z, H, S))
    y = Z * H * S
    d = [TensorDescriptor(q, shape=[y, D], strides=[D, 1], block_shape=[1, 1]) for _ in range(4)]
    grid = lambda META: (-(-S // META["BLOCK_M"]), Z * H, 1)
    kernels._attn_fwd[grid](0.5, Mt, Z, H, *d, N_CTX=S, HEAD_DIM=D, FP8_OUTPUT=False, STAGE=3, warp_specialize=True,
                            IS_HOPPER=False)
    call = recording[0]
    assert call["grid"] == (2, 6, 1)
    assert call["function"] == "_attn_fwd:STAGE=3,BLOCK_M=128"   # the grid is checked against BLOCK_M
    kinds = [k for k, _ in call["flat"]]
    assert kinds[0] == _lib.ARG_F32 and kinds[1] == _lib.ARG_PTR and len(kinds) == 4 + 40 + 1
    assert call["flat"][-1][1] == S


def test_kernel_argument_errors(recording):
    x = fake(torch.zeros(8))
    with pytest.raises(TypeError):
        kernels.add_kernel[(1,)](x, x, x, 8)                       # BLOCK_SIZE missing
    with pytest.raises(TypeError):
        kernels.add_kernel[(1,)](x, x, x, 8, BLOCK_SIZE=8, bogus=1)
    with pytest.raises(ValueError):
        kernels.add_kernel[(1,)](torch.zeros(8), x, x, 8, BLOCK_SIZE=8)  # host tensor
    kernels.add_kernel[(1,)](x, x, x, 8, BLOCK_SIZE=8, num_warps=4, num_stages=2)  # accepted and ignored
    assert len(recording) == 1


def test_tensor_descriptor_checks():
    t = torch.zeros(64, 24, dtype=torch.bfloat16)
    d = TensorDescriptor.from_tensor(t, [32, 32])
    assert d.shape == [64, 24] and d.strides == [24, 1] and d.padding == "zero"
    with pytest.raises(AssertionError):
        TensorDescriptor.from_tensor(torch.zeros(64, 20, dtype=torch.bfloat16), [32, 32])  # 40-byte rows
    with pytest.raises(AssertionError):
        TensorDescriptor(t, [64, 24], [1, 64], [32, 32])                                    # inner stride != 1


def test_load_binary_and_target():
    u = driver.B200Utils()
    mod, fn, n_regs, n_spills, max_threads = u.load_binary("matmul_kernel_tma", b"", 0, 0)
    assert fn == "matmul_kernel_tma"
    with pytest.raises(KeyError):
        u.load_binary("not_a_kernel", b"", 0, 0)
    assert driver.active.get_current_target() == ("cuda", 100, 32)
    assert driver.pack_metadata(4, 1, 1024) == (4, 1, 1024, 1, 1, 1)


@pytest.mark.parametrize("nb,workers", [(97, 8), (5, 8), (2048, 148), (0, 3), (16, 16)])
def test_block_range_matches_oracle_and_covers(nb, workers):
    covered = []
    for w in range(workers):
        r = sharding.block_range(nb, workers, w)
        assert r == oracle.block_range(nb, workers, w)
        covered.extend(range(*r))
    assert covered == list(range(nb))


def test_row_and_head_shards():
    assert [sharding.row_shard(8192, 8, r) for r in range(8)] == [(1024 * r, 1024 * (r + 1)) for r in range(8)]
    spans = [sharding.row_shard(1000, 3, r) for r in range(3)]      # 8 tiles of 128 rows -> 3,3,2 tiles
    assert spans == [(0, 384), (384, 768), (768, 1000)]
    assert [sharding.head_shard(128, 8, r) for r in (0, 7)] == [(0, 16), (112, 128)]


def test_ops_fail_loudly_without_cuda():
    from triton_tenstorrent_b200 import ops
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(Exception):
        ops.add(torch.zeros(8), torch.zeros(8))


@pytest.mark.parametrize("ZH,S,D,ctas", [(128, 4096, 128, 148), (3, 384, 128, 148), (16, 2048, 256, 148), (40, 8192, 64, 132),
                                         (1, 128, 128, 148)])
def test_causal_attention_schedule_covers_and_balances(ZH, S, D, ctas):
    # every (head, row pair) item exactly once; per-CTA work (K/V blocks + 1 per item) within one longest item of the mean
    import ctypes
    lib = _lib.load()
    ntile = 2 if D <= 128 else 1
    mblk = S // 128
    pairs = -(-mblk // ntile)
    items = ZH * pairs
    ctas = min(ctas, items)
    cap = (items + ctas) * 2
    table = (ctypes.c_int * cap)()
    rounds = ctypes.c_int()
    assert lib.b200k_attn_causal_schedule(ZH, S, D, ctas, table, cap, ctypes.byref(rounds)) == _lib.OK
    t = [table[i] for i in range(rounds.value * ctas)]
    seen = sorted(x for x in t if x >= 0)
    assert seen == list(range(items))

    def blocks(item):
        pr = pairs - 1 - item % pairs
        m0, m1 = ntile * pr, ntile * pr + 1
        return max(m0 + 1, m1 + 1 if (ntile == 2 and m1 < mblk) else 0) + 1

    load = [sum(blocks(t[k * ctas + c]) for k in range(rounds.value) if t[k * ctas + c] >= 0) for c in range(ctas)]
    mean = sum(load) / ctas
    assert max(load) <= mean + blocks(0)              # list scheduling: at most one (longest) item above the mean
    if items >= 8 * ctas:
        assert max(load) <= 1.05 * mean               # many items per CTA: within 5 %
    # items are taken head by head (which keeps concurrently running CTAs on the same few heads) except for the last
    # one and a half rounds, which are taken longest first
    tail_heads = min(ZH, -(-(3 * ctas // 2) // pairs))
    for c in range(ctas):
        mine = [x for x in (t[k * ctas + c] for k in range(rounds.value)) if 0 <= x < (ZH - tail_heads) * pairs]
        assert mine == sorted(mine)
    assert lib.b200k_attn_causal_schedule(ZH, S, D, ctas, table, 0, ctypes.byref(rounds)) == _lib.ERR_INVALID_ARG


def _tail_plan(M, N, K, sm_count=148):
    import ctypes
    out = (ctypes.c_int * 5)()
    _lib.check(_lib.load().b200k_matmul_tail_plan(M, N, K, sm_count, out))
    return dict(mode=out[0], rest=out[1], pairs=out[2], full_waves=out[3], last_wave_items=out[4])


def test_matmul_tail_cost_model():
    # the M-row shards of the 8192^3 problem over 1, 2, 4 and 8 GPUs (CTA pairs on 256 x 256 tiles, 74 pairs)
    assert _tail_plan(8192, 8192, 8192) == dict(mode=0, rest=62, pairs=74, full_waves=13, last_wave_items=62)
    assert _tail_plan(4096, 8192, 8192) == dict(mode=0, rest=68, pairs=74, full_waves=6, last_wave_items=68)
    assert _tail_plan(2048, 8192, 8192) == dict(mode=1, rest=34, pairs=74, full_waves=3, last_wave_items=68)
    assert _tail_plan(1024, 8192, 8192) == dict(mode=0, rest=54, pairs=74, full_waves=1, last_wave_items=54)
    # the other sizes of the workload: 4096^3 (256 tiles) and 16384^3 (4096 tiles = 55 waves + 26)
    assert _tail_plan(4096, 4096, 4096)["mode"] == 1 and _tail_plan(16384, 16384, 16384) == dict(
        mode=1, rest=26, pairs=74, full_waves=55, last_wave_items=52)
    # column halves only while they fit into one wave, never for an exact number of waves or a single partial wave
    for M in range(256, 8192 + 1, 256):
        plan = _tail_plan(M, 8192, 8192)
        assert plan["mode"] == (1 if 0 < 2 * plan["rest"] <= plan["pairs"] and plan["rest"] < plan["pairs"] else 0)
        assert plan["last_wave_items"] <= plan["pairs"]
    assert _tail_plan(256, 512, 64, sm_count=148) == dict(mode=0, rest=0, pairs=2, full_waves=1, last_wave_items=0)
