"""GPU parity of the tcgen05 tensor-core GEMM against the oracle.

Tolerance (relative Frobenius error): 2e-3 for the tf32 / bf16 / fp16 input
classes, as the benchmark states.  The oracle multiplies the same rounded
inputs in float64, so for inputs that are exactly representable the observed
error is accumulation order only; TIGHT = 2e-5 is asserted there so that a
dropped k-slice or a mis-addressed tile cannot hide inside 2e-3.
"""
import numpy as np
import pytest

from oracle import spiral_oracle as so

pytestmark = pytest.mark.gpu
TOL = 2e-3
TIGHT = 2e-5


def operands(seed, at, bt, m, n, k, in_dtype):
    g = so.rng(seed)
    a = so.round_input(g.normal(size=(k, m) if at else (m, k)).astype(np.float32), in_dtype)
    b = so.round_input(g.normal(size=(n, k) if bt else (k, n)).astype(np.float32), in_dtype)
    c = g.normal(size=(m, n)).astype(np.float32)
    return a, b, c


def storage(in_dtype):
    return "f32" if in_dtype == "tf32" else in_dtype


def run(gpu, at, bt, alpha, a, b, beta, c, in_dtype, out_dtype="f32", **kw):
    da = gpu.DeviceArray.from_numpy(a, storage(in_dtype))
    db = gpu.DeviceArray.from_numpy(b, storage(in_dtype))
    dc = gpu.DeviceArray.from_numpy(c, out_dtype)
    gpu.matmul(at, bt, alpha, da, db, beta, dc, in_dtype=in_dtype, **kw)
    return dc.numpy()


@pytest.mark.parametrize("in_dtype", ["bf16", "f16", "tf32"])
def test_single_tile_nt(gpu, in_dtype):
    a, b, c = operands(11, False, True, 128, 16, 64, in_dtype)
    got = run(gpu, False, True, 1.0, a, b, 0.0, c, in_dtype)
    assert so.rel_frobenius(got, so.matmul(False, True, 1.0, a, b, 0.0, None)) <= TIGHT


LAYOUTS = [(False, True), (False, False), (True, False), (True, True)]


@pytest.mark.parametrize("in_dtype", ["bf16", "f16", "tf32"])
@pytest.mark.parametrize("at,bt", LAYOUTS)
def test_512_cubed_layouts(gpu, at, bt, in_dtype):
    a, b, c = operands(12, at, bt, 512, 512, 512, in_dtype)
    got = run(gpu, at, bt, 1.0, a, b, 0.0, c, in_dtype)
    assert so.rel_frobenius(got, so.matmul(at, bt, 1.0, a, b, 0.0, None)) <= TIGHT


@pytest.mark.parametrize("in_dtype", ["bf16", "tf32"])
@pytest.mark.parametrize("at,bt", LAYOUTS[:3])
def test_ragged_4000x3000x1000(gpu, at, bt, in_dtype):
    """Tile tails in M, N and K (benchmark configuration 2's ragged case)."""
    a, b, c = operands(13, at, bt, 4000, 3000, 1000, in_dtype)
    got = run(gpu, at, bt, 1.0, a, b, 0.0, c, in_dtype)
    assert so.rel_frobenius(got, so.matmul(at, bt, 1.0, a, b, 0.0, None)) <= TIGHT


@pytest.mark.parametrize("in_dtype,out_dtype", [("bf16", "f32"), ("f16", "bf16"), ("tf32", "f32")])
@pytest.mark.parametrize("at,bt", LAYOUTS[:3])
def test_last_wave_of_half_width_tiles(gpu, at, bt, in_dtype, out_dtype):
    """More 256 x 256 tiles than CTA pairs, with a remainder of at most half the pairs: the last wave runs
    as half-width tiles (two work items per tile, their own instruction descriptor and B boxes).  Sized
    from the SM count so that the remainder is 9 tiles; a ragged M and N put the clipped tiles there."""
    pairs = gpu.sm_count() // 2
    tiles_m = pairs + 9
    m, n, k = 256 * tiles_m - 40, 248, 192
    a, b, c = operands(61, at, bt, m, n, k, in_dtype)
    bias = so.rng(62).normal(size=n).astype(np.float32)
    plan = gpu.matmul_plan(at, bt, m, n, k, in_dtype)
    assert plan["block_m"] == 256 and plan["block_n"] == 256       # CTA pairs, one tile column
    kw = {}
    if out_dtype != "f32":
        kw = dict(epilogue=("bias", "relu"), bias=gpu.DeviceArray.from_numpy(bias))
    got = run(gpu, at, bt, 1.0, a, b, 0.0, c, in_dtype, out_dtype=out_dtype, **kw)
    want = so.matmul(at, bt, 1.0, a, b, 0.0, None)
    if out_dtype != "f32":
        want = so.round_input(so.relu(want + bias), out_dtype)
        assert so.rel_frobenius(got, want) <= 3e-3
    else:
        assert so.rel_frobenius(got, want) <= TIGHT
    tail = slice(256 * (tiles_m - 9), m)          # the rows of the half-width tiles, by themselves
    assert so.rel_frobenius(got[tail], want[tail]) <= (3e-3 if out_dtype != "f32" else TIGHT)


@pytest.mark.parametrize("m,n,k", [(8, 8, 8), (136, 24, 72), (120, 264, 200), (304, 520, 136), (64, 1000, 8)])
@pytest.mark.parametrize("at,bt", LAYOUTS[:3])
def test_small_odd_shapes_bf16(gpu, at, bt, m, n, k):
    """Every contiguous dimension is a multiple of 8 elements (16-byte row pitch, as the reference
    also demands, corecuda/base.spi:158); tile tails in M, N and K are exercised."""
    a, b, c = operands(m + n + k, at, bt, m, n, k, "bf16")
    got = run(gpu, at, bt, 1.0, a, b, 0.0, c, "bf16")
    assert so.rel_frobenius(got, so.matmul(at, bt, 1.0, a, b, 0.0, None)) <= TIGHT


@pytest.mark.parametrize("m,n,k", [(1, 1, 8), (127, 3, 200), (333, 257, 72)])
def test_nt_needs_only_k_aligned(gpu, m, n, k):
    """The dense-layer layout (NT) has K contiguous in both operands: M and N may be anything."""
    a, b, c = operands(m * n + k, False, True, m, n, k, "bf16")
    got = run(gpu, False, True, 1.0, a, b, 0.0, c, "bf16")
    assert so.rel_frobenius(got, so.matmul(False, True, 1.0, a, b, 0.0, None)) <= TIGHT


def test_alpha_beta_in_place(gpu):
    a, b, c = operands(14, False, True, 384, 320, 192, "bf16")
    got = run(gpu, False, True, 0.75, a, b, -1.25, c, "bf16")
    assert so.rel_frobenius(got, so.matmul(False, True, 0.75, a, b, -1.25, c)) <= TIGHT


def test_reference_surface_matmul_tf32_unrounded_fp32(gpu):
    """matmul_tf32 on arbitrary fp32 data: the tensor core reads 10 mantissa bits, so the
    error against the TF32-rounded oracle is of TF32 size, inside the 2e-3 class."""
    g = so.rng(15)
    a = g.normal(size=(256, 384)).astype(np.float32)
    b = g.normal(size=(320, 384)).astype(np.float32)
    c = g.normal(size=(256, 320)).astype(np.float32)
    dc = gpu.DeviceArray.from_numpy(c)
    gpu.matmul_tf32(False, True, 1.0, gpu.DeviceArray.from_numpy(a), gpu.DeviceArray.from_numpy(b), 1.0, dc)
    err = so.rel_frobenius(dc.numpy(), so.matmul(False, True, 1.0, a, b, 1.0, c, in_dtype="tf32"))
    assert err <= TOL


def test_4096_cubed_sampled_rows_and_linearity(gpu):
    """Full benchmark size: oracle on 48 sampled rows, plus linearity C(2A) == 2 C(A) exactly."""
    at, bt = False, True
    a, b, c = operands(16, at, bt, 4096, 4096, 4096, "bf16")
    got = run(gpu, at, bt, 1.0, a, b, 0.0, c, "bf16")
    rows = so.rng(17).choice(4096, size=48, replace=False)
    want = so.matmul(at, bt, 1.0, a[rows], b, 0.0, None)
    assert so.rel_frobenius(got[rows], want) <= TIGHT
    got2 = run(gpu, at, bt, 1.0, 2 * a, b, 0.0, c, "bf16")
    np.testing.assert_array_equal(got2, 2 * got)


@pytest.mark.parametrize("out_dtype", ["f32", "bf16", "f16"])
def test_bias_relu_epilogue_and_output_dtypes(gpu, out_dtype):
    a, b, c = operands(18, False, True, 300, 264, 128, "bf16")
    bias = so.rng(19).normal(size=264).astype(np.float32)
    got = run(gpu, False, True, 1.0, a, b, 0.0, c, "bf16", out_dtype=out_dtype, epilogue=("bias", "relu"),
              bias=gpu.DeviceArray.from_numpy(bias))
    want = so.relu(so.matmul(False, True, 1.0, a, b, 0.0, None) + bias)
    if out_dtype != "f32":
        want = so.round_input(want, out_dtype)
        assert so.rel_frobenius(got, want) <= 3e-3     # one output rounding of 2^-9 (bf16) / 2^-11 (f16)
    else:
        assert so.rel_frobenius(got, want) <= TIGHT


def test_relu_grad_epilogue(gpu):
    a, b, c = operands(20, False, False, 256, 192, 64, "bf16")
    act = so.round_bf16(so.rng(21).normal(size=(256, 192)).astype(np.float32))
    got = run(gpu, False, False, 1.0, a, b, 0.0, c, "bf16", out_dtype="bf16", epilogue=("relu_grad",),
              aux_in=gpu.DeviceArray.from_numpy(act, "bf16"))
    want = so.round_bf16(np.where(act > 0, so.matmul(False, False, 1.0, a, b, 0.0, None), 0))
    assert so.rel_frobenius(got, want) <= 3e-3
    assert np.all(got[act <= 0] == 0)


def bits_to_bool(words, m, n):
    """uint32 [n/32, m] sign words (bit j of word [c, row] = column 32c+j of that row) -> bool [m, n]."""
    by_row = np.ascontiguousarray(words.view(np.uint32).reshape(n // 32, m).T)
    return np.unpackbits(by_row.view(np.uint8).reshape(m, -1), axis=1, bitorder="little").reshape(m, n).astype(bool)


def bool_to_bits(keep):
    m, n = keep.shape
    by_row = np.packbits(keep.reshape(m, n // 32, 32), axis=-1, bitorder="little").view(np.uint32).reshape(m, n // 32)
    return np.ascontiguousarray(by_row.T)


def test_relu_sign_bits_forward_and_backward_gate(gpu):
    """SB_EPI_RELU_MASK_OUT records bit j of word [c, row] = (value[row, 32c+j] > 0); gating a second
    GEMM by those bits equals gating by the activation tile itself."""
    m, n, k = 300, 320, 128
    a, b, c = operands(31, False, True, m, n, k, "bf16")
    bits = gpu.DeviceArray.zeros((n // 32, m), "i32")
    act = run(gpu, False, True, 1.0, a, b, 0.0, c, "bf16", out_dtype="bf16", epilogue=("relu", "relu_mask_out"),
              aux_out=bits)
    pre = so.matmul(False, True, 1.0, a, b, 0.0, None)
    got = bits_to_bool(bits.numpy(), m, n)
    decided = np.abs(pre) > 1e-3                       # leave out values within rounding of zero
    assert not ((got != (pre > 0)) & decided).any()
    np.testing.assert_array_equal(act > 0, got)
    np.testing.assert_array_equal(bool_to_bits(got), bits.numpy().view(np.uint32).reshape(n // 32, m))
    a2, b2, c2 = operands(32, False, False, m, n, 64, "bf16")
    by_bits = run(gpu, False, False, 1.0, a2, b2, 0.0, c2, "bf16", out_dtype="bf16", epilogue=("relu_grad_mask",), aux_in=bits)
    by_tile = run(gpu, False, False, 1.0, a2, b2, 0.0, c2, "bf16", out_dtype="bf16", epilogue=("relu_grad",),
                  aux_in=gpu.DeviceArray.from_numpy(act, "bf16"))
    np.testing.assert_array_equal(by_bits, by_tile)


@pytest.mark.parametrize("m,n,k,out_dtype", [(300, 320, 128, "bf16"), (1000, 512, 64, "f32"), (64, 32, 16, "f16")])
@pytest.mark.parametrize("gated", [False, True])
def test_column_sums_epilogue(gpu, m, n, k, out_dtype, gated):
    """SB_EPI_COLSUM_OUT adds the column sums of the (gated) product to aux_out, which may already
    hold a value; ragged last row blocks add nothing."""
    in_dtype = "f16" if out_dtype == "f16" else "bf16"
    a, b, c = operands(41, False, False, m, n, k, in_dtype)
    sums0 = so.rng(42).normal(size=n).astype(np.float32)
    sums = gpu.DeviceArray.from_numpy(sums0, "f32")
    prod = so.matmul(False, False, 1.0, a, b, 0.0, None)
    kw = dict(epilogue=("colsum_out",), aux_out=sums)
    if gated:
        gate = so.rng(43).integers(0, 2 ** 32, size=(n // 32, m), dtype=np.uint64).astype(np.uint32)
        keep = bits_to_bool(gate, m, n)
        prod = np.where(keep, prod, 0)
        kw = dict(epilogue=("relu_grad_mask", "colsum_out"), aux_in=gpu.DeviceArray.from_numpy(gate.view(np.int32), "i32"),
                  aux_out=sums)
    got = run(gpu, False, False, 1.0, a, b, 0.0, c, in_dtype, out_dtype=out_dtype, **kw)
    assert so.rel_frobenius(got, so.round_input(prod.astype(np.float32), out_dtype) if out_dtype != "f32" else prod) <= 3e-3
    want = sums0 + prod.sum(axis=0, dtype=np.float64)
    np.testing.assert_allclose(sums.numpy(), want, rtol=0, atol=2e-4 * np.sqrt(m * k))


def test_column_sums_rejects_unsupported_combinations(gpu):
    a, b, c = operands(44, False, True, 64, 64, 64, "bf16")
    sums = gpu.DeviceArray.zeros((64,), "f32")
    with pytest.raises(gpu.SpiralError):
        run(gpu, False, True, 1.0, a, b, 0.0, c, "bf16", epilogue=("relu", "colsum_out"), aux_out=sums)
    with pytest.raises(gpu.SpiralError):
        run(gpu, False, True, 2.0, a, b, 0.0, c, "bf16", epilogue=("colsum_out",), aux_out=sums)
    with pytest.raises(gpu.SpiralError):
        run(gpu, False, True, 1.0, a, b, 0.0, c, "bf16", epilogue=("colsum_out",))


@pytest.mark.parametrize("n", [3, 10, 16, 17, 32, 40])
@pytest.mark.parametrize("heads", [("masked_softmax",), ("regret_matching",), ("masked_softmax", "regret_matching")])
def test_fused_row_heads(gpu, n, heads):
    m, k = 333, 256
    a, b, c = operands(22 + n, False, True, m, n, k, "tf32")
    a = so.round_tf32(a * np.float32(0.2))     # keep the inputs exactly representable in TF32
    mask = (so.rng(23).random((m, n)) < 0.6).astype(np.uint8)
    mask[:, 0] = 1
    idx = gpu.DeviceArray((m,), "i32")
    got = run(gpu, False, True, 1.0, a, b, 0.0, c, "tf32", epilogue=heads + ("argmax",),
              mask=gpu.DeviceArray.from_numpy(mask), aux_out=idx)
    want = so.matmul(False, True, 1.0, a, b, 0.0, None)
    if "masked_softmax" in heads:
        want = so.masked_softmax(want, mask)
    if "regret_matching" in heads:
        want = so.masked_regret_matching(want, mask)
    np.testing.assert_allclose(got, want, atol=2e-5)
    np.testing.assert_array_equal(idx.numpy(), np.argmax(got, axis=1))      # fused argmax == argmax of its own output
    top2 = np.sort(want, axis=1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 1e-4
    np.testing.assert_array_equal(idx.numpy()[clear], so.argmax(want)[clear])


def test_edge_cases(gpu):
    from spiral_b200 import SpiralError
    # K = 0: C <- beta * C
    c = so.rng(24).normal(size=(5, 8)).astype(np.float32)
    dc = gpu.DeviceArray.from_numpy(c)
    gpu.matmul(False, True, 1.0, gpu.DeviceArray((5, 0), "bf16"), gpu.DeviceArray((8, 0), "bf16"), 2.0, dc)
    np.testing.assert_array_equal(dc.numpy(), 2 * c)
    # empty M
    gpu.matmul(False, True, 1.0, gpu.DeviceArray((0, 8), "bf16"), gpu.DeviceArray((8, 8), "bf16"), 0.0,
               gpu.DeviceArray((0, 8), "f32"))
    # a row pitch that is not a multiple of 16 bytes is refused, not mis-read
    with pytest.raises(SpiralError) as e:
        gpu.matmul(False, True, 1.0, gpu.DeviceArray((8, 12), "bf16"), gpu.DeviceArray((8, 12), "bf16"), 0.0,
                   gpu.DeviceArray((8, 8), "f32"))
    assert e.value.code == -2
