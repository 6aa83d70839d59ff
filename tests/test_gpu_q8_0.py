"""GPU parity of the Q8_0 path against the CPU oracle, through the C ABI.

Bar: activation quants, scale bits and per-block int32 sums exact; f32 outputs bit-exact in the
selected instruction-set semantics (stronger than the 1e-5 relative the path is held to), and
within 1e-5 relative (max|a-b|/max|ref|, src/ops/kernel/q8_0/avx2.rs:239-245) across semantics.
"""
import numpy as np
import pytest

from oracle import orc
from tests.helpers import bits, make_q8_0_weight, q8_0_uniform_row, ramp_input, rel_err

pytestmark = pytest.mark.gpu
SEMS = [orc.SEM_AVX2, orc.SEM_NEON, orc.SEM_SCALAR]


@pytest.fixture(scope="module")
def ctx(rmi):
    c = rmi.context(0)
    yield c
    c.set_semantics(rmi.SEM_AVX2)


def f32(b):
    return np.array(b, np.uint32).view(np.float32)


# ------------------------------------------------------------------ quantizer

@pytest.mark.parametrize("sem", SEMS)
def test_quantizer_golden_vectors(rmi, ctx, sem):
    ctx.set_semantics(sem)
    x = np.zeros(32, np.float32)
    x[0], x[1] = 1.0, f32([0x3d11213e])[0]           # src/ops/matmul_tests.rs:558-571
    q8, sc = rmi.quantize_q8_0(x, 32)
    assert list(q8.view(np.int8)[:3]) == [127, 4, 0] and bits(sc)[0] == 0x3c010000
    x = np.zeros(32, np.float32)
    x[:3] = [127.0, 0.5, -0.5]                         # tests/quantized_inference.rs:55-66
    q8, _ = rmi.quantize_q8_0(x, 32)
    assert list(q8.view(np.int8)[:3]) == ([127, 1, -1] if sem == orc.SEM_SCALAR else [127, 0, 0])
    x = np.zeros(32, np.float32)
    x[0], x[1] = 127.0, 34.5                           # src/ops/matmul_tests.rs:546-556
    q8, _ = rmi.quantize_q8_0(x, 32)
    assert q8.view(np.int8)[1] == (35 if sem == orc.SEM_SCALAR else 34)


@pytest.mark.parametrize("sem", SEMS)
@pytest.mark.parametrize("m,n", [(1, 32), (1, 1024), (3, 96), (32, 3072), (512, 1024)])
def test_quantizer_bit_exact_on_random_rows(rmi, ctx, sem, m, n):
    ctx.set_semantics(sem)
    rng = np.random.default_rng(m * 1000 + n)
    x = rng.standard_normal((m, n)).astype(np.float32)
    x[0, :32] = 0.0                       # an all-zero block
    x[-1, -32:] *= np.float32(1e-30)      # denormal-scale block
    x[m // 2, 7] = 3.0e4                  # outlier
    q8, sc = rmi.quantize_q8_0(x, n)
    rq, rs = orc.quantize_q8_0(x, sem)
    assert np.array_equal(q8.reshape(m, n), rq)
    assert np.array_equal(bits(sc.reshape(m, -1)), bits(rs))


def test_quantizer_rejects_bad_length_and_accepts_empty(rmi, ctx):
    with pytest.raises(rmi.RmiError) as e:
        rmi.quantize_q8_0(np.zeros(33, np.float32), 33)
    assert e.value.status == 2
    q8, sc = rmi.quantize_q8_0(np.zeros(0, np.float32), 32)
    assert q8.size == 0 and sc.size == 0


# ------------------------------------------------------------------ GEMV: the reference's own unit tests

@pytest.mark.parametrize("sem", SEMS)
def test_q8_kernel_uniform_multi_row_scale_and_forward(rmi, ctx, sem):
    # src/ops/kernel/q8_0/mod.rs:74-129
    ctx.set_semantics(sem)
    q8, sc = np.ones(32, np.uint8), np.ones(1, np.float32)
    k = rmi.Q8Kernel.new(q8_0_uniform_row(1, 1.0), 32, 1)
    out = np.zeros(1, np.float32)
    k.forward_prequantized(q8, sc, out, 32, 1, 0, 1)
    assert list(out) == [32.0]
    k2 = rmi.Q8Kernel.new(np.concatenate([q8_0_uniform_row(1, 1.0)] * 2), 32, 2)
    out = np.zeros(2, np.float32)
    k2.forward_prequantized(q8, sc, out, 32, 2, 0, 1)
    assert list(out) == [32.0, 32.0]
    k3 = rmi.Q8Kernel.new(q8_0_uniform_row(1, 0.5), 32, 1)
    out = np.zeros(1, np.float32)
    k3.forward_prequantized(q8, sc, out, 32, 1, 0, 1)
    assert list(out) == [16.0]
    out = np.zeros(1, np.float32)
    k.forward(np.ones(32, np.float32), out, 32, 1)
    assert abs(out[0] - 32.0) < 5e-3


@pytest.mark.parametrize("sem", SEMS)
def test_q8_kernel_thread_partition(rmi, ctx, sem):
    # src/ops/kernel/q8_0/mod.rs:131-156: each (ith, nth) writes only its own rows
    ctx.set_semantics(sem)
    k = rmi.Q8Kernel.new(np.concatenate([q8_0_uniform_row(1, 1.0)] * 4), 32, 4)
    q8, sc = np.ones(32, np.uint8), np.ones(1, np.float32)
    a, b = np.zeros(4, np.float32), np.zeros(4, np.float32)
    k.forward_prequantized(q8, sc, a, 32, 4, 0, 2)
    k.forward_prequantized(q8, sc, b, 32, 4, 1, 2)
    assert list(a) == [32.0, 32.0, 0.0, 0.0] and list(b) == [0.0, 0.0, 32.0, 32.0]


def test_neon_q8_matmul_pinned_bits(rmi, ctx):
    # src/ops/matmul_tests.rs:288-306
    ctx.set_semantics(rmi.SEM_NEON)
    blk = np.zeros(34, np.uint8)
    blk[0:2] = np.array([0x1800], np.uint16).view(np.uint8)
    blk[2] = 127
    k = rmi.Q8Kernel.new(np.concatenate([blk, blk]), 64, 1)
    q8 = np.zeros(64, np.uint8)
    q8[0], q8[32] = np.uint8(-127 & 0xff), 127
    sc = np.array([np.array([0x1800], np.uint16).view(np.float16)[0], np.array([0x1a7d], np.uint16).view(np.float16)[0]], np.float32)
    out = np.zeros(1, np.float32)
    k.forward_prequantized(q8, sc, out, 64, 1, 0, 1)
    assert bits(out)[0] == 0x3d1cc57d


@pytest.mark.parametrize("sem", SEMS)
@pytest.mark.parametrize("n_out", [3584, 7168])
def test_parallel_matches_reference_bit_exact(rmi, ctx, sem, n_out):
    # tests/q8_0_parallel_matmul.rs:110-145: 1024 -> 3584 / 7168, threads 1/2/4/8
    ctx.set_semantics(sem)
    n_in = 1024
    wb = make_q8_0_weight(n_out, n_in, 7)
    w = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q8_0, n_in, n_out)
    q8, sc = rmi.quantize_q8_0(ramp_input(n_in), n_in)
    rq, rs = orc.quantize_q8_0(ramp_input(n_in), sem)
    assert np.array_equal(q8, rq) and np.array_equal(bits(sc), bits(rs))
    ref = orc.matmul_q8_0_range(wb, rq, rs, n_in, 0, n_out, sem)
    for nth in (1, 2, 4, 8):
        out = np.zeros(n_out, np.float32)
        for ith in range(nth):
            rmi.matmul_q8_0_quantized_parallel_rows(w, q8, sc, out, n_in, n_out, ith, nth)
        assert np.array_equal(bits(out), bits(ref)), f"nth={nth}"
    w.free()


@pytest.mark.parametrize("sem", SEMS)
def test_fused_vstack_matches_separate(rmi, ctx, sem):
    # tests/fused_ffn_matmul_parity.rs:92-127; src/ops/quant/fuse.rs:147-196
    ctx.set_semantics(sem)
    n_in, n = 1024, 3584
    gate = rmi.QuantizedTensor.from_bytes(make_q8_0_weight(n, n_in, 0), rmi.GGML_Q8_0, n_in, n)
    up = rmi.QuantizedTensor.from_bytes(make_q8_0_weight(n, n_in, 17), rmi.GGML_Q8_0, n_in, n)
    fused, rows = rmi.fuse_vstack_q8_0(gate, up)
    assert rows == 2 * n
    q8, sc = rmi.quantize_q8_0(ramp_input(n_in), n_in)
    og, ou, of = np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros(2 * n, np.float32)
    rmi.matmul_q8_0_quantized(gate, q8, sc, og, n_in, n)
    rmi.matmul_q8_0_quantized(up, q8, sc, ou, n_in, n)
    for ith in range(8):
        rmi.matmul_q8_0_quantized_parallel_rows(fused, q8, sc, of, n_in, 2 * n, ith, 8)
    assert np.array_equal(bits(of[:n]), bits(og)) and np.array_equal(bits(of[n:]), bits(ou))
    other = rmi.QuantizedTensor.from_bytes(make_q8_0_weight(4, 64, 0), rmi.GGML_Q8_0, 64, 4)
    assert rmi.fuse_vstack_q8_0(gate, other) is None
    # odd row counts: the second operand starts inside a 16-row tile
    a = rmi.QuantizedTensor.from_bytes(make_q8_0_weight(5, 64, 1), rmi.GGML_Q8_0, 64, 5)
    b = rmi.QuantizedTensor.from_bytes(make_q8_0_weight(21, 64, 9), rmi.GGML_Q8_0, 64, 21)
    f2, r2 = rmi.fuse_vstack_q8_0(a, b)
    q8s, scs = rmi.quantize_q8_0(ramp_input(64), 64)
    out = np.zeros(r2, np.float32)
    rmi.matmul_q8_0_quantized(f2, q8s, scs, out, 64, r2)
    ref = np.concatenate([orc.matmul_q8_0_range(make_q8_0_weight(5, 64, 1), q8s, scs, 64, 0, 5, sem),
                          orc.matmul_q8_0_range(make_q8_0_weight(21, 64, 9), q8s, scs, 64, 0, 21, sem)])
    assert np.array_equal(bits(out), bits(ref))


# ------------------------------------------------------------------ GEMV: shapes, ragged edges, M rows

@pytest.mark.parametrize("sem", SEMS)
@pytest.mark.parametrize("n,k", [(1, 32), (3, 64), (4, 32), (5, 256), (16, 1024), (17, 64), (127, 256), (128, 32),
                                 (129, 1024), (3072, 1024), (1024, 3072)])
def test_gemv_bit_exact_small_and_ragged_shapes(rmi, ctx, sem, n, k):
    ctx.set_semantics(sem)
    wb = rmi.synth.q8_0_weight(n, k, seed=n * 7 + k)
    w = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q8_0, k, n)
    x = rmi.synth.normal((k,), seed=k + 1)
    q8, sc = orc.quantize_q8_0(x, sem)
    canary = np.full(n + 8, np.float32(-777.0))
    out = canary[4:4 + n]
    tmp = np.zeros(n, np.float32)
    rmi.matmul_q8_0_quantized(w, q8, sc, tmp, k, n)
    out[:] = tmp
    ref = orc.matmul_q8_0_range(wb, q8, sc, k, 0, n, sem)
    assert np.array_equal(bits(tmp), bits(ref))
    # sub-ranges that start and end inside 16-row tiles
    for s, e in ((0, n), (1, n), (n // 3, max(n // 3, n - 1)), (n - 1, n)):
        o = np.full(n, np.float32(-5.0))
        rmi.matmul_q8_0_quantized_range(w, q8, sc, o, k, s, e)
        assert np.array_equal(bits(o[: e - s]), bits(ref[s:e])) and np.all(o[e - s:] == -5.0)
    w.free()


@pytest.mark.parametrize("sem", SEMS)
@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 9, 16, 31, 32])
def test_gemv_m_rows_bit_exact_and_m_independent(rmi, ctx, sem, m):
    ctx.set_semantics(sem)
    n, k = 515, 1024
    wb = rmi.synth.q8_0_weight(n, k, seed=3)
    w = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q8_0, k, n)
    x = rmi.synth.normal((m, k), seed=40 + m)
    got = rmi.matmul_q8_0(w, x)
    ref = orc.q8_forward_batched(wb, x, k, n, sem)
    assert np.array_equal(bits(got), bits(ref))
    w.free()


def test_config1_gemv_all_semantics_and_cross_semantics_tolerance(rmi, ctx):
    # BASELINE config 1: W [3072,1024] from N(0,0.02) seed 0, x [1,1024] N(0,1) seed 1
    wb = rmi.synth.q8_0_weight(3072, 1024, seed=0)
    x = rmi.synth.normal((1, 1024), seed=1)
    w = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q8_0, 1024, 3072)
    outs = {}
    for sem in SEMS:
        ctx.set_semantics(sem)
        outs[sem] = rmi.matmul_q8_0(w, x)[0]
        q8, sc = orc.quantize_q8_0(x[0], sem)
        assert np.array_equal(bits(outs[sem]), bits(orc.matmul_q8_0_range(wb, q8, sc, 1024, 0, 3072, sem)))
        again = rmi.matmul_q8_0(w, x)[0]
        assert np.array_equal(bits(again), bits(outs[sem]))  # run-to-run identical
    q8, sc = orc.quantize_q8_0(x[0], orc.SEM_AVX2)
    ref = orc.matmul_q8_0_range(wb, q8, sc, 1024, 0, 3072, orc.SEM_AVX2)
    assert rel_err(outs[orc.SEM_NEON], ref) < 1e-2  # different quantizer rounding: coarse bound only
    w.free()


def test_block_sums_exact_cuda_cores(rmi, ctx):
    n, k, m = 200, 512, 3
    wb = rmi.synth.q8_0_weight(n, k, seed=8)
    w = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q8_0, k, n)
    q8, _ = orc.quantize_q8_0(rmi.synth.normal((m, k), seed=9), orc.SEM_AVX2)
    got = rmi.q8_0_block_sums(w, q8, m)
    for t in range(m):
        assert np.array_equal(got[t], orc.q8_0_block_sums(wb, q8[t], k, 0, n))
    w.free()


def test_error_paths(rmi, ctx):
    with pytest.raises(rmi.RmiError) as e:
        rmi.QuantizedTensor.from_bytes(np.zeros(34, np.uint8), rmi.GGML_Q8_0, 33, 1)
    assert e.value.status == 2
    with pytest.raises(rmi.RmiError) as e:
        rmi.QuantizedTensor.from_bytes(np.zeros(33, np.uint8), rmi.GGML_Q8_0, 32, 1)   # short buffer
    assert e.value.status == 2
    with pytest.raises(rmi.RmiError) as e:
        rmi.QuantizedTensor.from_bytes(np.zeros(64, np.uint8), 3, 32, 1)               # Q4_1 is not on this path
    assert e.value.status == 6
    w = rmi.QuantizedTensor.from_bytes(make_q8_0_weight(4, 32, 0), rmi.GGML_Q8_0, 32, 4)
    with pytest.raises(rmi.RmiError) as e:
        rmi.matmul_q8_0_quantized_range(w, np.zeros(32, np.uint8), np.zeros(1, np.float32), np.zeros(4, np.float32), 32, 2, 9)
    assert e.value.status == 2
    empty = rmi.QuantizedTensor.from_bytes(make_q8_0_weight(4, 32, 0), rmi.GGML_Q8_0, 32, 4, row_begin=2, row_end=2)
    assert empty.n_out == 0
    assert rmi.matmul_q8_0(empty, np.zeros((1, 32), np.float32)).shape == (1, 0)


def test_row_sharded_upload_equals_slices_of_the_full_result(rmi, ctx):
    # PlacementSlice::Rows (src/format/load_plan.rs:19-22): rank r of g uploads rows [r*N/g,(r+1)*N/g)
    ctx.set_semantics(rmi.SEM_AVX2)
    n, k, g = 1024, 256, 4
    wb = rmi.synth.q8_0_weight(n, k, seed=21)
    x = rmi.synth.normal((5, k), seed=22)
    full = rmi.matmul_q8_0(rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q8_0, k, n), x)
    for r in range(g):
        shard = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q8_0, k, n, row_begin=r * n // g, row_end=(r + 1) * n // g)
        assert np.array_equal(bits(rmi.matmul_q8_0(shard, x)), bits(full[:, r * n // g:(r + 1) * n // g]))


@pytest.mark.parametrize("sem", SEMS)
@pytest.mark.parametrize("n,k,m", [(16389, 2048, 1), (15000, 2080, 2), (20000, 8192, 1)])
def test_streaming_gemv_many_long_rows_bit_exact(rmi, ctx, sem, n, k, m):
    """More 16-row tiles than the one-copy-per-tile kernel takes and rows of 64 blocks or more: persistent CTAs
    stream the records through a ring of bulk copies.  Ragged last tile, a chunk count that does not divide the
    row (2080 = 65 blocks), a row range, and run-twice equality."""
    ctx.set_semantics(sem)
    wb = rmi.synth.q8_0_weight(n, k, seed=n % 97)
    w = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q8_0, k, n)
    x = rmi.synth.normal((m, k), seed=3)
    got = rmi.matmul_q8_0(w, x)
    ref = orc.q8_forward_batched(wb, x, k, n, sem, threads=8)
    assert np.array_equal(bits(got), bits(ref))
    assert np.array_equal(bits(rmi.matmul_q8_0(w, x)), bits(got))
    q8, sc = orc.quantize_q8_0(x, sem)
    part = rmi.matmul_q8_0_prequantized_rows(w, q8, sc, m, row_begin=17, row_end=n - 33)
    assert np.array_equal(bits(part[:, 17:n - 33]), bits(ref[:, 17:n - 33]))
    w.free()


# ------------------------------------------------------------------ f32-input matmul (ops::matmul_q8_0)

@pytest.mark.parametrize("sem", SEMS)
@pytest.mark.parametrize("n,k,m", [(40, 96, 1), (1024, 1024, 3), (300, 2048, 2)])
def test_f32_input_matmul_q8_0_bit_exact(rmi, ctx, sem, n, k, m):
    """rmi_matmul_q8_0_f32 = ops::matmul_q8_0 (src/ops/kernel/q8_0/parallel.rs:317-341): the AVX2 order under AVX2
    semantics, the scalar order otherwise; ragged last tile, several activation rows, host and device entry points."""
    torch = pytest.importorskip("torch")
    ctx.set_semantics(sem)
    wb = make_q8_0_weight(n, k, 2)
    w = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q8_0, k, n)
    x = np.random.default_rng(n + m).standard_normal((m, k)).astype(np.float32)
    ref = orc.matmul_q8_0_f32(wb, x, k, n, sem)
    got = rmi.matmul_q8_0_f32(w, x)
    assert np.array_equal(bits(got), bits(ref))
    xd = torch.from_numpy(x).cuda()
    od = torch.empty((m, n), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    rmi.matmul_q8_0_f32_dev(w, xd.data_ptr(), m, od.data_ptr())
    ctx.sync()
    assert np.array_equal(bits(od.cpu().numpy()), bits(ref))
    # the quantize-then-GEMV path of the same weight agrees within the quantization error of the activation
    q = rmi.matmul_q8_0(w, x)
    assert rel_err(q, ref) < 2e-2
    w.free()
