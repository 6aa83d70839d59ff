"""Q4_K paths on the GPU vs the oracle: Q8_K quantizer (exact), Q4_K x Q8_K dot (exact integer
sums, bit-exact f32 in AVX2 and scalar order), dequantize (exact), dequant-matmul (1e-4 relative)."""
import numpy as np
import pytest

from oracle import orc
from tests.helpers import bits, f16_bits, ramp_input, rel_err

pytestmark = pytest.mark.gpu
KSEMS = [orc.SEM_AVX2, orc.SEM_SCALAR]


@pytest.fixture(scope="module")
def ctx(rmi):
    c = rmi.context(0)
    yield c
    c.set_semantics(rmi.SEM_AVX2)


@pytest.mark.parametrize("sem", KSEMS)
def test_q8_k_quantizer_exact(rmi, ctx, sem):
    ctx.set_semantics(sem)
    x = np.zeros(256, np.float32)
    x[:5] = [-127.0, 0.5, 1.5, 2.5, -0.5]                    # tests/quantized_inference.rs:174-186
    d, qs, bs = rmi.quantize_row_q8_k(x)
    assert list(qs[0, :5]) == [-127, 0, 2, 2, 0]
    x = np.array([(i - 127) * 0.03125 for i in range(256)], np.float32)   # :152-172
    d, qs, bs = rmi.quantize_row_q8_k(x)
    assert bs.astype(np.int64).sum() == qs.astype(np.int64).sum()
    x = rmi.synth.normal((4096,), seed=1)
    x[256:512] = 0.0
    x[700], x[701] = 5.0, -5.0                               # tie in |x|: the first one wins
    d, qs, bs = rmi.quantize_row_q8_k(x)
    rd, rq, rb = orc.q8k_to_numpy(orc.quantize_row_q8_k(x, sem))
    assert np.array_equal(bits(d), bits(rd)) and np.array_equal(qs, rq) and np.array_equal(bs, rb)


def test_q4_k_uniform_block_known_answer(rmi, ctx):
    # tests/quantized_inference.rs:233-249
    w = np.zeros(144, np.uint8)
    w[0:2] = np.array([f16_bits(1.0)], np.uint16).view(np.uint8)
    w[4:16] = [1, 1, 1, 1, 0, 0, 0, 0, 1, 1, 1, 1]
    w[16:] = 0x11
    k = rmi.Q4_KKernel.new(w, 256, 1)
    out = np.zeros(1, np.float32)
    k.forward_prequantized(np.ones(256, np.uint8), np.ones(8, np.float32), out, 256, 1, 0, 1)
    assert list(out) == [256.0]
    assert np.array_equal(rmi.dequantize_q4_k_weight(k.weight), np.ones((1, 256), np.float32))
    lin = rmi.QuantizedLinear.from_weight_slice(w, None, 256, 1, "uniform")
    o = np.zeros(1, np.float32)
    lin.forward_dequant(np.ones(256, np.float32), o)
    assert list(o) == [256.0] and lin.input_dim() == 256 and lin.output_dim() == 1 and lin.name() == "uniform"


def test_q4_k_dequantize_exact(rmi, ctx):
    wb = rmi.synth.q4_k_weight(64, 1024, seed=5)
    w = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q4_K, 1024, 64)
    assert np.array_equal(bits(rmi.dequantize_q4_k_weight(w)), bits(orc.dequantize_q4_k_weight(wb, 64, 1024)))


@pytest.mark.parametrize("sem", KSEMS)
def test_q4_k_prepared_path_bit_exact(rmi, ctx, sem):
    # Q4_KKernel::forward_prepared (src/ops/kernel/q4_k.rs:56-93), bytes as in
    # tests/quantized_inference.rs:188-210 and a random stream; (ith, nth) partition
    ctx.set_semantics(sem)
    w1 = ((np.arange(144) * 29 + 7) & 0xff).astype(np.uint8)
    x1 = np.array([((i % 23) - 11) / 7.0 for i in range(256)], np.float32)
    k1 = rmi.Q4_KKernel.new(w1, 256, 1)
    o = np.zeros(1, np.float32)
    k1.forward_prepared(x1, None, None, None, o, 256, 1, 0, 1)
    assert bits(o)[0] == bits(orc.q4k_forward_prepared(w1, x1, 256, 1, sem=sem))[0]
    n_in, n_out = 2048, 300
    wb = rmi.synth.q4_k_weight(n_out, n_in, seed=3)
    x = rmi.synth.normal((n_in,), seed=4)
    k = rmi.Q4_KKernel.new(wb, n_in, n_out)
    ref = orc.q4k_forward_prepared(wb, x, n_in, n_out, sem=sem)
    for nth in (1, 3, 8):
        out = np.zeros(n_out, np.float32)
        for ith in range(nth):
            k.forward_prepared(x, None, None, None, out, n_in, n_out, ith, nth)
        assert np.array_equal(bits(out), bits(ref)), nth


@pytest.mark.parametrize("sem", KSEMS)
def test_q4_k_partition_seq_parallel_fused(rmi, ctx, sem):
    # tests/fused_ffn_matmul_parity.rs:234-319
    ctx.set_semantics(sem)
    n_in, n_out = 512, 24
    rb = n_in // 256 * 144

    def mk(seed):
        return ((seed + np.arange(n_out)[:, None] + np.arange(rb)[None, :]) & 0xff).astype(np.uint8).reshape(-1)

    gate, up = mk(0), mk(17)
    x = ramp_input(n_in)
    tg = rmi.QuantizedTensor.from_bytes(gate, rmi.GGML_Q4_K, n_in, n_out)
    tu = rmi.QuantizedTensor.from_bytes(up, rmi.GGML_Q4_K, n_in, n_out)
    fused, rows = rmi.fuse_vstack_q4_k(tg, tu)
    out = np.zeros(rows, np.float32)
    kf = fused.into_kernel()
    for ith in range(4):
        kf.forward_prepared(x, None, None, None, out, n_in, rows, ith, 4)
    assert np.array_equal(bits(out[:n_out]), bits(orc.q4k_forward_prepared(gate, x, n_in, n_out, sem=sem)))
    assert np.array_equal(bits(out[n_out:]), bits(orc.q4k_forward_prepared(up, x, n_in, n_out, sem=sem)))


@pytest.mark.parametrize("m", [1, 8, 256])
def test_config3_q4_k_dequant_matmul(rmi, ctx, m):
    # BASELINE config 3: W [4096,4096] Q4_K, x [M,4096] N(0,1); tolerance 1e-4 relative
    n = 4096
    wb = rmi.synth.q4_k_weight(n, n, seed=0)
    lin = rmi.QuantizedLinear.from_weight_slice(wb, None, n, n, "c3")
    x = rmi.synth.normal((m, n), seed=1)
    out = np.zeros((m, n), np.float32)
    lin.forward_dequant(x, out)
    rows = list(range(m)) if m <= 8 else [0, 100, 255]
    deq = orc.dequantize_q4_k_weight(wb, n, n)
    for t in rows:
        ref_seq = orc.q4k_forward_dequant(wb, n, n, x[t]) if t == rows[0] else None
        ref64 = (deq.astype(np.float64) @ x[t].astype(np.float64)).astype(np.float32)
        assert rel_err(out[t], ref64) < 1e-4
        if ref_seq is not None:
            assert rel_err(out[t], ref_seq) < 1e-4   # the reference's sequential f32 order


@pytest.mark.parametrize("m,n,k", [(37, 200, 512), (64, 128, 256), (130, 260, 1024)])
def test_q4_k_dequant_gemm_ragged_tiles(rmi, ctx, m, n, k):
    """m >= 32 runs the tiled f32 GEMM with on-the-fly decode: ragged weight rows and activation rows,
    every output against the f64 product of the dequantized weight (1e-4 relative)."""
    wb = rmi.synth.q4_k_weight(n, k, seed=5)
    lin = rmi.QuantizedLinear.from_weight_slice(wb, None, k, n, "ragged")
    x = rmi.synth.normal((m, k), seed=6)
    out = np.full((m, n), np.nan, np.float32)
    lin.forward_dequant(x, out)
    deq = orc.dequantize_q4_k_weight(wb, n, k)
    ref = (x.astype(np.float64) @ deq.astype(np.float64).T).astype(np.float32)
    assert np.isfinite(out).all()
    assert rel_err(out, ref) < 1e-4
    # the small-batch kernel gives the same values within the same tolerance
    out8 = np.zeros((8, n), np.float32)
    lin.forward_dequant(x[:8], out8)
    assert rel_err(out8, ref[:8]) < 1e-4


@pytest.mark.parametrize("sem", ["SEM_AVX2", "SEM_SCALAR"])
@pytest.mark.parametrize("m", [1, 4, 7, 9])
def test_q4_k_q8k_device_entry_point_matches_host_entry_point(rmi, ctx, sem, m):
    """rmi_matmul_q4_k_q8k_dev (groups of four activation rows per pass + remainder) == rmi_matmul_q4_k_q8k bits."""
    torch = pytest.importorskip("torch")
    ctx.set_semantics(getattr(rmi, sem))
    n, k = 96, 512
    wb = rmi.synth.q4_k_weight(n, k, seed=9)
    w = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q4_K, k, n)
    x = rmi.synth.normal((m, k), seed=10)
    xd = torch.from_numpy(x).cuda()
    od = torch.empty((m, n), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    rmi.matmul_q4_k_q8k_dev(w, xd.data_ptr(), m, od.data_ptr())
    ctx.sync()
    ref = np.stack([orc.q4k_forward_prepared(wb, x[t], k, n, sem=getattr(orc, sem)) for t in range(m)])
    assert np.array_equal(bits(od.cpu().numpy()), bits(ref))
    w.free()
    ctx.set_semantics(rmi.SEM_AVX2)


@pytest.mark.parametrize("m,n,k", [(32, 64, 512), (70, 100, 1024), (256, 256, 4096)])
def test_q4k_q8k_many_rows_tiled_kernel_bit_exact(rmi, ctx, m, n, k):
    """m >= 32 under AVX2 semantics takes the tiled kernel (32 weight rows x 16 activation rows per CTA): every
    output carries the bits of the per-row reference order; ragged tiles in both directions and a row range."""
    ctx.set_semantics(rmi.SEM_AVX2)
    wb = rmi.synth.q4_k_weight(n, k, seed=m + n)
    w = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q4_K, k, n)
    x = rmi.synth.normal((m, k), seed=7)
    import ctypes as C

    def run(out, row_begin, row_end):
        st = rmi.lib().rmi_matmul_q4_k_q8k(ctx.handle, w._h, C.c_void_p(x.ctypes.data), C.c_size_t(m),
                                           C.c_void_p(out.ctypes.data), C.c_size_t(row_begin), C.c_size_t(row_end))
        assert st == 0, rmi.lib().rmi_last_error()

    got = np.zeros((m, n), np.float32)
    run(got, 0, n)
    for t in (0, 1, m // 2, m - 1):
        ref = orc.q4k_forward_prepared(wb, x[t], k, n, 0, 1, orc.SEM_AVX2)
        assert np.array_equal(bits(got[t]), bits(ref)), t
    part = np.zeros((m, n), np.float32)
    run(part, 5, n - 3)
    assert np.array_equal(bits(part[:, 5:n - 3]), bits(got[:, 5:n - 3]))
    assert not part[:, :5].any() and not part[:, n - 3:].any()
    w.free()


@pytest.mark.parametrize("m", [2, 5, 8, 13, 31])
def test_q4k_q8k_few_rows_stream_and_split_k_kernels_bit_exact(rmi, ctx, m):
    """m < 32 under AVX2 semantics: groups of 8 / 4 rows through the streaming kernel, the last 2 / 1 rows through
    the split-K kernel.  Six super-blocks per row (one full chunk of four and a short one), a weight row count that
    is no multiple of the 16- and 4-row tiles, and a row range that starts and ends inside a tile."""
    ctx.set_semantics(rmi.SEM_AVX2)
    n, k = 100, 1536
    wb = rmi.synth.q4_k_weight(n, k, seed=20 + m)
    w = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q4_K, k, n)
    x = rmi.synth.normal((m, k), seed=8)
    import ctypes as C

    def run(out, row_begin, row_end):
        st = rmi.lib().rmi_matmul_q4_k_q8k(ctx.handle, w._h, C.c_void_p(x.ctypes.data), C.c_size_t(m),
                                           C.c_void_p(out.ctypes.data), C.c_size_t(row_begin), C.c_size_t(row_end))
        assert st == 0, rmi.lib().rmi_last_error()

    got = np.zeros((m, n), np.float32)
    run(got, 0, n)
    ref = np.stack([orc.q4k_forward_prepared(wb, x[t], k, n, 0, 1, orc.SEM_AVX2) for t in range(m)])
    assert np.array_equal(bits(got), bits(ref))
    part = np.zeros((m, n), np.float32)
    run(part, 5, n - 3)
    assert np.array_equal(bits(part[:, 5:n - 3]), bits(ref[:, 5:n - 3]))
    assert not part[:, :5].any() and not part[:, n - 3:].any()
    w.free()
