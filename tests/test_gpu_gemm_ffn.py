"""Prefill-shaped calls (M > 32): tcgen05 int8 GEMM and the fused SwiGLU FFN vs the oracle."""
import numpy as np
import pytest

from oracle import orc
from tests.helpers import bits, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx(rmi):
    c = rmi.context(0)
    yield c
    c.set_semantics(rmi.SEM_AVX2)


@pytest.mark.parametrize("m,n,k", [(33, 128, 128), (128, 128, 32), (128, 256, 1024), (130, 200, 96), (512, 3072, 1024),
                                   (256, 1024, 3072), (64, 40, 64)])
def test_tensor_core_block_sums_are_exact(rmi, ctx, m, n, k):
    wb = rmi.synth.q8_0_weight(n, k, seed=n + k)
    w = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q8_0, k, n)
    q8, _ = orc.quantize_q8_0(rmi.synth.normal((m, k), seed=m), orc.SEM_AVX2)
    if m * n * (k // 32) > 6_000_000:   # keep the debug dump small: check a row subset on the host
        m_chk = 130
        q8 = q8[:m_chk]
        m = m_chk
    got = rmi.q8_0_block_sums(w, q8, m, use_tensor_cores=True)
    ref = rmi.q8_0_block_sums(w, q8, m, use_tensor_cores=False)
    assert np.array_equal(got, ref)
    for t in (0, m - 1):
        assert np.array_equal(got[t], orc.q8_0_block_sums(wb, q8[t], k, 0, n))
    w.free()


@pytest.mark.parametrize("sem", [orc.SEM_NEON, orc.SEM_SCALAR])
@pytest.mark.parametrize("m,n,k", [(33, 128, 128), (128, 256, 1024), (130, 200, 96), (512, 3072, 1024), (200, 1024, 3072)])
def test_gemm_bit_exact_in_whole_block_semantics(rmi, ctx, sem, m, n, k):
    ctx.set_semantics(sem)
    wb = rmi.synth.q8_0_weight(n, k, seed=n * 3 + k)
    w = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q8_0, k, n)
    x = rmi.synth.normal((m, k), seed=m + 5)
    got = rmi.matmul_q8_0(w, x)
    ref = orc.q8_forward_batched(wb, x, k, n, sem, threads=8)
    assert np.array_equal(bits(got), bits(ref))
    # the M <= 32 GEMV kernels give the same bits as the GEMM for the same rows
    assert np.array_equal(bits(rmi.matmul_q8_0(w, x[:7])), bits(got[:7]))
    w.free()


def test_gemm_avx2_exact_path_and_tensor_core_path(rmi, ctx):
    """AVX2 semantics, m > 32.  rmi_set_prefill_exact(1): CUDA cores, the reference's eight-lane order bit for
    bit.  Default: tcgen05 -- the device's output carries the bits of the oracle's whole-block chain over the
    AVX2-quantized activations and lies within 1e-5 of the eight-lane order."""
    m, n, k = 160, 512, 1024
    wb = rmi.synth.q8_0_weight(n, k, seed=77)
    w = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q8_0, k, n)
    x = rmi.synth.normal((m, k), seed=78)
    ctx.set_semantics(rmi.SEM_AVX2)
    ref = orc.q8_forward_batched(wb, x, k, n, orc.SEM_AVX2, threads=8)
    ctx.set_prefill_exact(True)
    try:
        launches = ctx.launch_count()
        got = rmi.matmul_q8_0(w, x)
        assert np.array_equal(bits(got), bits(ref))
    finally:
        ctx.set_prefill_exact(False)
    tc = rmi.matmul_q8_0(w, x)                      # read from the device: the tensor-core result
    block = orc.q8_forward_batched(wb, x, k, n, orc.SEM_AVX2_BLOCK, threads=8)
    assert np.array_equal(bits(tc), bits(block))
    assert rel_err(tc, ref) < 1e-5                  # tolerance stated by the path's contract
    assert not np.array_equal(bits(tc), bits(ref))  # the two orders do differ in the last bits
    assert ctx.launch_count() > launches
    w.free()


def _c2_weights(rmi, e, ff):
    return (rmi.synth.q8_0_weight(ff, e, seed=0), rmi.synth.q8_0_weight(ff, e, seed=1),
            rmi.synth.q8_0_weight(e, ff, seed=2))


def test_config2_avx2_default_runs_on_tensor_cores_within_contract(rmi, ctx):
    """BASELINE config 2 (M=512, K=1024, n_ff=3072) under the library's default setting (AVX2 semantics,
    tensor cores).  Checked on the device's output: activation bytes and scale bits equal the AVX2 quantizer,
    int32 block sums equal the oracle's, gate and up projections within 1e-5 of the eight-lane order, the down
    projection within 1e-5 on identical quantized activations, and the whole FFN bit-equal to the oracle's
    statement of this path."""
    m, e, ff = 512, 1024, 3072
    ctx.set_semantics(rmi.SEM_AVX2)
    g, u, d = _c2_weights(rmi, e, ff)
    wg = rmi.QuantizedTensor.from_bytes(g, rmi.GGML_Q8_0, e, ff)
    wu = rmi.QuantizedTensor.from_bytes(u, rmi.GGML_Q8_0, e, ff)
    wd = rmi.QuantizedTensor.from_bytes(d, rmi.GGML_Q8_0, ff, e)
    wgu = wg.fuse_vstack(wu)
    x = rmi.synth.normal((m, e), seed=3)
    # (1) quantizer: bytes and scale bits
    q8, sc = rmi.quantize_q8_0(x.reshape(-1), e)
    rq, rs = orc.quantize_q8_0(x, orc.SEM_AVX2)
    assert np.array_equal(q8.reshape(m, e), rq) and np.array_equal(bits(sc).reshape(m, -1), bits(rs))
    # (2) block sums out of the int8 MMA (a row subset keeps the dump small)
    rows = np.r_[0:40, 200:230, 480:512]
    sums = rmi.q8_0_block_sums(wg, rq[rows], len(rows), use_tensor_cores=True)
    for i in (0, 39, 40, len(rows) - 1):
        assert np.array_equal(sums[i], orc.q8_0_block_sums(g, rq[rows[i]], e, 0, ff))
    # (3) gate | up projection on the tensor cores vs the eight-lane order
    gu = rmi.matmul_q8_0(wgu, x)
    ref_gu = np.concatenate([orc.q8_forward_batched(g, x, e, ff, orc.SEM_AVX2, threads=8),
                             orc.q8_forward_batched(u, x, e, ff, orc.SEM_AVX2, threads=8)], axis=1)
    assert rel_err(gu, ref_gu) < 1e-5
    # (4) whole FFN: bits of the oracle's statement of the path; the eight-lane FFN differs only where the
    # re-quantization of the activation (a discontinuous step) flips a byte or a scale bit
    got = rmi.ffn_swiglu_q8_0(wgu, wd, x)
    blk, act_blk = orc.ffn_swiglu_q8_0(g, u, d, x, e, ff, orc.SEM_AVX2_BLOCK, threads=8, want_act=True)
    assert np.array_equal(bits(got), bits(blk))
    avx, act_avx = orc.ffn_swiglu_q8_0(g, u, d, x, e, ff, orc.SEM_AVX2, threads=8, want_act=True)
    assert rel_err(act_blk, act_avx) < 1e-5
    qa, sa = orc.quantize_q8_0(act_avx, orc.SEM_AVX2)
    qb, sb = orc.quantize_q8_0(act_blk, orc.SEM_AVX2)
    same_rows = np.flatnonzero((qa == qb).all(axis=1) & (bits(sa) == bits(sb)).all(axis=1))
    assert len(same_rows) > m * 0.9
    assert rel_err(got[same_rows], avx[same_rows]) < 1e-5
    assert rel_err(got, avx) < 5e-3
    # (5) down projection alone on identical quantized activations
    dn = rmi.matmul_q8_0(wd, act_avx)
    assert rel_err(dn, orc.q8_forward_batched(d, act_avx, ff, e, orc.SEM_AVX2, threads=8)) < 1e-5
    for w in (wg, wu, wd, wgu):
        w.free()


def test_config5_shard_avx2_default_within_contract(rmi, ctx):
    """One 8-GPU shard of BASELINE config 5 (rows [4096, 8192) of W [32768, 8192]) at M=256 under the default
    setting: device output bit-equal to the oracle's whole-block chain and within 1e-5 of the eight-lane order."""
    n, k, m, s, e = 32768, 8192, 256, 4096, 8192
    ctx.set_semantics(rmi.SEM_AVX2)
    wb = rmi.synth.q8_0_weight_rows(n, k, seed=0, row_begin=s, row_end=e)
    w = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q8_0, k, e - s)
    x = rmi.synth.normal((m, k), seed=1)
    got = rmi.matmul_q8_0(w, x)
    assert np.array_equal(bits(got), bits(orc.q8_forward_batched(wb, x, k, e - s, orc.SEM_AVX2_BLOCK, threads=8)))
    assert rel_err(got, orc.q8_forward_batched(wb, x, k, e - s, orc.SEM_AVX2, threads=8)) < 1e-5
    w.free()


@pytest.mark.parametrize("sem", [orc.SEM_NEON, orc.SEM_SCALAR])
@pytest.mark.parametrize("m,n,k", [(9, 128, 128), (16, 1000, 96), (32, 384, 1024), (33, 130, 160), (40, 256, 3072),
                                   (96, 200, 64), (16, 4096, 1024)])
def test_small_batch_gemm_with_swapped_operands_is_bit_exact(rmi, ctx, sem, m, n, k):
    """8 < m <= 96: the weight is the 128-row MMA operand and the activation rows are tile columns
    (transposed store); ragged n (rows of the last weight tile) and ragged m (columns of the last block)."""
    ctx.set_semantics(sem)
    wb = rmi.synth.q8_0_weight(n, k, seed=n + 7 * k)
    w = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q8_0, k, n)
    x = rmi.synth.normal((m, k), seed=m + 11)
    got = rmi.matmul_q8_0(w, x)
    ref = orc.q8_forward_batched(wb, x, k, n, sem, threads=8)
    assert np.array_equal(bits(got), bits(ref))
    assert np.array_equal(bits(rmi.matmul_q8_0(w, x)), bits(got))   # run twice: same bits
    w.free()


@pytest.mark.parametrize("sem", [orc.SEM_AVX2, orc.SEM_NEON, orc.SEM_SCALAR])
@pytest.mark.parametrize("m", [1, 5, 32])
def test_ffn_decode_shapes_bit_exact(rmi, ctx, sem, m):
    ctx.set_semantics(sem)
    e, ff = 256, 768
    g, u, d = (rmi.synth.q8_0_weight(ff, e, seed=1), rmi.synth.q8_0_weight(ff, e, seed=2),
               rmi.synth.q8_0_weight(e, ff, seed=3))
    wg = rmi.QuantizedTensor.from_bytes(g, rmi.GGML_Q8_0, e, ff)
    wu = rmi.QuantizedTensor.from_bytes(u, rmi.GGML_Q8_0, e, ff)
    wd = rmi.QuantizedTensor.from_bytes(d, rmi.GGML_Q8_0, ff, e)
    wgu = wg.fuse_vstack(wu)
    x = rmi.synth.normal((m, e), seed=4)
    got = rmi.ffn_swiglu_q8_0(wgu, wd, x)
    ref = orc.ffn_swiglu_q8_0(g, u, d, x, e, ff, sem)
    assert np.array_equal(bits(got), bits(ref))


@pytest.mark.parametrize("sem", [orc.SEM_NEON, orc.SEM_SCALAR, orc.SEM_AVX2, "avx2-exact"])
@pytest.mark.parametrize("m,e,ff", [(512, 1024, 3072), (130, 256, 768), (40, 128, 192)])
def test_ffn_prefill_bit_exact(rmi, ctx, sem, m, e, ff):
    # BASELINE config 2 at (512, 1024, 3072): gate/up seeds 0/1, down seed 2, x seed 3.
    # AVX2 on the tensor cores (default) is compared with the oracle's whole-block statement of that path,
    # "avx2-exact" (rmi_set_prefill_exact) with the reference's eight-lane order.
    exact = sem == "avx2-exact"
    dev_sem = orc.SEM_AVX2 if exact else sem
    ref_sem = orc.SEM_AVX2_BLOCK if sem == orc.SEM_AVX2 else dev_sem
    ctx.set_semantics(dev_sem)
    ctx.set_prefill_exact(exact)
    try:
        g, u, d = _c2_weights(rmi, e, ff)
        wgu = rmi.QuantizedTensor.from_bytes(g, rmi.GGML_Q8_0, e, ff).fuse_vstack(
            rmi.QuantizedTensor.from_bytes(u, rmi.GGML_Q8_0, e, ff))
        wd = rmi.QuantizedTensor.from_bytes(d, rmi.GGML_Q8_0, ff, e)
        x = rmi.synth.normal((m, e), seed=3)
        got = rmi.ffn_swiglu_q8_0(wgu, wd, x)
        ref = orc.ffn_swiglu_q8_0(g, u, d, x, e, ff, ref_sem, threads=8)
        assert np.array_equal(bits(got), bits(ref))
        again = rmi.ffn_swiglu_q8_0(wgu, wd, x)
        assert np.array_equal(bits(again), bits(got))
        if dev_sem != orc.SEM_AVX2:
            avx = orc.ffn_swiglu_q8_0(g, u, d, x[:8], e, ff, orc.SEM_AVX2)
            assert rel_err(got[:8], avx) < 2e-2  # different activation rounding; sanity bound only
    finally:
        ctx.set_prefill_exact(False)


@pytest.mark.parametrize("sem,m", [(orc.SEM_NEON, 130), (orc.SEM_AVX2, 3), (orc.SEM_SCALAR, 40)])
def test_ffn_pipelined_batches_equal_the_oracle_per_batch(rmi, ctx, sem, m):
    """Seven batches over two alternating weight sets, copies overlapped with the arithmetic:
    every batch must carry the oracle's bits (and so those of the one-batch entry point)."""
    torch = pytest.importorskip("torch")
    ctx.set_semantics(sem)
    e, ff, n = 256, 768, 7
    raw, sets = [], []
    for k in range(2):
        g, u, d = (rmi.synth.q8_0_weight(ff, e, seed=10 + k), rmi.synth.q8_0_weight(ff, e, seed=20 + k),
                   rmi.synth.q8_0_weight(e, ff, seed=30 + k))
        raw.append((g, u, d))
        sets.append((rmi.QuantizedTensor.from_bytes(g, rmi.GGML_Q8_0, e, ff).fuse_vstack(
            rmi.QuantizedTensor.from_bytes(u, rmi.GGML_Q8_0, e, ff)), rmi.QuantizedTensor.from_bytes(d, rmi.GGML_Q8_0, ff, e)))
    xs = [torch.from_numpy(rmi.synth.normal((m, e), seed=40 + i)).pin_memory() for i in range(n)]
    outs = [torch.full((m, e), float("nan")).pin_memory() for _ in range(n)]
    rmi.ffn_swiglu_q8_0_pipelined([sets[i % 2][0] for i in range(n)], [sets[i % 2][1] for i in range(n)],
                                  [x.data_ptr() for x in xs], [o.data_ptr() for o in outs], m)
    for i in range(n):
        g, u, d = raw[i % 2]
        ref = orc.ffn_swiglu_q8_0(g, u, d, xs[i].numpy(), e, ff, sem, threads=4)
        assert np.array_equal(bits(outs[i].numpy()), bits(ref)), i
    # pageable buffers: still correct
    x_np, o_np = rmi.synth.normal((m, e), seed=77), np.zeros((m, e), np.float32)
    rmi.ffn_swiglu_q8_0_pipelined([sets[0][0]], [sets[0][1]], [x_np.ctypes.data], [o_np.ctypes.data], m)
    assert np.array_equal(bits(o_np), bits(rmi.ffn_swiglu_q8_0(sets[0][0], sets[0][1], x_np)))
    with pytest.raises(ValueError):
        rmi.ffn_swiglu_q8_0_pipelined([sets[0][0]], [], [x_np.ctypes.data], [o_np.ctypes.data], m)


def test_silu_mul_matches_oracle_bits(rmi, ctx):
    g = rmi.synth.normal((3072,), seed=5) * np.float32(3.0)
    u = rmi.synth.normal((3072,), seed=6)
    got = u.copy()
    rmi.silu_mul_inplace(g, got)
    ref = u.copy()
    orc.silu_mul_inplace(g, ref)
    assert np.array_equal(bits(got), bits(ref))
    pin_g = np.array([0xbf44c6b5], np.uint32).view(np.float32)   # tests/quantized_inference.rs:20-29
    pin_u = np.array([0x3ddf57e5], np.uint32).view(np.float32).copy()
    rmi.silu_mul_inplace(pin_g, pin_u)
    assert bits(pin_u)[0] == 0xbcd98667


@pytest.mark.parametrize("sem,n_tokens", [(orc.SEM_NEON, 70), (orc.SEM_AVX2, 6)])
def test_qwen35_forward_ffn_parallel_matches_the_per_token_reference(rmi, ctx, sem, n_tokens):
    """src/models/qwen35.rs:762-782: gate/up per token, silu_mul over all tokens, down per token."""
    ctx.set_semantics(sem)
    e, ff = 256, 512
    g, u, d = (rmi.synth.q8_0_weight(ff, e, seed=61), rmi.synth.q8_0_weight(ff, e, seed=62),
               rmi.synth.q8_0_weight(e, ff, seed=63))
    ffn = rmi.Qwen35Ffn(rmi.QuantizedTensor.from_bytes(g, rmi.GGML_Q8_0, e, ff),
                        rmi.QuantizedTensor.from_bytes(u, rmi.GGML_Q8_0, e, ff),
                        rmi.QuantizedTensor.from_bytes(d, rmi.GGML_Q8_0, ff, e))
    hidden = rmi.synth.normal((n_tokens, e), seed=64)
    got = ffn.forward_ffn_parallel(hidden.reshape(-1), n_tokens)
    # the reference order, step by step, with the oracle's single-token kernels
    gate = orc.q8_forward_batched(g, hidden, e, ff, sem)
    up = orc.q8_forward_batched(u, hidden, e, ff, sem)
    act = np.ascontiguousarray(up.reshape(-1))
    orc.silu_mul_inplace(gate.reshape(-1), act)       # up[i] *= silu(gate[i]) over all tokens at once
    ref = orc.q8_forward_batched(d, act.reshape(n_tokens, ff), ff, e, sem)
    assert np.array_equal(bits(got), bits(ref))
    ffn.free()
