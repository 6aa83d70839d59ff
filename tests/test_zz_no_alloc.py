"""The allocation-free matmul entry point against the regular one.

Some hosts cannot let a plug-in call cudaMalloc: their own allocator already owns the device's
memory, or their serving loop cannot absorb the device-wide synchronisation an allocation causes.
rmi_matmul_q8_0_dev_noalloc keeps its scratch (the quantized activations) in a fixed array inside
the library instead.  This file is collected last on purpose: a failure here must not hide the
result of any other test in a run that stops at the first failure.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _dev(ctx, arr):
    p = ctx.dev_alloc(arr.nbytes)
    ctx.h2d(p, arr)
    return p


def test_noalloc_matches_the_regular_entry_point_on_two_consecutive_calls(rmi):
    ctx = rmi.context(0)
    ctx.set_semantics(rmi.SEM_AVX2)
    ctx.prof_enable(False)
    # two calls in a row with different shapes: the second one is smaller, so stale bytes of the
    # first call stay in the shared array and must not influence the result
    cases = [(3072, 1024, 8, 11), (515, 256, 3, 12)]
    weights = [rmi.QuantizedTensor.from_bytes(rmi.synth.q8_0_weight(n, k, seed=s), rmi.GGML_Q8_0, k, n)
               for n, k, _, s in cases]
    for (n, k, m, seed), w in zip(cases, weights):
        x = rmi.synth.normal((m, k), seed=seed + 100)
        dx = _dev(ctx, x)
        d_ref, d_new = ctx.dev_alloc(m * n * 4), ctx.dev_alloc(m * n * 4)
        rmi.matmul_q8_0_dev(w, dx, m, d_ref)
        rmi.matmul_q8_0_dev_noalloc(w, dx, m, d_new)
        ref, got = np.zeros((m, n), np.float32), np.zeros((m, n), np.float32)
        ctx.d2h(ref, d_ref)
        ctx.d2h(got, d_new)
        # same kernels, same inputs: bit-identical (the bar used for every f32 output in this suite)
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32)), (n, k, m)
        assert np.abs(ref).max() > 0
        for p in (dx, d_ref, d_new):
            ctx.dev_free(p)
    ctx.set_semantics(rmi.SEM_AVX2)


@pytest.mark.parametrize("sem", ["SEM_NEON", "SEM_SCALAR"])
def test_noalloc_equals_the_regular_entry_point_where_their_kernels_differ(rmi, sem):
    """Whole-block semantics with 9..32 rows: the regular entry point runs the swapped-operand tensor-core
    GEMM, the allocation-free one the GEMV.  Both must carry the oracle's bits.  The last case fills the
    fixed array exactly (32 x 16384 = 524288 values)."""
    from oracle import orc
    ctx = rmi.context(0)
    ctx.set_semantics(getattr(rmi, sem))
    ctx.prof_enable(False)
    try:
        for n, k, m, seed in [(1000, 256, 16, 5), (384, 1024, 32, 6), (48, 16384, 32, 7)]:
            wb = rmi.synth.q8_0_weight(n, k, seed=seed)
            w = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q8_0, k, n)
            x = rmi.synth.normal((m, k), seed=seed + 50)
            dx = _dev(ctx, x)
            d_ref, d_new = ctx.dev_alloc(m * n * 4), ctx.dev_alloc(m * n * 4)
            rmi.matmul_q8_0_dev(w, dx, m, d_ref)
            rmi.matmul_q8_0_dev_noalloc(w, dx, m, d_new)
            ref, got = np.zeros((m, n), np.float32), np.zeros((m, n), np.float32)
            ctx.d2h(ref, d_ref)
            ctx.d2h(got, d_new)
            assert np.array_equal(got.view(np.uint32), ref.view(np.uint32)), (n, k, m)
            want = orc.q8_forward_batched(wb, x, k, n, getattr(orc, sem), threads=4)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (n, k, m)
            for p in (dx, d_ref, d_new):
                ctx.dev_free(p)
            w.free()
    finally:
        ctx.set_semantics(rmi.SEM_AVX2)


def test_noalloc_rejects_sizes_beyond_the_fixed_array(rmi):
    ctx = rmi.context(0)
    w = rmi.QuantizedTensor.from_bytes(rmi.synth.q8_0_weight(16, 32768, seed=1), rmi.GGML_Q8_0, 32768, 16)
    dx, dout = ctx.dev_alloc(33 * 32768 * 4), ctx.dev_alloc(33 * 16 * 4)
    with pytest.raises(rmi.RmiError) as e:          # 17 * 32768 > 524288 values
        rmi.matmul_q8_0_dev_noalloc(w, dx, 17, dout)
    assert e.value.status == 2 and "fixed scratch array" in e.value.message
    with pytest.raises(rmi.RmiError) as e:          # more than 32 rows
        rmi.matmul_q8_0_dev_noalloc(w, dx, 33, dout)
    assert e.value.status == 2
    ctx.dev_free(dx)
    ctx.dev_free(dout)
