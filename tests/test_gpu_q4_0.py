"""Q4_0 through the C ABI against the oracle (bit-exact) and the reference's known answers."""
import numpy as np
import pytest

from helpers import bits
from oracle import orc

pytestmark = pytest.mark.gpu


def _block(scale, lo, hi=None):
    hi = lo if hi is None else hi
    return np.concatenate([np.array([scale], np.float16).view(np.uint8), np.full(16, lo | (hi << 4), np.uint8)])


def test_q4_0_reference_known_answers(rmi):
    # src/ops/kernel/q4_0/mod.rs:99-123
    q8, sc = np.full(32, 1, np.int8).view(np.uint8), np.ones(1, np.float32)
    for nib, want in ((8, 0.0), (9, 32.0)):
        out = np.full(1, np.nan, np.float32)
        rmi.Q4_0Kernel.new(_block(1.0, nib), 32, 1).forward_prequantized(q8, sc, out, 32, 1, 0, 1)
        assert out[0] == want


@pytest.mark.parametrize("n,k", [(1, 32), (33, 96), (64, 1024), (130, 2080)])
def test_q4_0_bit_exact_and_partition(rmi, n, k):
    wb = rmi.synth.q4_0_weight(n, k, seed=n + k)
    kern = rmi.Q4_0Kernel.new(wb, k, n)
    x = rmi.synth.normal((1, k), seed=7)
    q8, sc = orc.quantize_q8_0(x[0], orc.SEM_AVX2)
    out = np.zeros(n, np.float32)
    for ith in range(3):
        kern.forward_prequantized(q8, sc, out, k, n, ith, 3)
    assert np.array_equal(bits(out), bits(orc.q4_0_forward_prequantized(wb, q8, sc, k, n)))


def test_q4_0_extreme_blocks(rmi):
    # the edge inputs of src/ops/kernel/q4_0/avx2.rs:247-330
    for nib, q in [(0, np.full(32, -128, np.int8)), (15, np.full(32, 127, np.int8)), (0, np.full(32, 127, np.int8)),
                   (11, np.array([127 if i % 2 else -127 for i in range(32)], np.int8))]:
        w = _block(0.5, nib, 15 - nib)
        out = np.zeros(1, np.float32)
        sc = np.array([0.25], np.float32)
        rmi.Q4_0Kernel.new(w, 32, 1).forward_prequantized(q.view(np.uint8), sc, out, 32, 1, 0, 1)
        assert np.array_equal(bits(out), bits(orc.q4_0_forward_prequantized(w, q.view(np.uint8), sc, 32, 1)))


@pytest.mark.parametrize("sem", ["SEM_AVX2", "SEM_NEON", "SEM_SCALAR"])
def test_q4_0_forward_quantizes_with_the_context_semantics(rmi, sem):
    ctx = rmi.context(0)
    ctx.set_semantics(getattr(rmi, sem))
    n, k, m = 48, 256, 5
    wb = rmi.synth.q4_0_weight(n, k, seed=2)
    w = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q4_0, k, n)
    x = rmi.synth.normal((m, k), seed=3)
    got = rmi.matmul_q4_0(w, x)
    ref = np.zeros((m, n), np.float32)
    for t in range(m):
        q8, sc = orc.quantize_q8_0(x[t], getattr(orc, sem))
        ref[t] = orc.q4_0_forward_prequantized(wb, q8, sc, k, n)
    assert np.array_equal(bits(got), bits(ref))
    w.free()
    ctx.set_semantics(rmi.SEM_AVX2)
