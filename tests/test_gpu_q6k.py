"""Q6_K through the C ABI against the oracle: vec_dot_q6k_q8k bit-exact in the AVX2 and scalar orders,
the Q8_0-activation path within tolerance, the dequantizer exact, the (ith, nth) partition."""
import numpy as np
import pytest

from helpers import bits, rel_err
from oracle import orc

pytestmark = pytest.mark.gpu


@pytest.fixture
def ctx(rmi):
    c = rmi.context(0)
    yield c
    c.set_semantics(rmi.SEM_AVX2)


def test_q6_k_dequantize_exact(rmi, ctx):
    n, k = 24, 512
    wb = rmi.synth.q6_k_weight(n, k, seed=3)
    w = rmi.QuantizedTensor.from_bytes(wb, rmi.GGML_Q6_K, k, n)
    got = rmi.dequantize_q6_k(w)
    ref = np.stack([orc.dequantize_row_q6_k(wb[r * 420:(r + 1) * 420], k) for r in range(n)])
    assert np.array_equal(bits(got), bits(ref))
    w.free()


@pytest.mark.parametrize("sem", [orc.SEM_AVX2, orc.SEM_SCALAR])
@pytest.mark.parametrize("m,n,k", [(1, 40, 256), (1, 130, 1024), (5, 33, 512), (9, 64, 768)])
def test_q6_k_q8k_bit_exact(rmi, ctx, sem, m, n, k):
    ctx.set_semantics(sem)
    wb = rmi.synth.q6_k_weight(n, k, seed=n + k)
    kern = rmi.Q6_KKernel.new(wb, k, n)
    x = rmi.synth.normal((m, k), seed=m + 2)
    out = np.zeros((m, n), np.float32)
    kern.forward_prepared(x, None, None, None, out, k, n, 0, 1)
    ref = np.stack([orc.q6k_forward_prepared(wb, x[t], k, n, sem=sem) for t in range(m)])
    assert np.array_equal(bits(out), bits(ref))


def test_q6_k_reference_fixture_and_partition(rmi, ctx):
    # the four-block fixture of src/ops/quant/mod.rs:1187-1211 as a one-row weight, then a row partition
    blocks = []
    for i in range(4):
        v = np.zeros(210, np.uint8)
        v[:128] = [(i * 11 + j * 3) % 4 for j in range(128)]
        v[128:192] = [(i + j * 7) % 4 for j in range(64)]
        v[192:208] = np.array([(i * 5 + kk) - 6 for kk in range(16)], np.int8).view(np.uint8)
        v[208:210] = np.array([0.01 + i * 0.1], np.float16).view(np.uint8)
        blocks.append(v)
    wb = np.concatenate(blocks)
    x = np.array([(i - 512.0) * 0.01 for i in range(1024)], np.float32)
    for sem in (orc.SEM_AVX2, orc.SEM_SCALAR):
        ctx.set_semantics(sem)
        kern = rmi.Q6_KKernel.new(wb, 1024, 1)
        out = np.zeros(1, np.float32)
        kern.forward_prepared(x, None, None, None, out, 1024, 1, 0, 1)
        assert np.array_equal(bits(out), bits(orc.q6k_forward_prepared(wb, x, 1024, 1, sem=sem)))
    ctx.set_semantics(orc.SEM_AVX2)
    n, k = 37, 512
    wb = rmi.synth.q6_k_weight(n, k, seed=8)
    kern = rmi.Q6_KKernel.new(wb, k, n)
    x = rmi.synth.normal((1, k), seed=9)
    out = np.zeros(n, np.float32)
    for ith in range(5):
        kern.forward_prepared(x, None, None, None, out, k, n, ith, 5)
    assert np.array_equal(bits(out), bits(orc.q6k_forward_prepared(wb, x[0], k, n)))


def test_q6_k_prequantized_path_within_tolerance(rmi, ctx):
    n, k = 48, 1024
    wb = rmi.synth.q6_k_weight(n, k, seed=4)
    kern = rmi.Q6_KKernel.new(wb, k, n)
    x = rmi.synth.normal((1, k), seed=5)
    q8, sc = orc.quantize_q8_0(x[0], orc.SEM_AVX2)
    out = np.zeros(n, np.float32)
    for ith in range(3):
        kern.forward_prequantized(q8, sc, out, k, n, ith, 3)
    ref = orc.q6k_forward_prequantized(wb, q8, sc, k, n)
    assert rel_err(out, ref) < 1e-4


def test_q6_k_rejects_neon_and_wrong_type(rmi, ctx):
    wb = rmi.synth.q6_k_weight(8, 256, seed=1)
    kern = rmi.Q6_KKernel.new(wb, 256, 8)
    ctx.set_semantics(rmi.SEM_NEON)
    with pytest.raises(rmi.RmiError):
        kern.forward_prepared(np.zeros(256, np.float32), None, None, None, np.zeros(8, np.float32), 256, 8, 0, 1)
    ctx.set_semantics(rmi.SEM_AVX2)
    q4 = rmi.QuantizedTensor.from_bytes(rmi.synth.q4_k_weight(8, 256, seed=1), rmi.GGML_Q4_K, 256, 8)
    with pytest.raises(rmi.RmiError):
        rmi.dequantize_q6_k(q4)
    q4.free()


@pytest.mark.parametrize("ggml,gen,row_bytes", [(8, "q8_0_weight", 34 / 32), (2, "q4_0_weight", 18 / 32), (14, "q6_k_weight", 210 / 256)])
def test_embedding_lookup_bit_exact(rmi, ctx, ggml, gen, row_bytes):
    """src/ops/embedding.rs:3-47 for the three table types."""
    vocab, n_embd = 50, 512
    wb = getattr(rmi.synth, gen)(vocab, n_embd, seed=ggml)
    w = rmi.QuantizedTensor.from_bytes(wb, ggml, n_embd, vocab)
    ids = [0, 49, 17, 17, 33]
    got = rmi.embedding_lookup(w, ids)
    ref = np.stack([orc.embedding_lookup(wb, t, n_embd, ggml) for t in ids])
    assert np.array_equal(bits(got), bits(ref))
    with pytest.raises(rmi.RmiError):
        rmi.embedding_lookup(w, [50])
    w.free()
