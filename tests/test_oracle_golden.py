"""Pins the CPU oracle against the known-answer vectors held by the reference's own tests.

Each test names the reference test it restates (path:line inside the reference project).
The vectors were read from the reference's test sources; nothing here runs the reference.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import orc
from tests.helpers import (bits, f16_bits, make_q8_0_weight, q8_0_uniform_row, ramp_input,
                           rel_err, synth_q8_0)

SEMS = [orc.SEM_AVX2, orc.SEM_NEON, orc.SEM_SCALAR]


def f32(bits_):
    return np.array(bits_, np.uint32).view(np.float32)


# ---------------------------------------------------------------- f16 conversion

def test_f16_roundtrip_all_half_values():
    allh = np.arange(65536, dtype=np.uint16)
    ref = allh.view(np.float16).astype(np.float32)
    got = np.array([orc.lib().orc_f16_to_f32(int(h)) for h in allh[::7]], np.float32)
    assert np.array_equal(bits(got)[~np.isnan(got)], bits(ref[::7])[~np.isnan(got)])


def test_f32_to_f16_matches_ieee_rne():
    rng = np.random.default_rng(5)
    x = np.concatenate([
        rng.standard_normal(200000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 200000).astype(np.float32),
        f32([0x33000000, 0x33000001, 0x477fefff, 0x477ff000, 0x38800000, 0x387fffff, 0x33800000,
             0x00000001, 0x80000000, 0x7f800000, 0xff800000, 0x3f801000, 0x3f803000, 0x3f801001]),
    ]).astype(np.float32)
    with np.errstate(over="ignore"):
        ref = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(orc.f32_to_f16_bits(x), ref)


def test_f16_from_bytes_is_the_same_decode():
    # src/ops/quant/mod.rs:13-22 vs src/ops/float.rs:177-191 on finite values
    for h in list(range(0, 0x7c00, 37)) + [0x8001, 0xbc00, 0x0001, 0x03ff, 0x0400]:
        b = np.array([h], np.uint16).view(np.uint8)
        a = orc.lib().orc_f16_from_bytes(b.ctypes.data_as(C.c_void_p), 2, 0)
        assert np.float32(a) == np.float32(orc.lib().orc_f16_to_f32(h))


# ---------------------------------------------------------------- Q8_0 quantizer

@pytest.mark.parametrize("sem", SEMS)
def test_q8_quantization_stores_f16_scale_without_requantizing_values(sem):
    # src/ops/matmul_tests.rs:558-571
    x = np.zeros(32, np.float32)
    x[0] = 1.0
    x[1] = f32([0x3d11213e])[0]
    q8, sc = orc.quantize_q8_0(x, sem)
    assert q8.view(np.int8)[0] == 127 and q8.view(np.int8)[1] == 4
    assert not q8[2:].any()
    assert bits(sc)[0] == 0x3c010000


def test_parity_q8_0_uses_llama_scalar_rounding():
    # tests/quantized_inference.rs:55-66 (half away from zero)
    x = np.zeros(32, np.float32)
    x[:3] = [127.0, 0.5, -0.5]
    q8, _ = orc.quantize_q8_0(x, orc.SEM_SCALAR)
    assert list(q8.view(np.int8)[:3]) == [127, 1, -1]


@pytest.mark.parametrize("sem", [orc.SEM_NEON, orc.SEM_AVX2])
def test_q8_quantization_uses_ties_to_even(sem):
    # src/ops/matmul_tests.rs:546-556 (NEON); the AVX2 path rounds the same way (q8_0.rs:211)
    x = np.zeros(32, np.float32)
    x[0], x[1] = 127.0, 34.5
    q8, _ = orc.quantize_q8_0(x, sem)
    assert q8.view(np.int8)[1] == 34


def test_neon_q8_quantization_matches_scalar():
    # src/ops/matmul_tests.rs:528-543
    x = np.array([((i % 17) - 8) * 0.125 for i in range(64)], np.float32)
    qs, ss = orc.quantize_q8_0(x, orc.SEM_SCALAR)
    qn, sn = orc.quantize_q8_0(x, orc.SEM_NEON)
    assert np.array_equal(qs, qn) and np.array_equal(bits(ss), bits(sn))


def test_quantizer_zero_block_and_intrinsics_agree():
    rng = np.random.default_rng(1)
    x = rng.standard_normal(4096).astype(np.float32)
    x[64:96] = 0.0
    q, s = orc.quantize_q8_0(x, orc.SEM_AVX2)
    assert not q[64:96].any() and s[2] == 0.0
    if orc.lib().orc_has_avx2_fast():
        qf, sf = orc.quantize_q8_0(x, orc.SEM_AVX2, fast=True)
        assert np.array_equal(q, qf) and np.array_equal(bits(s), bits(sf))


# ---------------------------------------------------------------- Q8_0 GEMV

@pytest.mark.parametrize("sem", SEMS)
def test_q8_kernel_uniform_weights_multi_row_and_scale(sem):
    # src/ops/kernel/q8_0/mod.rs:74-116
    q8 = np.ones(32, np.uint8)
    sc = np.ones(1, np.float32)
    w = q8_0_uniform_row(1, 1.0)
    assert list(orc.matmul_q8_0_range(w, q8, sc, 32, 0, 1, sem)) == [32.0]
    w2 = np.concatenate([w, w])
    assert list(orc.matmul_q8_0_range(w2, q8, sc, 32, 0, 2, sem)) == [32.0, 32.0]
    assert list(orc.matmul_q8_0_range(q8_0_uniform_row(1, 0.5), q8, sc, 32, 0, 1, sem)) == [16.0]


@pytest.mark.parametrize("sem", SEMS)
def test_q8_kernel_forward_quantizes_internally(sem):
    # src/ops/kernel/q8_0/mod.rs:118-129
    out = orc.q8_forward_batched(q8_0_uniform_row(1, 1.0), np.ones(32, np.float32), 32, 1, sem)
    assert abs(out[0, 0] - 32.0) < 5e-3


@pytest.mark.parametrize("sem", SEMS)
def test_q8_kernel_thread_partition(sem):
    # src/ops/kernel/q8_0/mod.rs:131-156
    w = np.concatenate([q8_0_uniform_row(1, 1.0)] * 4)
    q8, sc = np.ones(32, np.uint8), np.ones(1, np.float32)
    a = np.zeros(4, np.float32)
    orc.matmul_q8_0_parallel_rows(w, q8, sc, a, 32, 4, 0, 2, sem)
    b = np.zeros(4, np.float32)
    orc.matmul_q8_0_parallel_rows(w, q8, sc, b, 32, 4, 1, 2, sem)
    assert list(a) == [32.0, 32.0, 0.0, 0.0] and list(b) == [0.0, 0.0, 32.0, 32.0]


def test_neon_q8_matmul_matches_repacked_fused_block_accumulation():
    # src/ops/matmul_tests.rs:288-306
    blk = np.zeros(34, np.uint8)
    blk[0:2] = np.array([0x1800], np.uint16).view(np.uint8)
    blk[2] = 127
    w = np.concatenate([blk, blk])
    q8 = np.zeros(64, np.uint8)
    q8[0] = np.uint8(-127 & 0xff)
    q8[32] = 127
    sc = np.array([orc.lib().orc_f16_to_f32(0x1800), orc.lib().orc_f16_to_f32(0x1a7d)], np.float32)
    out = orc.matmul_q8_0_range(w, q8, sc, 64, 0, 1, orc.SEM_NEON)
    assert bits(out)[0] == 0x3d1cc57d


@pytest.mark.parametrize("n_out", [3584, 7168])
@pytest.mark.parametrize("sem", SEMS)
def test_parallel_matches_reference_bit_exact(n_out, sem):
    # tests/q8_0_parallel_matmul.rs:110-145 (threads 1/2/4/8, bit equality)
    n_in = 1024
    w = make_q8_0_weight(n_out, n_in, 7)
    q8, sc = orc.quantize_q8_0(ramp_input(n_in), sem)
    ref = orc.matmul_q8_0_range(w, q8, sc, n_in, 0, n_out, sem)
    assert np.isfinite(ref).all() and np.abs(ref).max() > 0
    for nth in (1, 2, 4, 8):
        out = np.zeros(n_out, np.float32)
        for ith in range(nth):
            orc.matmul_q8_0_parallel_rows(w, q8, sc, out, n_in, n_out, ith, nth, sem)
        assert np.array_equal(bits(out), bits(ref)), f"nth={nth}"


def test_avx2_intrinsics_kernel_is_bit_identical_to_the_restatement():
    if not orc.lib().orc_has_avx2_fast():
        pytest.skip("no AVX2 on this host")
    for n_in, n_out in ((1024, 3072), (64, 7), (3072, 1023)):
        w = synth_q8_0(n_out, n_in, seed=n_out)
        x = np.random.default_rng(2).standard_normal(n_in).astype(np.float32)
        q8, sc = orc.quantize_q8_0(x, orc.SEM_AVX2)
        a = orc.matmul_q8_0_range(w, q8, sc, n_in, 1, n_out, orc.SEM_AVX2)
        b = orc.matmul_q8_0_range(w, q8, sc, n_in, 1, n_out, orc.SEM_AVX2, fast=True)
        assert np.array_equal(bits(a), bits(b))


def test_three_isa_variants_agree_within_the_stated_tolerance():
    # docs/OPTIMIZATION.md:330-332 records the drift between variants; 1e-5 relative is the bar.
    w = synth_q8_0(3072, 1024, seed=0)
    x = np.random.default_rng(1).standard_normal(1024).astype(np.float32)
    q8, sc = orc.quantize_q8_0(x, orc.SEM_AVX2)
    ref = orc.matmul_q8_0_range(w, q8, sc, 1024, 0, 3072, orc.SEM_SCALAR)
    for sem in (orc.SEM_AVX2, orc.SEM_NEON):
        assert rel_err(orc.matmul_q8_0_range(w, q8, sc, 1024, 0, 3072, sem), ref) < 1e-5


def test_micro_bench_self_check_auto_vs_scalar():
    # src/bin/micro_bench.rs:110-120: 1e-4 + 1e-4*|ref| per row
    rng = np.random.default_rng(42)
    n_in, n_out = 1024, 3072
    wq = rng.integers(-127, 128, size=(n_out, n_in // 32, 32)).astype(np.int8)
    ws = rng.uniform(0.005, 0.025, size=(n_out, n_in // 32)).astype(np.float16).view(np.uint16)
    w = np.zeros((n_out, n_in // 32, 34), np.uint8)
    w[:, :, 0], w[:, :, 1], w[:, :, 2:] = ws & 0xff, ws >> 8, wq.view(np.uint8)
    q8, sc = orc.quantize_q8_0(rng.uniform(-1, 1, n_in).astype(np.float32), orc.SEM_AVX2)
    a = orc.matmul_q8_0_range(w, q8, sc, n_in, 0, n_out, orc.SEM_AVX2)
    s = orc.matmul_q8_0_range(w, q8, sc, n_in, 0, n_out, orc.SEM_SCALAR)
    assert np.all(np.abs(a - s) <= 1e-4 + 1e-4 * np.abs(s))


def test_block_sums_are_exact_integers():
    w = synth_q8_0(16, 256, seed=3)
    q8, _ = orc.quantize_q8_0(np.random.default_rng(4).standard_normal(256).astype(np.float32))
    got = orc.q8_0_block_sums(w, q8, 256, 0, 16)
    wq = w.reshape(16, 8, 34)[:, :, 2:].view(np.int8).astype(np.int64)
    ref = (wq * q8.view(np.int8).reshape(1, 8, 32).astype(np.int64)).sum(-1)
    assert np.array_equal(got, ref)


# ---------------------------------------------------------------- fusion

@pytest.mark.parametrize("sem", SEMS)
def test_fused_q8_0_matches_separate(sem):
    # tests/fused_ffn_matmul_parity.rs:92-127, src/ops/quant/fuse.rs:147-184
    n_in, n = 1024, 3584
    gate, up = make_q8_0_weight(n, n_in, 0), make_q8_0_weight(n, n_in, 17)
    q8, sc = orc.quantize_q8_0(ramp_input(n_in), sem)
    fused, rows = orc.fuse_vstack(gate, n, up, n)
    assert rows == 2 * n
    og = orc.matmul_q8_0_range(gate, q8, sc, n_in, 0, n, sem)
    ou = orc.matmul_q8_0_range(up, q8, sc, n_in, 0, n, sem)
    of = np.zeros(2 * n, np.float32)
    for ith in range(8):
        orc.matmul_q8_0_parallel_rows(fused, q8, sc, of, n_in, 2 * n, ith, 8, sem)
    assert np.array_equal(bits(of[:n]), bits(og)) and np.array_equal(bits(of[n:]), bits(ou))


def test_fuse_vstack_rejects_mismatched_rows():
    # src/ops/quant/fuse.rs:186-196
    assert orc.fuse_vstack(np.zeros(34 * 2, np.uint8), 2, np.zeros(68 * 2, np.uint8), 2) is None


# ---------------------------------------------------------------- activations / norms / rope

@pytest.mark.parametrize("mode", [orc.EXP_LIBM, orc.EXP_CR])
def test_silu_mul_llama_scalar_order(mode):
    # tests/quantized_inference.rs:20-29
    orc.set_exp_mode(mode)
    try:
        gate = np.zeros(4, np.float32)
        up = np.zeros(4, np.float32)
        gate[3] = f32([0xbf44c6b5])[0]
        up[3] = f32([0x3ddf57e5])[0]
        orc.silu_mul_inplace(gate, up)
        assert bits(up)[3] == 0xbcd98667
    finally:
        orc.set_exp_mode(orc.EXP_CR)


def test_rms_norm_accumulates_f32_squares_in_f64():
    # src/ops/matmul_tests.rs:127-144
    x = f32([0x3f800000, 0x39800000, 0x39800000])
    out = orc.rms_norm(x, np.ones(3, np.float32), 0.0)
    assert list(bits(out)) == [0x3fddb3d6, 0x39ddb3d6, 0x39ddb3d6]


def test_rms_norm_inplace_matches_ggml_sequential_f64_accumulation():
    # src/ops/matmul_tests.rs:146-183
    x = f32([0x3e57d77b, 0xbd828687, 0xbe102e16, 0x3d2f9fea, 0x3df48d0b, 0x3ded164c, 0x3bcc65ad, 0xbe18b60f])
    w = f32([0x40910000, 0x3f9f0000, 0xbf3c0000, 0x3fda0000, 0x40260000, 0x3fc70000, 0x3f8c0000, 0x3fbb0000])
    out = orc.rms_norm(x, w, float(f32([0x358637bd])[0]))
    assert list(bits(out)) == [0x40f971a9, 0xbf2568fe, 0x3f580a09, 0x3f18930b, 0x4021c6f1,
                               0x3fbc04bd, 0x3d641282, 0xbfe39aea]


def test_rope_neox_matches_pinned_ggml_recurrence_and_fused_rotation():
    # src/ops/matmul_tests.rs:185-199
    v = np.zeros(128, np.float32)
    v[[0, 1, 64, 65]] = f32([0x402a4f21, 0x3fadb711, 0xbe0e7273, 0x3ef5b8f9])
    out = orc.rope_neox(v, 1, 128, 1_000_000.0)
    assert list(bits(out[[0, 1, 64, 65]])) == [0x3fc70519, 0x3f17f682, 0x400a7ff8, 0x3fa7dc8a]


def test_dot_f16_f64_loop_matches_pinned_bits():
    # src/ops/matmul_tests.rs:462-497, non-native-fp16 tuple: the plain f64-accumulate loop
    # (src/ops/dot.rs:115-118 and :146-149 are the same loop) gives these bits.
    for n, expect in ((32, 0xc086612e), (37, 0x4035d999), (64, 0x4122a161)):
        i = np.arange(n)
        x = (np.where(i % 3 == 0, 0x8000, 0) | ((14 + i % 3) << 10) | ((i * 73 + 19) & 0x3ff)).astype(np.uint16)
        y = (np.where((i % 5 == 1) | (i % 5 == 2), 0x8000, 0) | ((13 + i % 4) << 10) | ((i * 151 + 7) & 0x3ff)).astype(np.uint16)
        assert bits(np.array([orc.dot_f16(x, y)]))[0] == expect, n


def test_softmax_basic_and_padding():
    s = orc.softmax(np.array([-1.0, 0.0, 1.0, -np.inf], np.float32))
    assert s[3] == 0.0 and abs(s.sum() - 1.0) < 1e-6
    assert np.allclose(s[:3], np.exp([-2.0, -1.0, 0.0]) / np.exp([-2.0, -1.0, 0.0]).sum(), rtol=1e-6)


def test_exp_modes_agree_almost_everywhere():
    # The CUDA path implements the correctly rounded f32 exp; this host's libm expf (what the
    # reference calls) may differ from it by one ulp on a small fraction of inputs.
    x = -np.abs(np.random.default_rng(0).standard_normal(200000).astype(np.float32)) * 8
    orc.set_exp_mode(orc.EXP_LIBM)
    a = np.array([orc.lib().orc_expf(float(v)) for v in x[:20000]], np.float32)
    orc.set_exp_mode(orc.EXP_CR)
    b = np.array([orc.lib().orc_expf(float(v)) for v in x[:20000]], np.float32)
    diff = np.abs(bits(a).astype(np.int64) - bits(b).astype(np.int64))
    assert diff.max() <= 1
    assert (diff != 0).mean() < 0.01


def test_greedy_sampling_uses_first_maximum_and_rejects_nan():
    # src/models/qwen3.rs:1518-1522
    assert orc.greedy_token(np.array([1.0, 2.0, 2.0], np.float32)) == 1
    assert orc.greedy_token(np.array([1.0, np.nan], np.float32)) == -1


def test_embedding_row_decode():
    w = synth_q8_0(5, 64, seed=9)
    out = orc.embedding_lookup_q8_0(w, 3, 64)
    blk = w.reshape(5, 2, 34)[3]
    d = blk[:, :2].copy().view(np.float16).astype(np.float32)
    ref = (d * blk[:, 2:].view(np.int8).astype(np.float32)).reshape(-1)
    assert np.array_equal(bits(out), bits(ref))


# ---------------------------------------------------------------- K-quants

def test_q8_k_quantizer_returns_one_complete_block():
    # tests/quantized_inference.rs:152-172
    x = np.array([(i - 127) * 0.03125 for i in range(256)], np.float32)
    for sem in (orc.SEM_AVX2, orc.SEM_SCALAR):
        blocks = orc.quantize_row_q8_k(x, sem)
        d, qs, bs = orc.q8k_to_numpy(blocks)
        assert len(blocks) == 1 and bs.astype(np.int64).sum() == qs.astype(np.int64).sum()


def test_q8_k_quantizer_uses_llama_nearest_even_rounding():
    # tests/quantized_inference.rs:174-186
    x = np.zeros(256, np.float32)
    x[:5] = [-127.0, 0.5, 1.5, 2.5, -0.5]
    for sem in (orc.SEM_AVX2, orc.SEM_SCALAR):
        _, qs, _ = orc.q8k_to_numpy(orc.quantize_row_q8_k(x, sem))
        assert list(qs[0, :5]) == [-127, 0, 2, 2, 0]


def _numpy_q4k_dequant(block: np.ndarray) -> np.ndarray:
    """Independent decode of one 144-byte super-block (src/ops/quant/mod.rs:25-33, 456-490)."""
    d = block[0:2].copy().view(np.float16).astype(np.float32)[0]
    dmin = block[2:4].copy().view(np.float16).astype(np.float32)[0]
    s = block[4:16]
    out = np.zeros(256, np.float32)
    for j in range(8):
        if j < 4:
            sc, mn = s[j] & 63, s[j + 4] & 63
        else:
            sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4)
            mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4)
        qs = block[16 + (j // 2) * 32: 16 + (j // 2) * 32 + 32]
        q = (qs & 0xF) if j % 2 == 0 else (qs >> 4)
        out[j * 32:(j + 1) * 32] = (d * np.float32(sc)) * q.astype(np.float32) - (dmin * np.float32(mn))
    return out


def test_q4_k_kernel_multiplies_uniform_block():
    # tests/quantized_inference.rs:233-249
    w = np.zeros(144, np.uint8)
    w[0:2] = np.array([f16_bits(1.0)], np.uint16).view(np.uint8)
    w[4:16] = [1, 1, 1, 1, 0, 0, 0, 0, 1, 1, 1, 1]
    w[16:] = 0x11
    out = orc.q4k_forward_prequantized(w, np.ones(256, np.uint8), np.ones(8, np.float32), 256, 1)
    assert list(out) == [256.0]
    assert np.array_equal(orc.dequantize_q4_k_weight(w, 1, 256), np.ones((1, 256), np.float32))
    assert list(orc.q4k_forward_dequant(w, 1, 256, np.ones(256, np.float32))) == [256.0]


def test_q4_k_dequant_matches_independent_decode():
    w = ((np.arange(144 * 6) * 29 + 7) & 0xff).astype(np.uint8)
    w.reshape(6, 144)[:, 1] = 0x2c  # keep d finite and small
    w.reshape(6, 144)[:, 3] = 0x28
    got = orc.dequantize_q4_k_weight(w, 2, 768)
    ref = np.concatenate([_numpy_q4k_dequant(b) for b in w.reshape(6, 144)]).reshape(2, 768)
    assert np.array_equal(bits(got), bits(ref))


def test_q4_k_prepared_path_ints_and_scalar_dot():
    # tests/quantized_inference.rs:188-210 builds these bytes; the file is stale against the
    # current trait, so the pinned property is: scalar dot == an independent evaluation, the
    # AVX2 variant shares the exact integer sums and agrees within mod.rs:1112-1162's 1e-3.
    w = ((np.arange(144) * 29 + 7) & 0xff).astype(np.uint8)
    x = np.array([((i % 23) - 11) / 7.0 for i in range(256)], np.float32)
    for sem in (orc.SEM_AVX2, orc.SEM_SCALAR):
        blocks = orc.quantize_row_q8_k(x, sem)
        d8, qs, bs = orc.q8k_to_numpy(blocks)
        a, m = orc.q4k_q8k_block_ints(w, blocks[0])
        deq = _numpy_q4k_dequant(w)
        # independent integer sums
        s = w[4:16]
        scs, mns = [], []
        for j in range(8):
            if j < 4:
                scs.append(int(s[j] & 63)); mns.append(int(s[j + 4] & 63))
            else:
                scs.append(int((s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4)))
                mns.append(int((s[j + 4] >> 4) | ((s[j] >> 6) << 4)))
        q4 = np.zeros(256, np.int64)
        for g in range(4):
            q4[64 * g:64 * g + 32] = w[16 + 32 * g:48 + 32 * g] & 0xF
            q4[64 * g + 32:64 * g + 64] = w[16 + 32 * g:48 + 32 * g] >> 4
        a_ref = sum(scs[j] * int((q4[32 * j:32 * j + 32] * qs[0, 32 * j:32 * j + 32].astype(np.int64)).sum()) for j in range(8))
        m_ref = sum(int(bs[0, j]) * mns[j // 2] for j in range(16))
        assert (a, m) == (a_ref, m_ref)
        got = orc.vec_dot_q4k_q8k(w, blocks, sem)
        ref = float((deq.astype(np.float64) * (qs[0].astype(np.float64) * float(d8[0]))).sum())
        assert abs(got - ref) <= 1e-3 * max(abs(ref), 1.0)
    ga = orc.vec_dot_q4k_q8k(w, orc.quantize_row_q8_k(x, orc.SEM_AVX2), orc.SEM_AVX2)
    gs = orc.vec_dot_q4k_q8k(w, orc.quantize_row_q8_k(x, orc.SEM_SCALAR), orc.SEM_SCALAR)
    assert abs(ga - gs) <= 1e-3 * max(abs(gs), 1.0)  # src/ops/quant/mod.rs:1112-1162


@pytest.mark.parametrize("sem", [orc.SEM_AVX2, orc.SEM_SCALAR])
def test_q4_k_partition_seq_parallel_fused(sem):
    # tests/fused_ffn_matmul_parity.rs:234-319: weights seed+r+j bytes; seq == parallel == fused
    n_in, n_out = 512, 24
    row_bytes = n_in // 256 * 144

    def mk(seed):
        r = np.arange(n_out)[:, None]
        j = np.arange(row_bytes)[None, :]
        return ((seed + r + j) & 0xff).astype(np.uint8).reshape(-1)

    gate, up = mk(0), mk(17)
    x = ramp_input(n_in)
    seq_g = orc.q4k_forward_prepared(gate, x, n_in, n_out, sem=sem)
    seq_u = orc.q4k_forward_prepared(up, x, n_in, n_out, sem=sem)
    fused, rows = orc.fuse_vstack(gate, n_out, up, n_out)
    out = np.zeros(rows, np.float32)
    for ith in range(4):
        orc.q4k_forward_prepared(fused, x, n_in, rows, ith, 4, sem, output=out)
    assert np.array_equal(bits(out[:n_out]), bits(seq_g)) and np.array_equal(bits(out[n_out:]), bits(seq_u))


# ---------------------------------------------------------------- session sizing

def test_session_sizing_steps_and_token_count():
    # src/models/qwen3.rs:1487-1496: capacity = prompt+gen, steps = prompt+gen-1
    from tests.synth_model import tiny_model
    cfg, tensors = tiny_model(seed=0)
    m = orc.Qwen3(cfg, tensors)
    prompt = np.array([1, 2, 3], np.uint32)
    toks, trace = m.generate(prompt, 4, want_trace=True)
    assert len(toks) == 4 and trace.shape[0] == 3 + 4 - 1


# ---------------------------------------------------------------- Q6_K (src/ops/quant/mod.rs)

def _q6k_block(ql, qh, scales, d):
    """make_q6k_block, src/ops/quant/mod.rs:1097-1111"""
    v = np.zeros(210, np.uint8)
    v[:128], v[128:192] = ql, qh
    v[192:208] = np.asarray(scales, np.int8).view(np.uint8)
    v[208:210] = np.array([d], np.float16).view(np.uint8)
    return v


def _q8k_test_blocks(values):
    """block_q8k of the reference's test module (mod.rs:1070-1087): d = amax/127, q = round-half-away(v*127/amax)."""
    values = np.asarray(values, np.float32)
    blocks = (orc.BlockQ8K * (values.size // 256))()
    for b, chunk in enumerate(values.reshape(-1, 256)):
        amax = np.float32(np.abs(chunk).max())
        idv = np.float32(0) if amax == 0 else np.float32(127.0) / amax
        blocks[b].d = float(np.float32(0) if amax == 0 else amax / np.float32(127.0))
        t = (chunk * idv).astype(np.float32)
        q = np.clip(np.where(t >= 0, np.floor(t + np.float32(0.5)), np.ceil(t - np.float32(0.5))), -127, 127).astype(np.int8)
        for i in range(256):
            blocks[b].qs[i] = int(q[i])
        for g in range(16):
            blocks[b].bsums[g] = int(q[16 * g:16 * g + 16].astype(np.int32).sum())
    return blocks


def test_q6k_reference_fixture_one_block_avx2_vs_scalar():
    # q6k_avx2_matches_scalar_one_block, src/ops/quant/mod.rs:1165-1184
    ql = np.array([i % 4 for i in range(128)], np.uint8)
    qh = np.array([i * 5 % 4 for i in range(64)], np.uint8)
    w = _q6k_block(ql, qh, [i - 4 for i in range(16)], 0.5)
    x = np.array([(i - 128.0) * 0.01 for i in range(256)], np.float32)
    q8k = _q8k_test_blocks(x)
    avx2, scalar = orc.vec_dot_q6k_q8k(w, q8k, orc.SEM_AVX2), orc.vec_dot_q6k_q8k(w, q8k, orc.SEM_SCALAR)
    rel = abs(avx2 - scalar) / abs(scalar) if abs(scalar) > 1e-3 else abs(avx2 - scalar)
    assert rel < 1e-3
    # both equal the dot of the dequantized row with the dequantized activation to f32 accuracy
    deq = orc.dequantize_row_q6_k(w, 256).astype(np.float64)
    d8, qs, _ = orc.q8k_to_numpy(q8k)
    ref = float((deq * (qs[0].astype(np.float64) * float(d8[0]))).sum())
    assert abs(avx2 - ref) <= 1e-5 * max(1.0, abs(ref)) and abs(scalar - ref) <= 1e-5 * max(1.0, abs(ref))


def test_q6k_reference_fixture_four_blocks_avx2_vs_scalar():
    # q6k_avx2_matches_scalar_multi_block, src/ops/quant/mod.rs:1187-1211
    w = np.concatenate([_q6k_block(np.array([(i * 11 + j * 3) % 4 for j in range(128)], np.uint8),
                                   np.array([(i + j * 7) % 4 for j in range(64)], np.uint8),
                                   [(i * 5 + k) - 6 for k in range(16)], 0.01 + i * 0.1) for i in range(4)])
    x = np.array([(i - 512.0) * 0.01 for i in range(1024)], np.float32)
    q8k = _q8k_test_blocks(x)
    avx2, scalar = orc.vec_dot_q6k_q8k(w, q8k, orc.SEM_AVX2), orc.vec_dot_q6k_q8k(w, q8k, orc.SEM_SCALAR)
    rel = abs(avx2 - scalar) / abs(scalar) if abs(scalar) > 1e-3 else abs(avx2 - scalar)
    assert rel < 1e-3


def test_q6k_lane_sums_equal_the_scalar_integer_sums():
    """The eight AVX2 int32 lanes (with the -32 offset folded through bsums) sum to the scalar kernel's
    Σ scale·q8·(q6-32) exactly, on random bytes."""
    rng = np.random.default_rng(11)
    blk = rng.integers(0, 256, 210, dtype=np.uint8)
    x = rng.standard_normal(256).astype(np.float32)
    q8k = orc.quantize_row_q8_k(x, orc.SEM_AVX2)
    lanes = orc.q6k_q8k_block_lanes(blk, q8k[0])
    _, qs, _ = orc.q8k_to_numpy(q8k)
    sc = blk[192:208].view(np.int8).astype(np.int64)
    deq_int = np.array([0] * 256, np.int64)
    row = orc.dequantize_row_q6_k(np.concatenate([blk[:208], np.array([1.0], np.float16).view(np.uint8)]), 256)
    # with d = 1 the dequantized value is sc * (q - 32) exactly
    total = int((row.astype(np.int64) * qs[0].astype(np.int64)).sum())
    assert int(lanes.astype(np.int64).sum()) == total
    del deq_int, sc


def test_q6k_forward_partition_and_prequantized_path():
    rng = np.random.default_rng(12)
    n_in, n_out = 512, 24
    w = rng.integers(0, 256, n_out * (n_in // 256) * 210, dtype=np.uint8)
    for r in range(n_out * (n_in // 256)):   # sane f16 scales
        w[r * 210 + 208:r * 210 + 210] = np.array([0.01 + 0.001 * (r % 7)], np.float16).view(np.uint8)
    x = rng.standard_normal(n_in).astype(np.float32)
    for sem in (orc.SEM_AVX2, orc.SEM_SCALAR):
        whole = orc.q6k_forward_prepared(w, x, n_in, n_out, sem=sem)
        parts = np.zeros(n_out, np.float32)
        for ith in range(5):
            orc.q6k_forward_prepared(w, x, n_in, n_out, ith, 5, sem=sem, output=parts)
        assert np.array_equal(whole.view(np.uint32), parts.view(np.uint32))
    q8, sc = orc.quantize_q8_0(x, orc.SEM_AVX2)
    pre = orc.q6k_forward_prequantized(w, q8, sc, n_in, n_out)
    deq = np.stack([orc.dequantize_row_q6_k(w[r * 420:(r + 1) * 420], n_in) for r in range(n_out)]).astype(np.float64)
    xin = q8.reshape(-1).view(np.int8).astype(np.float64) * np.repeat(sc.reshape(-1).astype(np.float64), 32)
    ref = deq @ xin
    assert np.abs(pre - ref).max() <= 1e-4 * max(1.0, np.abs(ref).max())


# ---------------------------------------------------------------- Q4_0 (src/ops/kernel/q4_0)

def _q4_0_block(scale, lo, hi=None):
    hi = lo if hi is None else hi
    return np.concatenate([np.array([scale], np.float16).view(np.uint8), np.full(16, lo | (hi << 4), np.uint8)])


def test_q4_0_reference_known_answers():
    # q4_0/mod.rs:99-123: nibble 8 -> 0.0; nibble 9 with q8 = 1, scale 1 -> 32.0
    q8, sc = np.full(32, 1, np.int8).view(np.uint8), np.ones(1, np.float32)
    assert orc.q4_0_forward_prequantized(_q4_0_block(1.0, 8), q8, sc, 32, 1)[0] == 0.0
    assert orc.q4_0_forward_prequantized(_q4_0_block(1.0, 9), q8, sc, 32, 1)[0] == 32.0


def test_q4_0_reference_edge_blocks():
    # the inputs of q4_0/avx2.rs:247-330 (zero / max / min activations, zero / max nibbles, linspace, alternating
    # signs): the exact integer dot times d times scale
    cases = [(0, np.zeros(32, np.int8)), (15, np.zeros(32, np.int8)), (0, np.full(32, 127, np.int8)),
             (0, np.full(32, -128, np.int8)), (15, np.full(32, 127, np.int8)),
             (5, np.linspace(-127, 127, 32).astype(np.int8)), (11, np.array([127 if i % 2 else -127 for i in range(32)], np.int8))]
    for nib, q in cases:
        w = _q4_0_block(0.5, nib, 15 - nib)
        got = orc.q4_0_forward_prequantized(w, q.view(np.uint8), np.array([0.25], np.float32), 32, 1)[0]
        dot = int(((nib - 8) * q[:16].astype(np.int64)).sum() + ((15 - nib - 8) * q[16:].astype(np.int64)).sum())
        assert got == np.float32(np.float32(np.float32(dot) * np.float32(0.5)) * np.float32(0.25))


def test_q4_0_partition_equals_whole():
    rng = np.random.default_rng(5)
    n_in, n_out = 256, 19
    w = rng.integers(0, 256, n_out * (n_in // 32) * 18, dtype=np.uint8)
    for r in range(n_out * (n_in // 32)):
        w[r * 18:r * 18 + 2] = np.array([0.01 + 0.002 * (r % 5)], np.float16).view(np.uint8)
    x = rng.standard_normal(n_in).astype(np.float32)
    q8, sc = orc.quantize_q8_0(x, orc.SEM_AVX2)
    whole = orc.q4_0_forward_prequantized(w, q8, sc, n_in, n_out)
    parts = np.zeros(n_out, np.float32)
    for ith in range(4):
        orc.q4_0_forward_prequantized(w, q8, sc, n_in, n_out, ith, 4, output=parts)
    assert np.array_equal(whole.view(np.uint32), parts.view(np.uint32))


# ---------------------------------------------------------------- the CLI forward's attention (src/app/text.rs)

def test_cli_attention_helpers_and_tie_break():
    lib = orc.lib()
    lib.orc_dot_f16_f32.restype = orc.C.c_float
    rng = np.random.default_rng(3)
    a = rng.standard_normal(128).astype(np.float32)
    b16 = rng.standard_normal(128).astype(np.float16)
    ref = float((a.astype(np.float64) * b16.astype(np.float64)).sum())
    for sem in (orc.SEM_AVX2, orc.SEM_NEON, orc.SEM_SCALAR):
        got = lib.orc_dot_f16_f32(orc._p(a), orc._p(b16.view(np.uint16)), orc.C.c_size_t(128), orc.C.c_int(sem))
        assert abs(got - ref) < 1e-4
    # n = 5 exercises only the scalar tail in every variant: identical bits
    tails = {sem: lib.orc_dot_f16_f32(orc._p(a), orc._p(b16.view(np.uint16)), orc.C.c_size_t(3), orc.C.c_int(sem))
             for sem in (orc.SEM_AVX2, orc.SEM_NEON, orc.SEM_SCALAR)}
    assert len({np.float32(v).tobytes() for v in tails.values()}) == 1
    lib.orc_greedy_token_last.restype = orc.C.c_int64
    x = np.array([1, 2, 2], np.float32)
    assert lib.orc_greedy_token_last(orc._p(x), orc.C.c_size_t(3)) == 2       # max_by keeps the last maximum
    assert orc.greedy_token(x) == 1                                           # Qwen3Session keeps the first
    x[1] = np.nan
    assert lib.orc_greedy_token_last(orc._p(x), orc.C.c_size_t(3)) == -1


def test_dot_f32_neon_pinned_vector_and_lane_orders():
    """src/ops/matmul_tests.rs:240-258: the four-accumulator NEON reduction on 16 pinned inputs."""
    lib = orc.lib()
    lib.orc_dot_f32.restype = orc.C.c_float
    a = np.array([1035226804, 3189287613, 3181886457, 3193572547, 1042787479, 3172027867, 1034549374, 3188264325,
                  1056115932, 3201905443, 3188891406, 1051732974, 1049988604, 3191259790, 3197162127, 1039754039],
                 np.uint32).view(np.float32)
    b = np.array([1075433967, 1074732927, 1057635659, 3215511252, 3198768119, 1079784837, 1023408184, 3203974092,
                  3215464821, 3191576483, 1049344900, 1021989171, 3207345090, 3229966761, 3189361871, 1036416888],
                 np.uint32).view(np.float32)
    got = np.float32(lib.orc_dot_f32(orc._p(a), orc._p(b), orc.C.c_size_t(16), orc.C.c_int(orc.SEM_NEON)))
    assert int(got.view(np.uint32)) == 0x3d071678
    rng = np.random.default_rng(11)
    x, y = rng.standard_normal(256).astype(np.float32), rng.standard_normal(256).astype(np.float32)
    ref = float((x.astype(np.float64) * y.astype(np.float64)).sum())
    for sem in (orc.SEM_AVX2, orc.SEM_NEON, orc.SEM_SCALAR):
        assert abs(lib.orc_dot_f32(orc._p(x), orc._p(y), orc.C.c_size_t(256), orc.C.c_int(sem)) - ref) < 1e-4
    # the scalar order, restated in numpy f32
    s = np.float32(0)
    for i in range(40):
        s = np.float32(s + np.float32(x[i] * y[i]))
    got = np.float32(lib.orc_dot_f32(orc._p(x), orc._p(y), orc.C.c_size_t(40), orc.C.c_int(orc.SEM_SCALAR)))
    assert got.tobytes() == s.tobytes()


def test_cli_f32_cache_oracle_runs_and_tracks_the_f16_cache_variant():
    """The F32-cache branch of the CLI loop differs from the F16-cache branch only by the cache rounding and the
    soft-max form: hidden states stay close on a small model, and the first position (one cached key, weight
    exactly 1) is identical except for the f16 rounding of V."""
    from synth_model import tiny_model
    cfg, tensors = tiny_model(seed=2)
    oracle = orc.Qwen3(cfg, tensors)
    prompt = np.arange(1, 13, dtype=np.uint32) % cfg["vocab"]
    t32, tr32 = oracle.generate(prompt, 6, want_trace=True, cli=True, kv_f32=True)
    t16, tr16 = oracle.generate(prompt, 6, want_trace=True, cli=True)
    assert t32.shape == t16.shape == (6,)
    assert np.isfinite(tr32).all()
    assert np.abs(tr32[0] - tr16[0]).max() <= 2e-2 * max(1.0, np.abs(tr16[0]).max())
    with pytest.raises(ValueError):
        oracle.generate(prompt, 6, kv_f32=True)
    for sem in (orc.SEM_NEON, orc.SEM_SCALAR):
        alt = oracle.generate(prompt, 6, sem=sem, want_trace=True, cli=True, kv_f32=True)[1]
        assert np.abs(alt - tr32).max() <= 1e-2 * max(1.0, np.abs(tr32).max())
    # the logits tool's loop: same scores and soft-max, sequential value chains; first maximal index
    for kv_f32 in (False, True):
        tl, trl = oracle.generate(prompt, 6, want_trace=True, logits_tool=True, kv_f32=kv_f32)
        assert tl.shape == (6,) and np.isfinite(trl).all()
        assert np.abs(trl - (tr32 if kv_f32 else tr16)).max() <= 1e-2 * max(1.0, np.abs(tr16).max())


def test_f32_input_matmul_q8_0_exact_on_integer_data_in_both_orders():
    """ops::matmul_q8_0 (src/ops/kernel/q8_0/parallel.rs:317-341) has no vector in the reference's own tests, so its
    restatements (AVX2: avx2.rs:180-217, scalar: scalar.rs:3-29) are pinned on data where every product and every
    partial sum is an exactly representable integer multiple of the scale: both accumulation orders must then give the
    exact value, which is computed in int64."""
    rng = np.random.default_rng(5)
    n_out, n_in = 19, 160
    blocks = n_in // 32
    q = rng.integers(-127, 128, size=(n_out, blocks, 32), dtype=np.int64)
    e = rng.integers(-3, 4, size=(n_out, blocks))                # scales 2^-3 .. 2^3
    x = rng.integers(-8, 9, size=n_in).astype(np.float32)
    weight = bytearray()
    for r in range(n_out):
        for b in range(blocks):
            weight += np.float16(2.0 ** float(e[r, b])).tobytes() + q[r, b].astype(np.int8).tobytes()
    weight = np.frombuffer(bytes(weight), np.uint8)
    exact = np.array([sum(float(2.0 ** float(e[r, b])) * float((q[r, b] * x[b * 32:(b + 1) * 32].astype(np.int64)).sum())
                          for b in range(blocks)) for r in range(n_out)], np.float64)
    for sem in (orc.SEM_AVX2, orc.SEM_SCALAR, orc.SEM_NEON):
        got = orc.matmul_q8_0_f32(weight, x, n_in, n_out, sem)[0]
        assert np.array_equal(got.astype(np.float64), exact), sem


def test_f32_input_matmul_q8_0_orders_agree_within_tolerance_and_differ_in_bits():
    weight = make_q8_0_weight(64, 1024, 3)
    x = np.random.default_rng(4).standard_normal(1024).astype(np.float32)
    a = orc.matmul_q8_0_f32(weight, x, 1024, 64, orc.SEM_AVX2)[0]
    s = orc.matmul_q8_0_f32(weight, x, 1024, 64, orc.SEM_SCALAR)[0]
    assert np.max(np.abs(a - s)) / np.max(np.abs(s)) < 1e-5
    assert not np.array_equal(bits(a), bits(s))      # sixteen fused chains vs one chain with separate mul and add
    assert np.array_equal(bits(s), bits(orc.matmul_q8_0_fallback_range(weight, x, 1024, 0, 64)))
