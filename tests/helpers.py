"""Shared builders for test inputs. The weight/ramp patterns restate the deterministic
generators of the reference's own integration tests (cited per function)."""
import numpy as np

from oracle import orc


def f16_bits(x: float) -> int:
    return int(np.array([x], np.float32).astype(np.float16).view(np.uint16)[0])


def q8_0_uniform_row(value: int, scale: float) -> np.ndarray:
    """src/ops/kernel/q8_0/mod.rs:64-72: one 34-byte block, all quants = value."""
    row = np.zeros(34, np.uint8)
    row[0:2] = np.array([f16_bits(scale)], np.uint16).view(np.uint8)
    row[2:] = np.uint8(value & 0xff)
    return row


def make_q8_0_weight(n_rows: int, n_cols: int, row_offset: int) -> np.ndarray:
    """tests/q8_0_parallel_matmul.rs:26-42 and tests/fused_ffn_matmul_parity.rs (same pattern):
    scale = f16(0.5 + 0.01 r); quant j = (row_offset + r + b + j/4) as i8."""
    blocks = n_cols // 32
    r = np.arange(n_rows, dtype=np.int64)[:, None, None]
    b = np.arange(blocks, dtype=np.int64)[None, :, None]
    j = np.arange(32, dtype=np.int64)[None, None, :]
    q = ((row_offset + r + b + j // 4) & 0xff).astype(np.uint8)
    scale = (np.float32(0.5) + np.float32(0.01) * np.arange(n_rows, dtype=np.float32)).astype(np.float32)
    sbits = scale.astype(np.float16).view(np.uint16)
    out = np.zeros((n_rows, blocks, 34), np.uint8)
    out[:, :, 0] = (sbits & 0xff)[:, None]
    out[:, :, 1] = (sbits >> 8)[:, None]
    out[:, :, 2:] = q
    return out.reshape(-1)


def ramp_input(n: int) -> np.ndarray:
    """tests/q8_0_parallel_matmul.rs:113: (i as f32) * 0.013 - 4.0"""
    return (np.arange(n, dtype=np.float32) * np.float32(0.013) - np.float32(4.0)).astype(np.float32)


def encode_q8_0(w: np.ndarray) -> np.ndarray:
    """f32 [N,K] -> GGUF Q8_0 bytes [N, K/32, 34] using the AVX2-semantics quantizer
    (d = f16(amax/127), q = rne(w * 127/amax))."""
    w = np.ascontiguousarray(w, np.float32)
    n, k = w.shape
    q8, sc = orc.quantize_q8_0(w, orc.SEM_AVX2, fast=bool(orc.lib().orc_has_avx2_fast()))
    sbits = sc.astype(np.float16).view(np.uint16)  # scales are already f16-representable
    out = np.zeros((n, k // 32, 34), np.uint8)
    out[:, :, 0] = sbits & 0xff
    out[:, :, 1] = sbits >> 8
    out[:, :, 2:] = q8.reshape(n, k // 32, 32)
    return out.reshape(-1)


def synth_q8_0(n: int, k: int, seed: int, std: float = 0.02) -> np.ndarray:
    w = np.random.default_rng(seed).standard_normal((n, k), dtype=np.float32) * np.float32(std)
    return encode_q8_0(w)


def synth_q4_k(n: int, k: int, seed: int) -> np.ndarray:
    """Valid Q4_K super-block stream [N, K/256, 144]: random 6-bit scales/mins and nibbles,
    f16 d/dmin sized so dequantized weights look like N(0, 0.02). The reference has no
    f32->Q4_K encoder; parity is defined on decoding these bytes."""
    rng = np.random.default_rng(seed)
    nb = k // 256
    out = rng.integers(0, 256, size=(n, nb, 144), dtype=np.uint8)
    d = (rng.uniform(0.5, 1.5, size=(n, nb)) * 0.02 / 63.0 / 4.0).astype(np.float16).view(np.uint16)
    dmin = (rng.uniform(0.5, 1.5, size=(n, nb)) * 0.02 / 63.0 * 1.8).astype(np.float16).view(np.uint16)
    out[:, :, 0] = d & 0xff
    out[:, :, 1] = d >> 8
    out[:, :, 2] = dmin & 0xff
    out[:, :, 3] = dmin >> 8
    return out.reshape(-1)


def rel_err(a: np.ndarray, ref: np.ndarray) -> float:
    """src/ops/kernel/q8_0/avx2.rs:239-245: max|a-b| / max|ref|"""
    return float(np.max(np.abs(a.astype(np.float64) - ref.astype(np.float64))) /
                 max(float(np.max(np.abs(ref))), 1e-30))


def bits(a) -> np.ndarray:
    return np.ascontiguousarray(a, np.float32).view(np.uint32)
