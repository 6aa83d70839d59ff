"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (no datasets or checkpoints exist offline).

RNG: numpy.random.default_rng(seed).standard_normal(shape, dtype=float32) (PCG64); weights
are multiplied by float32(0.02).  Q8_0 weight encoding uses the x86 production quantizer's
arithmetic of the reference (src/ops/quant/q8_0.rs:176-230): d = amax/127 stored as f16,
q = round_half_even(w * (127/amax)) -- the reference has no f32->Q8_0 weight encoder.
"""
from __future__ import annotations

import numpy as np

from . import gguf

QWEN3_0_6B = dict(n_embd=1024, n_layer=28, n_head=16, n_head_kv=8, head_dim=128, n_ff=3072,
                  vocab=151936, eps=1e-6, freq_base=1_000_000.0, n_ctx=40960)


def normal(shape, seed: int, std: float = 1.0) -> np.ndarray:
    x = np.random.default_rng(seed).standard_normal(shape, dtype=np.float32)
    return x if std == 1.0 else x * np.float32(std)


def encode_q8_0(w: np.ndarray) -> np.ndarray:
    """f32 [N,K] -> uint8 [N*K/32*34] GGUF Q8_0 blocks ([f16 d][32 x i8])."""
    w = np.ascontiguousarray(w, np.float32)
    n, k = w.shape
    blk = w.reshape(n, k // 32, 32)
    amax = np.abs(blk).max(axis=2)
    with np.errstate(divide="ignore", invalid="ignore"):
        d = np.where(amax == 0, np.float32(0), amax / np.float32(127.0)).astype(np.float32)
        inv = np.where(amax == 0, np.float32(0), np.float32(127.0) / amax).astype(np.float32)
    q = np.clip(np.rint(blk * inv[:, :, None]), -128, 127).astype(np.int8)
    dbits = d.astype(np.float16).view(np.uint16)
    out = np.empty((n, k // 32, 34), np.uint8)
    out[:, :, 0] = dbits & 0xff
    out[:, :, 1] = dbits >> 8
    out[:, :, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def q8_0_weight(n: int, k: int, seed: int, std: float = 0.02) -> np.ndarray:
    """Q8_0 bytes of an [n,k] N(0,std) matrix, generated in row chunks to bound memory."""
    rng = np.random.default_rng(seed)
    out = np.empty(n * (k // 32) * 34, np.uint8)
    rb = k // 32 * 34
    step = max(1, (1 << 24) // k)
    for r in range(0, n, step):
        m = min(step, n - r)
        w = rng.standard_normal((m, k), dtype=np.float32) * np.float32(std)
        out[r * rb:(r + m) * rb] = encode_q8_0(w)
    return out


def q8_0_weight_rows(n: int, k: int, seed: int, row_begin: int, row_end: int, std: float = 0.02,
                     chunk: int = 1024) -> np.ndarray:
    """Rows [row_begin,row_end) of an [n,k] matrix whose row chunk c is drawn from
    default_rng([seed, c]): every rank can generate exactly its shard of the same matrix."""
    rb = k // 32 * 34
    out = np.empty((row_end - row_begin) * rb, np.uint8)
    r = row_begin
    while r < row_end:
        c = r // chunk
        lo, hi = c * chunk, min((c + 1) * chunk, n)
        w = np.random.default_rng([seed, c]).standard_normal((hi - lo, k), dtype=np.float32) * np.float32(std)
        take_hi = min(hi, row_end)
        out[(r - row_begin) * rb:(take_hi - row_begin) * rb] = encode_q8_0(w[r - lo:take_hi - lo])
        r = take_hi
    return out


def q4_k_weight(n: int, k: int, seed: int) -> np.ndarray:
    """A valid Q4_K super-block stream [n, k/256, 144]: uniform random 6-bit scales/mins and
    nibbles with f16 d/dmin sized so decoded weights have roughly N(0,0.02) spread.  Parity
    is defined on decoding these bytes (the reference has no f32->Q4_K encoder)."""
    rng = np.random.default_rng(seed)
    nb = k // 256
    out = rng.integers(0, 256, size=(n, nb, 144), dtype=np.uint8)
    d = (rng.uniform(0.5, 1.5, size=(n, nb)) * (0.02 / 63.0 / 4.0)).astype(np.float16).view(np.uint16)
    dmin = (rng.uniform(0.5, 1.5, size=(n, nb)) * (0.02 / 63.0 * 1.8)).astype(np.float16).view(np.uint16)
    out[:, :, 0], out[:, :, 1] = d & 0xff, d >> 8
    out[:, :, 2], out[:, :, 3] = dmin & 0xff, dmin >> 8
    return out.reshape(-1)


def q4_0_weight(n: int, k: int, seed: int) -> np.ndarray:
    """A valid Q4_0 block stream [n, k/32, 18]: random nibbles, f16 d sized for roughly N(0,0.02) weights."""
    rng = np.random.default_rng(seed)
    out = rng.integers(0, 256, size=(n, k // 32, 18), dtype=np.uint8)
    d = (rng.uniform(0.5, 1.5, size=(n, k // 32)) * (0.02 / 4.0)).astype(np.float16).view(np.uint16)
    out[:, :, 0], out[:, :, 1] = d & 0xff, d >> 8
    return out.reshape(-1)


def q6_k_weight(n: int, k: int, seed: int) -> np.ndarray:
    """A valid Q6_K super-block stream [n, k/256, 210]: uniform random ql/qh bytes and int8 scales, f16 d sized so
    that decoded weights have roughly N(0,0.02) spread.  Parity is defined on decoding these bytes."""
    rng = np.random.default_rng(seed)
    nb = k // 256
    out = rng.integers(0, 256, size=(n, nb, 210), dtype=np.uint8)
    d = (rng.uniform(0.5, 1.5, size=(n, nb)) * (0.02 / 64.0 / 20.0)).astype(np.float16).view(np.uint16)
    out[:, :, 208], out[:, :, 209] = d & 0xff, d >> 8
    return out.reshape(-1)


def prompt_tokens(vocab: int, n: int, seed: int) -> np.ndarray:
    return np.random.default_rng(seed).integers(0, vocab, size=n, dtype=np.uint32)


def qwen3_tensors(cfg: dict, seed: int = 0) -> dict:
    """Random-init Qwen3-architecture weights: all linears and the tied embedding Q8_0 from
    N(0,0.02); norm weights f32 N(1,0.02)."""
    nq, nk = cfg["n_head"] * cfg["head_dim"], cfg["n_head_kv"] * cfg["head_dim"]
    e, ff = cfg["n_embd"], cfg["n_ff"]
    t = {}
    s = seed * 100003

    def nrm(n, sd):
        return (np.float32(1.0) + normal((n,), sd, 0.02)).astype(np.float32)

    t["token_embd.weight"] = q8_0_weight(cfg["vocab"], e, s + 1)
    t["output_norm.weight"] = nrm(e, s + 2)
    for i in range(cfg["n_layer"]):
        b = s + 1000 * (i + 1)
        p = f"blk.{i}."
        t[p + "attn_norm.weight"] = nrm(e, b + 1)
        t[p + "ffn_norm.weight"] = nrm(e, b + 2)
        t[p + "attn_q_norm.weight"] = nrm(cfg["head_dim"], b + 3)
        t[p + "attn_k_norm.weight"] = nrm(cfg["head_dim"], b + 4)
        t[p + "attn_q.weight"] = q8_0_weight(nq, e, b + 5)
        t[p + "attn_k.weight"] = q8_0_weight(nk, e, b + 6)
        t[p + "attn_v.weight"] = q8_0_weight(nk, e, b + 7)
        t[p + "attn_output.weight"] = q8_0_weight(e, nq, b + 8)
        t[p + "ffn_gate.weight"] = q8_0_weight(ff, e, b + 9)
        t[p + "ffn_up.weight"] = q8_0_weight(ff, e, b + 10)
        t[p + "ffn_down.weight"] = q8_0_weight(e, ff, b + 11)
    return t


def write_qwen3_gguf(path: str, cfg: dict, tensors: dict) -> None:
    """GGUF v3 with general.architecture = "qwen3" and the keys the reference reads
    (src/core/loader.rs:410-460, src/models/qwen3.rs:44-52)."""
    G = gguf
    md = [("general.architecture", G.T_STR, "qwen3"),
          ("general.alignment", G.T_U32, 32),
          ("qwen3.embedding_length", G.T_U32, cfg["n_embd"]),
          ("qwen3.block_count", G.T_U32, cfg["n_layer"]),
          ("qwen3.attention.head_count", G.T_U32, cfg["n_head"]),
          ("qwen3.attention.head_count_kv", G.T_U32, cfg["n_head_kv"]),
          ("qwen3.attention.key_length", G.T_U32, cfg["head_dim"]),
          ("qwen3.attention.value_length", G.T_U32, cfg["head_dim"]),
          ("qwen3.feed_forward_length", G.T_U32, cfg["n_ff"]),
          ("qwen3.context_length", G.T_U32, cfg.get("n_ctx", 40960)),
          ("qwen3.vocab_size", G.T_U32, cfg["vocab"]),
          ("qwen3.rope.freq_base", G.T_F32, cfg["freq_base"]),
          ("qwen3.attention.layer_norm_rms_epsilon", G.T_F32, cfg["eps"])]
    nq, nk = cfg["n_head"] * cfg["head_dim"], cfg["n_head_kv"] * cfg["head_dim"]
    e, ff = cfg["n_embd"], cfg["n_ff"]
    dims = {"attn_q.weight": [e, nq], "attn_k.weight": [e, nk], "attn_v.weight": [e, nk],
            "attn_output.weight": [nq, e], "ffn_gate.weight": [e, ff], "ffn_up.weight": [e, ff],
            "ffn_down.weight": [ff, e], "attn_norm.weight": [e], "ffn_norm.weight": [e],
            "attn_q_norm.weight": [cfg["head_dim"]], "attn_k_norm.weight": [cfg["head_dim"]]}
    tl = []
    for name, arr in tensors.items():
        if name == "token_embd.weight" or name == "output.weight":
            tl.append((name, [e, cfg["vocab"]], G.GGML_Q8_0, arr))
        elif name == "output_norm.weight":
            tl.append((name, [e], G.GGML_F32, arr.view(np.uint8)))
        else:
            suffix = name.split(".", 2)[2]
            d = dims[suffix]
            if len(d) == 1:
                tl.append((name, d, G.GGML_F32, arr.view(np.uint8)))
            else:
                tl.append((name, d, G.GGML_Q8_0, arr))
    G.write_gguf(path, md, tl)
