"""ctypes binding of the CPU oracle (oracle/rmi_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by the
cpu-baseline / reference legs of bench.py -- never by the product package.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "librmi_oracle.so")

SEM_AVX2, SEM_NEON, SEM_SCALAR = 0, 1, 2
SEM_AVX2_BLOCK = 3   # x86 quantizer + whole-block accumulation: what the tensor-core GEMM computes for an x86 host
EXP_LIBM, EXP_CR = 0, 1


def build(force: bool = False) -> str:
    src = [os.path.join(_HERE, f) for f in ("rmi_oracle.c", "rmi_oracle.h", "Makefile")]
    stale = force or not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in src if os.path.exists(s))
    if stale:
        subprocess.check_call(["make", "-C", _HERE, "-s"] + (["-B"] if force else []))
    return _LIB_PATH


class BlockQ8K(C.Structure):
    _fields_ = [("d", C.c_float), ("qs", C.c_int8 * 256), ("bsums", C.c_int16 * 16)]


class Qwen3Config(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in
                ("n_embd", "n_layer", "n_head", "n_head_kv", "head_dim", "n_ff", "vocab")] + \
               [("eps", C.c_float), ("freq_base", C.c_float)]


class Qwen3Layer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in
                ("attn_norm", "ffn_norm", "q_norm", "k_norm", "wq", "wk", "wv", "wo",
                 "w_gate", "w_up", "w_down")]


class Qwen3Model(C.Structure):
    _fields_ = [("cfg", Qwen3Config), ("layers", C.POINTER(Qwen3Layer)),
                ("output_norm", C.c_void_p), ("token_embd", C.c_void_p), ("output", C.c_void_p)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_expf.restype = C.c_float
        _lib.orc_expf.argtypes = [C.c_float]
        _lib.orc_f32_to_f16.restype = C.c_uint16
        _lib.orc_f32_to_f16.argtypes = [C.c_float]
        _lib.orc_f16_to_f32.restype = C.c_float
        _lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_f16_from_bytes.restype = C.c_float
        _lib.orc_f16_from_bytes.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t]
        _lib.orc_vec_dot_q4k_q8k.restype = C.c_float
        _lib.orc_dot_f16.restype = C.c_float
        _lib.orc_greedy_token.restype = C.c_int64
        _lib.orc_qwen3_generate.restype = C.c_int64
        _lib.orc_fuse_vstack.restype = C.c_size_t
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _u8(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint8).reshape(-1)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def set_exp_mode(mode: int):
    lib().orc_set_exp_mode(C.c_int(mode))


def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    x = _f32(x).reshape(-1)
    out = np.empty(x.size, np.uint16)
    lib().orc_f32_slice_to_f16(_p(x), _p(out), C.c_size_t(x.size))
    return out


def quantize_q8_0(x, sem=SEM_AVX2, fast=False):
    """-> (q8 uint8[n], scales f32[n/32]) for one row or a [M,n] matrix (row-wise)."""
    x = _f32(x)
    n = x.shape[-1]
    flat = x.reshape(-1, n)
    q8 = np.empty(flat.shape, np.uint8)
    sc = np.empty((flat.shape[0], n // 32), np.float32)
    for i in range(flat.shape[0]):
        if fast:
            ok = lib().orc_quantize_q8_0_avx2_fast(_p(flat[i]), C.c_size_t(n), _p(q8[i]), _p(sc[i]))
            assert ok, "AVX2 intrinsics path not built"
        else:
            lib().orc_quantize_q8_0(_p(flat[i]), C.c_size_t(n), _p(q8[i]), _p(sc[i]), C.c_int(sem))
    return q8.reshape(x.shape), sc.reshape(x.shape[:-1] + (n // 32,))


def matmul_q8_0_range(weight, q8, scales, n_in, row_start, row_end, sem=SEM_AVX2, fast=False):
    weight, q8, scales = _u8(weight), _u8(q8), _f32(scales)
    out = np.zeros(row_end - row_start, np.float32)
    if fast:
        ok = lib().orc_matmul_q8_0_range_avx2_fast(_p(weight), _p(q8), _p(scales), _p(out),
                                                   C.c_size_t(n_in), C.c_size_t(row_start),
                                                   C.c_size_t(row_end))
        assert ok
    else:
        lib().orc_matmul_q8_0_range(_p(weight), _p(q8), _p(scales), _p(out), C.c_size_t(n_in),
                                    C.c_size_t(row_start), C.c_size_t(row_end), C.c_int(sem))
    return out


def matmul_q8_0_parallel_rows(weight, q8, scales, output, n_in, n_out, ith, nth, sem=SEM_AVX2):
    weight, q8, scales = _u8(weight), _u8(q8), _f32(scales)
    assert output.dtype == np.float32 and output.flags.c_contiguous
    lib().orc_matmul_q8_0_parallel_rows(_p(weight), _p(q8), _p(scales), _p(output),
                                        C.c_size_t(n_in), C.c_size_t(n_out), C.c_size_t(ith),
                                        C.c_size_t(nth), C.c_int(sem))


def q8_0_block_sums(weight, q8, n_in, row_start, row_end):
    weight, q8 = _u8(weight), _u8(q8)
    out = np.zeros((row_end - row_start, n_in // 32), np.int32)
    lib().orc_q8_0_block_sums(_p(weight), _p(q8), _p(out), C.c_size_t(n_in),
                              C.c_size_t(row_start), C.c_size_t(row_end))
    return out


def matmul_q8_0_fallback_range(weight, x, n_in, row_start, row_end):
    weight, x = _u8(weight), _f32(x)
    out = np.zeros(row_end - row_start, np.float32)
    lib().orc_matmul_q8_0_fallback_range(_p(weight), _p(x), _p(out), C.c_size_t(n_in),
                                         C.c_size_t(row_start), C.c_size_t(row_end))
    return out


def matmul_q8_0_f32(weight, x, n_in, n_out, sem=SEM_AVX2):
    """ops::matmul_q8_0 (f32 input, src/ops/kernel/q8_0/parallel.rs:317-341) for every row of x."""
    weight, x = _u8(weight), _f32(x).reshape(-1, n_in)
    out = np.zeros((x.shape[0], n_out), np.float32)
    for t in range(x.shape[0]):
        lib().orc_matmul_q8_0_f32(_p(weight), _p(x[t]), _p(out[t]), C.c_size_t(n_in), C.c_size_t(n_out), C.c_int(sem))
    return out


def q8_forward_batched(weight, x, n_in, n_out, sem=SEM_AVX2, threads=1):
    weight, x = _u8(weight), _f32(x).reshape(-1, n_in)
    out = np.zeros((x.shape[0], n_out), np.float32)
    lib().orc_q8_forward_batched(_p(weight), _p(x), _p(out), C.c_size_t(x.shape[0]),
                                 C.c_size_t(n_in), C.c_size_t(n_out), C.c_int(sem), C.c_int(threads))
    return out


def fuse_vstack(a, a_rows, b, b_rows):
    a, b = _u8(a), _u8(b)
    out = np.empty(a.size + b.size, np.uint8)
    rows = lib().orc_fuse_vstack(_p(a), C.c_size_t(a.size), C.c_size_t(a_rows), _p(b),
                                 C.c_size_t(b.size), C.c_size_t(b_rows), _p(out))
    return (out, rows) if rows else None


def silu_mul_inplace(gate, up):
    gate = _f32(gate)
    assert up.dtype == np.float32 and up.flags.c_contiguous
    lib().orc_silu_mul_inplace(_p(gate), _p(up), C.c_size_t(gate.size))


def ffn_swiglu_q8_0(w_gate, w_up, w_down, x, n_embd, n_ff, sem=SEM_AVX2, threads=1, want_act=False):
    x = _f32(x).reshape(-1, n_embd)
    out = np.zeros_like(x)
    act = np.zeros((x.shape[0], n_ff), np.float32) if want_act else None
    lib().orc_ffn_swiglu_q8_0(_p(_u8(w_gate)), _p(_u8(w_up)), _p(_u8(w_down)), _p(x), _p(out),
                              _p(act), C.c_size_t(x.shape[0]), C.c_size_t(n_embd),
                              C.c_size_t(n_ff), C.c_int(sem), C.c_int(threads))
    return (out, act) if want_act else out


def quantize_row_q8_k(x, sem=SEM_AVX2):
    x = _f32(x).reshape(-1)
    nb = x.size // 256
    blocks = (BlockQ8K * nb)()
    lib().orc_quantize_row_q8_k(_p(x), C.c_size_t(x.size), blocks, C.c_int(sem))
    return blocks


def q8k_to_numpy(blocks):
    nb = len(blocks)
    d = np.array([b.d for b in blocks], np.float32)
    qs = np.array([list(b.qs) for b in blocks], np.int8).reshape(nb, 256)
    bs = np.array([list(b.bsums) for b in blocks], np.int16).reshape(nb, 16)
    return d, qs, bs


def vec_dot_q4k_q8k(q4k, blocks, sem=SEM_AVX2):
    q4k = _u8(q4k)
    return float(lib().orc_vec_dot_q4k_q8k(_p(q4k), C.c_size_t(q4k.size), blocks,
                                           C.c_size_t(len(blocks)), C.c_int(sem)))


def q4k_q8k_block_ints(q4k_block, block):
    q4k_block = _u8(q4k_block)
    a, m = C.c_int32(), C.c_int32()
    lib().orc_q4k_q8k_block_ints(_p(q4k_block), C.byref(block), C.byref(a), C.byref(m))
    return a.value, m.value


def dequantize_q4_k_weight(w, n_rows, n_cols):
    w = _u8(w)
    out = np.zeros((n_rows, n_cols), np.float32)
    lib().orc_dequantize_q4_k_weight(_p(w), C.c_size_t(w.size), C.c_size_t(n_rows),
                                     C.c_size_t(n_cols), _p(out))
    return out


def q4k_forward_dequant(w, out_features, in_features, x):
    w, x = _u8(w), _f32(x)
    out = np.zeros(out_features, np.float32)
    scratch = np.zeros(out_features * in_features, np.float32)
    lib().orc_q4k_forward_dequant(_p(w), C.c_size_t(w.size), C.c_size_t(out_features),
                                  C.c_size_t(in_features), _p(x), _p(out), _p(scratch),
                                  C.c_size_t(scratch.size))
    return out


def q4k_forward_prepared(w, x, n_in, n_out, ith=0, nth=1, sem=SEM_AVX2, output=None):
    w, x = _u8(w), _f32(x)
    out = np.zeros(n_out, np.float32) if output is None else output
    lib().orc_q4k_forward_prepared(_p(w), C.c_size_t(w.size), _p(x), _p(out), C.c_size_t(n_in),
                                   C.c_size_t(n_out), C.c_size_t(ith), C.c_size_t(nth), C.c_int(sem))
    return out


def q4k_forward_prequantized(w, q8, scales, n_in, n_out, ith=0, nth=1, output=None):
    w, q8, scales = _u8(w), _u8(q8), _f32(scales)
    out = np.zeros(n_out, np.float32) if output is None else output
    lib().orc_q4k_forward_prequantized(_p(w), C.c_size_t(w.size), _p(q8), _p(scales), _p(out),
                                       C.c_size_t(n_in), C.c_size_t(n_out), C.c_size_t(ith),
                                       C.c_size_t(nth))
    return out


def q4_0_forward_prequantized(w, q8, scales, n_in, n_out, ith=0, nth=1, output=None):
    w, q8, scales = _u8(w), _u8(q8), _f32(scales)
    out = np.zeros(n_out, np.float32) if output is None else output
    lib().orc_q4_0_forward_prequantized(_p(w), _p(q8), _p(scales), _p(out), C.c_size_t(n_in), C.c_size_t(n_out),
                                        C.c_size_t(ith), C.c_size_t(nth))
    return out


def dequantize_row_q6_k(w, n):
    w = _u8(w)
    out = np.zeros(n, np.float32)
    lib().orc_dequantize_row_q6_k(_p(w), C.c_size_t(w.size), _p(out), C.c_size_t(n))
    return out


def vec_dot_q6k_q8k(q6k, blocks, sem=SEM_AVX2):
    q6k = _u8(q6k)
    fn = lib().orc_vec_dot_q6k_q8k
    fn.restype = C.c_float
    return float(fn(_p(q6k), C.c_size_t(q6k.size), blocks, C.c_size_t(len(blocks)), C.c_int(sem)))


def q6k_q8k_block_lanes(q6k_block, block):
    q6k_block = _u8(q6k_block)
    lanes = (C.c_int32 * 8)()
    lib().orc_q6k_q8k_block_lanes(_p(q6k_block), C.byref(block), lanes)
    return np.array(list(lanes), np.int32)


def q6k_forward_prepared(w, x, n_in, n_out, ith=0, nth=1, sem=SEM_AVX2, output=None):
    w, x = _u8(w), _f32(x)
    out = np.zeros(n_out, np.float32) if output is None else output
    lib().orc_q6k_forward_prepared(_p(w), C.c_size_t(w.size), _p(x), _p(out), C.c_size_t(n_in),
                                   C.c_size_t(n_out), C.c_size_t(ith), C.c_size_t(nth), C.c_int(sem))
    return out


def q6k_forward_prequantized(w, q8, scales, n_in, n_out, ith=0, nth=1, output=None):
    w, q8, scales = _u8(w), _u8(q8), _f32(scales)
    out = np.zeros(n_out, np.float32) if output is None else output
    lib().orc_q6k_forward_prequantized(_p(w), C.c_size_t(w.size), _p(q8), _p(scales), _p(out),
                                       C.c_size_t(n_in), C.c_size_t(n_out), C.c_size_t(ith),
                                       C.c_size_t(nth))
    return out


def rms_norm(x, w, eps):
    x, w = _f32(x), _f32(w)
    out = np.zeros_like(x)
    lib().orc_rms_norm(_p(x), _p(w), _p(out), C.c_size_t(x.size), C.c_float(eps))
    return out


def rope_neox(x, pos, head_dim, freq_base):
    x = _f32(x).copy()
    lib().orc_rope_neox(_p(x), C.c_size_t(x.size), C.c_size_t(pos), C.c_size_t(head_dim),
                        C.c_float(freq_base))
    return x


def rope_table(n_pos, head_dim, freq_base):
    """[n_pos, head_dim/2, 2] (cos, sin) exactly as rope_neox evaluates them."""
    t = np.zeros((n_pos, head_dim // 2, 2), np.float32)
    for p in range(n_pos):
        lib().orc_rope_table(C.c_size_t(p), C.c_size_t(head_dim), C.c_float(freq_base), _p(t[p]))
    return t


def softmax(x):
    x = _f32(x).copy()
    lib().orc_softmax(_p(x), C.c_size_t(x.size))
    return x


def dot_f16(a, b):
    a = np.ascontiguousarray(a, np.uint16)
    b = np.ascontiguousarray(b, np.uint16)
    return np.float32(lib().orc_dot_f16(_p(a), _p(b), C.c_size_t(a.size)))


def embedding_lookup(w, token, n_embd, ggml_type):
    """src/ops/embedding.rs:3-10 dispatch: 8 = Q8_0, 2 = Q4_0, 14 = Q6_K"""
    w = _u8(w)
    out = np.zeros(n_embd, np.float32)
    fn = {8: lib().orc_embedding_lookup_q8_0, 2: lib().orc_embedding_lookup_q4_0, 14: lib().orc_embedding_lookup_q6_k}[ggml_type]
    fn(_p(w), C.c_uint32(token), C.c_size_t(n_embd), _p(out))
    return out


def embedding_lookup_q8_0(w, token, n_embd):
    w = _u8(w)
    out = np.zeros(n_embd, np.float32)
    lib().orc_embedding_lookup_q8_0(_p(w), C.c_uint32(token), C.c_size_t(n_embd), _p(out))
    return out


def greedy_token(logits):
    logits = _f32(logits)
    return int(lib().orc_greedy_token(_p(logits), C.c_size_t(logits.size)))


class Qwen3:
    """Holds numpy views of a synthetic Qwen3-architecture model for orc_qwen3_generate.
    `tensors` maps GGUF tensor names to numpy arrays (uint8 for Q8_0, float32 for norms)."""

    def __init__(self, cfg: dict, tensors: dict):
        self._keep = []
        self.cfg = cfg
        layers = (Qwen3Layer * cfg["n_layer"])()

        def ptr(name, dtype):
            a = np.ascontiguousarray(tensors[name]).view(dtype).reshape(-1)
            self._keep.append(a)
            return a.ctypes.data

        for i in range(cfg["n_layer"]):
            L = layers[i]
            L.attn_norm = ptr(f"blk.{i}.attn_norm.weight", np.float32)
            L.ffn_norm = ptr(f"blk.{i}.ffn_norm.weight", np.float32)
            L.q_norm = ptr(f"blk.{i}.attn_q_norm.weight", np.float32)
            L.k_norm = ptr(f"blk.{i}.attn_k_norm.weight", np.float32)
            L.wq = ptr(f"blk.{i}.attn_q.weight", np.uint8)
            L.wk = ptr(f"blk.{i}.attn_k.weight", np.uint8)
            L.wv = ptr(f"blk.{i}.attn_v.weight", np.uint8)
            L.wo = ptr(f"blk.{i}.attn_output.weight", np.uint8)
            L.w_gate = ptr(f"blk.{i}.ffn_gate.weight", np.uint8)
            L.w_up = ptr(f"blk.{i}.ffn_up.weight", np.uint8)
            L.w_down = ptr(f"blk.{i}.ffn_down.weight", np.uint8)
        self._layers = layers
        m = Qwen3Model()
        for k in ("n_embd", "n_layer", "n_head", "n_head_kv", "head_dim", "n_ff", "vocab"):
            setattr(m.cfg, k, cfg[k])
        m.cfg.eps = cfg["eps"]
        m.cfg.freq_base = cfg["freq_base"]
        m.layers = layers
        m.output_norm = ptr("output_norm.weight", np.float32)
        m.token_embd = ptr("token_embd.weight", np.uint8)
        m.output = ptr("output.weight", np.uint8) if "output.weight" in tensors else m.token_embd
        self._m = m

    def generate(self, prompt, n_gen, sem=SEM_AVX2, threads=1, want_trace=False, want_logits=False, cli=False,
                 kv_f32=False, logits_tool=False):
        """cli=False: Qwen3Session (src/models/qwen3.rs); cli=True: the CLI's forward (src/app/text.rs:257-648),
        with kv_f32 its `--kv-cache f32` branch; logits_tool=True: the logits tool's loop (src/app/logits.rs)."""
        prompt = np.ascontiguousarray(prompt, np.uint32)
        out = np.zeros(max(n_gen, 1), np.uint32)
        steps = prompt.size + n_gen - 1
        trace = np.zeros((steps, self.cfg["n_embd"]), np.float32) if want_trace else None
        logits = np.zeros(self.cfg["vocab"], np.float32) if want_logits else None
        fn = lib().orc_qwen3_generate_cli if cli else lib().orc_qwen3_generate
        extra = ()
        if logits_tool:
            fn = lib().orc_qwen3_generate_logits_tool
            extra = (C.c_int(1 if kv_f32 else 0),)
        elif kv_f32:
            if not cli:
                raise ValueError("the F32 cache exists only in the CLI forward")
            fn = lib().orc_qwen3_generate_cli_f32kv
        fn.restype = C.c_int64
        n = fn(C.byref(self._m), _p(prompt), C.c_size_t(prompt.size), C.c_size_t(n_gen), _p(out), C.c_int(sem),
               C.c_int(threads), _p(trace), _p(logits), *extra)
        if n == -2:
            raise RuntimeError("context longer than 512 positions (the reference's F32-cache value array)")
        if n < 0:
            raise RuntimeError("Cannot sample non-finite logits")
        res = [out[:n].copy()]
        if want_trace:
            res.append(trace)
        if want_logits:
            res.append(logits)
        return res[0] if len(res) == 1 else tuple(res)
