"""Host-side mirror of the reference's operator interface over librmi_cuda.so.

Everything here is a thin ctypes layer over the C ABI declared in include/rmi_cuda.h; the
names, argument meaning and error behaviour follow the Rust reference (paths are inside
the reference project):

  quantize_q8_0_into / quantize_q8_0          src/ops/quant/q8_0.rs:3-24, :232-238
  matmul_q8_0_quantized(_parallel_rows|_range) src/ops/kernel/q8_0/parallel.rs:25-139, dispatch.rs:27-108
  Kernel / Q8Kernel / Q4_KKernel              src/ops/kernel/trait_.rs:15-110, q8_0/mod.rs:22-56, q4_k.rs:7-93
  QuantizedTensor.from_bytes(..).into_kernel  src/ops/kernel/quantized_tensor.rs:120-189
  fuse_vstack_q8_0 / fuse_vstack_q4_k         src/ops/quant/fuse.rs:25-63
  QuantizedLinear (forward_dequant, forward)  src/core/model.rs:12-104
  GGUFLoader                                  src/core/loader.rs:189-395
  Qwen3Model / Qwen3Session                   src/models/qwen3.rs:212-243, :407-550

There is no CPU path in this package: if the CUDA library is missing or no B200 is
visible, `context()` raises.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import gguf, load_plan, sharding, synth  # noqa: F401  (host utilities: synthetic checkpoints, rank partition, placement plans)

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "librmi_cuda.so")

SEM_AVX2, SEM_NEON, SEM_SCALAR = 0, 1, 2
GGML_F32, GGML_Q4_0, GGML_Q8_0, GGML_Q4_K, GGML_Q6_K = 0, 2, 8, 12, 14
FORWARD_QWEN3_SESSION, FORWARD_APP_TEXT, FORWARD_APP_TEXT_F32KV, FORWARD_APP_LOGITS, FORWARD_APP_LOGITS_F32KV = 0, 1, 2, 3, 4
PREFILL_BATCHED, PREFILL_TOKEN_LOOP, PREFILL_BATCHED_TENSOR = 0, 1, 2
STATUS = {0: "RMI_OK", 1: "RMI_ERR_BAD_HANDLE", 2: "RMI_ERR_BAD_SHAPE", 3: "RMI_ERR_OOM", 4: "RMI_ERR_CUDA",
          5: "RMI_ERR_TIMEOUT", 6: "RMI_ERR_UNSUPPORTED", 7: "RMI_ERR_IO", 8: "RMI_ERR_FORMAT",
          9: "RMI_ERR_NONFINITE"}


class RmiError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS.get(status, status)}: {message}")
        self.status = status
        self.message = message


_lib = None


def lib() -> C.CDLL:
    """Loads librmi_cuda.so; raises when it has not been built (there is no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python __graft_entry__.py build` first")
        _lib = C.CDLL(LIB_PATH)
        _lib.rmi_last_error.restype = C.c_char_p
    return _lib


def _check(status: int):
    if status != 0:
        raise RmiError(status, lib().rmi_last_error().decode(errors="replace"))


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _sz(v):
    return C.c_size_t(int(v))


class Context:
    """rmi_ctx: one per device (src/vulkan.rs:31-59 is the precedent)."""

    def __init__(self, device: int = 0):
        self._h = C.c_void_p()
        _check(lib().rmi_init(C.c_int32(device), C.byref(self._h)))
        self.device = device

    def close(self):
        if self._h:
            lib().rmi_destroy(self._h)
            self._h = C.c_void_p()

    @property
    def handle(self):
        return self._h

    def set_semantics(self, sem: int):
        _check(lib().rmi_set_semantics(self._h, C.c_int32(sem)))

    def set_prefill_exact(self, on: bool):
        """AVX2 semantics: True keeps calls of more than 32 rows on the bit-exact CUDA-core kernels."""
        _check(lib().rmi_set_prefill_exact(self._h, C.c_int32(1 if on else 0)))

    def semantics(self) -> int:
        v = C.c_int32()
        _check(lib().rmi_get_semantics(self._h, C.byref(v)))
        return v.value

    def set_stream(self, cuda_stream: int | None):
        _check(lib().rmi_set_stream(self._h, C.c_void_p(cuda_stream or 0)))

    def sync(self):
        _check(lib().rmi_sync(self._h))

    def device_info(self):
        sm, l2, mem = C.c_int32(), C.c_size_t(), C.c_size_t()
        _check(lib().rmi_device_info(self._h, C.byref(sm), C.byref(l2), C.byref(mem)))
        return sm.value, l2.value, mem.value

    def launch_count(self) -> int:
        v = C.c_uint64()
        _check(lib().rmi_launch_count(self._h, C.byref(v)))
        return v.value

    def prof_enable(self, on: bool):
        _check(lib().rmi_prof_enable(self._h, C.c_int32(1 if on else 0)))

    def prof_read(self, tag: str):
        """-> (launches, total_ms) of the kernels tagged `tag` since prof_enable(True)."""
        n, ms = C.c_uint64(), C.c_float()
        _check(lib().rmi_prof_read(self._h, tag.encode(), C.byref(n), C.byref(ms)))
        return n.value, ms.value

    # raw device memory (for callers without an allocator of their own)
    def dev_alloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        _check(lib().rmi_dev_alloc(self._h, _sz(nbytes), C.byref(p)))
        return p.value

    def dev_free(self, ptr: int):
        _check(lib().rmi_dev_free(self._h, C.c_void_p(ptr)))

    def h2d(self, dst: int, src: np.ndarray):
        src = np.ascontiguousarray(src)
        _check(lib().rmi_h2d(self._h, C.c_void_p(dst), _p(src), _sz(src.nbytes)))

    def d2h(self, dst: np.ndarray, src: int):
        _check(lib().rmi_d2h(self._h, _p(dst), C.c_void_p(src), _sz(dst.nbytes)))

    def set_dependent_launch(self, on: bool):
        """Programmatic dependent launch for chains of decode-shaped kernels (see rmi_set_dependent_launch)."""
        _check(lib().rmi_set_dependent_launch(self._h, C.c_int32(1 if on else 0)))

    def set_wait_limit_ms(self, ms: int):
        """Time limit of the bounded device-side waits (flag rounds, GEMM barriers); default 2000 ms."""
        _check(lib().rmi_set_wait_limit_ms(self._h, C.c_uint32(ms)))

    def check_status(self):
        """Synchronise and raise RMI_ERR_TIMEOUT if a device-side wait gave up."""
        _check(lib().rmi_check_status(self._h))

    def ipc_export(self, dev_ptr: int) -> bytes:
        buf = (C.c_uint8 * 64)()
        _check(lib().rmi_ipc_export(self._h, C.c_void_p(dev_ptr), buf))
        return bytes(buf)

    def ipc_open(self, handle: bytes) -> int:
        buf = (C.c_uint8 * 64).from_buffer_copy(handle)
        out = C.c_void_p()
        _check(lib().rmi_ipc_open(self._h, buf, C.byref(out)))
        return out.value

    def ipc_close(self, ptr: int):
        _check(lib().rmi_ipc_close(self._h, C.c_void_p(ptr)))


_ctx = None


def context(device: int = 0) -> Context:
    """Process-wide context (the reference keeps its GPU context in a OnceLock,
    src/ops/float.rs:44-58). Unlike the reference, failure raises: no CPU fallback."""
    global _ctx
    if _ctx is None:
        _ctx = Context(device)
    return _ctx


def enable_gpu(device: int = 0) -> Context:
    """ops::enable_gpu (src/ops/float.rs:11-13)."""
    return context(device)


# ------------------------------------------------------------------------------ weights

class QuantizedTensor:
    """QuantizedTensor<'a> (src/ops/kernel/quantized_tensor.rs:32-41): weight bytes + type + shape.
    `from_bytes` uploads once; `into_kernel` returns the Kernel object for the type."""

    def __init__(self, handle, ggml_type: int, n_in: int, n_out: int, ctx: Context):
        self._h, self.ggml_type, self.n_in, self.n_out, self._ctx = handle, ggml_type, n_in, n_out, ctx

    @classmethod
    def from_bytes(cls, data, ggml_type: int, n_in: int, n_out: int, row_begin: int = 0, row_end: int | None = None,
                   ctx: Context | None = None) -> "QuantizedTensor":
        ctx = ctx or context()
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        row_end = n_out if row_end is None else row_end
        h = C.c_void_p()
        _check(lib().rmi_weight_upload(ctx.handle, C.c_int32(ggml_type), _p(data), _sz(data.size), _sz(n_in),
                                       _sz(n_out), _sz(row_begin), _sz(row_end), C.byref(h)))
        return cls(h, ggml_type, n_in, row_end - row_begin, ctx)

    @classmethod
    def from_gguf(cls, g: "GGUFLoader", name: str, row_begin: int = 0, row_end: int | None = None,
                  ctx: Context | None = None) -> "QuantizedTensor":
        ctx = ctx or context()
        info = g.tensor_info(name)
        if info is None:
            raise RmiError(8, f"Missing tensor: {name}")
        h = C.c_void_p()
        re = (1 << 64) - 1 if row_end is None else row_end
        _check(lib().rmi_weight_upload_gguf(ctx.handle, g._h, name.encode(), _sz(row_begin), _sz(re), C.byref(h)))
        n_rows = (info["dims"][1] if row_end is None else row_end) - row_begin
        return cls(h, info["ggml_type"], info["dims"][0], n_rows, ctx)

    def fuse_vstack(self, other: "QuantizedTensor") -> "QuantizedTensor | None":
        """QTensorOwned::fuse_vstack (src/ops/kernel/qtensor_owned.rs:138-164); None when the
        row layouts differ, as the reference does."""
        h = C.c_void_p()
        st = lib().rmi_weight_fuse_vstack(self._ctx.handle, self._h, other._h, C.byref(h))
        if st == 2:
            return None
        _check(st)
        return QuantizedTensor(h, self.ggml_type, self.n_in, self.n_out + other.n_out, self._ctx)

    def into_kernel(self) -> "Kernel":
        if self.ggml_type == GGML_Q8_0:
            return Q8Kernel(self)
        if self.ggml_type == GGML_Q4_K:
            return Q4_KKernel(self)
        if self.ggml_type == GGML_Q6_K:
            return Q6_KKernel(self)
        if self.ggml_type == GGML_Q4_0:
            return Q4_0Kernel(self)
        raise RmiError(6, f"ggml type {self.ggml_type} has no kernel on this path")

    def device_bytes(self) -> int:
        b = C.c_size_t()
        _check(lib().rmi_weight_info(self._h, None, None, None, C.byref(b)))
        return b.value

    def free(self):
        if self._h:
            _check(lib().rmi_weight_free(self._ctx.handle, self._h))
            self._h = C.c_void_p()


def fuse_vstack_q8_0(a: QuantizedTensor, b: QuantizedTensor):
    """src/ops/quant/fuse.rs:25-40 -> (fused, rows) or None."""
    f = a.fuse_vstack(b)
    return None if f is None else (f, f.n_out)


fuse_vstack_q4_k = fuse_vstack_q8_0


def _row_range(n_out: int, ith: int, nth: int):
    """src/ops/kernel/q8_0/parallel.rs:112-129"""
    if nth <= 1 or n_out == 0:
        return 0, n_out
    per = (n_out + nth - 1) // nth
    s = ith * per
    return s, max(s, min(s + per, n_out))


class Kernel:
    """trait Kernel (src/ops/kernel/trait_.rs:15-110)."""

    def __init__(self, tensor: QuantizedTensor):
        self.weight = tensor
        self._ctx = tensor._ctx

    def forward_prequantized(self, input_q8, input_scales, output, n_in, n_out, ith, nth):
        raise NotImplementedError

    def forward_prepared(self, input_f32, input_q8, input_scales, q8_k, output, n_in, n_out, ith, nth):
        self.forward_prequantized(input_q8, input_scales, output, n_in, n_out, ith, nth)

    def forward(self, input, output, n_in, n_out):
        input = np.ascontiguousarray(input, np.float32)
        q8 = np.zeros(n_in, np.uint8)
        scales = np.zeros((n_in + 31) // 32, np.float32)
        quantize_q8_0_into(input, n_in, q8, scales, ctx=self._ctx)
        self.forward_prepared(input, q8, scales, None, output, n_in, n_out, 0, 1)

    def forward_batched(self, input, output, n_in, n_out):
        input = np.ascontiguousarray(input, np.float32).reshape(-1)
        n_tokens = input.size // n_in
        assert input.size == n_tokens * n_in and output.size == n_tokens * n_out
        for t in range(n_tokens):
            self.forward(input[t * n_in:(t + 1) * n_in], output.reshape(-1)[t * n_out:(t + 1) * n_out], n_in, n_out)


class Q8Kernel(Kernel):
    """Q8Kernel (src/ops/kernel/q8_0/mod.rs:22-56)."""

    @classmethod
    def new(cls, weight_bytes, n_in: int, n_out: int, ctx: Context | None = None) -> "Q8Kernel":
        return cls(QuantizedTensor.from_bytes(weight_bytes, GGML_Q8_0, n_in, n_out, ctx=ctx))

    def forward_prequantized(self, input_q8, input_scales, output, n_in, n_out, ith, nth):
        matmul_q8_0_quantized_parallel_rows(self.weight, input_q8, input_scales, output, n_in, n_out, ith, nth)

    def forward_batched(self, input, output, n_in, n_out):
        """One call for all tokens: rmi_matmul_q8_0 quantizes row-wise and picks GEMV or GEMM."""
        input = np.ascontiguousarray(input, np.float32).reshape(-1, n_in)
        assert output.dtype == np.float32 and output.flags.c_contiguous and output.size == input.shape[0] * n_out
        assert n_in == self.weight.n_in and n_out == self.weight.n_out
        _check(lib().rmi_matmul_q8_0(self._ctx.handle, self.weight._h, _p(input), _sz(input.shape[0]), _p(output)))


class Q4_KKernel(Kernel):
    """Q4_KKernel (src/ops/kernel/q4_k.rs:7-93)."""

    @classmethod
    def new(cls, data, n_in: int, n_out: int, ctx: Context | None = None) -> "Q4_KKernel":
        return cls(QuantizedTensor.from_bytes(data, GGML_Q4_K, n_in, n_out, ctx=ctx))

    def forward_prepared(self, input_f32, input_q8, input_scales, q8_k, output, n_in, n_out, ith, nth):
        # q4_k.rs:56-93; a caller-prepared Q8_K (q8_k) is recomputed on the device from input_f32,
        # which yields the same blocks (the quantizer is deterministic).
        input_f32 = np.ascontiguousarray(input_f32, np.float32).reshape(-1, n_in)
        s, e = _row_range(n_out, ith, max(nth, 1)) if nth > 0 else (0, n_out)
        per = (n_out + nth - 1) // nth
        s = ith * per
        e = min(s + per, n_out)
        if s >= e:
            return
        _check(lib().rmi_matmul_q4_k_q8k(self._ctx.handle, self.weight._h, _p(input_f32), _sz(input_f32.shape[0]),
                                         _p(output), _sz(s), _sz(e)))

    def forward_prequantized(self, input_q8, input_scales, output, n_in, n_out, ith, nth):
        # q4_k.rs:20-54: dequantize the Q8_0 activation to f32, then the dequantized-weight dot
        q = np.ascontiguousarray(input_q8, np.uint8).view(np.int8)[:n_in].astype(np.float32)
        x = q * np.repeat(np.ascontiguousarray(input_scales, np.float32)[: n_in // 32], 32)
        per = (n_out + nth - 1) // nth
        s, e = ith * per, min(ith * per + per, n_out)
        if s >= e:
            return
        full = np.zeros(n_out, np.float32)
        _check(lib().rmi_matmul_q4_k_dequant(self._ctx.handle, self.weight._h, _p(x), _sz(1), _p(full)))
        output.reshape(-1)[s:e] = full[s:e]


class Q6_KKernel(Kernel):
    """Q6_KKernel (src/ops/kernel/q6_k.rs:7-80)."""

    @classmethod
    def new(cls, data, n_in: int, n_out: int, ctx: Context | None = None) -> "Q6_KKernel":
        return cls(QuantizedTensor.from_bytes(data, GGML_Q6_K, n_in, n_out, ctx=ctx))

    def forward_prepared(self, input_f32, input_q8, input_scales, q8_k, output, n_in, n_out, ith, nth):
        # q6_k.rs:44-80; a caller-prepared Q8_K is recomputed on the device from input_f32 (deterministic)
        input_f32 = np.ascontiguousarray(input_f32, np.float32).reshape(-1, n_in)
        per = (n_out + nth - 1) // nth
        s, e = ith * per, min(ith * per + per, n_out)
        if s >= e:
            return
        _check(lib().rmi_matmul_q6_k_q8k(self._ctx.handle, self.weight._h, _p(input_f32), _sz(input_f32.shape[0]),
                                         _p(output), _sz(s), _sz(e)))

    def forward_prequantized(self, input_q8, input_scales, output, n_in, n_out, ith, nth):
        # q6_k.rs:22-42 -> matmul_q6_k_scalar_range (q6_k.rs:83-115)
        q8 = np.ascontiguousarray(input_q8, np.uint8).reshape(-1)[:n_in]
        sc = np.ascontiguousarray(input_scales, np.float32).reshape(-1)[: n_in // 32]
        per = (n_out + nth - 1) // nth
        s, e = ith * per, min(ith * per + per, n_out)
        if s >= e:
            return
        _check(lib().rmi_matmul_q6_k_prequantized(self._ctx.handle, self.weight._h, _p(q8), _p(sc), _sz(1), _p(output),
                                                  _sz(s), _sz(e)))


class Q4_0Kernel(Kernel):
    """Q4_0Kernel (src/ops/kernel/q4_0/mod.rs:14-80)."""

    @classmethod
    def new(cls, data, n_in: int, n_out: int, ctx: Context | None = None) -> "Q4_0Kernel":
        return cls(QuantizedTensor.from_bytes(data, GGML_Q4_0, n_in, n_out, ctx=ctx))

    def forward_prequantized(self, input_q8, input_scales, output, n_in, n_out, ith, nth):
        q8 = np.ascontiguousarray(input_q8, np.uint8).reshape(-1)[:n_in]
        sc = np.ascontiguousarray(input_scales, np.float32).reshape(-1)[: n_in // 32]
        per = (n_out + nth - 1) // nth
        s, e = ith * per, min(ith * per + per, n_out)
        if s >= e:
            return
        _check(lib().rmi_matmul_q4_0_prequantized(self._ctx.handle, self.weight._h, _p(q8), _p(sc), _sz(1), _p(output),
                                                  _sz(s), _sz(e)))


def matmul_q4_0(weight: "QuantizedTensor", x) -> np.ndarray:
    """Kernel::forward for every row of x (quantize to Q8_0, then Q4_0 x Q8_0)."""
    x = np.ascontiguousarray(x, np.float32).reshape(-1, weight.n_in)
    out = np.zeros((x.shape[0], weight.n_out), np.float32)
    _check(lib().rmi_matmul_q4_0(weight._ctx.handle, weight._h, _p(x), _sz(x.shape[0]), _p(out)))
    return out


def embedding_lookup(weight: "QuantizedTensor", token_ids) -> np.ndarray:
    """embedding_lookup (src/ops/embedding.rs:3-47) for Q8_0 / Q4_0 / Q6_K tables: [len(token_ids), n_embd]."""
    ids = np.ascontiguousarray(token_ids, np.uint32).reshape(-1)
    out = np.zeros((ids.size, weight.n_in), np.float32)
    _check(lib().rmi_embedding_lookup(weight._ctx.handle, weight._h, _p(ids), _sz(ids.size), _p(out)))
    return out


def dequantize_q6_k(weight: "QuantizedTensor") -> np.ndarray:
    """dequant_q6k_weight (src/ops/quant/mod.rs:571-583)"""
    out = np.zeros((weight.n_out, weight.n_in), np.float32)
    _check(lib().rmi_dequantize_q6_k(weight._ctx.handle, weight._h, _p(out)))
    return out


# ------------------------------------------------------------------------------ free functions

def quantize_q8_0_into(input, n: int, q8: np.ndarray, scales: np.ndarray, ctx: Context | None = None):
    """src/ops/quant/q8_0.rs:3-24. `input` may hold several rows of length n (row-wise)."""
    ctx = ctx or context()
    input = np.ascontiguousarray(input, np.float32)
    m = input.size // n if n else 0
    assert q8.dtype == np.uint8 and q8.flags.c_contiguous and scales.dtype == np.float32
    _check(lib().rmi_quantize_q8_0(ctx.handle, _p(input), _sz(m), _sz(n), _p(q8), _p(scales)))


def quantize_q8_0(input, n: int, ctx: Context | None = None):
    """src/ops/quant/q8_0.rs:232-238 -> (q8, scales)"""
    input = np.ascontiguousarray(input, np.float32)
    m = input.size // n if n else 0
    q8 = np.zeros(m * n, np.uint8)
    scales = np.zeros(m * (n // 32), np.float32)
    quantize_q8_0_into(input, n, q8, scales, ctx)
    return q8, scales


def _as_tensor(weight, n_in, n_out) -> QuantizedTensor:
    if isinstance(weight, QuantizedTensor):
        return weight
    raise TypeError("weight must be a QuantizedTensor (upload once with QuantizedTensor.from_bytes)")


def matmul_q8_0_quantized_range(weight, input_q8, input_scales, output, n_in, row_start, row_end):
    """src/ops/kernel/q8_0/dispatch.rs:27-108: `output` has row_end-row_start elements."""
    w = _as_tensor(weight, n_in, None)
    full = np.zeros(w.n_out, np.float32)
    q8 = np.ascontiguousarray(input_q8, np.uint8)
    sc = np.ascontiguousarray(input_scales, np.float32)
    _check(lib().rmi_matmul_q8_0_prequantized(w._ctx.handle, w._h, _p(q8), _p(sc), _sz(1), _p(full), _sz(row_start),
                                              _sz(row_end)))
    output.reshape(-1)[: row_end - row_start] = full[row_start:row_end]


def matmul_q8_0_quantized_parallel_rows(weight, input_q8, input_scales, output, n_in, n_out, ith, nth):
    """src/ops/kernel/q8_0/parallel.rs:102-139: writes output[my_start..my_end] of the full slice."""
    w = _as_tensor(weight, n_in, n_out)
    s, e = _row_range(n_out, ith, nth)
    if s >= e:
        return
    q8 = np.ascontiguousarray(input_q8, np.uint8)
    sc = np.ascontiguousarray(input_scales, np.float32)
    assert output.dtype == np.float32 and output.flags.c_contiguous and output.size >= n_out
    _check(lib().rmi_matmul_q8_0_prequantized(w._ctx.handle, w._h, _p(q8), _p(sc), _sz(1), _p(output), _sz(s), _sz(e)))


def matmul_q8_0_quantized(weight, input_q8, input_scales, output, n_in, n_out):
    """src/ops/kernel/q8_0/parallel.rs:25-96"""
    matmul_q8_0_quantized_parallel_rows(weight, input_q8, input_scales, output, n_in, n_out, 0, 1)


def matmul_q8_0_prequantized_rows(weight: QuantizedTensor, q8, scales, m: int, row_begin=0, row_end=None):
    """m activation rows at once -> [m, n_out] (columns outside the range stay zero)."""
    row_end = weight.n_out if row_end is None else row_end
    out = np.zeros((m, weight.n_out), np.float32)
    q8 = np.ascontiguousarray(q8, np.uint8)
    sc = np.ascontiguousarray(scales, np.float32)
    _check(lib().rmi_matmul_q8_0_prequantized(weight._ctx.handle, weight._h, _p(q8), _p(sc), _sz(m), _p(out),
                                              _sz(row_begin), _sz(row_end)))
    return out


def matmul_q8_0(weight: QuantizedTensor, x) -> np.ndarray:
    """f32 activations [m, n_in] -> [m, n_out] (quantize rows, then the matmul)."""
    x = np.ascontiguousarray(x, np.float32).reshape(-1, weight.n_in)
    out = np.zeros((x.shape[0], weight.n_out), np.float32)
    _check(lib().rmi_matmul_q8_0(weight._ctx.handle, weight._h, _p(x), _sz(x.shape[0]), _p(out)))
    return out


def matmul_q8_0_f32(weight: QuantizedTensor, x) -> np.ndarray:
    """ops::matmul_q8_0 (src/ops/kernel/q8_0/parallel.rs:317-341): dequantized weight x f32 activations [m, n_in],
    no activation quantization; AVX2 or scalar accumulation order by the context's semantics."""
    x = np.ascontiguousarray(x, np.float32).reshape(-1, weight.n_in)
    out = np.zeros((x.shape[0], weight.n_out), np.float32)
    _check(lib().rmi_matmul_q8_0_f32(weight._ctx.handle, weight._h, _p(x), _sz(x.shape[0]), _p(out)))
    return out


def matmul_q8_0_f32_dev(weight: QuantizedTensor, x_ptr: int, m: int, out_ptr: int):
    _check(lib().rmi_matmul_q8_0_f32_dev(weight._ctx.handle, weight._h, C.c_void_p(x_ptr), _sz(m), C.c_void_p(out_ptr)))


def q8_0_block_sums(weight: QuantizedTensor, q8, m: int, use_tensor_cores: bool = False) -> np.ndarray:
    q8 = np.ascontiguousarray(q8, np.uint8)
    out = np.zeros((m, weight.n_out, weight.n_in // 32), np.int32)
    _check(lib().rmi_q8_0_block_sums(weight._ctx.handle, weight._h, _p(q8), _sz(m), _p(out),
                                     C.c_int32(1 if use_tensor_cores else 0)))
    return out


def silu_mul_inplace(gate, up: np.ndarray, ctx: Context | None = None):
    """src/ops/activation/mod.rs:137-151"""
    ctx = ctx or context()
    gate = np.ascontiguousarray(gate, np.float32)
    assert up.dtype == np.float32 and up.flags.c_contiguous and up.size == gate.size
    _check(lib().rmi_silu_mul(ctx.handle, _p(gate), _p(up), _sz(gate.size)))


def ffn_swiglu_q8_0(w_gate_up: QuantizedTensor, w_down: QuantizedTensor, x) -> np.ndarray:
    """src/models/qwen3.rs:981-1046 for every row of x."""
    x = np.ascontiguousarray(x, np.float32).reshape(-1, w_gate_up.n_in)
    out = np.zeros((x.shape[0], w_down.n_out), np.float32)
    _check(lib().rmi_ffn_swiglu_q8_0(w_gate_up._ctx.handle, w_gate_up._h, w_down._h, _p(x), _sz(x.shape[0]), _p(out)))
    return out


def ffn_swiglu_q8_0_pipelined(w_gate_up, w_down, x_ptrs, out_ptrs, m: int):
    """A run of FFN calls over host buffers (addresses as integers, pinned for overlap) with the copies of
    neighbouring batches overlapped with the arithmetic.  w_gate_up / w_down: one QuantizedTensor per batch."""
    n = len(x_ptrs)
    if not (len(w_gate_up) == len(w_down) == len(out_ptrs) == n):
        raise ValueError("one weight pair, one input and one output per batch")
    if n == 0:
        return
    wg = (C.c_void_p * n)(*[w._h for w in w_gate_up])
    wd = (C.c_void_p * n)(*[w._h for w in w_down])
    xs = (C.c_void_p * n)(*[C.c_void_p(p) for p in x_ptrs])
    outs = (C.c_void_p * n)(*[C.c_void_p(p) for p in out_ptrs])
    _check(lib().rmi_ffn_swiglu_q8_0_pipelined(w_gate_up[0]._ctx.handle, wg, wd, xs, outs, _sz(n), _sz(m)))


# Device-pointer variants (stream-ordered, no synchronisation): pointers are integers, e.g.
# torch.Tensor.data_ptr() or Context.dev_alloc().

def ffn_swiglu_q8_0_dev(w_gate_up: QuantizedTensor, w_down: QuantizedTensor, x_ptr: int, m: int, out_ptr: int):
    _check(lib().rmi_ffn_swiglu_q8_0_dev(w_gate_up._ctx.handle, w_gate_up._h, w_down._h, C.c_void_p(x_ptr), _sz(m),
                                         C.c_void_p(out_ptr)))


def matmul_q8_0_dev(weight: QuantizedTensor, x_ptr: int, m: int, out_ptr: int):
    _check(lib().rmi_matmul_q8_0_dev(weight._ctx.handle, weight._h, C.c_void_p(x_ptr), _sz(m), C.c_void_p(out_ptr)))


def matmul_q8_0_dev_noalloc(weight: QuantizedTensor, x_ptr: int, m: int, out_ptr: int):
    """Allocation-free variant of matmul_q8_0_dev (m <= 32, m * n_in <= 524288): see include/rmi_cuda.h."""
    _check(lib().rmi_matmul_q8_0_dev_noalloc(weight._ctx.handle, weight._h, C.c_void_p(x_ptr), _sz(m),
                                             C.c_void_p(out_ptr)))


def matmul_q8_0_prequantized_dev(weight: QuantizedTensor, q8_ptr: int, scales_ptr: int, m: int, out_ptr: int,
                                 row_begin: int = 0, row_end: int | None = None):
    row_end = weight.n_out if row_end is None else row_end
    _check(lib().rmi_matmul_q8_0_prequantized_dev(weight._ctx.handle, weight._h, C.c_void_p(q8_ptr),
                                                  C.c_void_p(scales_ptr), _sz(m), C.c_void_p(out_ptr), _sz(row_begin),
                                                  _sz(row_end)))


def quantize_q8_0_dev(ctx: Context, x_ptr: int, m: int, n: int, q8_ptr: int, scales_ptr: int):
    _check(lib().rmi_quantize_q8_0_dev(ctx.handle, C.c_void_p(x_ptr), _sz(m), _sz(n), C.c_void_p(q8_ptr),
                                       C.c_void_p(scales_ptr)))


def matmul_q4_k_q8k_dev(weight: QuantizedTensor, x_ptr: int, m: int, out_ptr: int):
    _check(lib().rmi_matmul_q4_k_q8k_dev(weight._ctx.handle, weight._h, C.c_void_p(x_ptr), _sz(m), C.c_void_p(out_ptr)))


def matmul_q4_k_dequant_dev(weight: QuantizedTensor, x_ptr: int, m: int, out_ptr: int):
    _check(lib().rmi_matmul_q4_k_dequant_dev(weight._ctx.handle, weight._h, C.c_void_p(x_ptr), _sz(m),
                                             C.c_void_p(out_ptr)))


def unshard_cols_dev(ctx: Context, gathered_ptr: int, g: int, m: int, n_per_rank: int, out_ptr: int):
    _check(lib().rmi_unshard_cols_dev(ctx.handle, C.c_void_p(gathered_ptr), _sz(g), _sz(m), _sz(n_per_rank),
                                      C.c_void_p(out_ptr)))


def matmul_q8_0_fanout_dev(w: "QuantizedTensor", x_ptr: int, m: int, out_ptrs, out_stride: int, col_offset: int):
    """y = x W^T stored into every buffer of `out_ptrs` ([m][out_stride] f32) at columns col_offset.."""
    arr = (C.c_void_p * len(out_ptrs))(*[C.c_void_p(p) for p in out_ptrs])
    _check(lib().rmi_matmul_q8_0_fanout_dev(w._ctx.handle, w._h, C.c_void_p(x_ptr), _sz(m), arr,
                                            C.c_int32(len(out_ptrs)), _sz(out_stride), _sz(col_offset)))


def peer_signal_wait_dev(ctx: Context, flag_ptrs, rank: int, epoch: int):
    arr = (C.c_void_p * len(flag_ptrs))(*[C.c_void_p(p) for p in flag_ptrs])
    _check(lib().rmi_peer_signal_wait_dev(ctx.handle, arr, C.c_int32(len(flag_ptrs)), C.c_int32(rank),
                                          C.c_uint32(epoch & 0xffffffff)))


EXCHANGE_FUSED_STORES, EXCHANGE_PEER_COPY, EXCHANGE_PEER_PUSH = 0, 1, 2


class ShardGroup:
    """rmi_shard_group: one rank's result buffers and flags of a row-sharded matmul, and the peers' mappings."""

    def __init__(self, ctx: Context, world: int, rank: int, n_out: int, m_max: int):
        self._ctx, self.world, self.rank, self.n_out, self.m_max = ctx, world, rank, n_out, m_max
        self._h = C.c_void_p()
        _check(lib().rmi_shard_group_create(ctx.handle, C.c_int32(world), C.c_int32(rank), _sz(n_out), _sz(m_max),
                                            C.byref(self._h)))

    def export(self) -> bytes:
        buf = (C.c_uint8 * 192)()
        _check(lib().rmi_shard_group_export(self._ctx.handle, self._h, buf))
        return bytes(buf)

    def connect(self, handles_by_rank: list):
        blob = b"".join(handles_by_rank)
        if len(blob) != 192 * self.world:
            raise ValueError("need one 192-byte handle block per rank")
        buf = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
        _check(lib().rmi_shard_group_connect(self._ctx.handle, self._h, buf))

    @property
    def epoch(self) -> int:
        v = C.c_uint32()
        _check(lib().rmi_shard_group_epoch(self._h, C.byref(v)))
        return v.value

    def matmul_dev(self, w_shard: "QuantizedTensor", x_ptr: int, m: int, exchange: int = EXCHANGE_FUSED_STORES) -> int:
        """-> device pointer of this round's [m, n_out] result (complete once the enqueued work has run)."""
        out = C.c_void_p()
        _check(lib().rmi_matmul_q8_0_sharded_dev(self._ctx.handle, self._h, w_shard._h, C.c_void_p(x_ptr), _sz(m),
                                                 C.c_int32(exchange), C.byref(out)))
        return out.value

    def free(self):
        if self._h:
            _check(lib().rmi_shard_group_free(self._ctx.handle, self._h))
            self._h = C.c_void_p()


class NcclComm:
    """An NCCL communicator created through the library (rmi_nccl_*): rank 0 draws the id, `bcast(id_or_None)`
    returns rank 0's id on every rank (e.g. a torch.distributed object broadcast)."""

    def __init__(self, ctx: Context, world: int, rank: int, bcast):
        buf = (C.c_uint8 * 128)()
        if rank == 0:
            _check(lib().rmi_nccl_unique_id(buf))
        ident = bcast(bytes(buf) if rank == 0 else None)
        buf = (C.c_uint8 * 128).from_buffer_copy(ident)
        self._ctx, self.world, self.rank = ctx, world, rank
        self._h = C.c_void_p()
        _check(lib().rmi_nccl_comm_create(ctx.handle, buf, C.c_int32(world), C.c_int32(rank), C.byref(self._h)))

    def allgather_cols_dev(self, y_local_ptr: int, m: int, n_per_rank: int, gathered_ptr: int, out_ptr: int):
        _check(lib().rmi_allgather_cols_dev(self._ctx.handle, self._h, C.c_void_p(y_local_ptr), _sz(m), _sz(n_per_rank),
                                            C.c_int32(self.world), C.c_void_p(gathered_ptr or 0), C.c_void_p(out_ptr)))

    def destroy(self):
        if self._h:
            self._ctx.sync()
            _check(lib().rmi_nccl_comm_destroy(self._h))
            self._h = C.c_void_p()


def quantize_row_q8_k(x, ctx: Context | None = None):
    """src/ops/quant/mod.rs:42-61 -> (d[nb], qs[nb,256], bsums[nb,16])"""
    ctx = ctx or context()
    x = np.ascontiguousarray(x, np.float32).reshape(-1)
    nb = x.size // 256
    d, qs, bs = np.zeros(nb, np.float32), np.zeros((nb, 256), np.int8), np.zeros((nb, 16), np.int16)
    _check(lib().rmi_quantize_q8_k(ctx.handle, _p(x), _sz(1), _sz(x.size), _p(d), _p(qs), _p(bs)))
    return d, qs, bs


def dequantize_q4_k_weight(weight: QuantizedTensor) -> np.ndarray:
    """src/ops/quant/mod.rs:492-508"""
    out = np.zeros((weight.n_out, weight.n_in), np.float32)
    _check(lib().rmi_dequantize_q4_k(weight._ctx.handle, weight._h, _p(out)))
    return out


class Qwen35Ffn:
    """The multi-token FFN of the reference's Qwen3.5 forward (`forward_ffn_parallel`,
    src/models/qwen35.rs:762-782) for Q8_0 weights: per token gate and up matmuls on the Q8_0-quantized
    hidden row, `silu_mul_inplace` over all tokens, per token down matmul on the re-quantized product.
    Here one fused call for all tokens: v-stacked gate|up weight, SiLU*up and the re-quantization in the
    GEMM epilogue (tcgen05 for more than 32 tokens under NEON/SCALAR semantics)."""

    def __init__(self, ffn_gate: "QuantizedTensor", ffn_up: "QuantizedTensor", ffn_down: "QuantizedTensor"):
        if ffn_gate.ggml_type != GGML_Q8_0 or ffn_up.ggml_type != GGML_Q8_0 or ffn_down.ggml_type != GGML_Q8_0:
            raise RmiError(5, "Qwen35Ffn: Q8_0 weights only")
        self.n_embd, self.n_ff = ffn_gate.n_in, ffn_gate.n_out
        self.gate_up = ffn_gate.fuse_vstack(ffn_up)
        self.down = ffn_down

    def forward_ffn_parallel(self, hidden, n_tokens: int) -> np.ndarray:
        hidden = np.ascontiguousarray(hidden, np.float32).reshape(n_tokens, self.n_embd)
        return ffn_swiglu_q8_0(self.gate_up, self.down, hidden)

    def free(self):
        self.gate_up.free()


class QuantizedLinear:
    """QuantizedLinear<'a> (src/core/model.rs:12-104): Q4_K dequantize-and-matmul Layer."""

    def __init__(self, tensor: QuantizedTensor, name: str = ""):
        self._t, self.layer_name = tensor, name

    @classmethod
    def from_weight_slice(cls, weight, bias, in_features: int, out_features: int, name: str = "",
                          ctx: Context | None = None) -> "QuantizedLinear":
        return cls(QuantizedTensor.from_bytes(weight, GGML_Q4_K, in_features, out_features, ctx=ctx), name)

    @classmethod
    def from_source(cls, source: "GGUFLoader", weight_name: str, bias_name, in_features: int, out_features: int,
                    name: str = ""):
        if source.tensor_info(weight_name) is None:
            return None
        return cls(QuantizedTensor.from_gguf(source, weight_name), name)

    def forward_dequant(self, input, output: np.ndarray, scratch=None):
        x = np.ascontiguousarray(input, np.float32).reshape(-1, self._t.n_in)
        assert output.dtype == np.float32 and output.flags.c_contiguous
        _check(lib().rmi_matmul_q4_k_dequant(self._t._ctx.handle, self._t._h, _p(x), _sz(x.shape[0]), _p(output)))

    def forward(self, input, output, ctx=None):
        self.forward_dequant(input, output)

    def input_dim(self):
        return self._t.n_in

    def output_dim(self):
        return self._t.n_out

    def name(self):
        return self.layer_name


# ------------------------------------------------------------------------------ GGUF / Qwen3

class GGUFLoader:
    """GGUFLoader (src/core/loader.rs:189-395) over the library's mmap reader."""

    def __init__(self, handle):
        self._h = handle

    @classmethod
    def from_file(cls, path: str) -> "GGUFLoader":
        h = C.c_void_p()
        _check(lib().rmi_gguf_open(str(path).encode(), C.byref(h)))
        return cls(h)

    def close(self):
        if self._h:
            lib().rmi_gguf_close(self._h)
            self._h = C.c_void_p()

    def n_tensors(self) -> int:
        n = C.c_size_t()
        _check(lib().rmi_gguf_n_tensors(self._h, C.byref(n)))
        return n.value

    def tensor_info(self, name: str):
        t, nd, dims = C.c_int32(), C.c_int32(), (C.c_uint64 * 4)()
        data, nb = C.c_void_p(), C.c_size_t()
        st = lib().rmi_gguf_tensor(self._h, name.encode(), C.byref(t), dims, C.byref(nd), C.byref(data), C.byref(nb))
        if st != 0:
            return None
        return {"ggml_type": t.value, "dims": [int(dims[i]) for i in range(nd.value)], "nbytes": nb.value,
                "ptr": data.value}

    def tensor_slice(self, name: str):
        info = self.tensor_info(name)
        if info is None:
            return None
        return np.ctypeslib.as_array((C.c_uint8 * info["nbytes"]).from_address(info["ptr"]))

    def metadata_u64(self, key: str):
        v = C.c_uint64()
        return v.value if lib().rmi_gguf_meta_u64(self._h, key.encode(), C.byref(v)) == 0 else None

    def metadata_f64(self, key: str):
        v = C.c_double()
        return v.value if lib().rmi_gguf_meta_f64(self._h, key.encode(), C.byref(v)) == 0 else None

    def metadata_str(self, key: str):
        buf = C.create_string_buffer(256)
        return buf.value.decode() if lib().rmi_gguf_meta_str(self._h, key.encode(), buf, _sz(256)) == 0 else None


class Qwen3Model:
    """Qwen3Model (src/models/qwen3.rs:212-243): weights resident in HBM."""

    def __init__(self, handle, ctx: Context):
        self._h, self._ctx = handle, ctx
        v = [C.c_size_t() for _ in range(7)]
        _check(lib().rmi_qwen3_config(self._h, *[C.byref(x) for x in v]))
        self.config = dict(zip(("n_embd", "n_layer", "n_head", "n_head_kv", "head_dim", "n_ff", "vocab"),
                               (x.value for x in v)))

    @classmethod
    def from_file(cls, path: str, ctx: Context | None = None) -> "Qwen3Model":
        ctx = ctx or context()
        h = C.c_void_p()
        _check(lib().rmi_qwen3_load(ctx.handle, str(path).encode(), C.byref(h)))
        return cls(h, ctx)

    def generate(self, prompts, max_new_tokens: int):
        """Qwen3Model::generate (src/models/qwen3.rs:407-437), greedy; prompts [batch, n_prompt]."""
        prompts = np.ascontiguousarray(prompts, np.uint32)
        prompts = prompts.reshape(1, -1) if prompts.ndim == 1 else prompts
        s = Qwen3Session(self, prompts.shape[1] + max_new_tokens, batch=prompts.shape[0])
        try:
            return s.generate(prompts, max_new_tokens)
        finally:
            s.free()

    def free(self):
        if self._h:
            _check(lib().rmi_qwen3_free(self._ctx.handle, self._h))
            self._h = C.c_void_p()


class Qwen3Session:
    """Qwen3Session (src/models/qwen3.rs:238-243, :440-550): F16 KV cache + scratch in HBM."""

    def __init__(self, model: Qwen3Model, capacity: int, batch: int = 1, forward: int = 0):
        self.model, self._ctx, self.batch, self.capacity = model, model._ctx, batch, capacity
        self._h = C.c_void_p()
        _check(lib().rmi_session_create(self._ctx.handle, model._h, _sz(batch), _sz(capacity), C.byref(self._h)))
        self.prefill_ms = self.gen_ms = 0.0
        if forward != FORWARD_QWEN3_SESSION:
            self.set_forward(forward)

    def set_forward(self, forward: int):
        """FORWARD_QWEN3_SESSION (src/models/qwen3.rs), FORWARD_APP_TEXT (the CLI's loop, src/app/text.rs:257-648) or
        FORWARD_APP_TEXT_F32KV (that loop with `--kv-cache f32`; at most 512 positions), FORWARD_APP_LOGITS /
        FORWARD_APP_LOGITS_F32KV (the logits tool's loop, src/app/logits.rs, over the F16 / F32 cache)."""
        _check(lib().rmi_session_set_forward(self._ctx.handle, self._h, C.c_int32(forward)))

    def set_prefill(self, mode: int):
        """PREFILL_BATCHED (default: prompt positions as rows through every operator, bit-identical to the token
        loop), PREFILL_TOKEN_LOOP (one position per step, the reference's order) or PREFILL_BATCHED_TENSOR (AVX2
        semantics also on the tensor cores: cache rows within the 1e-5 matmul contract instead of bit-equal)."""
        _check(lib().rmi_session_set_prefill(self._ctx.handle, self._h, C.c_int32(mode)))

    def generate(self, prompts, max_new_tokens: int) -> np.ndarray:
        prompts = np.ascontiguousarray(prompts, np.uint32).reshape(self.batch, -1)
        out = np.zeros((self.batch, max(max_new_tokens, 1)), np.uint32)
        pre, gen = C.c_float(), C.c_float()
        _check(lib().rmi_session_generate(self._ctx.handle, self._h, _p(prompts), _sz(prompts.shape[1]),
                                          _sz(max_new_tokens), _p(out), C.byref(pre), C.byref(gen)))
        self.prefill_ms, self.gen_ms = pre.value, gen.value
        return out[:, :max_new_tokens]

    # per-step interface: the host feeds tokens and samples itself
    def reset(self):
        _check(lib().rmi_session_reset(self._ctx.handle, self._h))

    def prefill(self, tokens):
        """tokens [batch, n]: positions 0..n-1 whose logits nobody needs (a prompt without its last token)."""
        tokens = np.ascontiguousarray(tokens, np.uint32).reshape(self.batch, -1)
        _check(lib().rmi_session_prefill(self._ctx.handle, self._h, _p(tokens), _sz(tokens.shape[1])))

    def step(self, tokens, want_logits: bool = False):
        """tokens [batch] at the current position -> greedy next tokens [batch] (and the logits [batch, vocab])."""
        tokens = np.ascontiguousarray(tokens, np.uint32).reshape(self.batch)
        nxt = np.zeros(self.batch, np.uint32)
        logits = np.zeros((self.batch, self.model.config["vocab"]), np.float32) if want_logits else None
        _check(lib().rmi_session_step(self._ctx.handle, self._h, _p(tokens), _p(nxt), _p(logits)))
        return (nxt, logits) if want_logits else nxt

    @property
    def position(self) -> int:
        v = C.c_size_t()
        _check(lib().rmi_session_position(self._h, C.byref(v)))
        return v.value

    def hidden(self) -> np.ndarray:
        out = np.zeros((self.batch, self.model.config["n_embd"]), np.float32)
        _check(lib().rmi_session_read_hidden(self._ctx.handle, self._h, _p(out)))
        return out

    def logits(self) -> np.ndarray:
        out = np.zeros((self.batch, self.model.config["vocab"]), np.float32)
        _check(lib().rmi_session_read_logits(self._ctx.handle, self._h, _p(out)))
        return out

    def free(self):
        if self._h:
            _check(lib().rmi_session_free(self._ctx.handle, self._h))
            self._h = C.c_void_p()
