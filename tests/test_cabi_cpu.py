"""CPU-side checks of the product library: it loads, exports every declared symbol, parses
GGUF like the reference loader, and its host helpers agree with the oracle. No device calls."""
import ctypes as C
import os
import re
import struct

import numpy as np
import pytest

from oracle import orc
from tests.helpers import bits
from tests.synth_model import tiny_model

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(rmi):
    hdr = open(os.path.join(ROOT, "include", "rmi_cuda.h")).read()
    names = sorted(set(re.findall(r"^(?:int32_t|const char\*)\s+(rmi_[a-z0-9_]+)\s*\(", hdr, re.M)))
    assert len(names) >= 45
    lib = rmi.lib()
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_init_without_a_device_is_an_error_not_a_fallback(rmi):
    try:
        import torch
        if torch.cuda.is_available():
            pytest.skip("a GPU is present")
    except ImportError:
        pass
    with pytest.raises(rmi.RmiError) as e:
        rmi.Context(0)
    assert e.value.status in (4, 6)


def test_numpy_weight_encoder_equals_the_oracle_quantizer(rmi):
    w = rmi.synth.normal((37, 256), seed=11, std=0.02)
    w[3, 32:64] = 0.0
    enc = rmi.synth.encode_q8_0(w).reshape(37, 8, 34)
    q8, sc = orc.quantize_q8_0(w, orc.SEM_AVX2)
    assert np.array_equal(enc[:, :, 2:].reshape(37, 256), q8)
    d = enc[:, :, :2].copy().view(np.float16).astype(np.float32).reshape(37, 8)
    assert np.array_equal(bits(d), bits(sc))


def test_row_partition_matches_parallel_rows(rmi):
    # src/ops/kernel/q8_0/parallel.rs:124-129
    for n_out in (0, 1, 4, 5, 3072, 3584, 7168, 151936):
        for nth in (1, 2, 3, 4, 8, 16):
            covered = []
            for ith in range(nth):
                s, e = rmi._row_range(n_out, ith, nth)
                covered += list(range(s, e)) if n_out < 10000 else [(s, e)]
                per = (n_out + nth - 1) // nth if nth > 1 else n_out
                assert (s, e) == ((0, n_out) if nth <= 1 or n_out == 0 else (ith * per, max(ith * per, min(ith * per + per, n_out))))
            if n_out < 10000 and nth > 1:
                assert covered == list(range(n_out))


@pytest.fixture(scope="module")
def tiny_gguf(tmp_path_factory, rmi):
    cfg, tensors = tiny_model(seed=0)
    path = str(tmp_path_factory.mktemp("gguf") / "tiny.gguf")
    rmi.synth.write_qwen3_gguf(path, cfg, tensors)
    return path, cfg, tensors


def test_gguf_loader_reads_what_the_writer_wrote(rmi, tiny_gguf):
    # src/core/loader.rs:846-902 (byte-built file, metadata + tensor table + data offset)
    path, cfg, tensors = tiny_gguf
    g = rmi.GGUFLoader.from_file(path)
    assert g.n_tensors() == len(tensors)
    assert g.metadata_str("general.architecture") == "qwen3"
    assert g.metadata_u64("qwen3.embedding_length") == cfg["n_embd"]
    assert g.metadata_u64("qwen3.block_count") == cfg["n_layer"]
    assert abs(g.metadata_f64("qwen3.rope.freq_base") - 1e6) < 1
    assert g.metadata_u64("missing.key") is None
    py = rmi.gguf.GGUFFile(path)
    for name, arr in tensors.items():
        info = g.tensor_info(name)
        assert info is not None, name
        got = g.tensor_slice(name)
        assert np.array_equal(got, arr.view(np.uint8).reshape(-1)), name
        assert np.array_equal(py.tensor(name), got)
        assert info["dims"] == py.tensors[name][0]
    assert g.tensor_info("blk.0.attn_q.weight")["dims"] == [cfg["n_embd"], cfg["n_head"] * cfg["head_dim"]]
    assert g.tensor_info("nope") is None
    g.close()


def _write(tmp_path, name, data):
    p = tmp_path / name
    p.write_bytes(data)
    return str(p)


def test_gguf_loader_rejects_malformed_files(rmi, tmp_path, tiny_gguf):
    # src/core/loader.rs:988-1170 (malformed-input rejections)
    good = open(tiny_gguf[0], "rb").read()
    cases = {
        "magic": b"GGUX" + good[4:],
        "version": good[:4] + struct.pack("<I", 1) + good[8:],
        "version4": good[:4] + struct.pack("<I", 4) + good[8:],
        "truncated_header": good[:40],
        "truncated_data": good[: len(good) - 4096],
        "huge_tensor_count": good[:8] + struct.pack("<Q", 1 << 60) + good[16:],
        "huge_kv_count": good[:16] + struct.pack("<Q", 1 << 60) + good[24:],
    }
    for name, data in cases.items():
        with pytest.raises(rmi.RmiError) as e:
            rmi.GGUFLoader.from_file(_write(tmp_path, name + ".gguf", data))
        assert e.value.status == 8, name
    with pytest.raises(rmi.RmiError) as e:
        rmi.GGUFLoader.from_file(str(tmp_path / "does_not_exist.gguf"))
    assert e.value.status == 7


def test_gguf_zero_alignment_is_rejected(rmi, tmp_path):
    G = rmi.gguf
    p = str(tmp_path / "a.gguf")
    G.write_gguf(p, [("general.alignment", G.T_U32, 0)], [])
    with pytest.raises(rmi.RmiError):
        rmi.GGUFLoader.from_file(p)


def test_oracle_decode_is_deterministic_and_thread_count_invariant():
    cfg, tensors = tiny_model(seed=1)
    m = orc.Qwen3(cfg, tensors)
    prompt = np.array([5, 9, 200, 17, 3], np.uint32)
    a = m.generate(prompt, 12, threads=1)
    b = m.generate(prompt, 12, threads=4)
    assert np.array_equal(a, b) and len(a) == 12


def test_oracle_libm_and_correctly_rounded_exp_give_the_same_tokens_on_a_small_model():
    cfg, tensors = tiny_model(seed=2)
    m = orc.Qwen3(cfg, tensors)
    prompt = np.arange(1, 17, dtype=np.uint32)
    orc.set_exp_mode(orc.EXP_LIBM)
    a = m.generate(prompt, 16)
    orc.set_exp_mode(orc.EXP_CR)
    b = m.generate(prompt, 16)
    assert np.array_equal(a, b)
