"""Qwen3-architecture decode on the device vs the oracle: identical greedy tokens and
bit-identical hidden state / logits of the final step."""
import os

import numpy as np
import pytest

from oracle import orc
from tests.helpers import bits
from tests.synth_model import tiny_cfg

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx(rmi):
    c = rmi.context(0)
    yield c
    c.set_semantics(rmi.SEM_AVX2)


def _model(rmi, tmp_path_factory, cfg, seed):
    tensors = rmi.synth.qwen3_tensors(cfg, seed)
    path = str(tmp_path_factory.mktemp("m") / "model.gguf")
    rmi.synth.write_qwen3_gguf(path, cfg, tensors)
    return path, tensors


@pytest.mark.parametrize("sem", [orc.SEM_AVX2, orc.SEM_NEON, orc.SEM_SCALAR])
def test_tiny_model_tokens_hidden_and_logits(rmi, ctx, tmp_path_factory, sem):
    ctx.set_semantics(sem)
    cfg = tiny_cfg()
    path, tensors = _model(rmi, tmp_path_factory, cfg, seed=0)
    model = rmi.Qwen3Model.from_file(path)
    assert model.config["n_embd"] == cfg["n_embd"] and model.config["vocab"] == cfg["vocab"]
    oracle = orc.Qwen3(cfg, tensors)
    prompt = rmi.synth.prompt_tokens(cfg["vocab"], 24, seed=7)
    s = rmi.Qwen3Session(model, 24 + 40)
    got = s.generate(prompt, 40)[0]
    ref, trace, logits = oracle.generate(prompt, 40, sem=sem, want_trace=True, want_logits=True)
    assert np.array_equal(got, ref)
    assert np.array_equal(bits(s.hidden()[0]), bits(trace[-1]))
    assert np.array_equal(bits(s.logits()[0]), bits(logits))
    # a second run on the same session reproduces the tokens (KV cache is overwritten in place)
    assert np.array_equal(s.generate(prompt, 40)[0], ref)
    s.free()
    model.free()


@pytest.mark.parametrize("sem", [orc.SEM_AVX2, orc.SEM_NEON, orc.SEM_SCALAR])
def test_cli_forward_online_softmax_tokens_hidden_and_logits(rmi, ctx, tmp_path_factory, sem):
    """The CLI's copy of the forward (src/app/text.rs:257-648): f32 query x f16 keys, online soft-max, last
    maximal index.  Tokens identical, hidden state and logits bit-identical, in all three lane orders."""
    ctx.set_semantics(sem)
    cfg = tiny_cfg()
    path, tensors = _model(rmi, tmp_path_factory, cfg, seed=2)
    model = rmi.Qwen3Model.from_file(path)
    oracle = orc.Qwen3(cfg, tensors)
    prompt = rmi.synth.prompt_tokens(cfg["vocab"], 21, seed=9)
    s = rmi.Qwen3Session(model, 21 + 30, forward=rmi.FORWARD_APP_TEXT)
    got = s.generate(prompt, 30)[0]
    ref, trace, logits = oracle.generate(prompt, 30, sem=sem, want_trace=True, want_logits=True, cli=True)
    assert np.array_equal(got, ref)
    assert np.array_equal(bits(s.hidden()[0]), bits(trace[-1]))
    assert np.array_equal(bits(s.logits()[0]), bits(logits))
    # switching the same session back gives the Qwen3Session results again
    s.set_forward(rmi.FORWARD_QWEN3_SESSION)
    assert np.array_equal(s.generate(prompt, 30)[0], oracle.generate(prompt, 30, sem=sem))
    with pytest.raises(rmi.RmiError):
        s.set_forward(7)
    s.free()
    model.free()


@pytest.mark.parametrize("sem", [orc.SEM_AVX2, orc.SEM_NEON, orc.SEM_SCALAR])
def test_cli_forward_f32_kv_cache_tokens_hidden_and_logits(rmi, ctx, tmp_path_factory, sem):
    """The CLI loop with `--kv-cache f32` (src/app/text.rs:393-405, :458-496): f32 K/V, dot_f32 scores, padded
    soft-max, one dot over the positions per output element.  Bit-identical in all three lane orders."""
    ctx.set_semantics(sem)
    cfg = tiny_cfg()
    path, tensors = _model(rmi, tmp_path_factory, cfg, seed=2)
    model = rmi.Qwen3Model.from_file(path)
    oracle = orc.Qwen3(cfg, tensors)
    prompt = rmi.synth.prompt_tokens(cfg["vocab"], 21, seed=9)
    s = rmi.Qwen3Session(model, 21 + 30, forward=rmi.FORWARD_APP_TEXT_F32KV)
    got = s.generate(prompt, 30)[0]
    ref, trace, logits = oracle.generate(prompt, 30, sem=sem, want_trace=True, want_logits=True, cli=True, kv_f32=True)
    assert np.array_equal(got, ref)
    assert np.array_equal(bits(s.hidden()[0]), bits(trace[-1]))
    assert np.array_equal(bits(s.logits()[0]), bits(logits))
    # the F16-cache variant on the same session still gives its own results afterwards
    s.set_forward(rmi.FORWARD_APP_TEXT)
    assert np.array_equal(s.generate(prompt, 30)[0], oracle.generate(prompt, 30, sem=sem, cli=True))
    s.free()
    model.free()


def test_cli_forward_f32_kv_qwen3_head_shape_batch_and_context_limit(rmi, ctx, tmp_path_factory):
    ctx.set_semantics(rmi.SEM_AVX2)
    cfg = tiny_cfg(n_embd=1024, n_layer=2, n_head=16, n_head_kv=8, head_dim=128, n_ff=3072, vocab=2048)
    path, tensors = _model(rmi, tmp_path_factory, cfg, seed=0)
    model = rmi.Qwen3Model.from_file(path)
    oracle = orc.Qwen3(cfg, tensors)
    B = 3
    prompts = np.stack([rmi.synth.prompt_tokens(cfg["vocab"], 270, seed=20 + b) for b in range(B)])
    s = rmi.Qwen3Session(model, 300, batch=B, forward=rmi.FORWARD_APP_TEXT_F32KV)
    got = s.generate(prompts, 30)
    for b in range(B):
        ref, trace = oracle.generate(prompts[b], 30, sem=orc.SEM_AVX2, threads=8, want_trace=True, cli=True, kv_f32=True)
        assert np.array_equal(got[b], ref), b
        assert np.array_equal(bits(s.hidden()[b]), bits(trace[-1])), b
    s.free()
    # the reference's 512-entry value array: longer sessions are rejected, and the session keeps its variant
    long = rmi.Qwen3Session(model, 513)
    with pytest.raises(rmi.RmiError):
        long.set_forward(rmi.FORWARD_APP_TEXT_F32KV)
    long.free()
    with pytest.raises(RuntimeError):
        oracle.generate(prompts[0], 300, cli=True, kv_f32=True)
    model.free()


@pytest.mark.parametrize("sem", [orc.SEM_AVX2, orc.SEM_NEON, orc.SEM_SCALAR])
@pytest.mark.parametrize("kv_f32", [False, True])
def test_logits_tool_forward_tokens_hidden_and_logits(rmi, ctx, tmp_path_factory, sem, kv_f32):
    """The logits tool's loop (src/app/logits.rs:474-560) over the F16 and the F32 cache: lane-ordered scores,
    soft-max, sequential chain per output element.  Bit-identical in all three lane orders."""
    ctx.set_semantics(sem)
    cfg = tiny_cfg()
    path, tensors = _model(rmi, tmp_path_factory, cfg, seed=4)
    model = rmi.Qwen3Model.from_file(path)
    oracle = orc.Qwen3(cfg, tensors)
    prompt = rmi.synth.prompt_tokens(cfg["vocab"], 37, seed=12)
    fwd = rmi.FORWARD_APP_LOGITS_F32KV if kv_f32 else rmi.FORWARD_APP_LOGITS
    s = rmi.Qwen3Session(model, 37 + 9, forward=fwd)
    got = s.generate(prompt, 9)[0]
    ref, trace, logits = oracle.generate(prompt, 9, sem=sem, want_trace=True, want_logits=True, logits_tool=True,
                                         kv_f32=kv_f32)
    assert np.array_equal(got, ref)
    assert np.array_equal(bits(s.hidden()[0]), bits(trace[-1]))
    assert np.array_equal(bits(s.logits()[0]), bits(logits))
    s.free()
    model.free()


def test_logits_tool_forward_qwen3_head_shape_beyond_512_positions(rmi, ctx, tmp_path_factory):
    ctx.set_semantics(rmi.SEM_AVX2)
    cfg = tiny_cfg(n_embd=512, n_layer=2, n_head=8, n_head_kv=4, head_dim=128, n_ff=1024, vocab=512)
    path, tensors = _model(rmi, tmp_path_factory, cfg, seed=6)
    model = rmi.Qwen3Model.from_file(path)
    oracle = orc.Qwen3(cfg, tensors)
    B, P, G = 2, 530, 4
    prompts = np.stack([rmi.synth.prompt_tokens(cfg["vocab"], P, seed=40 + b) for b in range(B)])
    for kv_f32 in (False, True):
        s = rmi.Qwen3Session(model, P + G, batch=B,
                             forward=rmi.FORWARD_APP_LOGITS_F32KV if kv_f32 else rmi.FORWARD_APP_LOGITS)
        got = s.generate(prompts, G)
        for b in range(B):
            ref, trace = oracle.generate(prompts[b], G, threads=8, want_trace=True, logits_tool=True, kv_f32=kv_f32)
            assert np.array_equal(got[b], ref), (kv_f32, b)
            assert np.array_equal(bits(s.hidden()[b]), bits(trace[-1])), (kv_f32, b)
        s.free()
    model.free()


def test_cli_forward_qwen3_head_shape_long_context_and_batch(rmi, ctx, tmp_path_factory):
    ctx.set_semantics(rmi.SEM_AVX2)
    cfg = tiny_cfg(n_embd=1024, n_layer=2, n_head=16, n_head_kv=8, head_dim=128, n_ff=3072, vocab=2048)
    path, tensors = _model(rmi, tmp_path_factory, cfg, seed=0)
    model = rmi.Qwen3Model.from_file(path)
    oracle = orc.Qwen3(cfg, tensors)
    B = 3
    prompts = np.stack([rmi.synth.prompt_tokens(cfg["vocab"], 270, seed=20 + b) for b in range(B)])
    s = rmi.Qwen3Session(model, 300, batch=B, forward=rmi.FORWARD_APP_TEXT)
    got = s.generate(prompts, 30)
    for b in range(B):
        ref, trace = oracle.generate(prompts[b], 30, sem=orc.SEM_AVX2, threads=8, want_trace=True, cli=True)
        assert np.array_equal(got[b], ref), b
        assert np.array_equal(bits(s.hidden()[b]), bits(trace[-1])), b
    s.free()
    model.free()


@pytest.mark.parametrize("sem", [orc.SEM_AVX2, orc.SEM_NEON])
def test_large_batch_uses_the_single_cta_attention_and_stays_bit_exact(rmi, ctx, tmp_path_factory, sem):
    """batch * n_head_kv >= 64 switches to attention_seq_kernel (one CTA per sequence and kv head, K/V streamed
    through shared-memory tiles); head_dim 128, 300 positions cross the tile and the 256-padding boundaries."""
    ctx.set_semantics(sem)
    cfg = tiny_cfg(n_embd=512, n_layer=2, n_head=8, n_head_kv=4, head_dim=128, n_ff=1024, vocab=512)
    path, tensors = _model(rmi, tmp_path_factory, cfg, seed=3)
    model = rmi.Qwen3Model.from_file(path)
    oracle = orc.Qwen3(cfg, tensors)
    B, P, G = 33, 280, 12
    prompts = np.stack([rmi.synth.prompt_tokens(cfg["vocab"], P, seed=300 + b) for b in range(B)])
    s = rmi.Qwen3Session(model, P + G, batch=B)
    got = s.generate(prompts, G)
    hidden = s.hidden()
    for b in (0, 17, 32):
        ref, trace = oracle.generate(prompts[b], G, sem=sem, threads=8, want_trace=True)
        assert np.array_equal(got[b], ref), b
        assert np.array_equal(bits(hidden[b]), bits(trace[-1])), b
    s.free()
    model.free()


def test_batch_of_independent_sequences(rmi, ctx, tmp_path_factory):
    ctx.set_semantics(rmi.SEM_AVX2)
    cfg = tiny_cfg(n_layer=3)
    path, tensors = _model(rmi, tmp_path_factory, cfg, seed=4)
    model = rmi.Qwen3Model.from_file(path)
    oracle = orc.Qwen3(cfg, tensors)
    B, P, G = 11, 16, 12
    prompts = np.stack([rmi.synth.prompt_tokens(cfg["vocab"], P, seed=100 + b) for b in range(B)])
    got = model.generate(prompts, G)
    for b in range(B):
        assert np.array_equal(got[b], oracle.generate(prompts[b], G, sem=orc.SEM_AVX2)), b
    model.free()


def test_qwen3_head_shape_and_long_context(rmi, ctx, tmp_path_factory):
    # head_dim 128, 16 q / 8 kv heads, QK-norm, theta 1e6 as in Qwen3-0.6B; 2 layers, small vocab;
    # 300 positions crosses the 256-padding boundary of the reference's score rows
    ctx.set_semantics(rmi.SEM_AVX2)
    cfg = tiny_cfg(n_embd=1024, n_layer=2, n_head=16, n_head_kv=8, head_dim=128, n_ff=3072, vocab=2048)
    path, tensors = _model(rmi, tmp_path_factory, cfg, seed=0)
    model = rmi.Qwen3Model.from_file(path)
    prompt = rmi.synth.prompt_tokens(cfg["vocab"], 270, seed=1)
    s = rmi.Qwen3Session(model, 300)
    got = s.generate(prompt, 30)[0]
    ref, trace = orc.Qwen3(cfg, tensors).generate(prompt, 30, sem=orc.SEM_AVX2, threads=8, want_trace=True)
    assert np.array_equal(got, ref)
    assert np.array_equal(bits(s.hidden()[0]), bits(trace[-1]))
    s.free()
    model.free()


@pytest.mark.parametrize("batch", [1, 3])
def test_capacity_beyond_the_shared_memory_score_rows(rmi, ctx, tmp_path_factory, batch):
    """A session may be as long as the model's context (src/models/qwen3.rs:442-447).  At 40960 positions the score
    rows of the attention kernels no longer fit in shared memory and the single-CTA kernel keeps them in a global
    scratch area: same tokens and the same hidden-state bits as the oracle, and as a short session of the same model."""
    ctx.set_semantics(rmi.SEM_AVX2)
    cfg = tiny_cfg(n_head=4, n_head_kv=2, head_dim=128, n_embd=256, n_ctx=40960)
    path, tensors = _model(rmi, tmp_path_factory, cfg, seed=3)
    model = rmi.Qwen3Model.from_file(path)
    prompts = np.stack([rmi.synth.prompt_tokens(cfg["vocab"], 40, seed=5 + b) for b in range(batch)])
    long_s = rmi.Qwen3Session(model, 40960, batch=batch)
    got = long_s.generate(prompts, 12)
    hid = long_s.hidden().copy()
    long_s.free()
    short_s = rmi.Qwen3Session(model, 64, batch=batch)
    assert np.array_equal(short_s.generate(prompts, 12), got)
    assert np.array_equal(bits(short_s.hidden()), bits(hid))
    short_s.free()
    ref, trace = orc.Qwen3(cfg, tensors).generate(prompts[0], 12, sem=orc.SEM_AVX2, threads=8, want_trace=True)
    assert np.array_equal(got[0], ref)
    assert np.array_equal(bits(hid[0]), bits(trace[-1]))
    model.free()


def test_session_errors(rmi, ctx, tmp_path_factory):
    cfg = tiny_cfg()
    path, _ = _model(rmi, tmp_path_factory, cfg, seed=0)
    model = rmi.Qwen3Model.from_file(path)
    with pytest.raises(rmi.RmiError) as e:          # src/models/qwen3.rs:442-447
        rmi.Qwen3Session(model, 0)
    assert e.value.status == 2
    s = rmi.Qwen3Session(model, 8)
    with pytest.raises(rmi.RmiError) as e:          # :569-578 capacity
        s.generate(np.arange(6, dtype=np.uint32), 4)
    assert e.value.status == 2
    with pytest.raises(rmi.RmiError) as e:          # token id outside the vocabulary
        s.generate(np.array([cfg["vocab"]], np.uint32), 1)
    assert e.value.status == 2
    s.free()
    model.free()
    with pytest.raises(rmi.RmiError) as e:
        rmi.Qwen3Model.from_file(os.path.join(os.path.dirname(path), "missing.gguf"))
    assert e.value.status == 7


def _full_model(rmi):
    """Qwen3-0.6B-architecture checkpoint with random-init weights (seed 0), cached in the temp dir."""
    import tempfile
    cfg = dict(rmi.synth.QWEN3_0_6B)
    path = os.path.join(tempfile.gettempdir(), "rmi_qwen3_0_6b_seed0.gguf")
    if not os.path.exists(path):
        tmp = path + f".{os.getpid()}.tmp"
        rmi.synth.write_qwen3_gguf(tmp, cfg, rmi.synth.qwen3_tensors(cfg, 0))
        os.replace(tmp, path)
    f = rmi.gguf.GGUFFile(path)
    tensors = {}
    for name, (dims, gtype, data) in f.tensors.items():
        tensors[name] = data if gtype == rmi.gguf.GGML_Q8_0 else data.view(np.float32)
    return cfg, path, tensors


def test_config4_full_size_greedy_tokens_identical_over_128_steps(rmi, ctx):
    # BASELINE config 4: 28 layers, hidden 1024, 16 Q / 8 KV heads x 128, FFN 3072, vocab 151936 tied,
    # F16 KV cache, 512 random prompt ids, 128 greedy tokens (x86 production semantics)
    ctx.set_semantics(rmi.SEM_AVX2)
    cfg, path, tensors = _full_model(rmi)
    model = rmi.Qwen3Model.from_file(path)
    B, P, G = 2, 512, 128
    prompts = np.stack([rmi.synth.prompt_tokens(cfg["vocab"], P, seed=1000 + b) for b in range(B)])
    s = rmi.Qwen3Session(model, P + G, batch=B)
    got = s.generate(prompts, G)
    oracle = orc.Qwen3(cfg, tensors)
    threads = min(os.cpu_count() or 1, 16)
    ref0, trace, logits = oracle.generate(prompts[0], G, sem=orc.SEM_AVX2, threads=threads, want_trace=True,
                                          want_logits=True)
    assert np.array_equal(got[0], ref0)
    assert np.array_equal(bits(s.hidden()[0]), bits(trace[-1]))
    assert np.array_equal(bits(s.logits()[0]), bits(logits))
    top2 = np.sort(logits)[-2:]
    print(f"final-step top-1/top-2 logit margin: {top2[1] - top2[0]:.6f}")
    ref1 = oracle.generate(prompts[1], G, sem=orc.SEM_AVX2, threads=threads)
    assert np.array_equal(got[1], ref1)
    s.free()
    model.free()


def test_config4_full_size_batch_32_token_identity_on_sampled_sequences(rmi, ctx):
    # BASELINE config 4 at batch 32 (the single-CTA attention kernel, eight activation rows per GEMV pass, batched
    # prompt processing): three of the 32 sequences against the oracle, tokens and final hidden-state bits
    ctx.set_semantics(rmi.SEM_AVX2)
    cfg, path, tensors = _full_model(rmi)
    model = rmi.Qwen3Model.from_file(path)
    B, P, G = 32, 40, 8
    prompts = np.stack([rmi.synth.prompt_tokens(cfg["vocab"], P, seed=2000 + b) for b in range(B)])
    s = rmi.Qwen3Session(model, P + G, batch=B)
    got = s.generate(prompts, G)
    hid = s.hidden()
    oracle = orc.Qwen3(cfg, tensors)
    threads = min(os.cpu_count() or 1, 16)
    for b in (0, 13, 31):
        ref, trace = oracle.generate(prompts[b], G, sem=orc.SEM_AVX2, threads=threads, want_trace=True)
        assert np.array_equal(got[b], ref), b
        assert np.array_equal(bits(hid[b]), bits(trace[-1])), b
    s.free()
    model.free()


@pytest.mark.parametrize("sem", [orc.SEM_AVX2, orc.SEM_NEON, orc.SEM_SCALAR])
@pytest.mark.parametrize("batch,n_prompt", [(1, 70), (3, 33), (40, 300)])
def test_batched_prefill_equals_the_token_loop(rmi, ctx, tmp_path_factory, sem, batch, n_prompt):
    """Prompt positions as rows through every operator (matmuls with M = positions, causal attention per position)
    against the reference's one-position-per-step loop on the same session: tokens identical, hidden state and
    logits of the last step bit-identical; sequence 0 also against the oracle.  (40, 300) makes the prefill run
    in two groups of sequences (more than 8192 rows) and uses attention tiles of several key blocks."""
    ctx.set_semantics(sem)
    cfg = tiny_cfg()
    path, tensors = _model(rmi, tmp_path_factory, cfg, seed=5)
    model = rmi.Qwen3Model.from_file(path)
    n_gen = 12
    prompts = np.stack([rmi.synth.prompt_tokens(cfg["vocab"], n_prompt, seed=40 + b) for b in range(batch)])
    s = rmi.Qwen3Session(model, n_prompt + n_gen, batch=batch)
    s.set_prefill(rmi.PREFILL_TOKEN_LOOP)
    loop_tok = s.generate(prompts, n_gen)
    loop_hidden, loop_logits, loop_ms = s.hidden(), s.logits(), s.prefill_ms
    s.set_prefill(rmi.PREFILL_BATCHED)
    tok = s.generate(prompts, n_gen)
    assert np.array_equal(tok, loop_tok)
    assert np.array_equal(bits(s.hidden()), bits(loop_hidden))
    assert np.array_equal(bits(s.logits()), bits(loop_logits))
    ref = orc.Qwen3(cfg, tensors).generate(prompts[0], n_gen, sem=sem)
    assert np.array_equal(tok[0], ref)
    print(f"prefill {n_prompt - 1} positions x {batch}: token loop {loop_ms:.2f} ms, batched {s.prefill_ms:.2f} ms")
    s.free()
    model.free()


def test_batched_prefill_on_tensor_cores_under_avx2_semantics(rmi, ctx, tmp_path_factory):
    """RMI_PREFILL_BATCHED_TENSOR: AVX2 quantizer, whole-block accumulation on tcgen05 for the prompt rows.  The cache
    rows are then not bit-equal to the eight-lane order; the hidden state of the last step stays within a small
    relative distance and, on this model, the greedy tokens are the same."""
    ctx.set_semantics(rmi.SEM_AVX2)
    cfg = tiny_cfg()
    path, tensors = _model(rmi, tmp_path_factory, cfg, seed=6)
    model = rmi.Qwen3Model.from_file(path)
    prompts = np.stack([rmi.synth.prompt_tokens(cfg["vocab"], 130, seed=60 + b) for b in range(2)])
    s = rmi.Qwen3Session(model, 130 + 8, batch=2)
    exact = s.generate(prompts, 8)
    h_exact = s.hidden()
    s.set_prefill(rmi.PREFILL_BATCHED_TENSOR)
    tens = s.generate(prompts, 8)
    h_tens = s.hidden()
    assert np.array_equal(tens, exact)
    assert float(np.max(np.abs(h_tens - h_exact))) <= 2e-2 * float(np.max(np.abs(h_exact)))
    s.free()
    model.free()


@pytest.mark.parametrize("sem", [orc.SEM_AVX2, orc.SEM_NEON])
@pytest.mark.parametrize("n_prompt", [5, 40])
def test_per_step_interface_reproduces_generate(rmi, ctx, tmp_path_factory, sem, n_prompt):
    """reset / prefill / step with host-side greedy sampling from the returned logits: the same tokens, hidden state
    and logits as rmi_session_generate and the oracle (n_prompt = 40 takes the batched prefill, 5 the token loop)."""
    ctx.set_semantics(sem)
    cfg = tiny_cfg()
    path, tensors = _model(rmi, tmp_path_factory, cfg, seed=8)
    model = rmi.Qwen3Model.from_file(path)
    batch, n_gen = 2, 10
    prompts = np.stack([rmi.synth.prompt_tokens(cfg["vocab"], n_prompt, seed=80 + b) for b in range(batch)])
    s = rmi.Qwen3Session(model, n_prompt + n_gen, batch=batch)
    want = s.generate(prompts, n_gen)
    want_hidden, want_logits = s.hidden(), s.logits()
    s.reset()
    assert s.position == 0
    s.prefill(prompts[:, :-1])
    assert s.position == n_prompt - 1
    tok = prompts[:, -1].copy()
    got = np.zeros((batch, n_gen), np.uint32)
    for i in range(n_gen):
        greedy, logits = s.step(tok, want_logits=True)
        mine = np.array([orc.greedy_token(logits[b]) for b in range(batch)], np.uint32)   # the host's own sampler
        assert np.array_equal(mine, greedy)
        got[:, i] = mine
        tok = mine
        if i == n_gen - 2:   # generate() stops one step earlier: its last step produced token n_gen-1
            pass
    assert np.array_equal(got, want)
    assert s.position == n_prompt - 1 + n_gen
    ref = orc.Qwen3(cfg, tensors).generate(prompts[0], n_gen, sem=sem)
    assert np.array_equal(got[0], ref)
    # a session that is full refuses another step; generate() leaves step mode
    s2 = rmi.Qwen3Session(model, 3, batch=batch)
    s2.reset()
    for _ in range(3):
        s2.step(prompts[:, 0])
    with pytest.raises(rmi.RmiError):
        s2.step(prompts[:, 0])
    s2.generate(prompts[:, :2], 1)
    with pytest.raises(rmi.RmiError):
        s2.step(prompts[:, 0])
    s2.free()
    del want_hidden, want_logits
    s.free()
    model.free()
