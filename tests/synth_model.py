"""Small Qwen3-architecture models for CPU-sized parity cases."""
from __graft_entry__ import load_package


def tiny_cfg(**over):
    cfg = dict(n_embd=128, n_layer=2, n_head=4, n_head_kv=2, head_dim=32, n_ff=256, vocab=512,
               eps=1e-6, freq_base=1_000_000.0, n_ctx=4096)
    cfg.update(over)
    return cfg


def tiny_model(seed=0, **over):
    synth = load_package().synth
    cfg = tiny_cfg(**over)
    return cfg, synth.qwen3_tensors(cfg, seed)
