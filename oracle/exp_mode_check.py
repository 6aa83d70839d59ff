"""Does the choice of exp() change the greedy tokens of the full-size benchmark model?

The device and the oracle evaluate exp() in soft-max and SiLU as the correctly rounded f32 exponential
(ORC_EXP_CR); the reference calls the platform libm (src/ops/attention.rs:28-38, src/ops/activation/mod.rs:8-10),
which the oracle also offers (ORC_EXP_LIBM).  This script runs the oracle's Qwen3Session on the
Qwen3-0.6B-architecture benchmark model (random init seed 0, 512 prompt ids, 128 greedy tokens) in both modes
and prints whether the tokens agree, and how far the final hidden states are apart.

TEST INFRASTRUCTURE (CPU only, a few minutes): python oracle/exp_mode_check.py [n_prompt] [n_gen] [threads]
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from __graft_entry__ import load_package  # noqa: E402
from oracle import orc  # noqa: E402


def main():
    n_prompt = int(sys.argv[1]) if len(sys.argv) > 1 else 512
    n_gen = int(sys.argv[2]) if len(sys.argv) > 2 else 128
    threads = int(sys.argv[3]) if len(sys.argv) > 3 else (os.cpu_count() or 1)
    pkg = load_package()
    cfg = dict(pkg.synth.QWEN3_0_6B)
    tensors = pkg.synth.qwen3_tensors(cfg, 0)
    model = orc.Qwen3(cfg, tensors)
    for seed in (1000, 1001):
        prompt = pkg.synth.prompt_tokens(cfg["vocab"], n_prompt, seed=seed)
        out = {}
        for name, mode in (("correctly_rounded", orc.EXP_CR), ("libm", orc.EXP_LIBM)):
            orc.set_exp_mode(mode)
            toks, trace = model.generate(prompt, n_gen, sem=orc.SEM_AVX2, threads=threads, want_trace=True)
            out[name] = (toks, trace[-1])
        orc.set_exp_mode(orc.EXP_CR)
        a, b = out["correctly_rounded"], out["libm"]
        same = bool(np.array_equal(a[0], b[0]))
        first = int(np.argmax(a[0] != b[0])) if not same else -1
        rel = float(np.max(np.abs(a[1] - b[1])) / max(float(np.max(np.abs(a[1]))), 1e-30))
        print(f"prompt seed {seed}: tokens identical = {same} (first difference at generated token {first}); "
              f"final hidden state max |a-b| / max |a| = {rel:.3e}; "
              f"bit-identical hidden = {bool(np.array_equal(a[1].view(np.uint32), b[1].view(np.uint32)))}", flush=True)


if __name__ == "__main__":
    main()
