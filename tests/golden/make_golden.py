"""Generates tests/golden/moe_7m_golden.npz by running the REFERENCE's own CPU model.

Needs the reference sources (default /root/reference; override with GPTOSS_REFERENCE_DIR): the
reference's run.cpp is compiled by oracle/Makefile into oracle/_ref/libref_cpu.so and its forward()
(run.cpp:501) is executed on a seeded random-init checkpoint with the gpt-oss-7m dimensions
(export_model_bin/gpt-oss-7m/config.json).  After each position the state left by the last layer's
MoE block (run.cpp:622-704) is captured: block input t, router scores, top-k ids, softmaxed gate
weights and the block output e_agg.  The greedy continuation (32 random prompt ids, 64 generated
tokens) is stored too, together with, per position, the argmax token, the gap between the two largest
logits and the logits at 64 fixed vocabulary ids (for the whole-model parity test).

Run from the repository root:   python tests/golden/make_golden.py
"""
from __future__ import annotations

import hashlib
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import __graft_entry__ as entry  # noqa: E402

entry.load_package()
from gptoss_b200 import binfmt, synth  # noqa: E402
import oracle_lib  # noqa: E402

SEED = 20240607
N_PROMPT, N_GEN = 32, 64
PROMPT_STREAM = 7


def main():
    ref = oracle_lib.reference()
    assert ref is not None, "reference sources not found"
    cfg = binfmt.config_7m()
    H, E, k, L = cfg.hidden_dim, cfg.n_experts, cfg.experts_per_token, cfg.n_layers
    with tempfile.TemporaryDirectory() as td:
        path = Path(td) / "gpt-oss-7m-synth.bin"
        binfmt.write_synthetic(str(path), cfg, SEED)
        sha = hashlib.sha256(path.read_bytes()).hexdigest()
        prompt = synth.uniform_ids(SEED, PROMPT_STREAM, N_PROMPT, cfg.vocab_size)
        h = ref.open(path)
        ts, vs, ids, aggs, scs, gen, nxts, margins, probes = [], [], [], [], [], [], [], [], []
        logits = np.empty(cfg.vocab_size, np.float32)
        probe_idx = synth.uniform_ids(SEED, PROMPT_STREAM + 1, 64, cfg.vocab_size)
        tok = int(prompt[0])
        for pos in range(N_PROMPT + N_GEN - 1):
            nxt = ref.forward(h, tok, pos, logits)
            top2 = np.partition(logits, -2)[-2:]
            nxts.append(nxt), margins.append(float(top2[1] - top2[0])), probes.append(logits[probe_idx].copy())
            t, v, i, agg, sc = ref.last_moe_state(h, H, E, k)
            ts.append(t), vs.append(v), ids.append(i), aggs.append(agg), scs.append(sc)
            if pos + 1 < N_PROMPT:
                tok = int(prompt[pos + 1])  # prompt tokens are forced
            else:
                gen.append(nxt)
                tok = nxt
        ref.close(h)
    out = Path(__file__).with_name("moe_7m_golden.npz")
    np.savez_compressed(
        out, seed=SEED, layer=L - 1, checkpoint_sha256=np.frombuffer(bytes.fromhex(sha), np.uint8),
        prompt=prompt, generated=np.array(gen, np.int32), t=np.stack(ts), topk_v=np.stack(vs),
        topk_i=np.stack(ids), e_agg=np.stack(aggs), router_score=np.stack(scs),
        next_token=np.array(nxts, np.int32), top2_margin=np.array(margins, np.float32),
        probe_idx=probe_idx, probe_logits=np.stack(probes))
    print(f"wrote {out} ({out.stat().st_size} bytes): {len(ts)} positions, {len(gen)} generated tokens")
    print("generated:", gen[:16], "...")


if __name__ == "__main__":
    main()
