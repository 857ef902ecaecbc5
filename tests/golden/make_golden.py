"""Generates tests/golden/moe_7m_golden.npz and tests/golden/attn_hd64_golden.npz by running the REFERENCE's own
CPU model.

Needs the reference sources (directory named by the environment variable GPTOSS_REFERENCE_DIR): the
reference's run.cpp is compiled by oracle/Makefile into oracle/_ref/libref_cpu.so and its forward()
(run.cpp:501) is executed on a seeded random-init checkpoint with the gpt-oss-7m dimensions
(export_model_bin/gpt-oss-7m/config.json).  After each position the state left by the last layer's
MoE block (run.cpp:622-704) is captured: block input t, router scores, top-k ids, softmaxed gate
weights and the block output e_agg.  The greedy continuation (32 random prompt ids, 64 generated
tokens) is stored too, together with, per position, the argmax token, the gap between the two largest
logits and the logits at 64 fixed vocabulary ids (for the whole-model parity test).

The second fixture covers the attention geometry of the 20b/120b checkpoints that the 7m one lacks (head_dim 64,
8 query heads per kv head) on a small two-layer model, over 200 teacher-forced positions with a sliding window
of 48: the windowed layer (layer 0, run.cpp:582) drops old positions, the other attends to all of them.  It
stores, per position, the argmax, the top-2 gap and the logits at 64 fixed ids.

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

# Seed of the checkpoint and the prompt.  The 7m model's logits have a spread of only ~0.1, so for most seeds some of
# the greedy steps are near-ties that a bf16 engine may legitimately resolve the other way, and many continuations
# collapse to one repeated token.  `--scan-seeds A B` prints, per seed, the smallest top-2 logit gap of the reference
# over the first 32 generated tokens and how many different tokens those are; this seed is the one of
# 20240607..20241008 with the widest such gap (0.0096: more than twice the 4e-3 to which the parity test holds every
# logit, and ten times the bf16-vs-fp32 noise actually seen) among the seeds whose first 32 tokens take more than 8
# different values, so "the first 32 greedy tokens are identical" can be asserted without any escape clause.
SEED = 20240618
N_PROMPT, N_GEN = 32, 64
PROMPT_STREAM = 7


def scan_seeds(first, last):
    """Prints the reference's smallest top-2 logit gap over the first 32 generated tokens for each seed."""
    ref = oracle_lib.reference()
    assert ref is not None, "reference sources not found"
    cfg = binfmt.config_7m()
    logits = np.empty(cfg.vocab_size, np.float32)
    for seed in range(first, last):
        with tempfile.TemporaryDirectory() as td:
            path = Path(td) / "m.bin"
            binfmt.write_synthetic(str(path), cfg, seed)
            prompt = synth.uniform_ids(seed, PROMPT_STREAM, N_PROMPT, cfg.vocab_size)
            h = ref.open(path)
            tok, margins, gen = int(prompt[0]), [], []
            for pos in range(N_PROMPT + N_GEN - 1):
                nxt = ref.forward(h, tok, pos, logits)
                top2 = np.partition(logits, -2)[-2:]
                margins.append(float(top2[1] - top2[0]))
                if pos + 1 < N_PROMPT:
                    tok = int(prompt[pos + 1])
                else:
                    gen.append(nxt)
                    tok = nxt
            ref.close(h)
        m = np.array(margins)
        print(f"{seed} min top-2 gap, first 32 generated {m[N_PROMPT - 1:N_PROMPT + 31].min():.4f}, all {m[N_PROMPT - 1:].min():.4f}, "
              f"distinct tokens in the first 32: {len(set(gen[:32]))}", flush=True)


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


ATTN_SEED = 20240611


def attn_config():
    """head_dim 64, 16 query heads over 2 kv heads, window 48; the other dims small so that the fixture stays cheap.
    Four experts, all four selected: the expert choice cannot flip between the fp32 reference and a path that
    rounds GEMM inputs to bf16 (a flip at one position would stay in the KV cache for the rest of the sequence),
    so the comparison stays at rounding-noise level over all positions."""
    return binfmt.Config(1024, 128, 4, 4, 128, 2, 64, 16, 2, 256, 4096, 150000.0, 32.0, 48, 7.0)


def make_attention_fixture(n_pos=200):
    ref = oracle_lib.reference()
    cfg = attn_config()
    with tempfile.TemporaryDirectory() as td:
        path = Path(td) / "attn-hd64-synth.bin"
        binfmt.write_synthetic(str(path), cfg, ATTN_SEED, sigma=0.05)
        ids = synth.uniform_ids(ATTN_SEED, PROMPT_STREAM, n_pos, cfg.vocab_size)
        probe_idx = synth.uniform_ids(ATTN_SEED, PROMPT_STREAM + 1, 64, cfg.vocab_size)
        logits = np.empty(cfg.vocab_size, np.float32)
        h = ref.open(path)
        nxts, margins, probes, stds = [], [], [], []
        for pos in range(n_pos):
            nxt = ref.forward(h, int(ids[pos]), pos, logits)
            top2 = np.partition(logits, -2)[-2:]
            nxts.append(nxt), margins.append(float(top2[1] - top2[0])), probes.append(logits[probe_idx].copy())
            stds.append(float(logits.std()))
        ref.close(h)
    out = Path(__file__).with_name("attn_hd64_golden.npz")
    np.savez_compressed(out, seed=ATTN_SEED, sigma=0.05, ids=ids, next_token=np.array(nxts, np.int32),
                        top2_margin=np.array(margins, np.float32), probe_idx=probe_idx,
                        probe_logits=np.stack(probes), logit_std=np.array(stds, np.float32))
    print(f"wrote {out} ({out.stat().st_size} bytes): {n_pos} positions, logit std {np.mean(stds):.4f}, "
          f"median top-2 gap {np.median(margins):.4f}")


if __name__ == "__main__":
    if "--scan-seeds" in sys.argv:
        i = sys.argv.index("--scan-seeds")
        scan_seeds(int(sys.argv[i + 1]), int(sys.argv[i + 2]))
        sys.exit(0)
    if "--attention-only" not in sys.argv:
        main()
    make_attention_fixture()
