"""Generates tests/golden/moe_7m_golden.npz, tests/golden/greedy_7m_golden.npz and tests/golden/attn_hd64_golden.npz by
running the REFERENCE's own CPU model.

Needs the reference sources (directory named by the environment variable GPTOSS_REFERENCE_DIR): the
reference's run.cpp is compiled by oracle/Makefile into oracle/_ref/libref_cpu.so and its forward()
(run.cpp:501) is executed on a seeded random-init checkpoint with the gpt-oss-7m dimensions
(export_model_bin/gpt-oss-7m/config.json).  After each position the state left by the last layer's
MoE block (run.cpp:622-704) is captured: block input t, router scores, top-k ids, softmaxed gate
weights and the block output e_agg.  The greedy continuation (32 random prompt ids, 64 generated
tokens) is stored too, together with, per position, the argmax token, the gap between the two largest
logits, the gap between the 4th and 5th router score of every layer, and the logits at 64 fixed vocabulary ids
(for the whole-model parity test).  greedy_7m_golden.npz holds only the greedy continuation of a second seed (see
SEED / GREEDY_SEED below for why there are two).

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

# Seeds.  The 7m model's logits have a spread of only ~0.1 and its router scores one of ~0.1 as well, so a bf16 engine
# can legitimately differ from the fp32 reference in two discrete ways: a greedy step whose two best logits are nearly
# equal, and a token whose 4th and 5th router scores are nearly equal (another expert is chosen, which moves that
# position's logits by a few 1e-2 and stays in the KV cache).  `--scan-seeds A B` prints per seed the reference's
# smallest 4th/5th router-score gap over both layers (first 63 positions / all 95), its smallest top-2 logit gap over
# the first 32 generated tokens, and how many different tokens those are.  No seed of the ~2000 scanned is comfortable on
# every count, so two checkpoints are used:
#  * SEED (teacher-forced fixture: block state, logits and argmax per position): the widest router gap over all 95
#    positions (5.5e-4, five times the gap at which such flips were seen to start), so no expert choice can flip and the
#    logits can be compared position by position;
#  * GREEDY_SEED (free-running fixture): top-2 logit gap >= 0.0096 over the first 32 generated tokens — more than twice
#    the 4e-3 to which the logits are held — and 11 different tokens among them, so "the first 32 greedy tokens are
#    identical" is asserted without any escape clause.
SEED = 20250311
GREEDY_SEED = 20240618
N_PROMPT, N_GEN = 32, 64
PROMPT_STREAM = 7


def route_gap(scores, k):
    s = np.sort(scores)
    return float(s[-k] - s[-k - 1])


def run_reference(ref, cfg, seed, capture_state):
    """Greedy decode of the reference on the seeded checkpoint: 32 forced prompt ids, 64 generated tokens."""
    H, E, k, L = cfg.hidden_dim, cfg.n_experts, cfg.experts_per_token, cfg.n_layers
    out = {key: [] for key in ("t", "topk_v", "topk_i", "e_agg", "router_score", "gen", "next", "margin", "probe", "route_gap")}
    with tempfile.TemporaryDirectory() as td:
        path = Path(td) / "gpt-oss-7m-synth.bin"
        binfmt.write_synthetic(str(path), cfg, seed)
        out["sha"] = hashlib.sha256(path.read_bytes()).hexdigest()
        prompt = synth.uniform_ids(seed, PROMPT_STREAM, N_PROMPT, cfg.vocab_size)
        probe_idx = synth.uniform_ids(seed, PROMPT_STREAM + 1, 64, cfg.vocab_size)
        h = ref.open(path)
        logits = np.empty(cfg.vocab_size, np.float32)
        tok = int(prompt[0])
        for pos in range(N_PROMPT + N_GEN - 1):
            gaps = []
            for n_layers in range(1, L):  # the router scores of the earlier layers (the full forward leaves the last one's)
                ref.forward_prefix(h, tok, pos, n_layers)
                gaps.append(route_gap(ref.last_moe_state(h, H, E, k)[4], k))
            nxt = ref.forward(h, tok, pos, logits)
            t, v, i, agg, sc = ref.last_moe_state(h, H, E, k)
            gaps.append(route_gap(sc, k))
            top2 = np.partition(logits, -2)[-2:]
            out["next"].append(nxt), out["margin"].append(float(top2[1] - top2[0])), out["route_gap"].append(gaps)
            if capture_state:
                out["probe"].append(logits[probe_idx].copy())
                out["t"].append(t), out["topk_v"].append(v), out["topk_i"].append(i), out["e_agg"].append(agg), out["router_score"].append(sc)
            if pos + 1 < N_PROMPT:
                tok = int(prompt[pos + 1])  # prompt tokens are forced
            else:
                out["gen"].append(nxt)
                tok = nxt
        ref.close(h)
    out["prompt"], out["probe_idx"] = prompt, probe_idx
    return out


def scan_seeds(first, last):
    ref = oracle_lib.reference()
    assert ref is not None, "reference sources not found"
    cfg = binfmt.config_7m()
    for seed in range(first, last):
        r = run_reference(ref, cfg, seed, capture_state=False)
        g, m = np.array(r["route_gap"]).min(axis=1), np.array(r["margin"])
        print(f"{seed} router gap, first 63 positions {g[:63].min():.5f}, all {g.min():.5f}; top-2 logit gap over the first 32 "
              f"generated {m[N_PROMPT - 1:N_PROMPT + 31].min():.4f}; different tokens among them {len(set(r['gen'][:32]))}", flush=True)


def main():
    ref = oracle_lib.reference()
    assert ref is not None, "reference sources not found"
    cfg = binfmt.config_7m()
    r = run_reference(ref, cfg, SEED, capture_state=True)
    out = Path(__file__).with_name("moe_7m_golden.npz")
    np.savez_compressed(
        out, seed=SEED, layer=cfg.n_layers - 1, checkpoint_sha256=np.frombuffer(bytes.fromhex(r["sha"]), np.uint8),
        prompt=r["prompt"], generated=np.array(r["gen"], np.int32), t=np.stack(r["t"]), topk_v=np.stack(r["topk_v"]),
        topk_i=np.stack(r["topk_i"]), e_agg=np.stack(r["e_agg"]), router_score=np.stack(r["router_score"]),
        next_token=np.array(r["next"], np.int32), top2_margin=np.array(r["margin"], np.float32),
        route_gap=np.array(r["route_gap"], np.float32), probe_idx=r["probe_idx"], probe_logits=np.stack(r["probe"]))
    print(f"wrote {out} ({out.stat().st_size} bytes): {len(r['t'])} positions, smallest router gap {np.min(r['route_gap']):.5f}")
    g = run_reference(ref, cfg, GREEDY_SEED, capture_state=False)
    out = Path(__file__).with_name("greedy_7m_golden.npz")
    np.savez_compressed(out, seed=GREEDY_SEED, checkpoint_sha256=np.frombuffer(bytes.fromhex(g["sha"]), np.uint8),
                        prompt=g["prompt"], generated=np.array(g["gen"], np.int32),
                        top2_margin=np.array(g["margin"], np.float32), route_gap=np.array(g["route_gap"], np.float32))
    m = np.array(g["margin"])
    print(f"wrote {out} ({out.stat().st_size} bytes): generated {g['gen'][:12]} ..., smallest top-2 gap over the first 32 "
          f"generated tokens {m[N_PROMPT - 1:N_PROMPT + 31].min():.4f}")


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
