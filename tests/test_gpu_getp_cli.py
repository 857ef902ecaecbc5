"""The reference's own command line (run.cpp + tokenizer.cpp + getp_eval.cpp) linked with this repository's
getp_run.cpp: `run_b200 model.bin -z tokenizer.bin -m getp -i in.txt -o out.txt -n steps` must write the
token ids that the same model produces when driven step by step from Python with the scheduler's rules
(lock-step positions, prompt tokens force-fed, first generated token at index 0, -1 terminator)."""
import subprocess
from pathlib import Path

import numpy as np
import pytest

from gptoss_b200 import binfmt

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

EXE = Path(__file__).resolve().parent.parent / "gpt-oss-team01_b200" / "host" / "_ref_build" / "run_b200"


@pytest.mark.skipif(not EXE.exists(), reason="run_b200 not built (needs the reference sources: make -C gpt-oss-team01_b200/host)")
def test_getp_mode_writes_the_tokens_of_the_stepwise_decode(tmp_path):
    from gptoss_b200 import model
    cfg = binfmt.config_7m()
    ckpt, tok, inp, out = (tmp_path / n for n in ("m.bin", "tokenizer.bin", "in.txt", "out.txt"))
    binfmt.write_synthetic(str(ckpt), cfg, 4242)
    binfmt.write_synthetic_tokenizer(str(tok), cfg.vocab_size)
    prompts = ["hello world", "a", "The quick brown fox", "B200", "mixture of experts"]
    inp.write_text(f"{len(prompts)}\n" + "\n".join(prompts) + "\n")
    steps = 40
    r = subprocess.run([str(EXE), str(ckpt), "-z", str(tok), "-m", "getp", "-i", str(inp), "-o", str(out), "-n", str(steps)],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300,
                       env={"GPTOSS_BATCH": "4", "GPTOSS_MAX_SEQ": str(steps), "PATH": "/usr/bin:/bin"})
    assert r.returncode == 0, r.stdout[-2000:]
    assert "achieved throughput TPS" in r.stdout
    got = [[int(x) for x in line.split()] for line in out.read_text().splitlines()]
    assert len(got) == len(prompts)

    # the same schedule from Python: batches of 4 (GPTOSS_BATCH), positions 0 .. steps-2
    m = model.Model(cfg, max_batch=4, max_seq=steps)
    m.load_bin(ckpt)
    want = []
    for first in range(0, len(prompts), 4):
        batch = [list(p.encode()) for p in prompts[first:first + 4]]
        n = len(batch)
        cur = np.array([b[0] for b in batch], np.int32)
        pos_of, active, outs = [0] * n, [True] * n, [[] for _ in range(n)]
        for pos in range(steps - 1):
            if not any(active):
                break
            nxt = m.step(cur, pos)
            for i in range(n):
                if not active[i]:
                    continue
                t = int(nxt[i])
                if pos_of[i] < len(batch[i]) - 1:
                    t = batch[i][pos_of[i] + 1]
                else:
                    outs[i].append(t)
                if t in (199999, 200002):
                    active[i] = False
                cur[i] = t
                pos_of[i] += 1
        for i in range(n):
            gen_len = max(0, pos_of[i] - len(batch[i]))
            want.append(outs[i][:gen_len + 1])
    m.close()
    assert got == want


@pytest.mark.skipif(not EXE.exists(), reason="run_b200 not built (needs the reference sources: make -C gpt-oss-team01_b200/host)")
def test_getp_mode_drops_finished_sequences_without_changing_the_output(tmp_path):
    """Sequences that stop early (here: on an extra stop id that some of them generate) leave the batch; the rows
    written for every request must be the same with and without that compaction, and the early stoppers' rows end
    at the stop id."""
    cfg = binfmt.config_7m()
    ckpt, tok, inp = (tmp_path / n for n in ("m.bin", "tokenizer.bin", "in.txt"))
    binfmt.write_synthetic(str(ckpt), cfg, 4242)
    binfmt.write_synthetic_tokenizer(str(tok), cfg.vocab_size)
    prompts = ["hello world", "a", "The quick brown fox", "B200", "mixture of experts", "peer memory", "x y z", "q"]
    inp.write_text(f"{len(prompts)}\n" + "\n".join(prompts) + "\n")
    steps = 40

    def run(name, **env):
        out = tmp_path / name
        r = subprocess.run([str(EXE), str(ckpt), "-z", str(tok), "-m", "getp", "-i", str(inp), "-o", str(out), "-n", str(steps)],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300,
                           env={"GPTOSS_BATCH": "8", "GPTOSS_MAX_SEQ": str(steps), "PATH": "/usr/bin:/bin", **env})
        assert r.returncode == 0, r.stdout[-2000:]
        return [[int(x) for x in line.split()] for line in out.read_text().splitlines()]

    plain = run("plain.txt")
    # a token that some, but not all, requests generate, and not as their first token
    candidates = {}
    for row in plain:
        for j, t in enumerate(row[1:12], start=1):
            if t > 255:
                candidates.setdefault(t, set()).add(j)
    stop = next(t for t in sorted(candidates) if sum(t in row[:12] for row in plain) < len(plain))
    a = run("compact.txt", GPTOSS_STOP_IDS=str(stop), GPTOSS_NO_CONTINUOUS="1")
    b = run("nocompact.txt", GPTOSS_STOP_IDS=str(stop), GPTOSS_NO_CONTINUOUS="1", GPTOSS_NO_COMPACT="1")
    assert a == b
    assert run("continuous.txt", GPTOSS_STOP_IDS=str(stop)) == a
    lengths = {len(r) for r in a}
    assert len(lengths) > 1                                  # some stopped early, some ran on
    for row, full in zip(a, plain):
        assert row == full[:len(row)]                        # a prefix of the unstopped run ...
        if len(row) < len(full):
            assert row[-1] == stop                           # ... that ends at the stop id


@pytest.mark.skipif(not EXE.exists(), reason="run_b200 not built (needs the reference sources: make -C gpt-oss-team01_b200/host)")
def test_getp_mode_refills_free_slots_without_changing_the_output(tmp_path):
    """Continuous batching: 11 requests on 3 slots, prompts of different lengths, some requests stopping early on an
    extra stop id.  A slot that falls free is taken by the next request at once, so sequences at different positions
    share every step; each request's row must equal the one the batch-at-a-time schedule writes."""
    cfg = binfmt.config_7m()
    ckpt, tok, inp = (tmp_path / n for n in ("m.bin", "tokenizer.bin", "in.txt"))
    binfmt.write_synthetic(str(ckpt), cfg, 4242)
    binfmt.write_synthetic_tokenizer(str(tok), cfg.vocab_size)
    prompts = ["hello world", "a", "The quick brown fox jumps over the lazy dog", "B200", "mixture of experts", "peer memory",
               "x y z", "q", "tensor memory accumulators", "zz", "one more request"]
    inp.write_text(f"{len(prompts)}\n" + "\n".join(prompts) + "\n")
    steps = 48

    def run(name, **env):
        out = tmp_path / name
        r = subprocess.run([str(EXE), str(ckpt), "-z", str(tok), "-m", "getp", "-i", str(inp), "-o", str(out), "-n", str(steps)],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300,
                           env={"GPTOSS_BATCH": "3", "GPTOSS_MAX_SEQ": str(steps), "PATH": "/usr/bin:/bin", **env})
        assert r.returncode == 0, r.stdout[-2000:]
        return [[int(x) for x in line.split()] for line in out.read_text().splitlines()], r.stdout

    plain, _ = run("plain.txt", GPTOSS_NO_CONTINUOUS="1")
    counts = {}
    for row in plain:
        for t in set(row[1:20]):
            if t > 255:
                counts[t] = counts.get(t, 0) + 1
    stop = next(t for t in sorted(counts) if 1 <= counts[t] < len(plain))
    want, _ = run("batches.txt", GPTOSS_STOP_IDS=str(stop), GPTOSS_NO_CONTINUOUS="1")
    got, log_c = run("continuous.txt", GPTOSS_STOP_IDS=str(stop))
    assert got == want
    assert len({len(r) for r in got}) > 1  # some stopped early
    assert "achieved throughput TPS" in log_c


@pytest.mark.skipif(not EXE.exists(), reason="run_b200 not built (needs the reference sources: make -C gpt-oss-team01_b200/host)")
def test_getp_mode_group_of_gpus_writes_the_same_tokens(tmp_path):
    """GPTOSS_EP=1: the GPUs decode every batch together (experts sharded, sequences in slices, one host thread per
    GPU); the written ids must equal those of the single-GPU run of the same command."""
    n_gpus = torch.cuda.device_count()
    if n_gpus < 2:
        pytest.skip("needs at least two GPUs")
    world = 2 if n_gpus < 4 else 4
    cfg = binfmt.config_7m()
    ckpt, tok, inp = (tmp_path / n for n in ("m.bin", "tokenizer.bin", "in.txt"))
    binfmt.write_synthetic(str(ckpt), cfg, 4242)
    binfmt.write_synthetic_tokenizer(str(tok), cfg.vocab_size)
    prompts = ["hello world", "a", "The quick brown fox", "B200", "mixture of experts", "peer memory", "x y z"]
    inp.write_text(f"{len(prompts)}\n" + "\n".join(prompts) + "\n")
    steps = 40
    outs = []
    for env in ({"GPTOSS_GPUS": "1"}, {"GPTOSS_GPUS": str(world), "GPTOSS_EP": "1"}):
        out = tmp_path / f"out{len(outs)}.txt"
        r = subprocess.run([str(EXE), str(ckpt), "-z", str(tok), "-m", "getp", "-i", str(inp), "-o", str(out), "-n", str(steps)],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300,
                           env={"GPTOSS_BATCH": "5", "GPTOSS_MAX_SEQ": str(steps), "PATH": "/usr/bin:/bin",
                                "NCCL_NVLS_ENABLE": "0", **env})
        assert r.returncode == 0, r.stdout[-2000:]
        outs.append(out.read_text())
    assert outs[0] == outs[1] and len(outs[0].splitlines()) == len(prompts)


@pytest.mark.skipif(not EXE.exists(), reason="run_b200 not built (needs the reference sources: make -C gpt-oss-team01_b200/host)")
def test_getp_mode_replicas_draw_requests_from_one_queue(tmp_path):
    """GPTOSS_GPUS=2 without GPTOSS_EP: two data-parallel replicas (the reference's 20B mode), each refilling its
    slots from the same queue of requests; which replica serves a request must not show in its output row."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    cfg = binfmt.config_7m()
    ckpt, tok, inp = (tmp_path / n for n in ("m.bin", "tokenizer.bin", "in.txt"))
    binfmt.write_synthetic(str(ckpt), cfg, 4242)
    binfmt.write_synthetic_tokenizer(str(tok), cfg.vocab_size)
    prompts = [f"request number {i} " + "x" * (i % 5) for i in range(13)]
    inp.write_text(f"{len(prompts)}\n" + "\n".join(prompts) + "\n")
    steps = 36
    outs = []
    for env in ({"GPTOSS_GPUS": "1"}, {"GPTOSS_GPUS": "2"}, {"GPTOSS_GPUS": "2", "GPTOSS_NO_CONTINUOUS": "1"}):
        out = tmp_path / f"out{len(outs)}.txt"
        r = subprocess.run([str(EXE), str(ckpt), "-z", str(tok), "-m", "getp", "-i", str(inp), "-o", str(out), "-n", str(steps)],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300,
                           env={"GPTOSS_BATCH": "3", "GPTOSS_MAX_SEQ": str(steps), "PATH": "/usr/bin:/bin", **env})
        assert r.returncode == 0, r.stdout[-2000:]
        outs.append(out.read_text())
    assert outs[0] == outs[1] == outs[2] and len(outs[0].splitlines()) == len(prompts)
