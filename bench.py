#!/usr/bin/env python
"""Benchmark of the MoE FFN block (one gpt-oss-20b layer call per step).

    python bench.py --gpus N --steps K --warmup W                  our arm (CUDA, through the C ABI)
    python bench.py --impl reference --gpus N --steps K --warmup W the reference's CPU path on the host

A step is one pass of the block over one batch of synthetic tokens.  N = 1: hidden 2880, 32 experts,
top-4, T = 1024 tokens (the single-GPU configuration the headline metric is quoted on).  N > 1 (one
process per GPU under torchrun): the same layer with its experts sharded E/N per GPU and T = 1024*N
replicated tokens; the gate-weighted expert rows are pushed to the GPU that owns the token by peer stores
from the down-GEMM epilogue, summed there and delivered to every rank (an NCCL all-reduce of per-rank
partials is timed beside it as the baseline) — per-GPU work is fixed, so the scaling is weak.  Weights rotate over several distinct layers (each 1.6 GB >> the 126 MB L2), so
every step streams its weights from HBM.

Prints ONE JSON line (rank 0).  `value` is timed with inputs resident in HBM; `e2e` goes through the
host-buffer entry point with pinned host memory (H2D + block + D2H inside the timed region).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

entry.load_package()
from gptoss_b200 import synth  # noqa: E402

H = I = 2880
E, K_TOP = 32, 4
TOKENS_PER_GPU = 1024
SEED = 2024
SIGMA = 0.02
N_WEIGHT_SETS = 4  # distinct layers the steps rotate over
FLOP_PER_TOKEN = 2 * H * E + 2 * K_TOP * H * (2 * I) + 2 * K_TOP * I * H  # 199,249,920

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the gate/up GEMM kernel at this workload,
# from the ncu capture summarised in profiles/ (None until captured).
NCU_TRAFFIC_MLP1_BYTES = 1_105_950_368  # dram read 1,102,148,000 + write 3,802,368 per launch (ncu capture of this workload, summarised under profiles/)


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"], d["bf16_tflops"], d.get("bf16_tflops_sustained", d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs.  nvidia-smi needs up to a
    second before its first line on a box with many GPUs, so the sampler may be started ahead of the region
    (``start()``, e.g. before the warm-up steps); only the lines read between ``with`` entry and exit count (the last
    one before and the first one after stand in when the region was shorter than one sampling period)."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, enabled: bool = True):
        self.index, self.all_rows, self.rows, self.proc = index, [], [], None
        self.t_in = self.t_out = None
        self.enabled = enabled  # only the rank that prints the line samples

    def start(self):
        if self.proc is None and self.enabled:
            try:
                self.proc = subprocess.Popen(
                    ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                     "--format=csv,noheader,nounits", "-lms", "20"],
                    stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
                self.thread = threading.Thread(target=self._read, daemon=True)
                self.thread.start()
            except OSError:
                self.proc = None
        return self

    def __enter__(self):
        self.start()
        self.t_in = time.monotonic()
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.all_rows.append((time.monotonic(), [c.strip() for c in line.split(",")]))

    def __exit__(self, *a):
        self.t_out = time.monotonic()
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)
        inside = [r for t, r in self.all_rows if self.t_in <= t <= self.t_out]
        before = [r for t, r in self.all_rows if t < self.t_in][-1:]
        after = [r for t, r in self.all_rows if t > self.t_out][:1]
        self.rows = inside if inside else before + after  # idle samples around the region only if it held none

    def summary(self):
        sm = [int(r[0]) for r in self.rows if len(r) >= 6 and r[0].isdigit()]
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows if len(r) >= 6)]
        mx = [int(r[1]) for r in self.rows if len(r) >= 6 and r[1].isdigit()]
        return {"sm_mhz": int(statistics.median(sm)), "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def to_bf16_bits(x):
    return synth.f32_to_bf16_bits(x).reshape(x.shape)


# ----------------------------------------------------------------------------------------------------------
# reference / CPU arm
# ----------------------------------------------------------------------------------------------------------
def host_weights():
    sys.path.insert(0, str(ROOT / "tests"))
    import oracle_lib
    return oracle_lib, oracle_lib.oracle().layer_weights(H, I, E, SEED, layer=0, sigma=SIGMA)


def cpu_arm(T, target_seconds, repeats, warmup):
    """Times the reference's CPU implementation of the block (its own matmul/topk/softmax from run.cpp,
    compiled into oracle/_ref) on a bounded sample of the workload's token rows; falls back to the C
    port when the reference object is absent.  Returns (tok/s, info, per-repeat seconds)."""
    oracle_lib, w = host_weights()
    t = synth.activations(SEED, T, H)
    ref = oracle_lib.reference()
    if ref is not None:
        kind, cores = "reference", ref.num_threads()
        run = lambda n: ref.moe_rows(t, w, K_TOP, rows=(0, n))  # noqa: E731
    else:
        ora = oracle_lib.oracle()
        kind, cores = "port", ora.num_threads()

        def run(n):
            sc = ora.router_scores(t[:n], w.router_w, w.router_b)
            tw, ti, _, _ = ora.topk_softmax(sc, K_TOP, oracle_lib.RULE_QSORT)
            ora.moe_block(np.ascontiguousarray(t[:n]), tw, ti, w, mode=oracle_lib.MODE_CPU)
    run(8)  # first touch of the weights (page faults) is not representative
    t0 = time.perf_counter()
    run(8)
    per_row = (time.perf_counter() - t0) / 8
    rows = int(max(8, min(T, target_seconds / max(per_row, 1e-9))))
    for _ in range(warmup):
        run(min(rows, 16))
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        run(rows)
        times.append(time.perf_counter() - t0)
    tok_s = rows * len(times) / sum(times)
    info = {"value": tok_s, "unit": "tok/s", "cores": cores, "kind": kind,
            "sample": f"first {rows} of {T} token rows of the same seeded layer-0 workload, "
                      f"{len(times)} timed pass(es)"}
    return tok_s, info, times


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun pins OMP_NUM_THREADS to 1; the reference arm uses every host core (set before libgomp loads)
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    T = (args.tokens_per_gpu or TOKENS_PER_GPU) * args.gpus
    tok_s, info, times = cpu_arm(T, target_seconds=6.0, repeats=max(1, args.steps), warmup=min(args.warmup, 1))
    line = {
        "impl": "reference", "metric": "batched decode tok/s, gpt-oss-20b MoE FFN block (one layer call per step)",
        "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * sum(times) / len(times), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 (double accumulate)", "data": "synthetic",
        "config": workload_config(args.gpus, T), "cpu_baseline": info,
        "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print_line(line)


def workload_config(n_gpus, T):
    return {"workload": f"gpt-oss-20b MoE layer: T={T} tokens N(0,1) bf16, hidden {H}, {E} experts "
                        f"(gate_up {2 * I}x{H}, down {H}x{I}) N(0,0.02) bf16, top-{K_TOP} softmax, SwiGLU alpha 1.702 "
                        f"clamp 7.0; experts sharded {E // n_gpus} per GPU" if n_gpus > 1 else
                        f"gpt-oss-20b MoE layer: T={T} tokens N(0,1) bf16, hidden {H}, {E} experts "
                        f"(gate_up {2 * I}x{H}, down {H}x{I}) N(0,0.02) bf16, top-{K_TOP} softmax, SwiGLU alpha 1.702 "
                        f"clamp 7.0",
            "tokens_per_step": T, "parallelism": f"ep{n_gpus}" if n_gpus > 1 else "single",
            "l2": f"weights rotate over {N_WEIGHT_SETS} layers of 1.59 GB each (inputs larger than the 126 MB L2)",
            "seed": SEED}


# ----------------------------------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist
    from gptoss_b200 import moe

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun for N > 1")
    torch.cuda.set_device(local_rank)
    clocks = ClockSampler(local_rank, enabled=rank == 0).start()  # nvidia-smi needs a second or more before its first line on an 8-GPU box
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    T = (args.tokens_per_gpu or TOKENS_PER_GPU) * world
    K, W = args.steps, max(args.warmup, 3)

    global N_WEIGHT_SETS
    N_WEIGHT_SETS = args.weight_sets
    blk = moe.MoEBlock(hidden=H, intermediate=I, n_experts=E, top_k=K_TOP, n_layers=N_WEIGHT_SETS,
                       device=local_rank, rank=rank, world=world, max_tokens=T,
                       wire={"f32": 0, "bf16": 1}[args.wire])
    for layer in range(N_WEIGHT_SETS):
        blk.fill_layer_synthetic(layer, SEED, SIGMA)
        if args.zipf > 0:  # skewed routing (BASELINE config 3): router_bias[e] += -s * ln(e + 1), hottest expert first
            blk.set_router_bias(layer, synth.zipf_router_bias(SEED, layer, E, args.zipf))
    t_dev = moe.synth_normal_bf16(T * H, SEED, synth.tensor_id(synth.TID_ACTIVATION), 1.0).view(T, H)
    x = torch.zeros((T, H), dtype=torch.float32, device="cuda")
    partial = torch.empty_like(x) if world > 1 else None

    if world > 1:
        blk.attach_peers()  # CUDA IPC handles of the combine buffers, exchanged over the process group

    def step(i):  # x += MoE(t); N > 1: fused peer-store combine inside forward()
        blk.forward(i % N_WEIGHT_SETS, t_dev, x)

    def step_nccl(i):  # A/B baseline for N > 1: per-rank partial + NCCL all-reduce + add
        blk.forward_partial(i % N_WEIGHT_SETS, t_dev, partial)
        dist.all_reduce(partial)
        x.add_(partial)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(W):
        step(i)
    barrier()
    blk.status()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with clocks:
        barrier()
        ev0.record()
        for i in range(K):
            step(i)
        ev1.record()
        barrier()
    blk.status()
    ms = ev0.elapsed_time(ev1)
    if world > 1:
        tms = torch.tensor([ms], device="cuda")
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = float(tms.item())
    value = T * K / (ms * 1e-3)

    nccl_ms = stub_ms = stub_free_ms = None
    if world > 1:
        # The same kernels with the exchange stubbed: every rank computes the partial of its own experts (no push,
        # no delivery, no add).  Timed twice: with a device-side rendezvous of the ranks after every step (what the
        # expert-parallel step costs without moving any data: the ranks still wait for the most loaded one every
        # step) and free-running (each rank at its own pace; the gap between the two is load imbalance, not exchange).
        def timed_stub(sync):
            for i in range(3):
                blk.forward_partial(i % N_WEIGHT_SETS, t_dev, partial)
                if sync:
                    blk.rendezvous()
            barrier()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for i in range(K):
                blk.forward_partial(i % N_WEIGHT_SETS, t_dev, partial)
                if sync:
                    blk.rendezvous()
            s1.record()
            barrier()
            ts = torch.tensor([s0.elapsed_time(s1)], device="cuda")
            dist.all_reduce(ts, op=dist.ReduceOp.MAX)
            return float(ts.item()) / K
        stub_ms = timed_stub(True)
        stub_free_ms = timed_stub(False)
        blk.status()
    if world > 1:  # the NCCL baseline on the same steps
        for i in range(3):
            step_nccl(i)
        barrier()
        n0, n1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n0.record()
        for i in range(K):
            step_nccl(i)
        n1.record()
        barrier()
        tn = torch.tensor([n0.elapsed_time(n1)], device="cuda")
        dist.all_reduce(tn, op=dist.ReduceOp.MAX)
        nccl_ms = float(tn.item()) / K

    # per-stage device time (same steps, events between the stages), for the roofline of the top kernel
    if world == 1:
        names = ["route", "mlp1_swiglu", "mlp2", "combine"]
    else:
        names = ["route", "mlp1_swiglu", "mlp2_push", "owner_combine", "add_delta"]
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)] for _ in range(K)]
    barrier()
    for i in range(K):
        layer = i % N_WEIGHT_SETS
        evs[i][0].record()
        blk.route(layer, t_dev)
        evs[i][1].record()
        blk.mlp1_swiglu(layer)
        evs[i][2].record()
        if world == 1:
            blk.mlp2(layer)
            evs[i][3].record()
            blk.combine(x, residual=True)
            evs[i][4].record()
        else:
            blk.push_to_owners(layer)
            evs[i][3].record()
            blk.owner_combine()
            evs[i][4].record()
            blk.add_delta(x)
            evs[i][5].record()
    barrier()
    blk.status()
    stage_ms = {n: sum(evs[i][j].elapsed_time(evs[i][j + 1]) for i in range(K)) / K for j, n in enumerate(names)}

    hbm_peak, tf_burst, tf_sust, peak_kind = measured_peaks()
    n_local = E // world
    # rows of this rank's experts in the routing of the last step (T*k/world under uniform routing); the rank with the
    # most rows decides an expert-parallel step
    off = blk.tap("offsets", T)
    rows_here = int(off[(rank + 1) * n_local] - off[rank * n_local])
    rows_max = rows_here
    if world > 1:
        rm = torch.tensor([rows_here], device="cuda")
        dist.all_reduce(rm, op=dist.ReduceOp.MAX)
        rows_max = int(rm.item())
    pairs_local = rows_here
    mlp1_bytes = n_local * (2 * I * H * 2 + 2 * I * 4) + pairs_local * H * 2 + pairs_local * I * 2
    mlp1_flops = 2 * pairs_local * H * 2 * I
    mlp1_s = stage_ms["mlp1_swiglu"] * 1e-3
    hbm_t, tc_t = mlp1_bytes / (hbm_peak * 1e9), mlp1_flops / (tf_burst * 1e12)
    if hbm_t >= tc_t:
        roof = {"bound": "hbm", "achieved": mlp1_bytes / mlp1_s / 1e9, "peak": hbm_peak, "unit": "GB/s"}
    else:
        roof = {"bound": "tensor", "achieved": mlp1_flops / mlp1_s / 1e12, "peak": tf_burst, "unit": "TFLOP/s"}
    roof["frac"] = roof["achieved"] / roof["peak"]
    roof["traffic"] = NCU_TRAFFIC_MLP1_BYTES if world == 1 else None  # captured at the N=1 workload only
    roof.update({"kernel": "grouped_gemm_kernel<2,true> (gate/up GEMM + SwiGLU)", "peak_source": f"{peak_kind} (MEASURED_PEAKS.json)",
                 "algorithmic_bytes_per_launch": mlp1_bytes, "algorithmic_flops_per_launch": mlp1_flops,
                 "avg_launch_ms": stage_ms["mlp1_swiglu"], "tensor_frac_of_burst": mlp1_flops / mlp1_s / 1e12 / tf_burst})
    block_bytes = n_local * 3 * H * I * 2 + n_local * (2 * I + H) * 2 + (H * E + E) * 2 + T * H * 2 + T * H * 8
    block_flops = FLOP_PER_TOKEN * T / world
    block_roof_s = max(block_bytes / (hbm_peak * 1e9), block_flops / (tf_sust * 1e12))
    busiest_flops = 2.0 * rows_max * 3 * H * I + 2.0 * T * H * E
    busiest_roof_s = max(block_bytes / (hbm_peak * 1e9), busiest_flops / (tf_sust * 1e12))

    line = {
        "metric": "batched decode tok/s, gpt-oss-20b MoE FFN block (one layer call per step)",
        "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 (fp32 accumulate)",
        "data": "synthetic", "config": dict(workload_config(world, T), **({"router_skew": f"Zipf s={args.zipf} over expert id "
                                                                              "(router_bias[e] -= s*ln(e+1))"} if args.zipf > 0 else {})),
        "roofline": roof,
        "block_roofline": {"algorithmic_bytes": block_bytes, "algorithmic_flops": block_flops,
                           "roof_ms": block_roof_s * 1e3, "frac": block_roof_s * 1e3 / (ms / K),
                           "busiest_rank_rows": rows_max, "rows_per_rank_if_even": T * K_TOP // world,
                           "roof_ms_busiest_rank": busiest_roof_s * 1e3, "frac_busiest_rank": busiest_roof_s * 1e3 / (ms / K),
                           "bound": "hbm" if block_bytes / (hbm_peak * 1e9) >= block_flops / (tf_sust * 1e12) else "tensor"},
        "stage_ms": stage_ms, "gpu_launches": (7 if world == 1 else 8) * K,  # router GEMM, top-k, scan, scatter, 2 GEMMs, combine (N > 1: owner combine + add instead)
    }
    if world > 1:
        comm_ms = ms / K - stub_ms  # exposed exchange = step with the fused combine - step with the exchange stubbed
        line["combine"] = {"kind": "peer stores (fp32) from the down-GEMM epilogue to the token owner + owner sum in slot "
                                   f"order + peer delivery of the sums ({args.wire})",
                           "exposed_ms": comm_ms, "share_of_step": comm_ms / (ms / K),
                           "stubbed_exchange_ms_per_step": stub_ms,
                           "stubbed_exchange_without_rendezvous_ms_per_step": stub_free_ms,
                           "nccl_allreduce_baseline_ms_per_step": nccl_ms}

    if rank == 0:
        cs = clocks.summary()
        line["clocks"] = cs

    # end to end through the host-buffer entry point (single GPU: the C ABI call a host program makes)
    if args.no_e2e:
        pass
    elif world == 1:
        t_host = torch.empty((T, H), dtype=torch.int16).pin_memory()
        t_host.copy_(t_dev.view(torch.int16).cpu())
        x_host = torch.zeros((T, H), dtype=torch.float32).pin_memory()
        for i in range(3):
            blk.forward_host(i % N_WEIGHT_SETS, t_host, x_host)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(K):
            blk.forward_host(i % N_WEIGHT_SETS, t_host, x_host)
        e2e_s = time.perf_counter() - t0
        line["e2e"] = {"value": T * K / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": T * H * 2 + T * H * 4,
                       "d2h_bytes_per_step": T * H * 4, "ms_per_step": 1e3 * e2e_s / K}
    else:
        # The host holds the batch once; every rank moves ITS slice of the tokens over PCIe (t and x in, x out) and the
        # ranks exchange activations and expert rows over NVLink (token-sliced form of the block): per step the
        # batch crosses the host link once in total, not once per GPU.
        first, n_own = blk.slice(T)
        t_host = torch.empty((n_own, H), dtype=torch.int16).pin_memory()
        t_host.copy_(t_dev.view(torch.int16)[first:first + n_own].cpu())
        x_host = torch.zeros((n_own, H), dtype=torch.float32).pin_memory()
        for i in range(3):
            blk.forward_host_sliced(i % N_WEIGHT_SETS, T, t_host, x_host)
        barrier()
        t0 = time.perf_counter()
        for i in range(K):
            blk.forward_host_sliced(i % N_WEIGHT_SETS, T, t_host, x_host)
        barrier()
        e2e_s = torch.tensor([time.perf_counter() - t0], device="cuda")
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
        line["e2e"] = {"value": T * K / float(e2e_s.item()), "unit": "tok/s",
                       "h2d_bytes_per_step": T * H * 2 + T * H * 4, "d2h_bytes_per_step": T * H * 4,
                       "ms_per_step": 1e3 * float(e2e_s.item()) / K,
                       "note": "bytes over all GPUs; each GPU copies its own token slice (1/N of them)"}

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        _, info, _ = cpu_arm(T, target_seconds=12.0, repeats=1, warmup=0)
        line["cpu_baseline"] = info
    blk.close()
    if rank == 0:
        print_line(line)
    if world > 1:
        dist.destroy_process_group()


def run_decode(args):
    """Whole-model batched greedy decode (random-init weights generated on the device), sequences of random prompt
    ids force-fed one position per step, then greedy tokens.  decode20b: gpt-oss-20b architecture, 1024 x 128 prompt
    ids, 256 generated (BASELINE config 4); decode120b: gpt-oss-120b architecture, 2048 x 256, 256 generated
    (config 5; needs the experts spread over >= 4 GPUs).  With N > 1 (one process per GPU) the N GPUs decode the
    batch together: sequences in slices, experts sharded, per-layer exchange over peer memory.  Reported like the
    reference's getp mode: generated tokens / wall time of the whole inference loop (getp-csrc/getp_eval.cpp:125-131),
    the slowest rank's time."""
    import torch
    from gptoss_b200 import binfmt, model
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    big = args.workload == "decode120b"
    B = args.decode_batch or (2048 if big else 1024)
    n_prompt = args.decode_prompt or (256 if big else 128)
    n_gen = args.decode_gen or 256
    cfg = binfmt.config_120b(seq_len=1024) if big else binfmt.config_20b(seq_len=1024)
    if args.decode_layers:
        cfg.n_layers = args.decode_layers
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    m = model.Model(cfg, device=local_rank, max_batch=B, max_seq=args.decode_first_pos + n_prompt + n_gen, rank=rank, world=world)
    m.fill_synthetic(SEED, SIGMA)
    if world > 1:
        m.attach_peers()
    first, n = m.slice(B)
    prompts = synth.uniform_ids(SEED, 11, B * n_prompt, cfg.vocab_size).reshape(B, n_prompt)[first:first + n]
    m.generate(prompts[:, :2], 2, batch=B)  # warm-up: 3 steps
    if world > 1:
        dist.barrier()
    with ClockSampler(local_rank) as clocks:
        t0 = time.perf_counter()
        out = m.generate(prompts, n_gen, batch=B, first_pos=args.decode_first_pos)
        dt = time.perf_counter() - t0
    n_distinct = int(len(np.unique(out)))
    if world > 1:
        tt = torch.tensor([dt], device="cuda", dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dt = float(tt.item())
        dist.barrier()
    steps = n_prompt + n_gen - 1
    arch = "gpt-oss-120b" if big else "gpt-oss-20b"
    line = {"metric": f"batched decode tok/s, {arch} arch (whole model, greedy, lock-step)", "value": B * n_gen / dt,
            "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": 3, "ms_per_step": 1e3 * dt / steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 (fp32 accumulate)",
            "data": "synthetic",
            "config": {"workload": f"{arch} architecture, {cfg.n_layers} layers, batch {B} x {n_prompt} random prompt "
                                   f"ids, greedy decode {n_gen} tokens; tokens in/out over host memory every step",
                       "parallelism": "one GPU" if world == 1 else
                       f"{world} GPUs: sequences in {world} slices (data-parallel attention), {cfg.n_experts // world} "
                       "experts per GPU, activations and expert rows exchanged over NVLink peer memory",
                       "positions_per_second": B * steps / dt, "seed": SEED},
            "clocks": clocks.summary(), "distinct_tokens_generated_rank0": n_distinct}
    m.close()
    if rank == 0:
        print_line(line)
    if world > 1:
        dist.destroy_process_group()


def main():
    # libraries (NCCL's version banner) may write to stdout; keep fd 1 for the ONE JSON line
    real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    global print_line
    def print_line(obj):
        real_stdout.write(json.dumps(obj) + "\n")
        real_stdout.flush()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    ap.add_argument("--wire", choices=["f32", "bf16"], default="bf16",
                    help="N > 1: format in which owners deliver the summed rows (rows travel to the owner in fp32)")
    ap.add_argument("--workload", choices=["moe_layer", "decode20b", "decode120b"], default="moe_layer",
                    help="moe_layer: the MoE block (headline); decode20b: whole-model greedy decode on one GPU")
    ap.add_argument("--decode-batch", type=int, default=0, help="0 = the config's batch (1024 / 2048)")
    ap.add_argument("--decode-prompt", type=int, default=0, help="0 = the config's prompt length (128 / 256)")
    ap.add_argument("--decode-gen", type=int, default=0, help="0 = 256")
    ap.add_argument("--decode-layers", type=int, default=0, help="override the layer count (0 = 24)")
    ap.add_argument("--decode-first-pos", type=int, default=0,
                    help="profiling runs: start the timed decode at this position (cache rows before it are zeros)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--tokens-per-gpu", type=int, default=0,
                    help="tokens per step and GPU (0 = 1024, the headline workload; 8192 on one GPU = BASELINE config 3's "
                         "shape, where the block is tensor-bound)")
    ap.add_argument("--zipf", type=float, default=0.0,
                    help="skew the routing: router_bias[e] -= s*ln(e+1) (1.2 = BASELINE config 3); 0 = uniform")
    ap.add_argument("--weight-sets", type=int, default=N_WEIGHT_SETS,
                    help="distinct layers of weights the steps rotate over (1 keeps a profiling run small)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload in ("decode20b", "decode120b"):
        run_decode(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
