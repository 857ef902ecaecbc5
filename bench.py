#!/usr/bin/env python
"""Benchmark of the MoE FFN block (one gpt-oss-20b layer call per step).

    python bench.py --gpus N --steps K --warmup W                  our arm (CUDA, through the C ABI)
    python bench.py --impl reference --gpus N --steps K --warmup W the reference's CPU path on the host

A step is one pass of the block over one batch of synthetic tokens.  N = 1: hidden 2880, 32 experts,
top-4, T = 1024 tokens (the single-GPU configuration the headline metric is quoted on).  N > 1 (one
process per GPU under torchrun): the same layer with its experts sharded E/N per GPU and T = 1024*N tokens,
uniform routing; per-GPU work is fixed, so the scaling is weak.  `value` times the token-sliced form: every GPU holds
1/N of the tokens (activations and residual rows), routes them, dispatches each token row to the GPUs whose experts
it selected (peer stores from the grouping kernel), and the gate-weighted expert rows are pushed back to the token's
GPU from the down-GEMM epilogue and summed there.  The replicated form (tokens and residual on every GPU, sums
delivered to all), an NCCL all-reduce of per-rank partials, and the same GEMMs with the exchange stubbed are timed
beside it, and one step of each form is checked against the NCCL result.  Weights rotate over several distinct layers
(each 1.6 GB >> the 126 MB L2), so every step streams its weights from HBM.  The timed region of K steps is repeated
until half a second of device time has been measured; `value` is the median region.

Extra keys of the same line: `skewed_T8192` (T = 8192 tokens in total, Zipf s = 1.2 routing, experts sharded E/N) and
`decode` (whole-model greedy decode of the gpt-oss-20b architecture at N GPUs, gpt-oss-120b at N >= 4).

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
NCU_TRAFFIC_MLP1_BYTES = 1_106_306_536  # dram read 1,101,761,000 + write 4,545,536 per launch (ncu capture of this workload, summarised under profiles/)


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
def timed_regions(step, K, barrier, world, dist, torch, min_seconds=0.5, max_regions=400):
    """Times regions of exactly K steps (CUDA events on the launching stream, barrier + synchronize on both sides, the
    slowest rank's time per region) until at least min_seconds of device time has been measured; returns the per-region
    milliseconds.  The number of regions follows from the first one, so every rank runs the same number."""
    def one():
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for i in range(K):
            step(i)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms
    regions = [one()]
    n = int(min(max_regions, max(1, -(-min_seconds * 1e3 // max(regions[0], 1e-3)))))
    for _ in range(n - 1):
        regions.append(one())
    return regions


def rel_l2_t(a, b):
    return float(((a - b).double().norm() / b.double().norm().clamp_min(1e-30)).item())


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
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    T = (args.tokens_per_gpu or TOKENS_PER_GPU) * world
    K, W = args.steps, args.warmup
    if W < 3:
        print(f"bench.py: --warmup {W} raised to 3 (fewer warm-up steps give a cold-start number)", file=sys.stderr)
        W = 3
    T_SKEW = 8192  # tokens of the skewed-routing workload (total, over all GPUs)
    skew_layer = args.weight_sets  # an extra layer slot whose router bias carries the Zipf skew

    global N_WEIGHT_SETS
    N_WEIGHT_SETS = args.weight_sets
    wire = {"f32": 0, "bf16": 1}[args.wire]
    blk = moe.MoEBlock(hidden=H, intermediate=I, n_experts=E, top_k=K_TOP, n_layers=N_WEIGHT_SETS + (0 if args.no_extras else 1),
                       device=local_rank, rank=rank, world=world, max_tokens=max(T, 0 if args.no_extras else T_SKEW), wire=wire)
    for layer in range(N_WEIGHT_SETS):
        blk.fill_layer_synthetic(layer, SEED, SIGMA)
        if args.zipf > 0:  # skewed routing: router_bias[e] += -s * ln(e + 1), hottest expert first
            blk.set_router_bias(layer, synth.zipf_router_bias(SEED, layer, E, args.zipf))
    t_dev = moe.synth_normal_bf16(T * H, SEED, synth.tensor_id(synth.TID_ACTIVATION), 1.0).view(T, H)
    x = torch.zeros((T, H), dtype=torch.float32, device="cuda")
    partial = torch.empty_like(x) if world > 1 else None
    first, n_own = blk.slice(T)
    t_own = t_dev[first:first + n_own].contiguous() if world > 1 else None
    x_own = torch.zeros((n_own, H), dtype=torch.float32, device="cuda") if world > 1 else None

    if world > 1:
        blk.attach_peers()  # CUDA IPC handles of the exchange buffers, handed round over the process group

    def step_replicated(i):  # x += MoE(t) on replicated t and x; N > 1: fused peer-store combine inside forward()
        blk.forward(i % N_WEIGHT_SETS, t_dev, x)

    def step_dispatch(i):  # N > 1, token-sliced: every rank holds its rows of t and x only
        blk.forward_dispatch(i % N_WEIGHT_SETS, T, t_own, x_own)

    step = step_replicated if world == 1 or args.form == "replicated" else step_dispatch

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
    with clocks:
        l0 = moe.launch_count()
        regions = timed_regions(step, K, barrier, world, dist, torch)
        launches = (moe.launch_count() - l0) // len(regions)
    blk.status()
    ms = statistics.median(regions)
    value = T * K / (ms * 1e-3)

    def timed_once(fn, sync_each=None):
        """ms per step of another arm, timed like `value`: the median of K-step regions over 0.3 s, so that it runs
        under the same clocks (a single short region would run at burst clocks where `value` is power-capped)."""
        def one(i):
            fn(i)
            if sync_each:
                sync_each()
        for i in range(3):
            one(i)
        return statistics.median(timed_regions(one, K, barrier, world, dist, torch, min_seconds=0.3)) / K

    nccl_ms = stub_ms = stub_free_ms = other_form_ms = None
    parity = None
    if world > 1:
        # The same expert GEMMs with the exchange stubbed: every rank computes the partial of its own experts (no
        # dispatch, no push, no add).  Timed twice: with a device-side rendezvous of the ranks after every step (what
        # the expert-parallel step costs without moving any data: the ranks still wait for the most loaded one) and
        # free-running (each rank at its own pace; the gap between the two is load imbalance, not exchange).
        stub = lambda i: blk.forward_partial(i % N_WEIGHT_SETS, t_dev, partial)  # noqa: E731
        stub_ms = timed_once(stub, blk.rendezvous)
        stub_free_ms = timed_once(stub)
        blk.status()
        nccl_ms = timed_once(step_nccl)
        other_form_ms = timed_once(step_dispatch if step is step_replicated else step_replicated)
        blk.status()

        # Correctness of what crossed NVLink, outside the timed regions: one step of each form on the same inputs
        # against the per-rank partials summed by NCCL.
        gen = torch.Generator(device="cuda").manual_seed(1234)
        x0 = torch.randn((T, H), dtype=torch.float32, device="cuda", generator=gen)
        want = x0.clone()
        blk.forward_partial(0, t_dev, partial)
        dist.all_reduce(partial)
        want.add_(partial)
        xr = x0.clone()
        blk.forward(0, t_dev, xr)
        xs = x0[first:first + n_own].clone()
        blk.forward_dispatch(0, T, t_own, xs)
        blk.status()
        errs = torch.tensor([rel_l2_t(xr - x0, want - x0),
                             rel_l2_t(xs - x0[first:first + n_own], (want - x0)[first:first + n_own]) if n_own else 0.0],
                            device="cuda", dtype=torch.float64)
        dist.all_reduce(errs, op=dist.ReduceOp.MAX)
        # every rank's replicated residual stream must hold the same bits
        digest = xr.view(torch.int32).to(torch.int64).sum().reshape(1)
        digests = [torch.empty_like(digest) for _ in range(world)]
        dist.all_gather(digests, digest)
        identical = all(int(d.item()) == int(digests[0].item()) for d in digests)
        # fp32 rows summed in another order than NCCL's: 1e-5; rows or sums rounded to bf16 on the wire: 2^-9 per row
        tol = 1e-5 if wire == 0 else 4e-3
        parity = {"replicated_vs_nccl_rel_l2": float(errs[0].item()), "dispatch_vs_nccl_rel_l2": float(errs[1].item()),
                  "parity_rel_l2": float(errs.max().item()), "ranks_identical": identical, "tolerance": tol,
                  "checked": "one step of each form on the same inputs against forward_partial + NCCL all-reduce (fp32)"}

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
    dispatch_stage_ms = None
    if world > 1:
        dn = ["route_own_rows", "group_and_dispatch_rows", "mlp1_mlp2_push", "owner_sum"]
        evd = [[torch.cuda.Event(enable_timing=True) for _ in range(len(dn) + 1)] for _ in range(K)]
        barrier()
        for i in range(K):
            layer = i % N_WEIGHT_SETS
            evd[i][0].record()
            blk.dispatch_route(layer, T, t_own)
            evd[i][1].record()
            blk.dispatch_rows(layer, T, t_own)
            evd[i][2].record()
            blk.dispatch_push(layer)
            evd[i][3].record()
            blk.sliced_combine(x_own)
            evd[i][4].record()
        barrier()
        blk.status()
        dispatch_stage_ms = {n: sum(evd[i][j].elapsed_time(evd[i][j + 1]) for i in range(K)) / K for j, n in enumerate(dn)}

    hbm_peak, tf_burst, tf_sust, peak_kind = measured_peaks()
    n_local = E // world
    # rows of this rank's experts in the routing of the last step (T*k/world under uniform routing); the rank with the
    # most rows decides an expert-parallel step
    off = blk.tap("offsets", T)
    rows_here = int(off[(rank + 1) * n_local] - off[rank * n_local])
    rows_max = rows_here
    nvlink = None
    if world > 1:
        rm = torch.tensor([rows_here], device="cuda")
        dist.all_reduce(rm, op=dist.ReduceOp.MAX)
        rows_max = int(rm.item())
        # bytes this GPU sends over NVLink per step in the dispatch form: token rows to remote experts, expert rows to
        # remote owners (counted from the routing of the last step)
        ti = blk.tap("topk_i", T)
        owner_of_expert = ti // n_local
        per = moe.slice_bounds(0, world, T)[1]
        owner_of_token = np.minimum(np.arange(T) // max(per, 1), world - 1)[:, None]
        mine_tok = owner_of_token == rank
        rows_out = int(((owner_of_expert != rank) & mine_tok).sum())  # one row per (token, slot) with a remote expert
        push_out = int(((owner_of_expert == rank) & ~mine_tok).sum())
        esz = 2 if wire == 1 else 4
        out_bytes = rows_out * H * 2 + push_out * H * esz
        t_out = torch.tensor([out_bytes], device="cuda", dtype=torch.float64)
        dist.all_reduce(t_out, op=dist.ReduceOp.MAX)
        nvlink = {"bytes_out_per_gpu_per_step_max": int(t_out.item()), "dispatch_rows_out": rows_out, "pushed_rows_out": push_out,
                  "pushed_row_dtype": "bf16" if wire == 1 else "f32",
                  "time_at_900_GBs_ms": float(t_out.item()) / 900e9 * 1e3,
                  "achieved_GBs_over_step": float(t_out.item()) / (ms / K * 1e-3) / 1e9 if step is step_dispatch else None,
                  "bytes_counted_for": "the dispatch form (token rows out + expert rows out), whichever form `value` times"}
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
    roof["traffic"] = NCU_TRAFFIC_MLP1_BYTES if world == 1 and T == 1024 else None  # captured at the N=1 workload only
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
                                                                              "(router_bias[e] -= s*ln(e+1))"} if args.zipf > 0 else
                                                                             {"routing": "uniform (no router-bias skew)"})),
        "timing": {"regions": len(regions), "steps_per_region": K, "region_ms_median": ms, "region_ms_min": min(regions),
                   "region_ms_max": max(regions), "value_from": "median region"},
        "roofline": roof,
        "block_roofline": {"algorithmic_bytes": block_bytes, "algorithmic_flops": block_flops,
                           "roof_ms": block_roof_s * 1e3, "frac": block_roof_s * 1e3 / (ms / K),
                           "busiest_rank_rows": rows_max, "rows_per_rank_if_even": T * K_TOP // world,
                           "roof_ms_busiest_rank": busiest_roof_s * 1e3, "frac_busiest_rank": busiest_roof_s * 1e3 / (ms / K),
                           "bound": "hbm" if block_bytes / (hbm_peak * 1e9) >= block_flops / (tf_sust * 1e12) else "tensor"},
        "stage_ms": stage_ms, "gpu_launches": int(launches),  # counted by the library: launches inside one timed region
    }
    if world > 1:
        line["config"]["form"] = ("token-sliced: each GPU holds its 1/N of the tokens' activations and residual rows; token rows "
                                  "are dispatched to the experts' GPUs, expert rows pushed back to the token's GPU"
                                  if step is step_dispatch else "replicated tokens and residual on every GPU")
        comm_ms = ms / K - stub_ms  # exposed exchange = step with the exchange - step with the exchange stubbed
        line["combine"] = {"kind": ("dispatch of token rows (bf16) by peer stores from the grouping kernel + push of expert rows "
                                    f"({'bf16' if wire == 1 else 'fp32'}) from the down-GEMM epilogue to the token owner + owner sum in slot order"
                                    if step is step_dispatch else
                                    "peer stores (fp32) from the down-GEMM epilogue to the token owner + owner sum in slot "
                                    f"order + peer delivery of the sums ({args.wire})"),
                           "exposed_ms": comm_ms, "share_of_step": comm_ms / (ms / K),
                           "stubbed_exchange_ms_per_step": stub_ms,
                           "stubbed_exchange_without_rendezvous_ms_per_step": stub_free_ms,
                           "nccl_allreduce_baseline_ms_per_step": nccl_ms,
                           ("replicated_form_ms_per_step" if step is step_dispatch else "dispatch_form_ms_per_step"): other_form_ms,
                           "other_timings": "each the median of K-step regions over 0.3 s (sustained, like `value`)",
                           "dispatch_stage_ms": dispatch_stage_ms, "nvlink": nvlink}
        line["combine"].update(parity)

    if rank == 0:
        cs = clocks.summary()
        line["clocks"] = cs

    # End to end through the host-buffer entry points (the C ABI calls a host program makes): every step uploads its
    # inputs from pinned host memory and downloads its result.  A host that feeds batch after batch submits the next
    # call before it waits for the previous one (two calls in flight, two sets of host buffers), so that the result of
    # one step crosses PCIe while the next one's inputs cross it the other way and its kernels run; `value` is that
    # stream of calls, `sync_call_ms` one call at a time (submit + wait back to back).
    if args.no_e2e:
        pass
    else:
        sliced = world > 1
        rows, lo = (n_own, first) if sliced else (T, 0)
        t_host, x_host = [], []
        for _ in range(2):
            th = torch.empty((rows, H), dtype=torch.int16).pin_memory()
            th.copy_(t_dev.view(torch.int16)[lo:lo + rows].cpu())
            t_host.append(th)
            x_host.append(torch.zeros((rows, H), dtype=torch.float32).pin_memory())

        def submit(i):
            if sliced:
                # The host holds the batch once; every rank moves ITS slice of the tokens over PCIe (t and x in, x out)
                # and the ranks exchange token rows and expert rows over NVLink (dispatch form of the block)
                blk.forward_host_sliced_submit(i % N_WEIGHT_SETS, T, t_host[i & 1], x_host[i & 1])
            else:
                blk.forward_host_submit(i % N_WEIGHT_SETS, t_host[i & 1], x_host[i & 1])

        def stream_of_calls(n):
            submit(0)
            for i in range(1, n):
                submit(i)
                blk.forward_host_wait()  # call i - 1: its result is in x_host[(i - 1) & 1]
            blk.forward_host_wait()

        def one_at_a_time(n):
            for i in range(n):
                submit(i)
                blk.forward_host_wait()

        n_e2e = max(K, 50, int(0.3 / max(ms / K * 2.5e-3, 1e-6))) if not sliced else max(K, 50)  # about 0.3 s of calls
        timings = {}
        for name, fn, n in (("stream", stream_of_calls, n_e2e), ("sync", one_at_a_time, max(K, 20))):
            fn(4)
            torch.cuda.synchronize()
            barrier()
            t0 = time.perf_counter()
            fn(n)
            dt = time.perf_counter() - t0
            if sliced:
                tt = torch.tensor([dt], device="cuda", dtype=torch.float64)
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                dt = float(tt.item())
            timings[name] = dt / n
        line["e2e"] = {"value": T / timings["stream"], "unit": "tok/s", "h2d_bytes_per_step": T * H * 2 + T * H * 4,
                       "d2h_bytes_per_step": T * H * 4, "ms_per_step": 1e3 * timings["stream"], "calls_timed": n_e2e,
                       "calls_in_flight": 2, "sync_call_ms": 1e3 * timings["sync"],
                       "sync_call_tok_per_s": T / timings["sync"],
                       "api": ("gptoss_moe_forward_host_sliced_submit" if sliced else "gptoss_moe_forward_host_submit")
                              + " / gptoss_moe_forward_host_wait"}
        if sliced:
            line["e2e"]["note"] = "bytes over all GPUs; each GPU copies its own token slice (1/N of them)"

    # the skewed-routing workload: T = 8192 tokens in total, Zipf s = 1.2 over the expert ids, experts sharded E/N
    if not args.no_extras:
        try:
            line["skewed_T8192"] = run_skewed(blk, moe, torch, dist, world, rank, skew_layer, T_SKEW, K, barrier)
        except Exception as e:  # an extra must never cost the headline
            line["skewed_T8192"] = {"error": repr(e)}

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        _, info, _ = cpu_arm(T, target_seconds=12.0, repeats=1, warmup=0)
        line["cpu_baseline"] = info
    blk.close()
    del blk, t_dev, x, partial
    torch.cuda.empty_cache()

    # whole-model decode beside the layer numbers (own context; the MoE context above is gone)
    if not args.no_extras:
        line["decode"] = {}
        for wl in (["decode20b"] + (["decode120b"] if world >= 4 else [])):
            try:
                line["decode"][wl] = decode_leg(args, wl, dist if world > 1 else None)
            except Exception as e:
                line["decode"][wl] = {"error": repr(e)}

    bad = parity is not None and not (parity["parity_rel_l2"] <= parity["tolerance"] and parity["ranks_identical"])
    if rank == 0:
        print_line(line)
    if world > 1:
        dist.destroy_process_group()
    if bad:
        raise SystemExit(f"cross-GPU parity check failed: {parity}")


def run_skewed(blk, moe, torch, dist, world, rank, layer, T, K, barrier):
    """One gpt-oss-20b MoE layer at T = 8192 tokens with Zipf-skewed routing (router_bias[e] -= 1.2 ln(e+1): expert 0 the
    hottest), experts in contiguous shards of E/N per GPU: rank 0 holds the hot experts.  N = 1: replicated form on
    one GPU; N > 1: dispatch form.  Reports the step time against the tensor roofline of the busiest rank."""
    hbm_peak, tf_burst, tf_sust, _ = measured_peaks()
    blk.fill_layer_synthetic(layer, SEED, SIGMA)
    blk.set_router_bias(layer, synth.zipf_router_bias(SEED, layer, E, 1.2))
    t_dev = moe.synth_normal_bf16(T * H, SEED + 1, synth.tensor_id(synth.TID_ACTIVATION), 1.0).view(T, H)
    first, n_own = blk.slice(T)
    if world == 1:
        x = torch.zeros((T, H), dtype=torch.float32, device="cuda")
        fn = lambda i: blk.forward(layer, t_dev, x)  # noqa: E731
    else:
        t_own = t_dev[first:first + n_own].contiguous()
        x = torch.zeros((n_own, H), dtype=torch.float32, device="cuda")
        fn = lambda i: blk.forward_dispatch(layer, T, t_own, x)  # noqa: E731
    for i in range(3):
        fn(i)
    barrier()
    blk.status()
    steps = max(5, min(K, 20))
    with ClockSampler(int(os.environ.get("LOCAL_RANK", "0")), enabled=rank == 0) as cl:
        regions = timed_regions(fn, steps, barrier, world, dist, torch, min_seconds=0.3)
    blk.status()
    ms = statistics.median(regions) / steps
    off = blk.tap("offsets", T)
    n_local = E // world
    rows = [int(off[(r + 1) * n_local] - off[r * n_local]) for r in range(world)]
    busiest = max(rows)
    flops_busiest = 2.0 * busiest * 3 * H * I + 2.0 * (T // world if world > 1 else T) * H * E
    bytes_rank = n_local * 3 * H * I * 2 + T * H * 2 + T * H * 8 / world
    roof_ms = max(flops_busiest / (tf_sust * 1e12), bytes_rank / (hbm_peak * 1e9)) * 1e3
    out = {"tokens": T, "router_skew": "Zipf s=1.2 over expert id", "experts_per_gpu": n_local, "ms_per_step": ms,
           "tok_per_s": T / (ms * 1e-3), "rows_per_rank": rows, "busiest_rank_rows": busiest,
           "roof_ms_busiest_rank": roof_ms, "frac_busiest_rank": roof_ms / ms,
           "bound": "tensor (sustained bf16 peak)" if flops_busiest / (tf_sust * 1e12) >= bytes_rank / (hbm_peak * 1e9) else "hbm",
           "form": "one GPU" if world == 1 else "token-sliced dispatch form", "clocks": cl.summary() if rank == 0 else None,
           "regions": len(regions), "steps_per_region": steps}
    if world > 1:
        partial = torch.empty((T, H), dtype=torch.float32, device="cuda")
        stub = lambda i: (blk.forward_partial(layer, t_dev, partial), blk.rendezvous())  # noqa: E731
        for i in range(2):
            stub(i)
        stub_regions = timed_regions(stub, steps, barrier, world, dist, torch, min_seconds=0.1)
        stub_ms = statistics.median(stub_regions) / steps
        out["combine"] = {"exposed_ms": ms - stub_ms, "share_of_step": (ms - stub_ms) / ms, "stubbed_exchange_ms_per_step": stub_ms}
        blk.status()
    return out


def decode_leg(args, workload, dist):
    """Whole-model batched greedy decode (random-init weights generated on the device), sequences of random prompt
    ids force-fed one position per step, then greedy tokens.  decode20b: gpt-oss-20b architecture, 1024 x 128 prompt
    ids, 256 generated; decode120b: gpt-oss-120b architecture, 2048 x 256, 256 generated (needs the experts spread
    over >= 4 GPUs).  With N > 1 (one process per GPU, process group already up) the N GPUs decode the
    batch together: sequences in slices, experts sharded, per-layer exchange over peer memory.  Reported like the
    reference's getp mode: generated tokens / wall time of the whole inference loop (getp-csrc/getp_eval.cpp:125-131),
    the slowest rank's time.  Returns the result as a dict."""
    import torch
    from gptoss_b200 import binfmt, model
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    big = workload == "decode120b"
    B = args.decode_batch or (2048 if big else 1024)
    n_prompt = args.decode_prompt or (256 if big else 128)
    n_gen = args.decode_gen or 256
    cfg = binfmt.config_120b(seq_len=1024) if big else binfmt.config_20b(seq_len=1024)
    if args.decode_layers:
        cfg.n_layers = args.decode_layers
    m = model.Model(cfg, device=local_rank, max_batch=B, max_seq=args.decode_first_pos + n_prompt + n_gen, rank=rank, world=world)
    try:
        m.fill_synthetic(SEED, SIGMA)
        if world > 1:
            m.attach_peers()
        first, n = m.slice(B)
        prompts = synth.uniform_ids(SEED, 11, B * n_prompt, cfg.vocab_size).reshape(B, n_prompt)[first:first + n]
        m.generate(prompts[:, :2], 2, batch=B)  # warm-up: 3 steps
        if world > 1:
            dist.barrier()
        with ClockSampler(local_rank, enabled=rank == 0) as clocks:
            t0 = time.perf_counter()
            out = m.generate(prompts, n_gen, batch=B, first_pos=args.decode_first_pos)
            dt = time.perf_counter() - t0
        n_distinct = int(len(np.unique(out)))
        if world > 1:
            tt = torch.tensor([dt], device="cuda", dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            dt = float(tt.item())
            dist.barrier()
    finally:
        m.close()
    steps = n_prompt + n_gen - 1
    arch = "gpt-oss-120b" if big else "gpt-oss-20b"
    # HBM roofline of the decode: every step streams this GPU's weights once (its experts, the attention projections;
    # the classifier only on steps that produce a token) and the K/V rows of its sequences up to the position
    # (windowed on even layers)
    hbm_peak = measured_peaks()[0]
    c = cfg
    qd, kvd = c.head_dim * c.n_attn_heads, c.head_dim * c.n_kv_heads
    w_layer = (c.n_experts // world) * 3 * c.hidden_dim * c.intermediate_dim * 2 + ((qd + 2 * kvd) * c.hidden_dim + c.hidden_dim * qd) * 2
    seqs = -(-B // world)
    total = 0.0
    for pos in range(args.decode_first_pos, args.decode_first_pos + steps):
        kv = 0
        for l in range(c.n_layers):
            ctx_len = min(pos + 1, c.sliding_window) if (c.sliding_window > 0 and l % 2 == 0) else pos + 1
            kv += ctx_len * kvd * 2 * 2
        total += c.n_layers * w_layer + seqs * kv
        if pos - args.decode_first_pos >= n_prompt - 1:
            total += c.vocab_size * c.hidden_dim * 2
    roof_s = total / (hbm_peak * 1e9)
    return {"metric": f"batched decode tok/s, {arch} arch (whole model, greedy, lock-step)", "value": B * n_gen / dt,
            "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": 3, "ms_per_step": 1e3 * dt / steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 (fp32 accumulate)",
            "data": "synthetic",
            "config": {"workload": f"{arch} architecture, {cfg.n_layers} layers, batch {B} x {n_prompt} random prompt "
                                   f"ids, greedy decode {n_gen} tokens; tokens in/out over host memory every step",
                       "parallelism": "one GPU" if world == 1 else
                       f"{world} GPUs: sequences in {world} slices (data-parallel attention), {cfg.n_experts // world} "
                       "experts per GPU, activations and expert rows exchanged over NVLink peer memory",
                       "positions_per_second": B * steps / dt, "seed": SEED},
            "roofline": {"bound": "hbm", "bytes_per_gpu_whole_decode": total, "roof_ms_per_step": 1e3 * roof_s / steps,
                         "frac": roof_s / dt, "peak": hbm_peak, "unit": "GB/s",
                         "counts": "per step: this GPU's expert and attention weights once, classifier on generating steps, K/V rows of its sequences"},
            "clocks": clocks.summary() if rank == 0 else None, "distinct_tokens_generated_rank0": n_distinct}


def ragged_leg(args):
    """Whole-model decode of requests of unequal length on one GPU, under two schedules: batch-at-a-time (the
    reference's, getp-csrc/submit/getp_run_submit.cpp:33-96, plus the removal of finished sequences from the batch)
    and continuous batching (a free slot is refilled at once; sequences at different positions share a step).
    gpt-oss-20b architecture, random-init weights; 4 x batch requests of 16 random prompt ids, each generating a seeded
    number of tokens drawn uniformly from [32, 256] (standing in for where a stop id would fall in real text).
    Both schedules produce the same tokens; reported: generated tokens / wall time of each."""
    from gptoss_b200 import binfmt, model
    B = args.decode_batch or 1024
    n_prompt = args.decode_prompt or 16
    n_req = 4 * B
    rng = np.random.default_rng(SEED)
    gen_len = rng.integers(32, 257, size=n_req)
    cfg = binfmt.config_20b(seq_len=1024)
    if args.decode_layers:
        cfg.n_layers = args.decode_layers
    prompts = synth.uniform_ids(SEED, 12, n_req * n_prompt, cfg.vocab_size).reshape(n_req, n_prompt).astype(np.int32)
    last_pos = n_prompt - 1 + gen_len  # a request has finished once it has taken this many steps
    m = model.Model(cfg, device=0, max_batch=B, max_seq=n_prompt + 256)
    out = {}
    try:
        m.fill_synthetic(SEED, SIGMA)
        m.generate(prompts[:B, :2], 2)  # warm-up
        for schedule in ("batches", "continuous"):
            tokens_out = np.full((n_req, 256), -1, np.int32)
            steps = 0
            seq_steps = 0
            with ClockSampler(0) as clocks:
                t0 = time.perf_counter()
                if schedule == "batches":
                    for first in range(0, n_req, B):
                        req = np.arange(first, first + B)
                        cur = prompts[req, 0].copy()
                        live = np.arange(B, dtype=np.int32)
                        pos = 0
                        while live.size:
                            r = req[live]
                            gen = pos + 1 >= n_prompt  # inside the prompts nobody needs the model's token
                            nxt = m.step(cur, pos, need_next=gen) if live.size == B else m.step_rows(cur[live], live, pos, need_next=gen)
                            steps += 1
                            seq_steps += live.size
                            if gen:
                                tokens_out[r, pos + 1 - n_prompt] = nxt
                                cur[live] = nxt
                            else:
                                cur[live] = prompts[r, pos + 1]
                            pos += 1
                            live = live[last_pos[r] > pos]
                else:
                    slot_req = np.full(B, -1, np.int64)
                    slot_pos = np.zeros(B, np.int32)
                    cur = np.zeros(B, np.int32)
                    next_req = 0
                    while True:
                        free = np.flatnonzero(slot_req < 0)
                        take = min(free.size, n_req - next_req)
                        if take:
                            f = free[:take]
                            slot_req[f] = np.arange(next_req, next_req + take)
                            slot_pos[f] = 0
                            cur[f] = prompts[slot_req[f], 0]
                            next_req += take
                        live = np.flatnonzero(slot_req >= 0).astype(np.int32)
                        if not live.size:
                            break
                        r, p = slot_req[live], slot_pos[live]
                        nxt = m.step_seqs(cur[live], live, p)
                        steps += 1
                        seq_steps += live.size
                        gen = p + 1 >= n_prompt
                        tokens_out[r[gen], p[gen] + 1 - n_prompt] = nxt[gen]
                        cur[live] = np.where(gen, nxt, prompts[r, np.minimum(p + 1, n_prompt - 1)])
                        slot_pos[live] = p + 1
                        done = live[last_pos[r] <= p + 1]
                        slot_req[done] = -1
                dt = time.perf_counter() - t0
            out[schedule] = {"tok_s": float(gen_len.sum() / dt), "wall_s": dt, "steps": steps,
                             "mean_sequences_per_step": seq_steps / steps, "ms_per_step": 1e3 * dt / steps,
                             "clocks": clocks.summary(), "tokens": tokens_out}
    finally:
        m.close()
    same = bool(np.array_equal(out["batches"]["tokens"], out["continuous"]["tokens"]))
    for v in out.values():
        del v["tokens"]
    return {"metric": "batched decode tok/s, gpt-oss-20b arch (whole model, greedy), requests of unequal length",
            "value": out["continuous"]["tok_s"], "unit": "tok/s", "n_gpus": 1, "higher_is_better": True,
            "dtype": "bf16 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": f"gpt-oss-20b architecture, {cfg.n_layers} layers, {n_req} requests on {B} slots, {n_prompt} random "
                                   "prompt ids each, generated length uniform in [32, 256] (seeded)", "seed": SEED},
            "schedules": out, "speedup_continuous_over_batches": out["continuous"]["tok_s"] / out["batches"]["tok_s"],
            "same_tokens_under_both_schedules": same}


def run_decode(args):
    import torch
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))))
    line = ragged_leg(args) if args.workload == "decode20b_ragged" else decode_leg(args, args.workload, dist)
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
                    help="N > 1: wire format. Dispatch form: the expert rows pushed to the token's owner (summed there in "
                         "fp32). Replicated form: the sums the owners deliver (rows travel to the owner in fp32)")
    ap.add_argument("--workload", choices=["moe_layer", "decode20b", "decode120b", "decode20b_ragged"], default="moe_layer",
                    help="moe_layer: the MoE block (headline, with the other workloads as extra keys); decode20b / "
                         "decode120b: only the whole-model greedy decode; decode20b_ragged: requests of unequal length "
                         "on one GPU, batch-at-a-time against continuous batching")
    ap.add_argument("--decode-batch", type=int, default=0, help="0 = the config's batch (1024 / 2048)")
    ap.add_argument("--decode-prompt", type=int, default=0, help="0 = the config's prompt length (128 / 256)")
    ap.add_argument("--decode-gen", type=int, default=0, help="0 = 256")
    ap.add_argument("--decode-layers", type=int, default=0, help="override the layer count (0 = 24)")
    ap.add_argument("--decode-first-pos", type=int, default=0,
                    help="profiling runs: start the timed decode at this position (cache rows before it are zeros)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the extra legs of the line (skewed T=8192 workload, whole-model decode)")
    ap.add_argument("--form", choices=["dispatch", "replicated"], default="dispatch",
                    help="N > 1: which form of the expert-parallel block `value` times (the other is reported beside it, "
                         "timed over one short region)")
    ap.add_argument("--tokens-per-gpu", type=int, default=0,
                    help="tokens per step and GPU (0 = 1024, the headline workload; 8192 on one GPU: the block is tensor-bound)")
    ap.add_argument("--zipf", type=float, default=0.0,
                    help="skew the routing: router_bias[e] -= s*ln(e+1) (1.2: the skewed-routing workload); 0 = uniform")
    ap.add_argument("--weight-sets", type=int, default=N_WEIGHT_SETS,
                    help="distinct layers of weights the steps rotate over (1 keeps a profiling run small)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload in ("decode20b", "decode120b", "decode20b_ragged"):
        run_decode(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
