"""Benchmark of the hot path on B200.

``python bench.py --gpus N --steps K --warmup W`` prints ONE JSON line.  A step is one pass of
the FP8 block-scaled MoE expert layer at the DeepSeek-V3 shape (4096 tokens, hidden 7168, 256
experts, top-8, intermediate 2048; softmax top-k routing; e4m3 activations with 1x128 scales)
over synthetic inputs; with N > 1 (launched by torch.distributed.run) the layer is
expert-parallel: 4096/N tokens and 256/N experts per rank, dispatch and combine over NVLink,
and ``value`` is the whole job's TFLOP/s (total work fixed: strong scaling).

``value``  : inputs resident in HBM before the timed region (CUDA events, barrier + synchronize on
             both sides, max over ranks).  The region of K steps is repeated (``cohorts``); the
             headline is the median cohort and the line carries every cohort and their CV.
``e2e``    : the same metric through the public Python API with HOST buffers: every step copies
             the step's activations and router logits from pinned memory to the device and reads
             the bf16 output back; expert weights are model state and stay resident.
``roofline``: the dominant kernel (grouped GEMM1 + SwiGLU), algorithmic bytes / CUDA-event time
             against the measured HBM copy bandwidth.
``contract_mode``: the same layer in the configuration that meets the reference contract's own
             tolerance (DeepSeek-V3 group-limited routing, two-term FP8 intermediate).
``compute_bound``: the layer with 1024 tokens per expert (4096 tokens over 32 experts), where the
             grouped GEMMs are bound by the tensor pipe instead of by weight streaming.
``cpu_baseline`` / ``--impl reference``: the reference's CPU oracle arithmetic for the same layer
             (oracle/moe.py, a restatement pinned bit-for-bit to the reference's oracle), timed on
             the host cores over a bounded sample of the workload.
The four per-GPU operators (RMSNorm, block-scaled GEMM, paged GQA / MLA decode) are timed at N = 1
and reported under ``operators``, each with its own bounded CPU baseline.  With N > 1 the line
also carries ``ep_parity`` (the expert-parallel output checked against the CPU oracle before the
timed region; a failure exits non-zero) and per-stage times of one step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHAPE = dict(tokens=4096, hidden=7168, inter=2048, experts=256, top_k=8)
WORKLOAD = "fp8_moe_dsv3_T4096_H7168_E256_top8_I2048_softmax_routing_e4m3_act"


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        doc = json.loads(path.read_text())
        return {"hbm_gbs": float(doc["hbm_gbs"]), "bf16_tflops": float(doc["bf16_tflops"]),
                "bf16_tflops_sustained": float(doc.get("bf16_tflops_sustained", doc["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=self.file,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        self.file.flush()
        rows = [line.split(",") for line in Path(self.file.name).read_text().splitlines() if line.count(",") >= 8]
        os.unlink(self.file.name)
        sm, power = [], []
        reasons = set()
        max_mhz = None
        for r in rows:
            try:
                clock, watts = float(r[1]), float(r[3])
                max_mhz = float(r[2])
            except ValueError:
                continue
            sm.append(clock); power.append(watts)
            for name, cell in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if cell.strip().lower().startswith("active"):
                    reasons.add(name)
        # "under load" = samples drawing at least half of the highest power seen during the region
        top = max(power) if power else 0.0
        loaded = [c for c, w in zip(sm, power) if w >= 0.5 * top] or sm
        return {"sm_mhz": statistics.median(loaded) if loaded else None, "sm_max_mhz": max_mhz, "reasons": sorted(reasons),
                "samples": len(sm), "samples_under_load": len(loaded), "power_w_max": top}


HOST_BINDING = {"cpus": None}


def bind_host_to_gpu(local: int):
    """Keeps this rank's host threads, and with them the pinned buffers they allocate and touch first, on the CPU
    socket the rank's GPU hangs off: with one rank per GPU and every rank's pinned memory on the socket the launcher
    happened to start it on, the end-to-end copies of several ranks share one inter-socket link.  Returns the CPU
    list used, or None where the platform does not tell (then nothing is changed)."""
    try:
        props = torch.cuda.get_device_properties(local)
        address = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        text = Path(f"/sys/bus/pci/devices/{address}/local_cpulist").read_text().strip()
        cpus = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return text
    except Exception:                                   # noqa: BLE001 - an optimisation only; never fatal
        return None


def dist_setup(n_gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        HOST_BINDING["cpus"] = bind_host_to_gpu(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    elif n_gpus > 1:
        raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    return world, rank, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(value: float, world: int) -> float:
    if world == 1:
        return value
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_steps(step, steps: int, warmup: int, world: int) -> float:
    """Milliseconds per step: W untimed steps, then exactly K steps between two events bracketed by
    barrier + synchronize; max over ranks."""
    for _ in range(warmup):
        step()
    barrier(world)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        step()
    stop.record()
    barrier(world)
    return max_over_ranks(start.elapsed_time(stop) / steps, world)


def cohort_stats(samples):
    """Median, coefficient of variation and the samples of repeated timed regions (the reference's paired
    timing admits a cohort at CV <= 0.05, src/open_cake_ir/evaluation/timing.py:167-173)."""
    mean = statistics.mean(samples)
    cv = statistics.pstdev(samples) / mean if len(samples) > 1 and mean > 0 else 0.0
    return {"n": len(samples), "ms": [round(x, 5) for x in samples], "median_ms": statistics.median(samples), "cv": cv}


def time_rotating(launches, min_seconds=0.15, warmup=3):
    """Mean milliseconds per launch of a kernel shorter than the event overhead is worth: the launches of
    ``launches`` (one closure per buffer set; the sets together exceed twice the L2, so every launch finds
    its inputs in HBM) are issued back to back, in turn, between ONE pair of events, for at least
    ``min_seconds``; three such regions, the median is returned with the samples."""
    n = len(launches)
    for _ in range(warmup):
        for launch in launches:
            launch()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for launch in launches:
        launch()
    stop.record()
    torch.cuda.synchronize()
    rough = max(start.elapsed_time(stop) / n, 1e-3)
    rounds = max(2, int(min_seconds * 1e3 / rough / n) + 1)
    samples = []
    for _ in range(3):
        start.record()
        for _ in range(rounds):
            for launch in launches:
                launch()
        stop.record()
        torch.cuda.synchronize()
        samples.append(start.elapsed_time(stop) / (rounds * n))
    return statistics.median(samples), cohort_stats(samples), rounds * n


E2E_INPUTS = ("routing_logits", "hidden_states", "hidden_states_scale")


def pipelined_e2e(make_set, dev, out):
    """Builds the end-to-end step: host inputs -> device, layer, output -> host, with the copies of
    neighbouring steps overlapping this step's kernels.  ``make_set()`` returns (device inputs, device
    output, launch(stream)) for one of the two buffer sets.  Returns (step, h2d bytes, d2h bytes)."""
    host_in = {k: dev[k].cpu().pin_memory() for k in E2E_INPUTS}
    h2d = sum(t.numel() * t.element_size() for t in host_in.values())
    d2h = out.numel() * out.element_size()
    sets = []
    for _ in range(2):
        inputs, o, launch = make_set()
        sets.append({"in": inputs, "out": o, "launch": launch, "host_out": torch.empty_like(out, device="cpu").pin_memory(),
                     "h2d_done": torch.cuda.Event(), "compute_done": torch.cuda.Event(), "d2h_done": torch.cuda.Event()})
    copy_in, compute, copy_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    main = torch.cuda.current_stream()
    counter = {"k": 0}

    def step():
        k = counter["k"]; counter["k"] += 1
        b = sets[k & 1]
        if k == 0:
            for st in (copy_in, compute, copy_out):
                st.wait_stream(main)
        with torch.cuda.stream(copy_in):
            if k >= 2:
                copy_in.wait_event(b["compute_done"])        # step k-2 has consumed these inputs
            for name in E2E_INPUTS:
                b["in"][name].copy_(host_in[name], non_blocking=True)
            b["h2d_done"].record(copy_in)
        with torch.cuda.stream(compute):
            compute.wait_event(b["h2d_done"])
            if k >= 2:
                compute.wait_event(b["d2h_done"])            # step k-2's output has left the device
            b["launch"](compute)
            b["compute_done"].record(compute)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(b["compute_done"])
            b["host_out"].copy_(b["out"], non_blocking=True)
            b["d2h_done"].record(copy_out)
        main.wait_stream(copy_out)                           # the timing events live on the main stream

    return step, h2d, d2h


# ------------------------------------------------------------------------------------------------
# dram__bytes_read.sum + dram__bytes_write.sum of ONE gemm_fp8_kernel<kGateUp> launch, from an ncu capture of
# `bench.py --profile-case moe` (1024 tokens over 64 experts: 128 tokens per expert as at full size), and the
# algorithmic bytes of that case.  Every expert's weights are read once, so traffic grows with the number of
# experts and the full layer's figure is this ratio times its algorithmic bytes (1.006 x algorithmic: every weight
# byte is read from DRAM once; the second row tile of an expert finds it in L2).
NCU_GEMM1_CASE = {"traffic_bytes": 1.966e9, "algorithmic_bytes": 64 * 2 * 2048 * 7168 + 8192 * (7168 + 2048)}


def stage_times(op, steps):
    """Mean milliseconds of the four parts of the layer, events between the parts (the weights, 11 GB, are far
    larger than L2, so consecutive launches are cold anyway)."""
    events = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(steps)]
    for k in range(steps):
        events[k][0].record()
        for s in range(4):
            op.launch_stage(s)
            events[k][s + 1].record()
    torch.cuda.synchronize()
    return [sum(events[k][s].elapsed_time(events[k][s + 1]) for k in range(steps)) / steps for s in range(4)]


def moe_single(steps, warmup, peaks, cohorts):
    import open_cake_ir_b200 as cake
    dev = cake.workloads.moe_inputs(tokens=SHAPE["tokens"], hidden=SHAPE["hidden"], inter=SHAPE["inter"],
                                    experts=SHAPE["experts"], local_experts=SHAPE["experts"], local_offset=0,
                                    routing="softmax", device="cuda", gen_device="cuda")
    out = torch.empty((SHAPE["tokens"], SHAPE["hidden"]), dtype=torch.bfloat16, device="cuda")
    op = cake.Fp8Moe(dev, out, routing="softmax", act_mode="fp8")
    flops = cake.workloads.moe_flops(SHAPE["tokens"], SHAPE["hidden"], SHAPE["inter"])
    clocks = ClockSampler(torch.cuda.current_device())
    clocks.__enter__()                     # sampled until the end-to-end loop below has finished
    samples = [time_steps(op.launch, steps, warmup if c == 0 else 1, 1) for c in range(cohorts)]
    if op.status():
        raise RuntimeError("a device-side wait ran out")
    stage_ms = stage_times(op, steps)
    pairs = SHAPE["tokens"] * SHAPE["top_k"]
    gemm1_bytes = SHAPE["experts"] * 2 * SHAPE["inter"] * SHAPE["hidden"] + pairs * (SHAPE["hidden"] + SHAPE["inter"])
    achieved = gemm1_bytes / (stage_ms[1] * 1e-3) / 1e9
    roofline = {"kernel": "gemm_fp8_kernel<kGateUp> (grouped GEMM1 + SwiGLU + e4m3 requantisation)", "bound": "hbm",
                "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "peak_source": peaks["source"], "algorithmic_bytes": gemm1_bytes, "ms": stage_ms[1],
                "traffic": int(gemm1_bytes * NCU_GEMM1_CASE["traffic_bytes"] / NCU_GEMM1_CASE["algorithmic_bytes"]),
                "traffic_source": "ncu capture of the 64-expert profile case, scaled by the number of experts",
                "tflops": 2 * pairs * 2 * SHAPE["inter"] * SHAPE["hidden"] / (stage_ms[1] * 1e-3) / 1e12}
    # End to end with host buffers: steps are independent layers over fresh activations, so the copies of
    # neighbouring steps overlap this step's kernels (two buffer sets over the same resident weights).
    def make_set():
        inputs = dict(dev)
        for k in E2E_INPUTS:
            inputs[k] = torch.empty_like(dev[k])
        o = torch.empty_like(out)
        layer = cake.Fp8Moe(inputs, o, routing="softmax", act_mode="fp8")
        return inputs, o, layer.launch

    e2e_step, h2d, d2h = pipelined_e2e(make_set, dev, out)
    e2e_ms = time_steps(e2e_step, steps, warmup, 1)
    clocks.__exit__()
    summary = clocks.summary()
    # The configuration that passes the reference contract's own cases at its own tolerance: DeepSeek-V3
    # group-limited sigmoid routing and the SwiGLU output carried as two e4m3 terms (GEMM2's K doubles).
    ds = dict(dev)
    ds["routing_bias"] = (torch.rand(SHAPE["experts"], device="cuda", generator=torch.Generator(device="cuda").manual_seed(20261125))
                          * 0.015).to(torch.bfloat16)
    contract_op = cake.Fp8Moe(ds, out, routing="ds", act_mode="split")
    contract_ms = time_steps(contract_op.launch, steps, 2, 1)
    contract_stages = stage_times(contract_op, steps)
    if contract_op.status():
        raise RuntimeError("a device-side wait ran out")
    contract = {"workload": "the same layer with DeepSeek-V3 group-limited routing and a two-term FP8 intermediate "
                            "(passes the reference contract's cases at atol = rtol = 1e-2)",
                "value": flops / (contract_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": contract_ms,
                "stage_ms": dict(zip(cake.Fp8Moe.STAGES, contract_stages))}
    del contract_op, ds
    mhz = summary.get("sm_mhz") or 0.0
    return {"ms": statistics.median(samples), "cohorts": cohort_stats(samples), "flops": flops, "clocks": summary,
            "stage_ms": dict(zip(cake.Fp8Moe.STAGES, stage_ms)),
            "stage_cycles": {name: ms * 1e-3 * mhz * 1e6 for name, ms in zip(cake.Fp8Moe.STAGES, stage_ms)},
            "roofline": roofline, "e2e_ms": e2e_ms, "h2d": h2d, "d2h": d2h, "launches": 8 * steps, "contract_mode": contract}


def moe_compute_bound(steps, peaks):
    """4096 tokens over 32 experts (1024 tokens per expert, eight full row tiles each): the grouped GEMMs
    re-use every weight tile eight times, so the layer is bound by the tensor pipe and the promotion, not by
    weight streaming.  Reported against twice the measured bf16 rate and against the 4.5 PFLOP/s nominal."""
    import open_cake_ir_b200 as cake
    experts = 32
    dev = cake.workloads.moe_inputs(tokens=SHAPE["tokens"], hidden=SHAPE["hidden"], inter=SHAPE["inter"], experts=experts,
                                    local_experts=experts, local_offset=0, routing="softmax", device="cuda", gen_device="cuda")
    out = torch.empty((SHAPE["tokens"], SHAPE["hidden"]), dtype=torch.bfloat16, device="cuda")
    op = cake.Fp8Moe(dev, out, experts=experts, routing="softmax", act_mode="fp8")
    ms = time_steps(op.launch, steps, 3, 1)
    stages = stage_times(op, steps)
    if op.status():
        raise RuntimeError("a device-side wait ran out")
    flops = cake.workloads.moe_flops(SHAPE["tokens"], SHAPE["hidden"], SHAPE["inter"])
    tflops = flops / (ms * 1e-3) / 1e12
    gemm_ms = stages[1] + stages[2]
    return {"workload": "fp8_moe_T4096_H7168_E32_top8_I2048 (1024 tokens per expert)", "tflops": tflops, "ms_per_step": ms,
            "stage_ms": dict(zip(cake.Fp8Moe.STAGES, stages)), "grouped_gemm_tflops": flops / (gemm_ms * 1e-3) / 1e12,
            "frac_of_2x_measured_bf16": tflops / (2 * peaks["bf16_tflops_sustained"]),
            "frac_of_4500": tflops / 4500.0,
            "peak_note": "2 x the measured sustained cuBLAS bf16 rate (the kernels run inside a long step)"}


def gather_rows(local: torch.Tensor, world: int, rank: int):
    """All ranks' [T/R, H] outputs -> [T, H] on rank 0's host (None elsewhere)."""
    import torch.distributed as dist
    parts = [torch.empty_like(local) for _ in range(world)] if rank == 0 else None
    dist.gather(local.contiguous(), parts, dst=0)
    return torch.cat([p.cpu() for p in parts]) if rank == 0 else None


def ep_parity(world, rank, layer, dev, layer_class):
    """The expert-parallel path against the CPU oracle, before anything is timed (the oracle is the checker
    here and nothing else).  (a) A small layer (512 tokens, hidden 1024, intermediate 512, 32 experts) through the
    same exchange on all ranks, gathered and compared with the oracle over the WHOLE problem.  (b) At the bench
    shape, eight of rank 0's tokens are followed through every expert they use, the weights of those experts
    regenerated from their seeds whoever owns them.  Returns the record for the JSON line."""
    import open_cake_ir_b200 as cake
    from open_cake_ir_b200 import ep
    from oracle import compare, moe as oracle_moe, routing as oracle_routing
    small = dict(hidden=1024, inter=512, experts=32)
    tokens = 512
    t_local, e_local = tokens // world, small["experts"] // world
    sd = cake.workloads.moe_inputs(tokens=t_local, **small, local_experts=e_local, local_offset=rank * e_local, routing="softmax",
                                   device="cuda", gen_device="cpu", first_token=rank * t_local, total_tokens=tokens)
    small_layer = layer_class(sd, sd["routing_logits"], sd["routing_bias"], sd["hidden_states"],
                              sd["hidden_states_scale"], experts=small["experts"], routing="softmax")
    for _ in range(2):                       # twice: every buffer is reused between steps
        got_local = small_layer.forward()
    torch.cuda.synchronize()
    got = gather_rows(got_local, world, rank)
    record = {"world": world}
    if rank == 0:
        whole = cake.workloads.moe_inputs(tokens=tokens, **small, local_experts=small["experts"], local_offset=0,
                                          routing="softmax", device="cpu", gen_device="cpu")
        want = oracle_moe.moe_reference(whole, routing="softmax", act_quant="fp8", dtype=torch.float32)["output"]
        ok, bad, err = compare.compare(got, want, atol=2e-2, rtol=2e-2)
        record.update(small_case="512 tokens, hidden 1024, intermediate 512, 32 experts: every output element",
                      rel_frobenius=compare.rel_frobenius(got, want), max_abs=float(err), mismatches=int(bad), ok=bool(ok))
    small_layer.close()
    del small_layer, sd
    # (b) the bench shape (the ranks meet first: rank 0 has just spent seconds in the oracle above)
    import torch.distributed as dist
    dist.barrier()
    out_local = layer.forward()
    torch.cuda.synchronize()
    if rank == 0:
        t_bench = SHAPE["tokens"] // world
        pick = torch.arange(0, t_bench, t_bench // 8)[:8]
        sub = {"routing_logits": dev["routing_logits"][pick].cpu(), "hidden_states": dev["hidden_states"][pick].cpu(),
               "hidden_states_scale": dev["hidden_states_scale"][:, pick].cpu().contiguous(),
               "routed_scaling_factor": dev["routed_scaling_factor"].cpu(), "local_expert_offset": torch.zeros(1, dtype=torch.int32)}
        ids, _ = oracle_routing.routing_softmax_topk(sub["routing_logits"])
        used = sorted(set(ids.reshape(-1).tolist()))
        remap = {e: i for i, e in enumerate(used)}
        parts = [cake.workloads.moe_expert_weights(e, SHAPE["hidden"], SHAPE["inter"], gen_device="cuda") for e in used]
        for i, name in enumerate(("gemm1_weights", "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale")):
            sub[name] = torch.stack([p[i].cpu() for p in parts])
        logits = torch.full((pick.numel(), len(used)), -1e30)      # the same experts win in the compacted numbering
        for t in range(pick.numel()):
            for e in ids[t].tolist():
                logits[t, remap[e]] = sub["routing_logits"][t, e]
        sub["routing_logits"] = logits
        sub["routing_bias"] = torch.zeros(len(used), dtype=torch.bfloat16)
        want = oracle_moe.moe_reference(sub, routing="softmax", act_quant="fp8", dtype=torch.float32)["output"]
        rel = compare.rel_frobenius(out_local[pick.cuda()].cpu(), want)
        record.update(bench_shape_tokens=int(pick.numel()), bench_shape_experts_followed=len(used), bench_shape_rel_frobenius=rel)
        record["ok"] = bool(record["ok"] and record["rel_frobenius"] <= 1e-2 and rel <= 1e-2)
    return record


def moe_parallel(steps, warmup, world, rank, cohorts, exchange):
    import torch.distributed as dist

    import open_cake_ir_b200 as cake
    from open_cake_ir_b200 import ep
    t_local, e_local = SHAPE["tokens"] // world, SHAPE["experts"] // world
    dev = cake.workloads.moe_inputs(tokens=t_local, hidden=SHAPE["hidden"], inter=SHAPE["inter"], experts=SHAPE["experts"],
                                    local_experts=e_local, local_offset=rank * e_local, routing="softmax", device="cuda",
                                    gen_device="cuda", first_token=rank * t_local, total_tokens=SHAPE["tokens"])
    if exchange == "push":
        # the push exchange needs memory every rank can write; where the box cannot give it on every rank the NCCL
        # exchange of this library's pack/unpack kernels is used instead, and the line says so
        try:
            import torch.distributed._symmetric_memory as symm
            probe = symm.empty(4096, dtype=torch.uint8, device="cuda")
            have = 1 if len(symm.rendezvous(probe, group=dist.group.WORLD).buffer_ptrs) == world else 0
        except Exception as error:                      # noqa: BLE001 - any failure means "not available here"
            print(f"bench: symmetric memory unavailable on rank {rank}: {error!r}", file=sys.stderr, flush=True)
            have = 0
        flag = torch.tensor([have], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            exchange = "nccl"

    def build(kind):
        cls = ep.PushExpertParallelMoe if kind == "push" else ep.NativeExpertParallelMoe
        made = cls(dev, dev["routing_logits"], dev["routing_bias"], dev["hidden_states"],
                   dev["hidden_states_scale"], experts=SHAPE["experts"], top_k=SHAPE["top_k"], routing="softmax")
        checked = ep_parity(world, rank, made, dev, cls)
        fine = (rank != 0 or bool(checked.get("ok"))) and not (kind == "push" and made.status())
        return cls, made, checked, fine

    try:
        layer_class, layer, parity, fine = build(exchange)
    except Exception as error:                          # noqa: BLE001 - reported, then the other exchange is tried
        print(f"bench: the {exchange} exchange failed on rank {rank}: {error!r}", file=sys.stderr, flush=True)
        layer_class = layer = None
        parity, fine = {"ok": False, "error": repr(error)}, False
    verdict = torch.tensor([1 if fine else 0], device="cuda")
    dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
    if int(verdict.item()) == 0 and exchange == "push":
        # the push exchange did not hold on this box (a wait ran out, or parity failed): the NCCL form takes over
        if rank == 0:
            print(f"bench: push exchange rejected ({parity}); using the NCCL exchange", file=sys.stderr, flush=True)
        exchange = "nccl"
        layer = None
        layer_class, layer, parity, fine = build(exchange)
        verdict = torch.tensor([1 if fine else 0], device="cuda")
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
    if int(verdict.item()) == 0:
        if rank == 0:
            print(json.dumps({"metric": "fp8_moe_tflops", "ep_parity": parity, "error": "expert-parallel output differs from the oracle"}), flush=True)
        dist.destroy_process_group()
        raise SystemExit(1)
    result = {}

    def step():
        result["out"] = layer.forward()

    step()
    stage_ms = layer.stage_times(max(3, steps // 2))          # eager, events between the parts of one step
    graph = os.environ.get("CAKE_BENCH_NO_GRAPH") != "1"
    if graph:
        layer.capture()                    # one CUDA graph per step: kernels and the exchange
    clocks = ClockSampler(torch.cuda.current_device())
    clocks.__enter__()
    samples = [time_steps(step, steps, warmup if c == 0 else 1, world) for c in range(cohorts)]
    if exchange == "push" and layer.status():
        raise RuntimeError("a wait for another rank's rows ran out")

    def make_set():
        inputs = dict(dev)
        for k in E2E_INPUTS:
            inputs[k] = torch.empty_like(dev[k])
        twin = layer_class(inputs, inputs["routing_logits"], inputs["routing_bias"], inputs["hidden_states"],
                           inputs["hidden_states_scale"], experts=SHAPE["experts"], top_k=SHAPE["top_k"], routing="softmax")

        twin.forward()
        if graph:
            twin.capture()

        def launch(stream):
            with torch.cuda.stream(stream):
                twin.forward()
        return inputs, twin.output, launch

    e2e_step, h2d, d2h = pipelined_e2e(make_set, dev, layer.output)
    e2e_ms = time_steps(e2e_step, steps, warmup, world)
    clocks.__exit__()
    flops = cake.workloads.moe_flops(SHAPE["tokens"], SHAPE["hidden"], SHAPE["inter"])
    return {"ms": statistics.median(samples), "cohorts": cohort_stats(samples), "flops": flops, "clocks": clocks.summary(),
            "e2e_ms": e2e_ms, "h2d": h2d * world, "d2h": d2h * world, "launches": layer.launches_per_step * steps,
            "rows_sent_rank0": layer.rows_sent() if exchange == "push" else int((layer.slot_of >= 0).sum().item()),
            "ep_parity": parity, "stage_ms": stage_ms, "exchange": exchange,
            "step_mode": "one CUDA graph per step" if graph else "eager launches"}


def _timed_cpu(fn, min_seconds=2.0, max_runs=20):
    """Wall seconds per call of a host function, repeated for about ``min_seconds`` after one warm-up."""
    fn()
    runs, t0 = 0, time.perf_counter()
    while True:
        fn()
        runs += 1
        elapsed = time.perf_counter() - t0
        if elapsed >= min_seconds or runs >= max_runs:
            return elapsed / runs, runs


def per_gpu_operators(peaks, with_cpu=True):
    """RMSNorm, block-scaled GEMM, paged GQA and MLA decode at their serving shapes.  Every operator is
    launched back to back over a rotation of buffer sets that together exceed twice the L2 (so inputs come
    from HBM), between one pair of events; algorithmic bytes or flops over the mean launch time.  Each row
    also carries the oracle timed on the host cores over a bounded sample of the same workload."""
    import open_cake_ir_b200 as cake
    from oracle import add_rmsnorm as oracle_add_rmsnorm, attention as oracle_attention, block_scaled_gemm as oracle_gemm, rmsnorm as oracle_rmsnorm
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    rows = []

    # ---- RMSNorm: 67 MB per launch, six buffer sets ----
    sets = []
    for k in range(6):
        inputs, meta = cake.workloads.rmsnorm_inputs(4096, 4096, device="cuda", gen_device="cuda", salt=k)
        out = torch.empty_like(inputs["x"])
        sets.append((inputs, out, cake.RmsNorm(inputs["x"], inputs["weight"], out, meta["epsilon"])))
    ms, stats, launches = time_rotating([op.launch for _, _, op in sets])
    copy_ms, _, _ = time_rotating([(lambda i=i, o=o: o.copy_(i["x"])) for i, o, _ in sets])
    nbytes = 2 * 4096 * 4096 * 2 + 4096 * 2
    row = {"operator": "rmsnorm", "workload": "x bf16 [4096,4096], eps 1e-6", "ms": ms, "samples": stats, "launches_timed": launches,
           "bound": "hbm", "unit": "GB/s", "achieved": nbytes / ms / 1e6, "peak": peaks["hbm_gbs"],
           "frac": nbytes / ms / 1e6 / peaks["hbm_gbs"], "copy_baseline_ms": copy_ms,
           "copy_baseline_note": "torch copy of x into out over the same rotation: the same bytes with no arithmetic",
           "l2": "six buffer sets of 67 MB in rotation (402 MB > 2 x L2)"}
    if with_cpu:
        x, w = sets[0][0]["x"].cpu(), sets[0][0]["weight"].cpu()
        seconds, runs = _timed_cpu(lambda: oracle_rmsnorm.rmsnorm_fast(x, w, 1e-6))
        row["cpu_baseline"] = {"value": nbytes / seconds / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                               "sample": f"the whole 4096x4096 problem, fp64 torch restatement (oracle/rmsnorm.py), {runs} run(s)"}
    rows.append(row)

    # ---- two-output add + RMSNorm: 134 MB per launch; the six inputs above serve as delta / residual of three sets ----
    add_sets = []
    for k in range(3):
        delta, residual, weight = sets[2 * k][0]["x"], sets[2 * k + 1][0]["x"], sets[2 * k][0]["weight"]
        out, residual_out = torch.empty_like(delta), torch.empty_like(delta)
        add_sets.append((out, residual_out, cake.AddRmsNorm(delta, residual, weight, out, residual_out, 1e-6)))
    ms, stats, launches = time_rotating([op.launch for _, _, op in add_sets])
    nbytes = 4 * 4096 * 4096 * 2 + 4096 * 2
    row = {"operator": "add_rmsnorm", "workload": "delta, residual bf16 [4096,4096] -> out, residual_out; eps 1e-6", "ms": ms,
           "samples": stats, "launches_timed": launches, "bound": "hbm", "unit": "GB/s", "achieved": nbytes / ms / 1e6,
           "peak": peaks["hbm_gbs"], "frac": nbytes / ms / 1e6 / peaks["hbm_gbs"],
           "l2": "three buffer sets of 134 MB in rotation (403 MB > 2 x L2)"}
    if with_cpu:
        d, r, w = sets[0][0]["x"].cpu(), sets[1][0]["x"].cpu(), sets[0][0]["weight"].cpu()
        seconds, runs = _timed_cpu(lambda: oracle_add_rmsnorm.add_rmsnorm_reference(d, r, w, 1e-6))
        row["cpu_baseline"] = {"value": nbytes / seconds / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                               "sample": f"the whole 4096x4096 problem, torch restatement (oracle/add_rmsnorm.py), {runs} run(s)"}
    rows.append(row)
    del sets, add_sets

    # ---- block-scaled GEMM: 155 MB per launch, three buffer sets ----
    sets = []
    for k in range(3):
        g = cake.workloads.block_scaled_gemm_inputs(8192, 4096, 7168, device="cuda", gen_device="cuda", salt=k)
        c = torch.empty((8192, 4096), dtype=torch.bfloat16, device="cuda")
        sets.append((g, c, cake.BlockScaledGemm(g["a"], g["sfa"], g["b"], g["sfb"], c)))
    ms, stats, launches = time_rotating([op.launch for _, _, op in sets])
    flops = 2 * 8192 * 4096 * 7168
    fp8_peak = 2 * peaks["bf16_tflops"]
    row = {"operator": "block_scaled_gemm", "workload": "M8192 N4096 K7168 e4m3, 1x128 / 128x128 fp32 scales", "ms": ms,
           "samples": stats, "launches_timed": launches, "bound": "tensor", "unit": "TFLOP/s", "achieved": flops / ms / 1e9,
           "peak": fp8_peak, "peak_note": "2 x measured cuBLAS bf16 burst (fp8 dense is twice the bf16 rate)",
           "frac": flops / ms / 1e9 / fp8_peak, "frac_of_2x_bf16_sustained": flops / ms / 1e9 / (2 * peaks["bf16_tflops_sustained"]),
           "frac_of_nominal_4500": flops / ms / 1e9 / 4500.0, "status": max(op.status() for _, _, op in sets),
           "l2": "three buffer sets of 155 MB in rotation (465 MB > 2 x L2)"}
    if with_cpu:
        g = {k: v.cpu() for k, v in sets[0][0].items()}
        sample_m = 1024
        a, sfa = g["a"][:sample_m].contiguous(), g["sfa"][:, :sample_m].contiguous()
        seconds, runs = _timed_cpu(lambda: oracle_gemm.block_scaled_gemm_reference(a, sfa, g["b"], g["sfb"]), min_seconds=3.0)
        row["cpu_baseline"] = {"value": 2 * sample_m * 4096 * 7168 / seconds / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                               "sample": f"the first {sample_m} of 8192 rows against all of B, dequantise + fp32 matmul "
                                         f"(oracle/block_scaled_gemm.py), {runs} run(s)"}
    rows.append(row)
    del sets

    # ---- paged GQA decode: 620 MB of cache rows per launch, far more than the L2 ----
    dev, meta = cake.workloads.gqa_decode_inputs(device="cuda", gen_device="cuda")
    out = torch.empty_like(dev["q"]); lse = torch.empty((64, 32), dtype=torch.float32, device="cuda")
    op = cake.GqaPagedDecode(dev["q"], dev["k_cache"], dev["v_cache"], dev["kv_indptr"], dev["kv_indices"],
                             dev["kv_last_page_len"], dev["sm_scale"], out, lse, max_kv_len=meta["max_kv_len"])
    ms, stats, launches = time_rotating([op.launch])
    total = int(meta["kv_lens"].sum())
    nbytes = total * 2 * 8 * 128 * 2 + 2 * out.numel() * 2 + lse.numel() * 4 + dev["kv_indices"].numel() * 4
    row = {"operator": "gqa_paged_decode", "workload": f"batch 64, 32/8 heads, d128, page 16, sum kv_len {total}",
           "ms": ms, "samples": stats, "launches_timed": launches, "bound": "hbm", "unit": "GB/s", "achieved": nbytes / ms / 1e6,
           "peak": peaks["hbm_gbs"], "frac": nbytes / ms / 1e6 / peaks["hbm_gbs"],
           "l2": "one buffer set: a launch reads 620 MB of cache rows, five times the L2"}
    if with_cpu:
        n = 4
        cpu = {k: v.cpu() for k, v in dev.items()}
        cpu.update(q=cpu["q"][:n], kv_indptr=cpu["kv_indptr"][:n + 1], kv_last_page_len=cpu["kv_last_page_len"][:n])
        seconds, runs = _timed_cpu(lambda: oracle_attention.paged_decode_reference(cpu, mla=False, page_size=16, per_head_loop=False))
        sample_tokens = int(meta["kv_lens"][:n].sum())
        row["cpu_baseline"] = {"value": sample_tokens * 4096 / seconds / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                               "sample": f"the first {n} of 64 sequences ({sample_tokens} tokens), fp64 oracle (oracle/attention.py), {runs} run(s)"}
        del cpu
    rows.append(row)
    del dev, out, lse, op

    # ---- paged MLA decode: 172 MB per launch, three cache pools ----
    sets = []
    for k in range(3):
        dev, meta = cake.workloads.mla_decode_inputs(device="cuda", gen_device="cuda", salt=k)
        out = torch.empty_like(dev["q_nope"]); lse = torch.empty((32, 128), dtype=torch.float32, device="cuda")
        sets.append((dev, meta, cake.MlaPagedDecode(dev["q_nope"], dev["q_pe"], dev["ckv_cache"], dev["kpe_cache"], dev["kv_indptr"],
                                                    dev["kv_indices"], dev["kv_last_page_len"], dev["sm_scale"], out, lse,
                                                    max_kv_len=meta["max_kv_len"]), out, lse))
    ms, stats, launches = time_rotating([entry[2].launch for entry in sets])
    total = sum(int(entry[1]["kv_lens"].sum()) for entry in sets) / len(sets)
    dev = sets[0][0]
    nbytes = total * 1152 + dev["q_nope"].numel() * 2 + dev["q_pe"].numel() * 2 + sets[0][3].numel() * 2
    flops = total * 128 * 2176
    row = {"operator": "mla_paged_decode", "workload": f"batch 32, 128 heads, ckv 512 + kpe 64, page 64, mean sum kv_len {int(total)}",
           "ms": ms, "samples": stats, "launches_timed": launches, "bound": "hbm", "unit": "GB/s", "achieved": nbytes / ms / 1e6,
           "peak": peaks["hbm_gbs"], "frac": nbytes / ms / 1e6 / peaks["hbm_gbs"], "tflops": flops / ms / 1e9,
           "tensor_frac_of_bf16_burst": flops / ms / 1e9 / peaks["bf16_tflops"],
           "l2": "three cache pools in rotation (3 x 172 MB read per round > 2 x L2)"}
    if with_cpu:
        n = 2
        cpu = {k: v.cpu() for k, v in dev.items()}
        cpu.update(q_nope=cpu["q_nope"][:n], q_pe=cpu["q_pe"][:n], kv_indptr=cpu["kv_indptr"][:n + 1],
                   kv_last_page_len=cpu["kv_last_page_len"][:n])
        seconds, runs = _timed_cpu(lambda: oracle_attention.paged_decode_reference(cpu, mla=True, page_size=64, per_head_loop=False))
        sample_tokens = int(sets[0][1]["kv_lens"][:n].sum())
        row["cpu_baseline"] = {"value": sample_tokens * 1152 / seconds / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                               "sample": f"the first {n} of 32 sequences ({sample_tokens} tokens), fp64 oracle (oracle/attention.py), {runs} run(s)"}
    rows.append(row)
    rows.extend(next_operators(peaks))
    return rows


def next_operators(peaks):
    """The operators next to the headline path (two-output add-RMSNorm is timed above): the DeepSeek-V4 gate and
    indexer top-k, the sparse MLA decode and the causal-prefill forms, at their contracts' shapes or, for prefill, a
    chunk of the size the reference's cases use.  They are microsecond kernels over data that fits in L2, so the
    rows give time and algorithmic GB/s and name the bound as latency; parity is the tests' business."""
    import open_cake_ir_b200 as cake
    rows = []
    g = torch.Generator(device="cuda").manual_seed(7)

    def add(name, workload, op, nbytes):
        ms, stats, launches = time_rotating([op.launch])
        status = op.status() if hasattr(op, "status") else 0
        rows.append({"operator": name, "workload": workload, "ms": ms, "samples": stats, "launches_timed": launches,
                     "bound": "latency", "unit": "GB/s", "achieved": nbytes / ms / 1e6, "peak": peaks["hbm_gbs"],
                     "frac": nbytes / ms / 1e6 / peaks["hbm_gbs"], "status": status,
                     "l2": "one buffer set that fits in L2: a latency-bound kernel, timed back to back"})

    tokens, experts, top_k = 4096, 384, 6
    logits = torch.randn((tokens, experts), generator=g, device="cuda") * 2
    bias = torch.rand(experts, generator=g, device="cuda") * 0.5
    weights = torch.empty((tokens, top_k), dtype=torch.float32, device="cuda")
    ids = torch.empty((tokens, top_k), dtype=torch.int32, device="cuda")
    add("v4_moe_gate", f"router_logits fp32 [{tokens},{experts}], top {top_k}", cake.V4MoeGate(logits, bias, weights, ids, top_k=top_k, route_scale=2.5),
        logits.numel() * 4 + experts * 4 + 2 * tokens * top_k * 4)

    rows_q, candidates, keep = 512, 2048, 1024
    scores = torch.randn((rows_q, candidates), generator=g, device="cuda")
    indices = torch.empty((rows_q, keep), dtype=torch.int32, device="cuda")
    add("csa_topk", f"index_scores fp32 [{rows_q},{candidates}] -> top {keep}", cake.CsaTopk(scores, indices), scores.numel() * 4 + indices.numel() * 4)

    t, heads, pages, page, listed = 64, 16, 512, 64, 2048
    q_nope = (torch.rand((t, heads, 512), generator=g, device="cuda") - 0.5).to(torch.bfloat16)
    q_pe = (torch.rand((t, heads, 64), generator=g, device="cuda") - 0.5).to(torch.bfloat16)
    ckv = torch.randn((pages, page, 512), generator=g, device="cuda").to(torch.bfloat16)
    kpe = torch.randn((pages, page, 64), generator=g, device="cuda").to(torch.bfloat16)
    sparse = torch.stack([torch.randperm(pages * page, generator=g, device="cuda")[:listed] for _ in range(t)]).to(torch.int32)
    out = torch.empty_like(q_nope)
    add("sparse_mla_decode", f"{t} query rows, {heads} heads, {listed} listed cache rows each (page {page})",
        cake.SparseMlaDecode(q_nope, q_pe, ckv, kpe, sparse, out), t * listed * 1152 + 2 * q_nope.numel() * 2 + q_pe.numel() * 2 + sparse.numel() * 4)

    segments, q_len, kv_len, hq, hkv = 4, 32, 512, 32, 8
    page = 16
    total_q, pages_per = segments * q_len, kv_len // page
    q = (torch.rand((total_q, hq, 128), generator=g, device="cuda") - 0.5).to(torch.bfloat16)
    k = torch.randn((segments * pages_per, page, hkv, 128), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((segments * pages_per, page, hkv, 128), generator=g, device="cuda").to(torch.bfloat16)
    qo = torch.arange(0, total_q + 1, q_len, dtype=torch.int32, device="cuda")
    kvp = torch.arange(0, segments * pages_per + 1, pages_per, dtype=torch.int32, device="cuda")
    kv_indices = torch.arange(segments * pages_per, dtype=torch.int32, device="cuda")
    last = torch.full((segments,), page, dtype=torch.int32, device="cuda")
    scale = torch.tensor([128 ** -0.5], device="cuda")
    o = torch.empty_like(q)
    lse = torch.empty((total_q, hq), dtype=torch.float32, device="cuda")
    add("gqa_causal_prefill_paged", f"{segments} segments x {q_len} query rows over {kv_len} KV rows, {hq}/{hkv} heads, page {page}",
        cake.GqaCausalPrefill(q, k, v, qo, kvp, kv_indices, last, scale, o, lse, max_kv_len=kv_len),
        2 * k.numel() * 2 + 2 * q.numel() * 2 + lse.numel() * 4)

    heads, page = 16, 64
    pages_per = kv_len // page
    qn = (torch.rand((total_q, heads, 512), generator=g, device="cuda") - 0.5).to(torch.bfloat16)
    qp = (torch.rand((total_q, heads, 64), generator=g, device="cuda") - 0.5).to(torch.bfloat16)
    ckv2 = torch.randn((segments * pages_per, page, 512), generator=g, device="cuda").to(torch.bfloat16)
    kpe2 = torch.randn((segments * pages_per, page, 64), generator=g, device="cuda").to(torch.bfloat16)
    kvp2 = torch.arange(0, segments * pages_per + 1, pages_per, dtype=torch.int32, device="cuda")
    idx2 = torch.arange(segments * pages_per, dtype=torch.int32, device="cuda")
    last2 = torch.full((segments,), page, dtype=torch.int32, device="cuda")
    scale2 = torch.tensor([0.1352337788608801], device="cuda")
    o2 = torch.empty_like(qn)
    lse2 = torch.empty((total_q, heads), dtype=torch.float32, device="cuda")
    add("mla_causal_prefill_paged", f"{segments} segments x {q_len} query rows over {kv_len} latent rows, {heads} heads, page {page}",
        cake.MlaCausalPrefill(qn, qp, ckv2, kpe2, qo, kvp2, idx2, last2, scale2, o2, lse2, max_kv_len=kv_len),
        segments * kv_len * 1152 + 2 * qn.numel() * 2 + qp.numel() * 2 + lse2.numel() * 4)
    return rows


def profile_case(name: str, launches: int = 3):
    """Runs one small case of one operator a few times and exits: the command to put under ncu.
    Cases keep the serving shapes' per-unit geometry (tokens per expert, heads, page size) with fewer
    units, so that a capture holds a few GB at most and ends by itself."""
    import open_cake_ir_b200 as cake
    if name == "moe":            # 1024 tokens over 64 experts: 128 tokens per expert as at full size, 2.8 GB of weights
        dev = cake.workloads.moe_inputs(tokens=1024, hidden=SHAPE["hidden"], inter=SHAPE["inter"], experts=64, local_experts=64,
                                        routing="softmax", device="cuda", gen_device="cuda")
        out = torch.empty((1024, SHAPE["hidden"]), dtype=torch.bfloat16, device="cuda")
        op = cake.Fp8Moe(dev, out, experts=64, routing="softmax", act_mode="fp8")
    elif name == "gemm":         # half the serving M
        g = cake.workloads.block_scaled_gemm_inputs(4096, 4096, 7168, device="cuda", gen_device="cuda")
        c = torch.empty((4096, 4096), dtype=torch.bfloat16, device="cuda")
        op = cake.BlockScaledGemm(g["a"], g["sfa"], g["b"], g["sfb"], c)
    elif name == "rmsnorm":
        inputs, meta = cake.workloads.rmsnorm_inputs(4096, 4096, device="cuda", gen_device="cuda")
        out = torch.empty_like(inputs["x"])
        op = cake.RmsNorm(inputs["x"], inputs["weight"], out, meta["epsilon"])
    elif name == "gqa":          # the serving batch and lengths (1.3 GB of cache)
        dev, meta = cake.workloads.gqa_decode_inputs(device="cuda", gen_device="cuda")
        out = torch.empty_like(dev["q"]); lse = torch.empty((64, 32), dtype=torch.float32, device="cuda")
        op = cake.GqaPagedDecode(dev["q"], dev["k_cache"], dev["v_cache"], dev["kv_indptr"], dev["kv_indices"],
                                 dev["kv_last_page_len"], dev["sm_scale"], out, lse, max_kv_len=meta["max_kv_len"])
    elif name == "mla":          # the serving batch and lengths (0.3 GB of cache)
        dev, meta = cake.workloads.mla_decode_inputs(device="cuda", gen_device="cuda")
        out = torch.empty_like(dev["q_nope"]); lse = torch.empty((32, 128), dtype=torch.float32, device="cuda")
        op = cake.MlaPagedDecode(dev["q_nope"], dev["q_pe"], dev["ckv_cache"], dev["kpe_cache"], dev["kv_indptr"],
                                 dev["kv_indices"], dev["kv_last_page_len"], dev["sm_scale"], out, lse, max_kv_len=meta["max_kv_len"])
    else:
        raise SystemExit(f"unknown profile case {name}")
    for _ in range(launches):
        op.launch()
    torch.cuda.synchronize()
    if op.status():
        raise SystemExit("a device-side wait ran out")


# ------------------------------------------------------------------------------------------------
CPU_SAMPLE = dict(tokens=4096, local_experts=96, local_offset=0)


def cpu_reference_step(state):
    """One bounded sample of the workload on the host: CPU_SAMPLE["tokens"] tokens routed over all 256
    experts, the contributions of the first CPU_SAMPLE["local_experts"] experts computed by the oracle in
    fp32 on all host threads (an expert-parallel rank's share of the layer)."""
    from oracle import moe as oracle_moe
    t0 = time.perf_counter()
    result = oracle_moe.moe_reference(state["inputs"], routing="softmax", act_quant="fp8", dtype=torch.float32, return_parts=True)
    seconds = time.perf_counter() - t0
    local = (result["expert_ids"] >= CPU_SAMPLE["local_offset"]) & (result["expert_ids"] < CPU_SAMPLE["local_offset"] + CPU_SAMPLE["local_experts"])
    pairs = int(local.sum())
    flops = 2 * pairs * (SHAPE["hidden"] * 2 * SHAPE["inter"] + SHAPE["inter"] * SHAPE["hidden"])
    return flops, seconds


def cpu_state():
    import open_cake_ir_b200 as cake
    torch.set_num_threads(os.cpu_count() or 1)
    inputs = cake.workloads.moe_inputs(tokens=CPU_SAMPLE["tokens"], hidden=SHAPE["hidden"], inter=SHAPE["inter"],
                                       experts=SHAPE["experts"], local_experts=CPU_SAMPLE["local_experts"],
                                       local_offset=CPU_SAMPLE["local_offset"], routing="softmax", device="cpu")
    return {"inputs": inputs}


def cpu_baseline(steps=1, warmup=0):
    state = cpu_state()
    for _ in range(warmup):
        cpu_reference_step(state)
    flops = seconds = 0.0
    for _ in range(steps):
        f, s = cpu_reference_step(state)
        flops += f; seconds += s
    return {"value": flops / seconds / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{CPU_SAMPLE['tokens']} tokens routed over 256 experts, contributions of {CPU_SAMPLE['local_experts']} experts, "
                      f"fp32 oracle (oracle/moe.py), {steps} pass(es), {seconds:.1f} s",
            "seconds": seconds}


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base = cpu_baseline(steps=max(1, args.steps), warmup=min(1, args.warmup))
    ms = base["seconds"] / max(1, args.steps) * 1e3
    line = {"impl": "reference", "metric": "fp8_moe_tflops", "value": base["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32 host arithmetic over e4m3 inputs", "data": "synthetic",
            "config": {"workload": WORKLOAD, "note": "reference CPU oracle arithmetic on a bounded sample of the workload"},
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": base["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--cohorts", type=int, default=3, help="repetitions of the timed region of --steps steps")
    parser.add_argument("--impl", default="native", choices=["native", "reference"])
    parser.add_argument("--exchange", default="push", choices=["push", "nccl"],
                        help="expert-parallel exchange: ranks write into each other's memory (push) or NCCL all-to-all")
    parser.add_argument("--skip-operators", action="store_true", help="time only the MoE layer")
    parser.add_argument("--skip-cpu", action="store_true", help="do not time the CPU baselines")
    parser.add_argument("--profile-case", default=None, choices=["moe", "gemm", "rmsnorm", "gqa", "mla"],
                        help="launch one small case of one operator three times and exit (for ncu)")
    args = parser.parse_args()
    if args.profile_case:
        profile_case(args.profile_case)
        return
    if args.impl == "reference":
        reference_arm(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the native path has no CPU fallback")
    world, rank, _ = dist_setup(args.gpus)
    peaks = measured_peaks()
    warmup = max(3, args.warmup)
    cohorts = max(1, args.cohorts)
    operators = None
    if world == 1 and not args.skip_operators:
        # before the layer's long timed regions: a kernel timed alone is compared with the burst peaks
        with ClockSampler(torch.cuda.current_device()) as sampler:
            operators = per_gpu_operators(peaks, with_cpu=not args.skip_cpu)
        operators_clocks = sampler.summary()
    if world == 1:
        r = moe_single(args.steps, warmup, peaks, cohorts)
    else:
        r = moe_parallel(args.steps, warmup, world, rank, cohorts, args.exchange)
    line = {"metric": "fp8_moe_tflops", "value": r["flops"] / (r["ms"] * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": r["ms"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": WORKLOAD, "parallelism": f"ep{world}", "tokens_per_rank": SHAPE["tokens"] // world,
                       "experts_per_rank": SHAPE["experts"] // world,
                       "l2": "inputs larger than L2 (expert weights 11.3 GB over all ranks)",
                       "step_mode": r.get("step_mode", "eager launches")},
            "cohorts": r["cohorts"], "clocks": r["clocks"],
            "e2e": {"value": r["flops"] / (r["e2e_ms"] * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": r["e2e_ms"],
                    "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"]},
            "gpu_launches": r["launches"] * cohorts,
            "pct_of_fp8_nominal_peak": r["flops"] / (r["ms"] * 1e-3) / 1e12 / (4500.0 * world),
            "stage_ms": r["stage_ms"]}
    if world == 1:
        line["roofline"] = r["roofline"]
        line["stage_cycles"] = r["stage_cycles"]
        weight_bytes = SHAPE["experts"] * 3 * SHAPE["inter"] * SHAPE["hidden"]
        line["layer_hbm_floor_ms"] = weight_bytes / (peaks["hbm_gbs"] * 1e9) * 1e3
        line["contract_mode"] = r["contract_mode"]
        line["compute_bound"] = moe_compute_bound(args.steps, peaks)
        if operators is not None:
            line["operators"] = operators
            line["operators_clocks"] = operators_clocks
        if not args.skip_cpu:
            base = cpu_baseline(steps=3)
            line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
    else:
        line["rows_sent_rank0"] = r["rows_sent_rank0"]
        line["config"]["exchange"] = ("rows written into the owner's memory over NVLink by this library's kernels" if r["exchange"] == "push"
                                      else "NCCL all-to-all, equal splits")
        line["ep_parity"] = r["ep_parity"]
        line["config"]["host_cpus_rank0"] = HOST_BINDING["cpus"] or "as started"
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
