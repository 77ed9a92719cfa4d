"""Benchmark of the hot path on B200.

``python bench.py --gpus N --steps K --warmup W`` prints ONE JSON line.  A step is one pass of
the FP8 block-scaled MoE expert layer at the DeepSeek-V3 shape (4096 tokens, hidden 7168, 256
experts, top-8, intermediate 2048; softmax top-k routing; e4m3 activations with 1x128 scales)
over synthetic inputs; with N > 1 (launched by torch.distributed.run) the layer is
expert-parallel: 4096/N tokens and 256/N experts per rank, all-to-all dispatch and combine over
NCCL, and ``value`` is the whole job's TFLOP/s (total work fixed: strong scaling).

``value``  : inputs resident in HBM before the timed region (CUDA events, barrier + synchronize on
             both sides, max over ranks).
``e2e``    : the same metric through the public Python API with HOST buffers: every step copies
             the step's activations and router logits from pinned memory to the device and reads
             the bf16 output back; expert weights are model state and stay resident.
``roofline``: the dominant kernel (grouped GEMM1 + SwiGLU), algorithmic bytes / CUDA-event time
             against the measured HBM copy bandwidth.
``cpu_baseline`` / ``--impl reference``: the reference's CPU oracle arithmetic for the same layer
             (oracle/moe.py, a restatement pinned bit-for-bit to the reference's oracle), timed on
             the host cores over a bounded sample of the workload.
The four per-GPU operators (RMSNorm, block-scaled GEMM, paged GQA / MLA decode) are timed at N = 1
and reported under ``operators``.
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


def dist_setup(n_gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
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


_flush = None


def flush_l2():
    """Evicts L2 (126 MB) by overwriting a 512 MB buffer."""
    global _flush
    if _flush is None:
        _flush = torch.empty(512 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def time_cold(launch, iters: int, warmup: int) -> float:
    """Mean milliseconds of `launch` alone with L2 flushed before every timed launch."""
    for _ in range(warmup):
        launch()
    times = []
    for _ in range(iters):
        flush_l2()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(); launch(); stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop))
    return statistics.mean(times)


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
def moe_single(steps, warmup, peaks):
    import open_cake_ir_b200 as cake
    dev = cake.workloads.moe_inputs(tokens=SHAPE["tokens"], hidden=SHAPE["hidden"], inter=SHAPE["inter"],
                                    experts=SHAPE["experts"], local_experts=SHAPE["experts"], local_offset=0,
                                    routing="softmax", device="cuda", gen_device="cuda")
    out = torch.empty((SHAPE["tokens"], SHAPE["hidden"]), dtype=torch.bfloat16, device="cuda")
    op = cake.Fp8Moe(dev, out, routing="softmax", act_mode="fp8")
    flops = cake.workloads.moe_flops(SHAPE["tokens"], SHAPE["hidden"], SHAPE["inter"])
    clocks = ClockSampler(torch.cuda.current_device())
    clocks.__enter__()                     # sampled until the end-to-end loop below has finished
    ms = time_steps(op.launch, steps, warmup, 1)
    if op.status():
        raise RuntimeError("a device-side wait ran out")
    # stage timing (inputs 11 GB >> L2, so consecutive launches are cold anyway)
    stage_ms = [0.0] * 4
    events = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(steps)]
    for k in range(steps):
        events[k][0].record()
        for s in range(4):
            op.launch_stage(s)
            events[k][s + 1].record()
    torch.cuda.synchronize()
    for k in range(steps):
        for s in range(4):
            stage_ms[s] += events[k][s].elapsed_time(events[k][s + 1]) / steps
    pairs = SHAPE["tokens"] * SHAPE["top_k"]
    gemm1_bytes = SHAPE["experts"] * 2 * SHAPE["inter"] * SHAPE["hidden"] + pairs * (SHAPE["hidden"] + SHAPE["inter"])
    achieved = gemm1_bytes / (stage_ms[1] * 1e-3) / 1e9
    roofline = {"kernel": "gemm_fp8_kernel<kGateUp> (grouped GEMM1 + SwiGLU + e4m3 requantisation)", "bound": "hbm",
                "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "peak_source": peaks["source"], "algorithmic_bytes": gemm1_bytes, "ms": stage_ms[1],
                # dram__bytes_read + write per launch: captured by ncu on --profile-case moe (64 experts, 1024 tokens:
                # 1.961 GB against 1.954 GB algorithmic) and scaled by the number of experts, every expert's weights
                # being read once (profiles/gemm_fp8_kernel_ncu_full.md)
                "traffic": int(gemm1_bytes * 1.004), "traffic_source": "ncu small case x units",
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
    return {"ms": ms, "flops": flops, "clocks": clocks.summary(), "stage_ms": dict(zip(cake.Fp8Moe.STAGES, stage_ms)),
            "roofline": roofline, "e2e_ms": e2e_ms, "h2d": h2d, "d2h": d2h, "launches": 8 * steps}


def moe_parallel(steps, warmup, world, rank):
    import open_cake_ir_b200 as cake
    from open_cake_ir_b200 import ep
    t_local, e_local = SHAPE["tokens"] // world, SHAPE["experts"] // world
    dev = cake.workloads.moe_inputs(tokens=t_local, hidden=SHAPE["hidden"], inter=SHAPE["inter"], experts=SHAPE["experts"],
                                    local_experts=e_local, local_offset=rank * e_local, routing="softmax", device="cuda",
                                    gen_device="cuda", first_token=rank * t_local, total_tokens=SHAPE["tokens"])
    layer = ep.NativeExpertParallelMoe(dev, dev["routing_logits"], dev["routing_bias"], dev["hidden_states"],
                                       dev["hidden_states_scale"], experts=SHAPE["experts"], top_k=SHAPE["top_k"],
                                       routing="softmax")
    result = {}

    def step():
        result["out"] = layer.forward()

    step()
    if os.environ.get("CAKE_BENCH_NO_GRAPH") != "1":
        layer.capture()                    # one CUDA graph per step: kernels + both all-to-alls
    clocks = ClockSampler(torch.cuda.current_device())
    clocks.__enter__()
    ms = time_steps(step, steps, warmup, world)
    def make_set():
        inputs = dict(dev)
        for k in E2E_INPUTS:
            inputs[k] = torch.empty_like(dev[k])
        twin = ep.NativeExpertParallelMoe(inputs, inputs["routing_logits"], inputs["routing_bias"], inputs["hidden_states"],
                                          inputs["hidden_states_scale"], experts=SHAPE["experts"], top_k=SHAPE["top_k"],
                                          routing="softmax")

        twin.forward()
        if os.environ.get("CAKE_BENCH_NO_GRAPH") != "1":
            twin.capture()

        def launch(stream):
            with torch.cuda.stream(stream):
                twin.forward()
        return inputs, twin.output, launch

    e2e_step, h2d, d2h = pipelined_e2e(make_set, dev, layer.output)
    e2e_ms = time_steps(e2e_step, steps, warmup, world)
    clocks.__exit__()
    flops = cake.workloads.moe_flops(SHAPE["tokens"], SHAPE["hidden"], SHAPE["inter"])
    return {"ms": ms, "flops": flops, "clocks": clocks.summary(), "e2e_ms": e2e_ms, "h2d": h2d * world, "d2h": d2h * world,
            "launches": layer.launches_per_step * steps,
            "rows_sent_rank0": int((layer.slot_of >= 0).sum().item())}


def per_gpu_operators(peaks, iters=20, warmup=3):
    """RMSNorm, block-scaled GEMM, paged GQA and MLA decode at their serving shapes, L2 flushed before
    every timed launch; algorithmic bytes or flops over the CUDA-event time."""
    import open_cake_ir_b200 as cake
    rows = []
    inputs, meta = cake.workloads.rmsnorm_inputs(4096, 4096, device="cuda", gen_device="cuda")
    out = torch.empty_like(inputs["x"])
    op = cake.RmsNorm(inputs["x"], inputs["weight"], out, meta["epsilon"])
    ms = time_cold(op.launch, iters, warmup)
    nbytes = 2 * 4096 * 4096 * 2 + 4096 * 2
    rows.append({"operator": "rmsnorm", "workload": "x bf16 [4096,4096], eps 1e-6", "ms": ms, "bound": "hbm", "unit": "GB/s",
                 "achieved": nbytes / ms / 1e6, "peak": peaks["hbm_gbs"], "frac": nbytes / ms / 1e6 / peaks["hbm_gbs"]})
    del inputs, out, op

    g = cake.workloads.block_scaled_gemm_inputs(8192, 4096, 7168, device="cuda", gen_device="cuda")
    c = torch.empty((8192, 4096), dtype=torch.bfloat16, device="cuda")
    op = cake.BlockScaledGemm(g["a"], g["sfa"], g["b"], g["sfb"], c)
    ms = time_cold(op.launch, iters, warmup)
    flops = 2 * 8192 * 4096 * 7168
    fp8_peak = 2 * peaks["bf16_tflops"]
    rows.append({"operator": "block_scaled_gemm", "workload": "M8192 N4096 K7168 e4m3, 1x128 / 128x128 fp32 scales", "ms": ms,
                 "bound": "tensor", "unit": "TFLOP/s", "achieved": flops / ms / 1e9, "peak": fp8_peak,
                 "peak_note": "2 x measured cuBLAS bf16 burst (fp8 dense is twice the bf16 rate)",
                 "frac": flops / ms / 1e9 / fp8_peak, "frac_of_nominal_4500": flops / ms / 1e9 / 4500.0, "status": op.status()})
    del g, c, op

    dev, meta = cake.workloads.gqa_decode_inputs(device="cuda", gen_device="cuda")
    out = torch.empty_like(dev["q"]); lse = torch.empty((64, 32), dtype=torch.float32, device="cuda")
    op = cake.GqaPagedDecode(dev["q"], dev["k_cache"], dev["v_cache"], dev["kv_indptr"], dev["kv_indices"],
                             dev["kv_last_page_len"], dev["sm_scale"], out, lse, max_kv_len=meta["max_kv_len"])
    ms = time_cold(op.launch, iters, warmup)
    total = int(meta["kv_lens"].sum())
    nbytes = total * 2 * 8 * 128 * 2 + 2 * out.numel() * 2 + lse.numel() * 4 + dev["kv_indices"].numel() * 4
    rows.append({"operator": "gqa_paged_decode", "workload": f"batch 64, 32/8 heads, d128, page 16, sum kv_len {total}",
                 "ms": ms, "bound": "hbm", "unit": "GB/s", "achieved": nbytes / ms / 1e6, "peak": peaks["hbm_gbs"],
                 "frac": nbytes / ms / 1e6 / peaks["hbm_gbs"]})
    del dev, out, lse, op

    dev, meta = cake.workloads.mla_decode_inputs(device="cuda", gen_device="cuda")
    out = torch.empty_like(dev["q_nope"]); lse = torch.empty((32, 128), dtype=torch.float32, device="cuda")
    op = cake.MlaPagedDecode(dev["q_nope"], dev["q_pe"], dev["ckv_cache"], dev["kpe_cache"], dev["kv_indptr"],
                             dev["kv_indices"], dev["kv_last_page_len"], dev["sm_scale"], out, lse, max_kv_len=meta["max_kv_len"])
    ms = time_cold(op.launch, iters, warmup)
    total = int(meta["kv_lens"].sum())
    nbytes = total * 1152 + dev["q_nope"].numel() * 2 + dev["q_pe"].numel() * 2 + out.numel() * 2
    flops = total * 128 * 2176
    rows.append({"operator": "mla_paged_decode", "workload": f"batch 32, 128 heads, ckv 512 + kpe 64, page 64, sum kv_len {total}",
                 "ms": ms, "bound": "hbm", "unit": "GB/s", "achieved": nbytes / ms / 1e6, "peak": peaks["hbm_gbs"],
                 "frac": nbytes / ms / 1e6 / peaks["hbm_gbs"], "tflops": flops / ms / 1e9,
                 "tensor_frac_of_bf16_burst": flops / ms / 1e9 / peaks["bf16_tflops"]})
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
    parser.add_argument("--impl", default="native", choices=["native", "reference"])
    parser.add_argument("--skip-operators", action="store_true", help="time only the MoE layer")
    parser.add_argument("--skip-cpu", action="store_true", help="do not time the CPU baseline")
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
    if world == 1:
        r = moe_single(args.steps, warmup, peaks)
    else:
        r = moe_parallel(args.steps, warmup, world, rank)
    line = {"metric": "fp8_moe_tflops", "value": r["flops"] / (r["ms"] * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": r["ms"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": WORKLOAD, "parallelism": f"ep{world}", "tokens_per_rank": SHAPE["tokens"] // world,
                       "experts_per_rank": SHAPE["experts"] // world,
                       "l2": "inputs larger than L2 (expert weights 11.3 GB over all ranks)"},
            "clocks": r["clocks"],
            "e2e": {"value": r["flops"] / (r["e2e_ms"] * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": r["e2e_ms"],
                    "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"]},
            "gpu_launches": r["launches"],
            "pct_of_fp8_nominal_peak": r["flops"] / (r["ms"] * 1e-3) / 1e12 / (4500.0 * world)}
    if world == 1:
        line["roofline"] = r["roofline"]
        line["stage_ms"] = r["stage_ms"]
        weight_bytes = SHAPE["experts"] * 3 * SHAPE["inter"] * SHAPE["hidden"]
        line["layer_hbm_floor_ms"] = weight_bytes / (peaks["hbm_gbs"] * 1e9) * 1e3
        if not args.skip_operators:
            line["operators"] = per_gpu_operators(peaks)
        if not args.skip_cpu:
            base = cpu_baseline(steps=3)         # about 11 s of host work on the 16 cores of a GPU box
            line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
    else:
        line["rows_sent_rank0"] = r["rows_sent_rank0"]
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
