"""Benchmark of the render-to-observation path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one pass of the hot path over one batch of lanes: every lane of the
rank is rendered (walls, visplanes, sprites, weapon, area resize) and its 84x84
frame is pushed onto the four-frame stack.  Workload at every N: 4096 lanes per
GPU on the seeded 64-sector map with 12 things per lane (the configuration the
headline metric is quoted on); lane states are synthetic, resident in HBM, and
advanced between steps by the built-in lane stepper outside the timed region.
With N>1 (torchrun, one rank per GPU) every rank owns its own 4096 lanes (weak
scaling, no collective on the render path; the per-lane statistics are
all-gathered every 100 steps).

Prints one JSON line: `value` is whole-job frames/s with inputs resident on the
device; `e2e` is the same through the host-buffer entry point (host records in,
newest frames out, stream synchronised every step); `roofline` relates the
algorithmic bytes of one launch to its measured duration and to the measured
copy bandwidth of the GPU; `cpu_baseline` times the CPU port on a bounded
sample; `whole_step` drives the lanes through the environment API for context.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import threading
import time
from concurrent.futures import ThreadPoolExecutor

import numpy as np

import __graft_entry__ as entry

LANES_PER_GPU = 4096
THINGS = 12
WORKLOAD = "c2"
METRIC = "rendered env-frames/sec at 4096 lanes/GPU"
UNIT = "frames/s"
# algorithmic HBM bytes per env-frame: newest 84x84 slot + 64 B lane scalars + 16 B per thing
BYTES_PER_FRAME = 84 * 84 + 64 + 16 * THINGS
# The headline workload is c2.  --workload selects the other GPU configurations of the benchmark
# definition: c3 also streams the 320x240 RGB24 frame of every lane every step, c4 is the 256-sector
# map with diagonal lines at 8192 lanes and 32 things per lane.
WORKLOADS = {
    "c2": {"lanes": 4096, "things": 12, "rgb": False, "map": "64-sector 8x8 map"},
    "c3": {"lanes": 1024, "things": 12, "rgb": True, "map": "32-sector 4x8 map"},
    "c4": {"lanes": 8192, "things": 32, "rgb": False, "map": "256-sector 16x16 map with diagonals"},
}
PROFILE_FACTS = os.path.join(entry.ROOT, "profiles", "gd_render_kernel_c2_counters.json")


def kernel_sources_hash():
    import importlib.util

    spec = importlib.util.spec_from_file_location("gd_build", os.path.join(entry.PACKAGE_DIR, "csrc", "build.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module.sources_hash()


def recorded_counters(stack_policy):
    """ncu counters of one 4096-lane launch recorded under profiles/ (DRAM bytes per launch, L2 hit
    rate), or Nones when the record was taken on other kernel sources than the ones in the tree."""

    try:
        with open(PROFILE_FACTS) as f:
            facts = json.load(f)
    except (OSError, ValueError):
        return None, None, "no record under profiles/"
    if facts.get("sources_sha256") != kernel_sources_hash():
        return None, None, "the record under profiles/ was taken on other kernel sources"
    entry_ = facts.get(stack_policy, {})
    return entry_.get("dram_bytes_per_launch_4096_lanes"), facts.get("l2_hit_rate"), \
        "profiles/" + os.path.basename(PROFILE_FACTS)


def measured_peaks():
    path = os.path.join(entry.ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle samples while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows = []
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        inside = [r for t, r in self.rows if t0 <= t <= t1] or [r for _, r in self.rows]
        sm, reasons, sm_max = [], set(), None
        for r in inside:
            try:
                sm.append(float(r[1]))
                sm_max = float(r[2])
            except (ValueError, IndexError):
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": sm_max, "reasons": sorted(reasons),
                "samples": len(inside)}


def cpu_baseline(blob, lanes, things, oracle, seconds=12.0, threads=1):
    """Time the CPU port of the path on a bounded sample of the same workload."""

    chunk = 32
    done = 0
    t0 = time.perf_counter()

    def work(i):
        sl = slice(i * chunk, (i + 1) * chunk)
        oracle.render(blob, lanes[sl], things[sl], mask_hud=True, stage_mask=oracle.STAGE_WALLS
                      | oracle.STAGE_SPRITES | oracle.STAGE_WEAPON)
        return chunk

    n_chunks = lanes.shape[0] // chunk
    with ThreadPoolExecutor(max_workers=threads) as pool:
        i = 0
        while i < n_chunks and time.perf_counter() - t0 < seconds:
            batch = list(range(i, min(i + threads, n_chunks)))
            done += sum(pool.map(work, batch))
            i += len(batch)
    dt = time.perf_counter() - t0
    return done / dt, done, dt


def median_rate(call, units, warmup, repeats, steps):
    """Median of `repeats` samples of units/s, each over `steps` calls, after `warmup` calls."""

    for _ in range(warmup):
        call()
    samples = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        for _ in range(steps):
            call()
        samples.append(units * steps / (time.perf_counter() - t0))
    return statistics.median(samples), samples


def upstream_cpu_numbers(cores, workload, lanes_sample, steps, warmup):
    """The upstream Torch engine on the host cores (installed under oracle/_ref by build()):
    the five figures of the CPU configuration (16-sector map, 4 lanes, uniform actions) with a
    shortened warm-up / median protocol, and the render of `lanes_sample` lanes of `workload`."""

    import sys

    import torch

    sys.path.insert(0, os.path.join(entry.ROOT, "oracle"))
    sys.path.insert(0, os.path.join(entry.ROOT, "tests", "golden"))
    import ref_engine

    if ref_engine.source_dir() is None:
        return None
    import make_golden

    eng, scn, act = ref_engine.load_reference()
    from gradoom_b200 import scene as gdscene

    torch.set_num_threads(cores)
    am = make_golden.action_matrix(act)
    out = {"cores": cores, "torch": torch.__version__,
           "protocol": "3 warm-up calls, median of 3 samples x 5 calls (the upstream tool uses 20 + 5 x 100)"}

    def note(text):
        print(f"[reference arm] {text}", file=sys.stderr, flush=True)

    def engine(config, n, k, renderer):
        note(f"upstream engine: {config}, {n} lanes, {renderer} renderer")
        sc = gdscene.make_grid_scene(gdscene.GRID_CONFIGS[config])
        e, _g = make_golden.make_engine(eng, scn, sc, n, k, seed=1234)
        if renderer == "approximate":
            del e.render_frame                  # the constructor default of the upstream environment
        return e

    g = torch.Generator().manual_seed(make_golden.ACTION_SEED)
    for renderer in ("approximate", "reference"):
        e = engine("c1", 4, 4, renderer)
        n = 4

        def step():
            _f, _r, term, trunc = e.step(am[torch.randint(0, 17, (n,), generator=g)])
            done = term | trunc
            if bool(done.any()):
                e.reset(done, torch.arange(n) + 77)

        rate, samples = median_rate(step, n, 3, 3, 5)
        note(f"step loop: {rate:.2f} frames/s")
        out[f"c1_step_loop_{renderer}"] = {"frames_per_s": rate, "samples": samples}
        if renderer == "approximate":
            rate, samples = median_rate(lambda: type(e).render_frame(e), n, 3, 3, 5)
            out["c1_render_frame_approximate"] = {"frames_per_s": rate, "samples": samples}
        else:
            rate, samples = median_rate(e.render_reference_frame, n, 1, 3, 3)
            out["c1_render_reference_frame"] = {"frames_per_s": rate, "samples": samples}
            rate, samples = median_rate(lambda: e.render_native_frame(include_hud=True), n, 1, 3, 3)
            out["c1_render_native_frame_hud"] = {"frames_per_s": rate, "samples": samples}
    e = engine(workload, lanes_sample, WORKLOADS[workload]["things"], "reference")
    times = []
    for k in range(warmup + steps):
        t0 = time.perf_counter()
        e.render_reference_frame()
        if k >= warmup:
            times.append(time.perf_counter() - t0)
    out["headline"] = {"frames_per_s": lanes_sample * len(times) / sum(times), "lanes": lanes_sample,
                       "calls": len(times), "seconds": sum(times)}
    return out


def run_reference(args):
    """The reference arm: the upstream's own CPU implementation of the path on all host
    threads.  `value` is the upstream Torch engine's render_reference_frame on a bounded
    sample of the workload's lanes (oracle/_ref, installed by build()); beside it the C
    restatement of the same pipeline (the oracle) over all lanes of the workload, and the
    five figures of the upstream's CPU configuration.  Without an installed upstream the
    C restatement is the value."""

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    entry.load_package()
    from gradoom_b200 import scene as gdscene, stepper

    oracle = entry.load_oracle()
    workload = args.workload
    spec = WORKLOADS[workload]
    THINGS = spec["things"]
    sc = gdscene.make_grid_scene(gdscene.GRID_CONFIGS[workload])
    blob = gdscene.pack_scene(sc)
    cores = len(os.sched_getaffinity(0))
    # the C restatement over the lanes of one full step of the workload
    sample = min(spec["lanes"], 4096)
    lanes, things = stepper.random_lanes(sc, sample, THINGS, seed=11)
    port_steps = max(min(args.steps, 3), 1)
    times = []
    for step in range(1 + port_steps):
        stepper.advance(sc, lanes, seed=step)
        t0 = time.perf_counter()
        chunk = 16
        with ThreadPoolExecutor(max_workers=cores) as pool:
            list(pool.map(lambda i: oracle.render(blob, lanes[i:i + chunk], things[i:i + chunk], mask_hud=True,
                                                  stage_mask=7), range(0, sample, chunk)))
        if step >= 1:
            times.append(time.perf_counter() - t0)
    port_value = sample * len(times) / sum(times)
    port = {"value": port_value, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"all {sample} lanes of a {workload} step x {len(times)} steps, {cores} threads"}
    upstream = None if args.skip_upstream else upstream_cpu_numbers(cores, workload, 4, max(min(args.steps, 8), 1),
                                                                     min(args.warmup, 1))
    if upstream is not None:
        value = upstream["headline"]["frames_per_s"]
        ms_per_step = 1000.0 * upstream["headline"]["seconds"] / upstream["headline"]["calls"]
        baseline = {"value": value, "unit": UNIT, "cores": cores, "kind": "reference",
                    "sample": f"upstream render_reference_frame (torch {upstream['torch']}, device=cpu), 4 lanes of the "
                              f"{workload} map per call x {upstream['headline']['calls']} calls"}
        sample_text = f"4 of {spec['lanes']} lanes per step"
    else:
        value, ms_per_step, baseline = port_value, 1000.0 * sum(times) / len(times), port
        sample_text = f"{sample} of {spec['lanes']} lanes per step"
    line = {
        "impl": "reference", "metric": METRIC if workload == WORKLOAD else
        f"rendered env-frames/sec at {spec['lanes']} lanes/GPU ({workload})", "value": value, "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "i64+f32", "data": "synthetic",
        "config": {"workload": f"{workload}: {spec['lanes']} lanes/GPU, {spec['map']}, {THINGS} things/lane, "
                               + ("obs and RGB24 frame every step" if spec["rgb"] else "obs only"),
                   "lanes_per_gpu": spec["lanes"], "sample": sample_text, "l2": "n/a (CPU)"},
        "cpu_baseline": baseline, "cpu_port": port, "upstream_cpu": upstream,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "host_cores": cores,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist

    entry.load_package()
    from gradoom_b200 import native, scene as gdscene, stats, stepper

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    if args.gpus != world and rank == 0 and world > 1:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")

    workload = args.workload
    spec = WORKLOADS[workload]
    THINGS = spec["things"]
    import dataclasses

    grid = gdscene.GRID_CONFIGS[workload]
    sc = gdscene.make_grid_scene(dataclasses.replace(grid, decals=True) if args.decals > 0 else grid)
    blob = gdscene.pack_scene(sc)
    n = args.lanes if args.lanes else spec["lanes"]
    # every rank draws the same seeded lane population (its lanes differ only in their global ids), so
    # that the ranks' times measure the machine and not the seeds
    producer = stepper.LaneStepper(sc, n, device=device, k_things=THINGS, max_things=THINGS, seed=1000)
    renderer = native.Renderer(blob, device, THINGS)
    producer.bind_renderer(renderer)          # the players' kinematics run in the renderer's library
    stack = torch.zeros((n, 4, 84, 84), dtype=torch.uint8, device=device)
    rgb = torch.empty((n, 240, 320, 3), dtype=torch.uint8, device=device) if spec["rgb"] else None
    # timed leg: the reference's contiguous rolled stack (what GraDoomVecEnv hands out by default);
    # --stack-policy ring times the mirrored eight-slot ring (no old frame is moved) instead
    use_ring = args.stack_policy == "ring" and rgb is None
    ring = torch.zeros((n, 8, 84, 84), dtype=torch.uint8, device=device) if use_ring else None
    ring_head = 3

    def render_step():
        nonlocal ring_head
        if use_ring:
            ring_head = (ring_head + 1) & 3
            renderer.step_ring(lanes, things, ring, ring_head)
        elif rgb is None:
            renderer.step(lanes, things, stack)
        else:
            renderer.step_frames(lanes, things, stack, rgb=rgb)

    everyone = torch.ones(n, dtype=torch.bool, device=device)
    lane_ids = torch.arange(n, device=device, dtype=torch.int64) + rank * n
    producer.reset(everyone, lane_ids + 1)
    lanes, things = producer.render_inputs()
    if args.decals > 0:
        rings = stepper.random_decals(sc, lanes.cpu().numpy(), min(args.decals, 64), 64, seed=5)
        renderer.bind_decals(torch.from_numpy(rings).to(device))
    renderer.reset(lanes, things, everyone, stack)
    if use_ring:
        renderer.reset_ring(lanes, things, everyone, ring)
    actions = torch.randint(0, 17, (args.warmup + 2 * args.steps + 8, n), device=device,
                            generator=torch.Generator(device=device).manual_seed(20260813))
    from gradoom_b200.env import action_matrix

    buttons = action_matrix(device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)   # > 126 MB L2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    step_index = 0

    def advance():
        nonlocal step_index
        producer.step(buttons[actions[step_index % actions.shape[0]]])
        step_index += 1

    for _ in range(args.warmup):
        advance()
        render_step()
    barrier()

    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    gathered = None
    gather_every = min(100, args.steps)        # the statistics collective, once per 100 steps (or per run)
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gather_us = None
    barrier()
    wall0 = time.time()
    launches0 = renderer.launches
    for k in range(args.steps):
        advance()
        flush.fill_(k & 0xFF)                 # evict the previous step's stack and records from L2
        starts[k].record()
        render_step()
        ends[k].record()
        if (k + 1) % gather_every == 0:
            gathered = stats.gather_lane_stats(producer.signal_buffer)
    barrier()
    wall1 = time.time()
    if gathered is not None:
        # the collective alone: inside the loop its duration would mostly be the wait for the slowest
        # rank (the ranks drift apart by a fraction of a millisecond per step), so it is timed once
        # more here, right after a barrier
        g0.record()
        stats.gather_lane_stats(producer.signal_buffer)
        g1.record()
        torch.cuda.synchronize(device)
        gather_us = 1000.0 * g0.elapsed_time(g1)
    kernel_ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    launches = renderer.launches - launches0
    renderer.check_status()
    clocks = sampler.stop(wall0, wall1)
    elapsed_ms = torch.tensor([sum(kernel_ms)], dtype=torch.float64, device=device)
    per_rank_ms = [float(elapsed_ms.item()) / args.steps]
    if world > 1:
        every = [torch.zeros_like(elapsed_ms) for _ in range(world)]
        dist.all_gather(every, elapsed_ms)
        per_rank_ms = [float(t.item()) / args.steps for t in every]
        dist.all_reduce(elapsed_ms, op=dist.ReduceOp.MAX)
    total_ms = float(elapsed_ms.item())
    value = world * n * args.steps / (total_ms / 1000.0)
    sum_of_rank_rates = sum(n / (ms / 1000.0) for ms in per_rank_ms)

    # end to end through the host-buffer entry point: pinned records in, newest frames out
    host_lanes = torch.empty(lanes.shape, dtype=torch.int32).pin_memory()
    host_things = torch.empty(things.shape, dtype=torch.int32).pin_memory()
    host_obs = torch.empty((n, 84, 84), dtype=torch.uint8).pin_memory()
    dev_lanes, dev_things = torch.empty_like(lanes), torch.empty_like(things)
    pool = []
    for _ in range(4):
        advance()
        pool.append((lanes.cpu().clone(), things.cpu().clone()))
    e2e_steps = max(args.steps, 3)
    for w in range(2):
        host_lanes.copy_(pool[w % 4][0]); host_things.copy_(pool[w % 4][1])
        renderer.step_host(host_lanes, host_things, dev_lanes, dev_things, stack, host_obs)
    barrier()
    t0 = time.perf_counter()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for k in range(e2e_steps):
        host_lanes.copy_(pool[k % 4][0]); host_things.copy_(pool[k % 4][1])
        renderer.step_host(host_lanes, host_things, dev_lanes, dev_things, stack, host_obs)
        torch.cuda.current_stream(device).synchronize()     # the caller reads host_obs here
    s1.record()
    barrier()
    e2e_ms = torch.tensor([s0.elapsed_time(s1)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_value = world * n * e2e_steps / (float(e2e_ms.item()) / 1000.0)
    renderer.check_status()

    # context: the whole device step through the environment API (state producer + render + the
    # reset launch of the auto-reset), no host synchronisation between steps
    from gradoom_b200.env import GraDoomVecEnv

    env = GraDoomVecEnv(compiled_scenario=sc, num_envs=n, device=device, frame_skip=2, obs_crop=(0, 32, 0, 0),
                        obs_crop_mode="mask", max_things=THINGS, producer_seed=2000)
    env.reset_device(everyone, lane_ids + 1)
    api_steps = max(args.steps, 3)
    for k in range(3):
        env.step_and_reset_device(actions[k % actions.shape[0]], lane_ids + 7)
    barrier()
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a0.record()
    for k in range(api_steps):
        env.step_and_reset_device(actions[k % actions.shape[0]], lane_ids + 11 * (k + 1))
    a1.record()
    barrier()
    api_ms = torch.tensor([a0.elapsed_time(a1)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(api_ms, op=dist.ReduceOp.MAX)
    api_value = world * n * api_steps / (float(api_ms.item()) / 1000.0)
    # the same step replayed from a CUDA graph (actions and reseeds fed through static buffers): the
    # entry points allocate nothing and never synchronise, so the whole step captures as it is
    act_buf, seed_buf = actions[0].clone(), (lane_ids + 5).clone()
    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(side):
        env.step_and_reset_device(act_buf, seed_buf)
    torch.cuda.current_stream(device).wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        env.step_and_reset_device(act_buf, seed_buf)
    barrier()
    a0.record()
    for k in range(api_steps):
        act_buf.copy_(actions[k % actions.shape[0]])
        seed_buf.add_(n)
        graph.replay()
    a1.record()
    barrier()
    graph_ms = torch.tensor([a0.elapsed_time(a1)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(graph_ms, op=dist.ReduceOp.MAX)
    graph_value = world * n * api_steps / (float(graph_ms.item()) / 1000.0)
    env.check_status()
    del graph
    env.close()

    if rank == 0:
        oracle = entry.load_oracle()
        peak, peak_kind = measured_peaks()
        avg_ms = statistics.mean(kernel_ms)
        policy = "ring" if use_ring else "roll"
        traffic, l2_hit, counters_source = recorded_counters(policy)
        sm_hz = (clocks.get("sm_mhz") or 0) * 1e6 or None
        bytes_per_frame = 84 * 84 + 64 + 16 * THINGS + (240 * 320 * 3 if rgb is not None else 0)
        achieved = bytes_per_frame * n / (avg_ms / 1000.0) / 1e9
        cpu_lanes, cpu_things = stepper.random_lanes(sc, 2048, THINGS, seed=11)
        cpu_value, cpu_done, cpu_dt = cpu_baseline(blob, cpu_lanes, cpu_things, oracle,
                                                   seconds=0.5 if args.skip_cpu else 12.0, threads=1)
        line = {
            "metric": METRIC if (workload, n) == (WORKLOAD, LANES_PER_GPU) else
            f"rendered env-frames/sec at {n} lanes/GPU ({workload})",
            "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "i64+f32", "data": "synthetic",
            "config": {"workload": f"{workload}: {n} lanes/GPU, {spec['map']}, {THINGS} things/lane, "
                                   + ("obs and RGB24 frame every step" if rgb is not None else "obs only")
                                   + (f", {min(args.decals, 64)} bullet chips/lane" if args.decals > 0 else ""),
                       "lanes_per_gpu": n, "l2": "flushed with a 256 MiB write between timed steps",
                       "ctas": renderer.ctas,
                       "shared_bytes_per_cta": renderer.shared_bytes if rgb is not None else renderer.shared_bytes_view,
                       "stack_policy": "mirrored ring (write 2 of 8 slots per lane, no reads)" if use_ring
                       else "roll (read 3 + write 4 slots per lane)"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic if (workload, n, rgb, args.decals) == (WORKLOAD, 4096, None, 0) else None,
                         "traffic_source": counters_source + " (ncu capture of this command, recorded; not "
                         "measured by this run)", "peak_source": peak_kind,
                         "algorithmic_bytes_per_launch": bytes_per_frame * n,
                         "kernel_ms": avg_ms, "pixels_per_s": 320 * 208 * n / (avg_ms / 1000.0),
                         # the path is bound on chip, not by HBM: >= 5 B of shared-memory / L2 gathers per
                         # shaded pixel (texel, colormap, frame byte, masks) against 128 B/clk/SM of shared memory
                         # at the SM clock sampled during this run
                         "onchip": {"bytes_per_s": 5 * 320 * 208 * n / (avg_ms / 1000.0),
                                    "peak_bytes_per_s": 148 * 128 * sm_hz if sm_hz else None,
                                    "frac": 5 * 320 * 208 * n / (avg_ms / 1000.0) / (148 * 128 * sm_hz) if sm_hz else None,
                                    "l2_hit_rate_recorded": l2_hit}},
            "cpu_baseline": {"value": cpu_value, "unit": UNIT, "cores": 1, "kind": "port",
                             "sample": f"{cpu_done} lanes of the {workload} workload in {cpu_dt:.1f} s, one thread"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(host_lanes.numel() * 4
                                                                                 + host_things.numel() * 4),
                    "d2h_bytes_per_step": int(host_obs.numel()), "steps": e2e_steps},
            "whole_step": {"value": api_value, "as_cuda_graph": graph_value, "unit": UNIT, "steps": api_steps,
                           "api": "GraDoomVecEnv.step_and_reset_device, device tensors, no host sync",
                           "producer": "player kinematics kernel (gd_player_tics) + synthetic things"},
            "per_rank_ms_per_step": per_rank_ms, "sum_of_rank_rates": sum_of_rank_rates,
            "host_cores": len(os.sched_getaffinity(0)),
            "gpu_launches": launches,
            "clocks": clocks,
            "stats_gather": None if gathered is None else {
                "shape": list(gathered.shape), "every_steps": gather_every, "collective_us": gather_us,
                "backend": "nccl all_gather_into_tensor" if world > 1 else "single rank (no collective)"},
            "wall_s": wall1 - wall0,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_rollout(args):
    """The rollout workload of the benchmark definition (256 lanes x 16-step rollouts on the
    64-sector map, a random-init Nature-CNN under bf16 autocast picking the actions, +1 per kill,
    GAE(0.99, 0.95)): ``gradoom_b200.rollout.RolloutLoop`` around ``GraDoomVecEnv``.  The policy is
    plain PyTorch (context, not part of the render path); what is measured is env-frames/s with
    the render in the loop.  ``--steps`` counts rollouts; ``--update`` adds the clipped
    policy-gradient pass after every rollout."""

    import torch

    entry.load_package()
    from gradoom_b200 import rollout, scene as gdscene
    from gradoom_b200.env import GraDoomVecEnv

    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    lanes, horizon, things = args.lanes or 256, 16, 12
    sc = gdscene.make_grid_scene(gdscene.GRID_CONFIGS["c2"])
    env = GraDoomVecEnv(compiled_scenario=sc, num_envs=lanes, device=device, frame_skip=2, obs_crop=(0, 32, 0, 0),
                        obs_crop_mode="mask", max_things=things, producer_seed=5)
    torch.manual_seed(5)
    policy = rollout.NatureCnnPolicy().to(device)
    loop = rollout.RolloutLoop(env, policy, horizon=horizon, gamma=0.99, gae_lambda=0.95, seed=5)
    launches_before = env._renderer.launches

    for w in range(args.warmup):
        loop.collect()
        if args.update:
            loop.update()
    torch.cuda.synchronize(device)
    launches_per_rollout = (env._renderer.launches - launches_before) // max(args.warmup, 1)
    # The loop is launch-bound at 256 lanes (dozens of small launches per env step), so one whole rollout
    # is captured into a CUDA graph: the environment's calls allocate nothing and never synchronise.
    graph = None
    if not args.no_graph:
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            loop.collect()
        torch.cuda.current_stream(device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            loop.collect()
        torch.cuda.synchronize(device)
    sampler = ClockSampler(device.index)
    sampler.start()
    time.sleep(0.2)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.time()
    e0.record()
    mean_return = 0.0
    for k in range(args.steps):
        if graph is not None:
            graph.replay()
        else:
            loop.collect()
        if args.update:
            loop.update()
        mean_return = float(loop.store.returns.mean())              # the learner reads a scalar per rollout
    e1.record()
    torch.cuda.synchronize(device)
    wall1 = time.time()
    env.check_status()
    ms = e0.elapsed_time(e1)
    frames = lanes * horizon * args.steps
    value = frames / (ms / 1000.0)
    line = {
        "metric": f"env-frames/sec in a {lanes}-lane x {horizon}-step rollout loop (c5)", "value": value, "unit": UNIT,
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "i64+f32 render, bf16 policy",
        "data": "synthetic",
        "config": {"workload": f"c5: {lanes} lanes x {horizon}-step rollouts, 64-sector 8x8 map, {things} things/lane, "
                               "Nature-CNN policy (PyTorch) in the loop, GAE(0.99, 0.95)"
                               + (", one clipped policy-gradient pass per rollout" if args.update else ""),
                   "producer": "player kinematics kernel + synthetic things", "l2": "not flushed: the loop's own working set",
                   "cuda_graph": graph is not None},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 4,
                "note": "one scalar per rollout read by the host; observations stay on the device"},
        "gpu_launches": launches_per_rollout * args.steps, "mean_return": mean_return,
        "clocks": sampler.stop(wall0, wall1),
    }
    print(json.dumps(line), flush=True)
    env.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=WORKLOAD, choices=sorted(WORKLOADS) + ["c5"],
                    help="benchmark configuration (default: the headline one)")
    ap.add_argument("--lanes", type=int, default=0, help="lanes per GPU (default: the workload's own count)")
    ap.add_argument("--skip-cpu", action="store_true", help="omit the CPU baseline leg (profiling captures)")
    ap.add_argument("--stack-policy", default="roll", choices=["roll", "ring"],
                    help="frame stack of the timed leg: the reference's contiguous rolled stack (the drop-in "
                         "contract), or the mirrored eight-slot ring")
    ap.add_argument("--skip-upstream", action="store_true",
                    help="reference arm: time only the C restatement, not the upstream Torch engine")
    ap.add_argument("--no-graph", action="store_true", help="c5 only: launch the rollout eagerly instead of as a CUDA graph")
    ap.add_argument("--update", action="store_true", help="c5 only: a clipped policy-gradient pass after every rollout")
    ap.add_argument("--decals", type=int, default=0,
                    help="bullet chips per lane (rings of 64 slots, bitmaps added to the scene); 0 = the contract workload")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.workload == "c5":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the rollout workload has no CPU arm"}), flush=True)
        else:
            run_rollout(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
