#!/usr/bin/env python
"""Benchmark of the Monarch self-attention hot path (one JSON line on stdout).

A "step" is one self-attention call of one DiT layer on one 3-frame chunk at Wan-1.3B shape:
fused RoPE + layout + in-place KV-cache write of the 4680 new tokens, then Monarch attention of
the 4680 queries against the cache (default: framewise blocking, 7 chunks = 32760 cached tokens,
12 heads of 128).  Inputs are seeded synthetic N(0,1) bf16 tensors.  Successive steps rotate
through several layer caches so that every step streams its K/V from HBM, as in the real model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--blocking framewise|tied3frame|reduce2xh|reduce4xw2xh|dense] [--k 1..7]
                    [--sweep FILE]

With N > 1 (launched by torchrun, one rank per GPU) every rank runs its own chunk: independent
videos, no inter-GPU traffic on this path (weak scaling).  --impl reference times the CPU
restatement of the reference's PyTorch path on the host cores instead.
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

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import numpy as np
import torch

BLOCKINGS = {  # name -> (f_tied, h_reduce, w_reduce)
    "framewise": (1, 1, 1), "tied3frame": (3, 1, 1), "reduce2xh": (1, 2, 1), "reduce4xw2xh": (1, 2, 4),
}
H_GRID, W_GRID, HEADS, HEAD_DIM, CHUNK_FRAMES = 30, 52, 12, 128, 3
CHUNK = CHUNK_FRAMES * H_GRID * W_GRID          # 4680 tokens
N_LAYER_CACHES = 4                              # rotated so K/V (201 MB per layer at k=7) is never L2 resident


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of each kernel at the bench
# workload, from the ncu capture summarised in profiles/monarch_framewise_k7_ncu.md.
# dram__bytes_read.sum + dram__bytes_write.sum per launch from ncu captures of this bench at k = 7 (averaged over a
# step's launches where the bridge budget cuts the step into several); profiles/monarch_framewise_k7_ncu.md,
# profiles/sweep_blockings_k1_7.md and profiles/dense_k7_ncu.md give the commands
NCU_TRAFFIC = {
    ("framewise", 7): {"monarch_row_step": 261.1e6 + 561.3e6, "monarch_col_step": 624.0e6 + 9.4e6,
                       "layout_rope_cache_write": 43.2e6 + 2.5e6},
    ("tied3frame", 7): {"monarch_row_step": 216.4e6 + 157.1e6, "monarch_col_step": 217.5e6 + 6.0e6,
                        "layout_rope_cache_write": 43.2e6 + 2.5e6},
    ("reduce2xh", 7): {"monarch_row_step": (347.5e6 + 1123.6e6) / 2, "monarch_col_step": (1233.6e6 + 9.7e6) / 2,
                       "layout_rope_cache_write": 43.2e6 + 3.0e6},
    ("reduce4xw2xh", 7): {"monarch_row_step": (564.7e6 + 4543.0e6) / 6, "monarch_col_step": (4884.8e6 + 2.2e6) / 6,
                          "layout_rope_cache_write": 43.2e6 + 2.5e6},
    ("dense", 7): {"dense": 215.9e6 + 13.0e6},
}


def algorithmic(blocking: str, k: int, heads: int = HEADS, batch: int = 1):
    """Algorithmic FLOPs and HBM bytes of one call (T = 1)."""
    n_q, n_kv = CHUNK, CHUNK * k
    if blocking == "dense":
        flops = 4.0 * n_q * n_kv * HEAD_DIM * heads * batch
        r_flops, l_flops = flops, 0.0
    else:
        ft, hr, wr = BLOCKINGS[blocking]
        b1, b2 = ft * H_GRID // hr, W_GRID // wr
        r_flops = 6.0 / b1 * n_q * n_kv * HEAD_DIM * heads * batch
        l_flops = 4.0 / b2 * n_q * n_kv * HEAD_DIM * heads * batch
        flops = r_flops + l_flops
    bytes_ = (4 * n_q + 2 * n_kv) * heads * HEAD_DIM * 2 * batch
    return flops, bytes_, r_flops, l_flops


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons every 200 ms while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                 parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def bind_host_to_gpu(local_rank: int, world: int):
    """Best effort, multi-rank runs only: run this rank on the cores of its GPU's NUMA node (its share of them,
    when several ranks' GPUs hang off one node) and prefer that node for new pages, so that the pinned
    staging buffers of the end-to-end leg (57.5 MB per step and GPU) are not all served by the memory of
    one socket.  Whatever the container does not allow is skipped; returns what was applied."""
    info = {}
    try:
        allowed = sorted(os.sched_getaffinity(0))

        def node_of(i):
            pr = torch.cuda.get_device_properties(i)
            path = f"/sys/bus/pci/devices/{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0/numa_node"
            return int(Path(path).read_text().strip())

        nodes = [node_of(i) for i in range(world)]
        node = nodes[local_rank]
        info["numa_node"] = node
        cpus = allowed
        if node >= 0:
            lst = Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip()
            on_node = set()
            for part in lst.split(","):
                a, _, b = part.partition("-")
                on_node.update(range(int(a), int(b or a) + 1))
            if on_node & set(allowed):
                cpus = sorted(on_node & set(allowed))
        peers = [r for r in range(world) if nodes[r] == node] if cpus is not allowed else list(range(world))
        share = max(1, len(cpus) // len(peers))
        mine = cpus[peers.index(local_rank) * share:(peers.index(local_rank) + 1) * share] or cpus
        os.sched_setaffinity(0, mine)
        info["cpus"] = f"{mine[0]}-{mine[-1]} ({len(mine)})"
        if node >= 0:
            import ctypes
            import platform
            nr = {"x86_64": 238, "aarch64": 237}.get(platform.machine())
            if nr is not None:
                mask = ctypes.c_ulong(1 << node)
                rc = ctypes.CDLL(None, use_errno=True).syscall(nr, 1, ctypes.byref(mask), 64)   # MPOL_PREFERRED
                info["mempolicy"] = "preferred node" if rc == 0 else f"not applied (errno {ctypes.get_errno()})"
    except Exception as exc:                                             # sysfs layout, permissions, old torch
        info["skipped"] = repr(exc)[:120]
    return info


def make_inputs(k: int, seed: int, device, heads: int = HEADS):
    g = torch.Generator(device="cpu").manual_seed(seed)
    mk = lambda n: torch.randn(1, n, heads, HEAD_DIM, generator=g, dtype=torch.float32).to(torch.bfloat16)
    q, kn, vn = mk(CHUNK), mk(CHUNK), mk(CHUNK)
    caches = []
    for _ in range(N_LAYER_CACHES):
        kc = torch.zeros(1, 7 * CHUNK, heads, HEAD_DIM, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        kc[:, :(k - 1) * CHUNK] = torch.randn(1, (k - 1) * CHUNK, heads, HEAD_DIM, generator=g).to(torch.bfloat16)
        vc[:, :(k - 1) * CHUNK] = torch.randn(1, (k - 1) * CHUNK, heads, HEAD_DIM, generator=g).to(torch.bfloat16)
        caches.append((kc.to(device), vc.to(device)))
    return q, kn, vn, caches


def make_step(sfb, blocking, k, q, kn, vn, caches, num_iters=1):
    n_kv = k * CHUNK
    start = n_kv - CHUNK
    start_frame = CHUNK_FRAMES * (k - 1)
    state = {"i": 0}
    if blocking == "dense":
        def step(qd=q, kd=kn, vd=vn):
            kc, vc = caches[state["i"] % len(caches)]; state["i"] += 1
            rq = sfb.causal_rope_apply(qd, [[CHUNK_FRAMES, H_GRID, W_GRID]], None, start_frame)
            rk = sfb.causal_rope_apply(kd, [[CHUNK_FRAMES, H_GRID, W_GRID]], None, start_frame)
            return sfb.full_attention_with_kv_cache(rq, kc[:, :n_kv], vc[:, :n_kv], rk, vd, start, n_kv)
    else:
        ft, hr, wr = BLOCKINGS[blocking]

        def step(qd=q, kd=kn, vd=vn):
            kc, vc = caches[state["i"] % len(caches)]; state["i"] += 1
            return sfb.rope_monarch_attn_with_kv_cache(qd, kd, vd, kc[:, :n_kv], vc[:, :n_kv], start, n_kv,
                                                       start_frame, ft, hr, wr, H_GRID, W_GRID, num_iters=num_iters)
    return step


def time_steps(step, steps, warmup, dist_barrier):
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    dist_barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    dist_barrier()
    return e0.elapsed_time(e1)


def time_steps_repeated(step, steps, warmup, dist_barrier, min_region_s, reduce_max=None):
    """The K-step timed loop of time_steps, run as many times back to back as it takes to fill
    `min_region_s` seconds of timed region (a single 50-step loop of this op lasts a few milliseconds, too
    short for a stable number or for clock samples).  Every repeat times exactly K steps between barriers;
    the median repeat is reported.  `reduce_max` turns a local time into the maximum over ranks so that all
    ranks agree on the number of repeats and on each repeat's time."""
    red = reduce_max or (lambda x: x)
    first = red(time_steps(step, steps, warmup, dist_barrier))
    repeats = max(1, min(2000, int(min_region_s * 1e3 / max(first, 1e-3)) + 1))
    times = [red(time_steps(step, steps, 0, dist_barrier)) for _ in range(repeats)]
    return statistics.median(times), repeats, sum(times) * 1e-3


def cpu_reference_step(heads_sample: int, blocking: str, k: int, seed: int = 1234):
    """One step of the reference arithmetic on the CPU (fp32, all host threads) for
    `heads_sample` of the heads; returns seconds."""
    from oracle import monarch_oracle as orc
    rng = np.random.default_rng(seed)
    mk = lambda n: torch.from_numpy(rng.standard_normal((1, n, heads_sample, HEAD_DIM), dtype=np.float32))
    n_kv = k * CHUNK
    q, kn, vn = mk(CHUNK), mk(CHUNK), mk(CHUNK)
    kc, vc = mk(n_kv), mk(n_kv)
    t0 = time.perf_counter()
    if blocking == "dense":
        rq = orc.rope_apply(q, (CHUNK_FRAMES, H_GRID, W_GRID), CHUNK_FRAMES * (k - 1))
        rk = orc.rope_apply(kn, (CHUNK_FRAMES, H_GRID, W_GRID), CHUNK_FRAMES * (k - 1))
        kc[:, n_kv - CHUNK:] = rk; vc[:, n_kv - CHUNK:] = vn
        orc.dense_attention(rq, kc, vc)
    else:
        ft, hr, wr = BLOCKINGS[blocking]
        rq = orc.rope_apply(q, (CHUNK_FRAMES, H_GRID, W_GRID), CHUNK_FRAMES * (k - 1))
        rk = orc.rope_apply(kn, (CHUNK_FRAMES, H_GRID, W_GRID), CHUNK_FRAMES * (k - 1))
        orc.monarch_attn_with_kv_cache(rq, kc, vc, rk, vn, n_kv - CHUNK, n_kv, ft, hr, wr, H_GRID, W_GRID)
    return time.perf_counter() - t0


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    heads_sample = HEADS if args.blocking != "dense" else 4      # dense on the CPU: 4 heads per step, scaled
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_reference_step(4, args.blocking, args.k)
    t = []
    budget_s, t_start = 150.0, time.perf_counter()
    for _ in range(args.steps):
        t.append(cpu_reference_step(heads_sample, args.blocking, args.k))
        if time.perf_counter() - t_start > budget_s:
            break
    sec = statistics.mean(t) * (HEADS / heads_sample)
    fps = CHUNK_FRAMES / sec
    flops, bytes_, _, _ = algorithmic(args.blocking, args.k)
    line = {
        "impl": "reference", "metric": "monarch_attn_latent_frames_per_s", "value": fps,
        "unit": "latent frames/s (one attention layer call per 3-frame chunk)", "n_gpus": args.gpus,
        "steps": len(t), "warmup": args.warmup, "ms_per_step": sec * 1e3, "ms_per_chunk": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args),
        "cpu_baseline": {"value": fps, "unit": "latent frames/s", "cores": cores, "kind": "port",
                         "sample": (f"the whole step (all {HEADS} heads)" if heads_sample == HEADS else
                                    f"{heads_sample} of {HEADS} heads per step, time scaled x{HEADS // heads_sample}") +
                                   f"; {len(t)} steps; fp32 torch CPU restatement of the reference PyTorch path"},
        "e2e": {"value": fps, "unit": "latent frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args):
    return {"workload": f"Wan-1.3B self-attention op, {args.blocking}, 4680-token chunk vs {args.k * CHUNK}-token "
                        f"KV cache (k={args.k}), 12 heads x 128, B=1 per GPU, RoPE 44/42/42 fused"
                        + (f", {args.num_iters} alternating passes" if getattr(args, "num_iters", 1) > 1 else ""),
            "blocking": args.blocking, "k": args.k, "n_q": CHUNK, "n_kv": args.k * CHUNK, "heads": HEADS,
            "head_dim": HEAD_DIM, "l2": f"{N_LAYER_CACHES} rotating layer caches "
                                         f"({N_LAYER_CACHES * 2 * args.k * CHUNK * HEADS * HEAD_DIM * 2 / 1e6:.0f} MB) "
                                         "> 126 MB L2, no explicit flush",
            "parallelism": f"dp{args.gpus} (independent chunks per GPU, no collective)"}


def run_rollout(args, sfb, rank, world, device, barrier):
    """The self-attention share of one Wan-1.3B video rollout on each GPU: 21 latent frames in 7 chunks of 3,
    per chunk 4 denoising forwards plus the clean-context forward that refreshes the cache
    (pipeline/causal_inference.py:203-245), per forward 30 layers, each layer one call of the layer path
    (RMSNorm + RoPE + cache write in one kernel, then Monarch attention; dense attention for the first
    chunk when --dense-init).  The projections' outputs are seeded random tensors shared by all layers;
    every layer has its own KV cache (30 x 403 MB)."""
    layers, chunks, forwards = 30, 7, 5
    ft, hr, wr = BLOCKINGS[args.blocking]
    cfg = sfb.LayerConfig(use_framewise=(ft == 1), h_reduce=hr, w_reduce=wr, use_dense_init=args.dense_init,
                          max_attention_size=chunks * CHUNK)
    g = torch.Generator(device="cpu").manual_seed(300 + rank)
    mk = lambda: torch.randn(1, CHUNK, HEADS, HEAD_DIM, generator=g).to(torch.bfloat16).to(device)
    qkv = [(mk(), mk(), mk()) for _ in range(3)]
    wq = (torch.rand(HEADS * HEAD_DIM, generator=g) + 0.5).to(torch.bfloat16).to(device)
    wk = (torch.rand(HEADS * HEAD_DIM, generator=g) + 0.5).to(torch.bfloat16).to(device)
    caches = [sfb.KVCache.allocate(1, chunks * CHUNK, HEADS, device) for _ in range(layers)]

    def video():
        for c in caches:
            c.reset()
        out = None
        for chunk in range(chunks):
            for fwd in range(forwards):
                q, k, v = qkv[(chunk + fwd) % 3]
                for layer in range(layers):
                    out = sfb.self_attention_kv(q, k, v, caches[layer], chunk * CHUNK, (CHUNK_FRAMES, H_GRID, W_GRID),
                                                cfg, norm_q_weight=wq, norm_k_weight=wk)
        return out

    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    sampler.start()
    steps, warmup = max(1, args.steps), max(1, min(args.warmup, 2))
    ms = time_steps(video, steps, warmup, barrier) / steps
    clocks = sampler.stop()
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item()
    if rank == 0:
        calls = layers * chunks * forwards
        print(json.dumps({
            "metric": "attention_rollout_latent_frames_per_s", "value": 21 * world / (ms * 1e-3),
            "unit": "latent frames/s (self-attention layers of a Wan-1.3B rollout only)", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms, "ms_per_layer_call": ms / calls,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"self-attention of a 21-frame Wan-1.3B rollout: 7 chunks x 5 forwards x 30 layers = "
                                   f"{calls} layer calls (RMSNorm + RoPE + cache write + {args.blocking} Monarch"
                                   f"{', dense first chunk' if args.dense_init else ''}), 12 heads x 128, one video per GPU",
                       "parallelism": f"dp{world}"},
            "clocks": clocks}))


def run_model(args, rank, world, device, barrier):
    """BASELINE's full-model configurations: the reference's own CausalWanModel, WanDiffusionWrapper and
    CausalInferencePipeline, imported unmodified from a staged checkout (baseline/stage_reference.py), with
    random-init bf16 weights, a random 512x4096 text context and seeded latent noise; 21 frames in 7 chunks
    of 3, 4 denoising steps plus the clean-context pass per chunk.  --attention selects what the model's
    self-attention calls: "ours" = this package behind wan.modules.monarch_attn / wan.modules.attention,
    "patched" = additionally the fused layer path in place of the cache branch of
    CausalWanSelfAttention.forward, "reference" = the reference's Triton / flash-attn operators.  Times are
    the pipeline's own CUDA events (inference(profile=True)); every rank generates its own videos."""
    sys.path.insert(0, str(ROOT / "baseline"))
    import reference_harness as rh
    base = {"metric": "wan_latent_frames_per_s", "unit": "latent frames/s (4-step causal rollout, whole DiT)",
            "n_gpus": world, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (random-init weights, random text context, seeded noise)"}
    root = rh.reference_root()
    if root is None:
        if rank == 0:
            print(json.dumps({**base, "unavailable": "reference sources not staged: run baseline/stage_reference.py "
                                                     "with SF_REFERENCE_ROOT pointing at a Self-Forcing checkout"}))
        return
    rh.prepare_imports(root, attention="reference" if args.attention == "reference" else "ours")
    overrides = {"num_layers": args.layers} if args.layers else {}
    sp = bool(args.sp) and world > 1
    pipe = rh.build_pipeline(args.model, args.blocking, device=device, dense_init=args.dense_init,
                             num_iters=args.num_iters, seed=0 if sp else rank, sequence_parallel=sp,
                             exchange="peer" if args.p2p else "all_to_all", **overrides)
    if args.attention == "patched":
        import self_forcing_b200 as sfb
        from self_forcing_b200.install import patch_self_attention_forward
        from wan.modules.causal_model import CausalWanSelfAttention
        patch_self_attention_forward(CausalWanSelfAttention)
    from self_forcing_b200 import _lib
    lib = _lib.load() if args.attention != "reference" else None
    for _ in range(max(1, min(args.warmup, 2))):
        rh.run_rollout(pipe, batch=args.batch, device=device, seed=10 + (0 if sp else rank))
    torch.cuda.synchronize()
    barrier()
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    sampler.start()
    n0 = lib.sfm_launch_count() if lib else 0
    diff_ms, block_ms = [], []
    steps = max(1, args.steps)
    for i in range(steps):
        _, prof = rh.run_rollout(pipe, batch=args.batch, device=device, seed=20 + (0 if sp else rank) + i)
        diff_ms.append(prof["diffusion_ms"])
        block_ms.append(prof["block_ms"])
    launches = (lib.sfm_launch_count() - n0) // steps if lib else 0
    clocks = sampler.stop()
    barrier()
    ms = statistics.median(diff_ms)
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item()
    if rank == 0:
        chunks = [statistics.median(b[i] for b in block_ms) for i in range(len(block_ms[0]))]
        shape = rh.MODEL_SHAPES[args.model]
        videos = args.batch * (1 if sp else world)
        if sp:
            base["scaling"] = "strong"
        print(json.dumps({**base, "value": 21 * videos / (ms * 1e-3), "steps": steps,
                          "warmup": max(1, min(args.warmup, 2)), "ms_per_step": ms, "ms_per_chunk": chunks,
                          "config": {"workload": f"causal Wan-{args.model.upper()} DiT ({shape['num_layers'] if not args.layers else args.layers} blocks, dim "
                                                 f"{shape['dim']}, {shape['num_heads']} heads, FFN {shape['ffn_dim']}), 21x60x104 latent in 7 "
                                                 f"chunks of 3 frames, timesteps [1000, 750, 500, 250] + clean-context pass, "
                                                 f"{args.blocking} self-attention with KV cache, batch {args.batch} per GPU",
                                     "attention": args.attention, "blocking": args.blocking, "batch": args.batch,
                                     "parallelism": (f"sp{world} (one video over all GPUs: tokens sharded outside attention, heads "
                                                     f"inside, exchanged {'by the kernels over peer memory' if args.p2p else 'by two all-to-alls'} per layer; "
                                                     "weights replicated)") if sp else
                                                    f"dp{world} (independent videos per GPU)"},
                          "gpu_launches": int(launches), "clocks": clocks}), flush=True)


def run_probe_dsmem(device):
    """Store bandwidth between the CTAs of a cluster through distributed shared memory (sfm_probe_dsmem_store):
    the ceiling of an on-chip hand-off between the row step and the column step."""
    import ctypes as C
    from self_forcing_b200 import _lib
    lib = _lib.load()
    rows = []
    for cluster in (1, 2, 4, 8, 16):
        for remote in ((0,) if cluster == 1 else (0, 1)):
            for pattern in (0, 1):
                ms, ctas, nbytes = C.c_float(), C.c_int(), C.c_double()
                rc = lib.sfm_probe_dsmem_store(cluster, pattern, remote, 2000, C.byref(ms), C.byref(ctas), C.byref(nbytes))
                row = {"cluster": cluster, "remote": bool(remote), "pattern": "row-per-lane 32 B" if pattern == 0 else "coalesced 16 B"}
                if rc:
                    row["error"] = lib.sfm_error_string(rc).decode()
                else:
                    row.update(ctas=ctas.value, ms=ms.value, tb_per_s=nbytes.value / ms.value * 1e-9,
                               bytes_per_clk_per_sm=nbytes.value / (ms.value * 1e-3) / ctas.value / 1.965e9)
                rows.append(row)
    print(json.dumps({"probe": "dsmem_store", "sm_clock_assumed_mhz": 1965, "rows": rows}, indent=1))


def run_incumbent(args, device):
    """The reference's own Triton Monarch path (monarch_attn_with_kv_cache, num_iters=1: _al_cl_y_fwd + _z_fwd
    in 3x3 group chunks, monarch_attn.py:1227-1323), imported unmodified from the staged checkout and timed on
    this GPU beside this package's op on the same tensors (op only: both write the new keys and attend;
    RoPE is outside).  The first call autotunes (minutes); the timed calls come after it."""
    import importlib.util
    sys.path.insert(0, str(ROOT / "baseline"))
    import reference_harness as rh
    root = rh.reference_root()
    if root is None:
        print(json.dumps({"incumbent": "unavailable", "why": "reference sources not staged (baseline/stage_reference.py)"}))
        return
    spec = importlib.util.spec_from_file_location("ref_monarch_attn", root / "wan/modules/monarch_attn.py")
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    import self_forcing_b200 as sfb
    ft, hr, wr = BLOCKINGS[args.blocking]
    out = {"blocking": args.blocking, "triton": __import__("triton").__version__, "rows": []}
    for k in ([args.k] if args.k_only else [7, 4, 1]):
        g = torch.Generator(device="cpu").manual_seed(k)
        mk = lambda m: torch.randn(1, m, HEADS, HEAD_DIM, generator=g).to(torch.bfloat16).to(device)
        n_kv = k * CHUNK
        q, nk, nv, kc, vc = mk(CHUNK), mk(CHUNK), mk(CHUNK), mk(n_kv), mk(n_kv)
        kc2, vc2 = kc.clone(), vc.clone()
        ref_call = lambda: ref.monarch_attn_with_kv_cache(q, kc, vc, nk, nv, n_kv - CHUNK, n_kv, ft, hr, wr, H_GRID, W_GRID, num_iters=1)
        our_call = lambda: sfb.monarch_attn_with_kv_cache(q, kc2, vc2, nk, nv, n_kv - CHUNK, n_kv, ft, hr, wr, H_GRID, W_GRID)
        row = {"k": k}
        with torch.no_grad():
            t0 = time.perf_counter()
            try:
                zr = ref_call()
                torch.cuda.synchronize()
            except Exception as exc:                                   # Triton may not compile here: record why
                row["error"] = repr(exc)[:400]
                out["rows"].append(row)
                continue
            row["first_call_s"] = time.perf_counter() - t0
            zo = our_call()
            row["max_abs_diff"] = (zr.float() - zo.float()).abs().max().item()
            row["reference_triton_ms"] = time_steps(ref_call, args.steps, args.warmup, lambda: None) / args.steps
            row["ours_ms"] = time_steps(our_call, args.steps, args.warmup, lambda: None) / args.steps
        if args.backward:
            # forward + backward through both packages' autograd functions (gradients of q and of the chunk's own keys
            # and values, as a training rollout asks for them: grad_only_new_kv)
            do = mk(CHUNK)
            def fwd_bwd(mod):
                q1, nk1, nv1 = (t.clone().requires_grad_(True) for t in (q, nk, nv))
                z = mod.monarch_attn_with_kv_cache(q1, kc.clone(), vc.clone(), nk1, nv1, n_kv - CHUNK, n_kv, ft, hr, wr,
                                                   H_GRID, W_GRID, grad_only_new_kv=True)
                z.backward(do)
                return q1.grad, nk1.grad, nv1.grad
            try:
                gr = fwd_bwd(ref)
                torch.cuda.synchronize()
            except Exception as exc:
                row["backward_error"] = repr(exc)[:400]
                out["rows"].append(row)
                continue
            go = fwd_bwd(sfb)
            for name, a, b in zip(("dq", "dk_new", "dv_new"), gr, go):
                row["rel_l2_" + name] = ((a.float() - b.float()).norm() / a.float().norm()).item()
            row["reference_triton_fwd_bwd_ms"] = time_steps(lambda: fwd_bwd(ref), args.steps, args.warmup, lambda: None) / args.steps
            row["ours_fwd_bwd_ms"] = time_steps(lambda: fwd_bwd(sfb), args.steps, args.warmup, lambda: None) / args.steps
        out["rows"].append(row)
    print(json.dumps(out, indent=1))


def run_backward(args, sfb, rank, world, device, barrier):
    """Forward + backward of the Monarch attention op at the headline shape (one 3-frame chunk against k cached
    chunks, 12 heads): the call a training rollout makes per layer (gradients of q and of the chunk's own keys
    and values, as with grad_only_new_kv)."""
    ft, hr, wr = BLOCKINGS[args.blocking]
    n_kv = args.k * CHUNK
    g = torch.Generator(device="cpu").manual_seed(400 + rank)
    mk = lambda n: torch.randn(1, n, HEADS, HEAD_DIM, generator=g).to(torch.bfloat16).to(device)
    q, kc, vc, do = mk(CHUNK), mk(n_kv), mk(n_kv), mk(CHUNK)
    group = ft * H_GRID * W_GRID // (hr * wr)
    groups = (n_kv // group - CHUNK // group, n_kv // group)
    fwd = lambda: sfb.ops.monarch_attention_on_cache(q, kc, vc, ft, hr, wr, H_GRID, W_GRID)
    bwd = lambda: sfb.monarch_attn_with_kv_cache_backward(q, kc, vc, do, ft, hr, wr, H_GRID, W_GRID, kv_groups=groups)
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    sampler.start()
    ms_f = time_steps(fwd, args.steps, args.warmup, barrier) / args.steps
    ms_b = time_steps(bwd, args.steps, args.warmup, barrier) / args.steps
    clocks = sampler.stop()
    t = torch.tensor([ms_f, ms_b], device=device, dtype=torch.float64)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_f, ms_b = t.tolist()
    if rank == 0:
        print(json.dumps({
            "metric": "attention_fwd_bwd_latent_frames_per_s", "value": CHUNK_FRAMES * world / ((ms_f + ms_b) * 1e-3),
            "unit": "latent frames/s (forward + backward of the attention op)", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_f + ms_b, "forward_ms": ms_f, "backward_ms": ms_b,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 (tcgen05 GEMMs with fp32 accumulation; dq fp32)",
            "data": "synthetic",
            "config": {"workload": f"{args.blocking} Monarch attention forward + backward, one 3-frame chunk vs k={args.k} "
                                   f"cached chunks ({n_kv} tokens), 12 heads x 128, dK/dV of the chunk's own groups",
                       "parallelism": f"dp{world}"},
            "clocks": clocks}))


def run_ulysses(args, sfb, rank, world, device, barrier, emit=True):
    """Wan-14B self-attention layer (40 heads x 128) on one 3-frame chunk with the heads sharded over
    the ranks: every rank holds 4680/P tokens of q, k, v outside attention and 40/P heads (with their
    KV cache) inside it.  Strong scaling: the total work is fixed."""
    import torch.distributed as dist
    from self_forcing_b200.ulysses import UlyssesSelfAttention, tokens_to_heads, heads_to_tokens
    heads = 40
    if heads % world or CHUNK % world:
        raise SystemExit("--ulysses needs a GPU count that divides 40 heads and 4680 tokens")
    hp, sp = heads // world, CHUNK // world
    k = args.k
    n_kv = k * CHUNK
    g = torch.Generator(device="cpu").manual_seed(200 + rank)
    mk = lambda n, h: torch.randn(1, n, h, HEAD_DIM, generator=g, dtype=torch.float32).to(torch.bfloat16).to(device)
    q, kn, vn = mk(sp, heads), mk(sp, heads), mk(sp, heads)
    caches = []
    for _ in range(2):                                   # 2 x 2 x 32760 x (40/P) x 128 x 2 B: larger than L2 up to P = 4
        kc = torch.zeros(1, 7 * CHUNK, hp, HEAD_DIM, dtype=torch.bfloat16, device=device)
        vc = torch.zeros_like(kc)
        kc[:, :n_kv - CHUNK] = mk(n_kv - CHUNK, hp)
        vc[:, :n_kv - CHUNK] = mk(n_kv - CHUNK, hp)
        caches.append((kc, vc))
    ft, hr, wr = BLOCKINGS[args.blocking]
    attn = UlyssesSelfAttention((ft, hr, wr, H_GRID, W_GRID))
    state = {"i": 0}
    start, start_frame = n_kv - CHUNK, CHUNK_FRAMES * (k - 1)

    def step():
        kc, vc = caches[state["i"] % len(caches)]; state["i"] += 1
        return attn(q, kn, vn, kc, vc, start, n_kv, start_frame)

    if args.p2p:
        if world == 1:
            raise SystemExit("--p2p needs more than one GPU")
        from self_forcing_b200.ulysses import PeerShardedSelfAttention
        peer_attn = PeerShardedSelfAttention((ft, hr, wr, H_GRID, W_GRID), 1, CHUNK, heads, device)
        # the projections of the real model would write their outputs here
        peer_attn.q_in.copy_(q); peer_attn.k_in.copy_(kn); peer_attn.v_in.copy_(vn)
        expect = step()
        caches = [(kc.clone(), vc.clone()) for kc, vc in caches]     # same cache contents for the check
        kc0, vc0 = caches[0]
        got = peer_attn(kc0, vc0, start, n_kv, start_frame)
        torch.cuda.synchronize()
        if not torch.equal(got, expect):
            raise SystemExit(f"rank {rank}: peer-memory path differs from the all-to-all path")

        def step():
            kc, vc = caches[state["i"] % len(caches)]; state["i"] += 1
            return peer_attn(kc, vc, start, n_kv, start_frame)

    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    sampler.start()
    ms_total = time_steps(step, args.steps, args.warmup, barrier)
    clocks = sampler.stop()

    # split: the two exchanges alone, and the attention alone, over the same number of steps
    def a2a_in():
        return tokens_to_heads([q, kn, vn])
    qh, kh, vh = a2a_in()

    def attn_only():
        kc, vc = caches[state["i"] % len(caches)]; state["i"] += 1
        return sfb.rope_monarch_attn_with_kv_cache(qh, kh, vh, kc[:, :n_kv], vc[:, :n_kv], start, n_kv, start_frame,
                                                   ft, hr, wr, H_GRID, W_GRID)
    oh = attn_only()

    def a2a_out():
        return heads_to_tokens(oh)
    ms_in = time_steps(a2a_in, args.steps, 3, barrier)
    ms_attn = time_steps(attn_only, args.steps, 3, barrier)
    ms_out = time_steps(a2a_out, args.steps, 3, barrier)
    t = torch.tensor([ms_total, ms_in, ms_attn, ms_out], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, ms_in, ms_attn, ms_out = (x / args.steps for x in t.tolist())
    flops = algorithmic(args.blocking, k, heads=heads)[0]
    record = ({
            "metric": "monarch_attn_latent_frames_per_s", "value": CHUNK_FRAMES / (ms_total * 1e-3),
            "unit": "latent frames/s (one Wan-14B attention layer call per 3-frame chunk)",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_total,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"Wan-14B self-attention op, {args.blocking}, 4680-token chunk vs {n_kv}-token KV cache, "
                                   f"40 heads x 128 sharded {hp} per GPU, tokens sharded {sp} per GPU outside attention",
                       "parallelism": (f"ulysses{world} (kernels gather q,k,v and scatter the result over peer memory; "
                                       "two device barriers)") if args.p2p else
                                      f"ulysses{world} (all-to-all q,k,v in; all-to-all out; NCCL)"},
            "split_ms": {"all_to_all_qkv": ms_in, "rope_cache_attention": ms_attn, "all_to_all_out": ms_out},
            "algorithmic_gflop": flops / 1e9, "clocks": clocks})
    if emit and rank == 0:
        print(json.dumps(record))
    return record


def ulysses_subrecord(args, sfb, rank, world, device, barrier):
    """For the multi-GPU default run: the Wan-14B head-sharded attention layer (40 heads over the ranks, strong
    scaling) on both exchange paths, next to the same 40-head layer call on one GPU alone, so that the record
    holds the speed-up the head sharding gives at this GPU count."""
    import copy
    import torch.distributed as dist
    a = copy.copy(args)
    a.steps, a.warmup = min(args.steps, 20), 5
    sub = {"workload": "Wan-14B self-attention layer call (40 heads x 128, 4680-token chunk vs "
                       f"{a.k * CHUNK}-token cache, {a.blocking}); strong scaling over {world} GPUs"}
    # all 40 heads on one GPU (every rank does the same; the slowest counts)
    g = torch.Generator(device="cpu").manual_seed(77)
    mk = lambda n: torch.randn(1, n, 40, HEAD_DIM, generator=g).to(torch.bfloat16).to(device)
    q, kn, vn = mk(CHUNK), mk(CHUNK), mk(CHUNK)
    n_kv = a.k * CHUNK
    kc, vc = mk(7 * CHUNK), mk(7 * CHUNK)
    ft, hr, wr = BLOCKINGS[a.blocking]
    one = lambda: sfb.rope_monarch_attn_with_kv_cache(q, kn, vn, kc[:, :n_kv], vc[:, :n_kv], n_kv - CHUNK, n_kv,
                                                      CHUNK_FRAMES * (a.k - 1), ft, hr, wr, H_GRID, W_GRID)
    t = torch.tensor([time_steps(one, a.steps, a.warmup, barrier) / a.steps], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sub["one_gpu_ms"] = t.item()
    del q, kn, vn, kc, vc
    torch.cuda.empty_cache()
    for name, p2p in (("nccl_all_to_all", False), ("peer_memory", True)):
        a.p2p = p2p
        try:
            r = run_ulysses(a, sfb, rank, world, device, barrier, emit=False)
            sub[name] = {"ms_per_layer_call": r["ms_per_step"], "speedup_vs_one_gpu": sub["one_gpu_ms"] / r["ms_per_step"],
                         "efficiency": sub["one_gpu_ms"] / r["ms_per_step"] / world, "split_ms": r["split_ms"]}
        except (Exception, SystemExit) as exc:
            sub[name] = {"error": repr(exc)[:200]}
    return sub


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--blocking", default="framewise", choices=list(BLOCKINGS) + ["dense"])
    ap.add_argument("--k", type=int, default=7)
    ap.add_argument("--sweep", default=None, help="also time every blocking x k and write a JSON table here")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--min-region-s", type=float, default=0.5,
                    help="repeat the timed K-step loop until the timed region is at least this long; report the median repeat")
    ap.add_argument("--ulysses", action="store_true",
                    help="time the Wan-14B attention layer (40 heads) with heads sharded over the GPUs "
                         "(token shards outside attention, two all-to-alls per layer) instead of the headline workload")
    ap.add_argument("--rollout", action="store_true",
                    help="time the self-attention share of a whole 21-frame Wan-1.3B rollout (7 chunks x 5 forwards x "
                         "30 layers through the layer path) instead of the headline workload")
    ap.add_argument("--backward", action="store_true",
                    help="time forward + backward of the attention op at the headline shape instead of the headline workload")
    ap.add_argument("--dense-init", action="store_true", help="with --rollout: dense attention for the first chunk")
    ap.add_argument("--p2p", action="store_true",
                    help="with --ulysses or --model --sp: the kernels gather / scatter over peer memory instead of the two "
                         "NCCL all-to-alls")
    ap.add_argument("--probe-dsmem", action="store_true",
                    help="measure store bandwidth between the CTAs of a cluster (distributed shared memory) and exit")
    ap.add_argument("--incumbent", action="store_true",
                    help="time the reference's own Triton Monarch op beside this package's on the same tensors "
                         "(needs the staged reference sources) and exit")
    ap.add_argument("--k-only", action="store_true", help="with --incumbent: only the cache length given by --k")
    ap.add_argument("--model", default=None, choices=["1.3b", "14b"],
                    help="time the whole causal DiT rollout through the reference's unmodified model and pipeline code "
                         "(needs the staged reference sources, see baseline/stage_reference.py) instead of the headline workload")
    ap.add_argument("--attention", default="ours", choices=["ours", "patched", "reference"],
                    help="with --model: what the model's self-attention runs on")
    ap.add_argument("--batch", type=int, default=1, help="with --model: videos per GPU")
    ap.add_argument("--sp", action="store_true",
                    help="with --model and N > 1 GPUs: one video over all GPUs (sequence parallel outside attention, head "
                         "sharding inside) instead of independent videos per GPU")
    ap.add_argument("--layers", type=int, default=0, help="with --model: override the number of blocks (0 = the model's)")
    ap.add_argument("--num-iters", type=int, default=1, help="alternating passes T of the Monarch op (with --model: MONARCH_ATTN_NUM_ITERS); the roofline figures assume T = 1")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    use_dist = world > 1
    host_binding = bind_host_to_gpu(local_rank, world) if use_dist else None
    if use_dist:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
        barrier = lambda: dist.barrier()
    else:
        barrier = lambda: None

    if args.probe_dsmem or args.incumbent:
        if rank == 0:
            run_probe_dsmem(device) if args.probe_dsmem else run_incumbent(args, device)
        if use_dist:
            dist.destroy_process_group()
        return

    if args.model:
        run_model(args, rank, world, device, barrier)
        if use_dist:
            dist.destroy_process_group()
        return

    import self_forcing_b200 as sfb
    from self_forcing_b200 import _lib
    lib = _lib.load()

    if args.rollout:
        run_rollout(args, sfb, rank, world, device, barrier)
        if use_dist:
            dist.destroy_process_group()
        return

    if args.backward:
        run_backward(args, sfb, rank, world, device, barrier)
        if use_dist:
            dist.destroy_process_group()
        return

    if args.ulysses:
        run_ulysses(args, sfb, rank, world, device, barrier)
        if use_dist:
            dist.destroy_process_group()
        return

    q, kn, vn, caches = make_inputs(args.k, 100 + rank, device)
    qd, kd, vd = q.to(device), kn.to(device), vn.to(device)
    step = make_step(sfb, args.blocking, args.k, qd, kd, vd, caches, args.num_iters)

    # ---- headline: device-resident inputs -------------------------------------------------
    def reduce_max(ms):
        if not use_dist:
            return ms
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    n0 = lib.sfm_launch_count()
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    launches = (lib.sfm_launch_count() - n0) * args.steps // 3      # this library's launches in K steps
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms_total, repeats, region_s = time_steps_repeated(step, args.steps, args.warmup, barrier, args.min_region_s,
                                                      reduce_max)
    clocks = sampler.stop()

    # ---- per-kernel durations over the same steps (events around every launch) -------------
    import ctypes as C
    lib.sfm_profile_enable(1)
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize()
    ms_cls = (C.c_float * 6)()
    n_cls = (C.c_longlong * 6)()
    _lib.check(lib.sfm_profile_read(ms_cls, n_cls, 6), "sfm_profile_read")
    lib.sfm_profile_enable(0)
    cls_names = ["layout_rope_cache_write", "monarch_row_step", "monarch_col_step", "monarch_iter", "dense", "monarch_backward"]
    kernels = {cls_names[i]: {"launches_per_step": n_cls[i] / args.steps, "ms_per_step": ms_cls[i] / args.steps}
               for i in range(6) if n_cls[i]}

    # ---- end to end through the public API with host buffers --------------------------------
    qh, kh, vh = q.pin_memory(), kn.pin_memory(), vn.pin_memory()
    out_h = torch.empty(1, CHUNK, HEADS, HEAD_DIM, dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        qd2 = qh.to(device, non_blocking=True)
        kd2 = kh.to(device, non_blocking=True)
        vd2 = vh.to(device, non_blocking=True)
        out = step(qd2, kd2, vd2)
        out_h.copy_(out, non_blocking=True)

    ms_e2e_serial = time_steps(e2e_step, args.steps, args.warmup, barrier)
    ms_e2e_serial = min(ms_e2e_serial, time_steps(e2e_step, args.steps, 0, barrier))

    # The same work as a serving loop would issue it: inputs of step i+1 are copied in, and the result of
    # step i-1 is copied out, on two side streams while step i computes (double-buffered device inputs).
    # Every step's copies are still inside the timed region.
    s_in, s_out = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
    dev_in = [tuple(torch.empty_like(t) for t in (qd, kd, vd)) for _ in range(2)]
    outs_h = [torch.empty(1, CHUNK, HEADS, HEAD_DIM, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    pipe = {"i": 0, "free": [None, None], "out": None}

    def e2e_pipelined_step():
        cur = torch.cuda.current_stream()
        j = pipe["i"] % 2
        pipe["i"] += 1
        with torch.cuda.stream(s_in):
            if pipe["free"][j] is not None:
                s_in.wait_event(pipe["free"][j])             # the step that last read these buffers is done
            for dst, src in zip(dev_in[j], (qh, kh, vh)):
                dst.copy_(src, non_blocking=True)
            ev_in = torch.cuda.Event()
            ev_in.record(s_in)
        cur.wait_event(ev_in)
        out = step(*dev_in[j])
        ev_done = torch.cuda.Event()
        ev_done.record(cur)
        pipe["free"][j] = ev_done
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done)
            out.record_stream(s_out)
            outs_h[j].copy_(out, non_blocking=True)
            ev_out = torch.cuda.Event()
            ev_out.record(s_out)
        pipe["out"] = ev_out

    def e2e_run(steps, warmup):
        for _ in range(warmup):
            e2e_pipelined_step()
        torch.cuda.synchronize()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            e2e_pipelined_step()
        torch.cuda.current_stream().wait_event(pipe["out"])  # the last read-back belongs to the timed region
        e1.record()
        torch.cuda.synchronize()
        barrier()
        return e0.elapsed_time(e1)

    ms_e2e = reduce_max(e2e_run(args.steps, args.warmup))
    e2e_repeats = max(1, min(200, int(args.min_region_s * 1e3 / max(ms_e2e, 1e-3)) + 1))
    ms_e2e = statistics.median([reduce_max(e2e_run(args.steps, 0)) for _ in range(e2e_repeats)])

    if use_dist:
        t = torch.tensor([ms_e2e_serial], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e_serial = t.item()

    ms_step = ms_total / args.steps
    fps = CHUNK_FRAMES * world / (ms_step * 1e-3)
    fps_e2e = CHUNK_FRAMES * world / (ms_e2e / args.steps * 1e-3)
    flops, bytes_, r_flops, l_flops = algorithmic(args.blocking, args.k)
    hbm_peak, tf_peak, peak_kind = load_peaks()

    # dominant kernel = the class with the most time
    dom = max(kernels, key=lambda n: kernels[n]["ms_per_step"]) if kernels else None
    roofline = None
    if dom:
        dom_ms = kernels[dom]["ms_per_step"]
        dom_flops = {"monarch_row_step": r_flops, "monarch_col_step": l_flops, "dense": flops}.get(dom, 0.0)
        ach = dom_flops / (dom_ms * 1e-3) / 1e12 if dom_ms > 0 else 0.0
        traffic = NCU_TRAFFIC.get((args.blocking, args.k), {}).get(dom)
        roofline = {"kernel": dom, "bound": "tensor", "achieved": ach, "peak": tf_peak, "unit": "TFLOP/s",
                    "frac": ach / tf_peak, "peak_kind": f"of {peak_kind}", "traffic": traffic,
                    "launch_ms_per_step": dom_ms,
                    # what the kernel actually moves through HBM (bridge included), against the copy peak
                    "dram_traffic_gbs": (traffic / (dom_ms * 1e-3) / 1e9) if traffic and dom_ms > 0 else None,
                    "dram_traffic_frac": (traffic / (dom_ms * 1e-3) / 1e9 / hbm_peak) if traffic and dom_ms > 0 else None,
                    "whole_op": {"algorithmic_gflop": flops / 1e9, "algorithmic_mb": bytes_ / 1e6,
                                 "tensor_tflops": flops / (ms_step * 1e-3) / 1e12,
                                 "tensor_frac": flops / (ms_step * 1e-3) / 1e12 / tf_peak,
                                 "hbm_gbs": bytes_ / (ms_step * 1e-3) / 1e9,
                                 "hbm_frac": bytes_ / (ms_step * 1e-3) / 1e9 / hbm_peak}}

    line = {
        "metric": "monarch_attn_latent_frames_per_s", "value": fps,
        "unit": "latent frames/s (one attention layer call per 3-frame chunk)",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "ms_per_chunk": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args),
        "clocks": clocks,
        "timing": {"repeats": repeats, "timed_region_s": region_s,
                   "how": f"median of {repeats} back-to-back repeats of the {args.steps}-step loop (CUDA events, "
                          "barrier + synchronize around each repeat, max over ranks)"},
        "e2e": {"value": fps_e2e, "repeats": e2e_repeats, "unit": "latent frames/s", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": 3 * q.numel() * 2, "d2h_bytes_per_step": q.numel() * 2,
                "how": "copies of step i+1 / i-1 on side streams while step i computes (double-buffered device inputs)",
                "serial_ms_per_step": ms_e2e_serial / args.steps},
        "gpu_launches": int(launches),
        "host_binding": host_binding,
        "kernels": kernels,
        "roofline": roofline,
    }

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        cpu_reference_step(4, args.blocking, args.k)                       # warm-up (thread pool, allocator)
        ts = [cpu_reference_step(HEADS, args.blocking, args.k) for _ in range(3)]
        sec = statistics.median(ts)
        line["cpu_baseline"] = {"value": CHUNK_FRAMES / sec, "unit": "latent frames/s", "ms_per_chunk": sec * 1e3,
                                "cores": cores, "kind": "port",
                                "sample": f"the whole step (all {HEADS} heads), median of 3; fp32 torch CPU restatement "
                                          "of the reference PyTorch path (RoPE in fp64 + Monarch reference op)"}

    if use_dist and 40 % world == 0 and CHUNK % world == 0 and os.environ.get("SFM_BENCH_NO_ULYSSES") != "1":
        line["ulysses"] = ulysses_subrecord(args, sfb, rank, world, device, barrier)

    if args.sweep and rank == 0:
        table = []
        for blocking in list(BLOCKINGS) + ["dense"]:
            for k in range(1, 8):
                q2, kn2, vn2, caches2 = make_inputs(k, 7, device)
                st = make_step(sfb, blocking, k, q2.to(device), kn2.to(device), vn2.to(device), caches2)
                ms = time_steps(st, 20, 5, lambda: None) / 20
                fl, by, _, _ = algorithmic(blocking, k)
                table.append({"blocking": blocking, "k": k, "ms_per_chunk": ms, "gflop": fl / 1e9, "mb": by / 1e6,
                              "tflops": fl / ms / 1e9, "tensor_frac": fl / ms / 1e9 / tf_peak,
                              "hbm_gbs": by / ms / 1e6, "hbm_frac": by / ms / 1e6 / hbm_peak})
                del caches2
                torch.cuda.empty_cache()
        Path(args.sweep).parent.mkdir(parents=True, exist_ok=True)
        Path(args.sweep).write_text(json.dumps(table, indent=1))

    if rank == 0:
        print(json.dumps(line), flush=True)
    if use_dist:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
