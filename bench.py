"""Benchmark of the KV-cache quantization hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (one "step" = the whole hot path of one generated image batch): the VAR-d16 256px
configuration -- 16 blocks, 16 heads, head_dim 64, batch 32 with CFG doubling to 64, the ten
scales 1,2,3,4,5,6,8,10,13,16 (680 tokens), INT8 per-head symmetric KV cache.  For every block
and every scale the step quantizes+packs the scale's fresh K (fp32, L2-normalised, as the VAR
attention hands it over) and V (bf16, a strided view into the fused QKV activation) into the
packed cache and runs attention of the scale's queries over everything cached, writing bf16.
The surrounding transformer (QKV/MLP GEMMs, sampling, VQVAE) is not part of the path and not
run.  Inputs are seeded synthetic tensors of those shapes; the same ten (q, k, v) triples feed
all 16 blocks, each block owning its caches.

With --gpus N (launched through torch.distributed.run) every rank runs the same batch-32 job on
its own GPU -- batch-sharded replicas, no collective on the path -- and the value is the sum
over ranks divided by the slowest rank's device time (weak scaling).

--impl reference times the CPU restatement of the reference algorithm (oracle/) on the host
cores on a bounded sample (whole blocks of the same workload) and scales to the full step.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "var-q_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

PATCH_NUMS = (1, 2, 3, 4, 5, 6, 8, 10, 13, 16)
DEPTH, HEADS, HEAD_DIM, IMAGES = 16, 16, 64, 32
B2 = 2 * IMAGES
STEPS_L = tuple(p * p for p in PATCH_NUMS)
L_TOTAL = sum(STEPS_L)
Q_GAIN = 4.0            # exp(scale_mul_1H11) at initialisation (VAR/models/basic_var.py:86)
WORKLOAD = "VAR-d16 256px KV hot path: 16 blocks x 10 scales x (quantize+pack K, V; attention over packed cache), B=32 (+CFG=64), H=16, c=64, INT8 per-head symmetric"


# --------------------------------------------------------------------------- inputs
def make_inputs(device, seed=0, pin_host=False):
    """Per scale: q fp32 [B2,l,H,c] (unit rows x gain), k fp32 (unit rows), v bf16 strided view."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    out = []
    for l in STEPS_L:
        qkv = torch.randn((B2, l, 3, HEADS, HEAD_DIM), generator=g, dtype=torch.float32)
        qkv[..., :4] *= 6.0                      # a few large channels, as K/V activations show
        q = torch.nn.functional.normalize(qkv[:, :, 0], dim=-1) * Q_GAIN
        k = torch.nn.functional.normalize(qkv[:, :, 1], dim=-1)
        rec = {"q": q.contiguous(), "k": k.contiguous(), "qkv16": qkv.to(torch.bfloat16).contiguous()}
        rec["v16"] = rec["qkv16"][:, :, 2].contiguous()     # the V third alone: what the end-to-end leg uploads
        if pin_host:
            rec = {n: t.pin_memory() for n, t in rec.items()}
        out.append(rec)
    if device is None:
        return out
    dev = []
    for rec in out:
        qkv16 = rec["qkv16"].to(device)
        dev.append({"q": rec["q"].to(device), "k": rec["k"].to(device), "qkv16": qkv16, "v": qkv16.unbind(dim=2)[2]})
    return dev, out


def algorithmic_bytes_attn(lq, lk):
    """Packed K+V codes, their per-(token, head) scales, Q in and O out, for one launch."""
    kv = B2 * HEADS * lk * HEAD_DIM * (8 + 8) // 8
    params = 2 * lk * HEADS * 4
    return kv + params + B2 * HEADS * lq * HEAD_DIM * (4 + 2)


def algorithmic_bytes_quant(l, in_bytes):
    n = B2 * l * HEADS * HEAD_DIM
    return n * in_bytes + n + l * HEADS * 4


# --------------------------------------------------------------------------- GPU arm
def new_quantizers():
    from VAR_Q.quant import VAR_Q
    mk = lambda blk: VAR_Q(quant_bits=8, qkv_format="BLHc", quant_method="G_TOKEN_HEAD", blk_idx=blk, max_tokens=L_TOTAL)
    return [(mk(b), mk(b)) for b in range(DEPTH)]


def hot_path_step(inputs, probe=None):
    """One image batch through the path.  `probe(kind, si)` may return (start, end) events to
    record around a call; it is used to time single launches without perturbing the rest."""
    from VAR_Q.attention import attend_cached
    out = None
    for kq, vq in new_quantizers():
        for si, rec in enumerate(inputs):
            ev = probe("quant_k", si) if probe else None
            if ev: ev[0].record()
            kq.append(rec["k"])
            if ev: ev[1].record()
            ev = probe("quant_v", si) if probe else None
            if ev: ev[0].record()
            vq.append(rec["v"])
            if ev: ev[1].record()
            ev = probe("attn", si) if probe else None
            if ev: ev[0].record()
            out = attend_cached(rec["q"], kq, vq, 1.0, out_dtype=torch.bfloat16)
            if ev: ev[1].record()
    return out


def e2e_step(host_inputs, device, dev_bufs, host_out, side=None):
    """Same path through the public API with HOST buffers: every call's inputs (q and k in fp32, v in
    bf16) are copied from pinned host memory and its result is copied back, inside the timed region.  The copies run
    on two side streams (`side` = (h2d_stream, d2h_stream)) so that the upload of the next call,
    this call's kernels and the download of the previous result overlap; every buffer reuse is
    ordered by events, and the calling stream joins both side streams before returning."""
    from VAR_Q.attention import attend_cached
    main = torch.cuda.current_stream(device)
    up, down = side if side is not None else (main, main)
    h2d = d2h = 0
    in_free = [None] * len(host_inputs)          # recorded on `main` once a scale's device inputs have been consumed
    for kq, vq in new_quantizers():
        for si, rec in enumerate(host_inputs):
            buf = dev_bufs[si]
            with torch.cuda.stream(up):
                if in_free[si] is not None:
                    up.wait_event(in_free[si])
                buf["q"].copy_(rec["q"], non_blocking=True)
                buf["k"].copy_(rec["k"], non_blocking=True)
                buf["v16"].copy_(rec["v16"], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(up)
            h2d += rec["q"].numel() * 4 + rec["k"].numel() * 4 + rec["v16"].numel() * 2
            main.wait_event(ready)
            kq.append(buf["k"])
            vq.append(buf["v16"])
            out = attend_cached(buf["q"], kq, vq, 1.0, out_dtype=torch.bfloat16)
            in_free[si] = torch.cuda.Event()
            in_free[si].record(main)
            down.wait_event(in_free[si])
            with torch.cuda.stream(down):
                host_out[si].copy_(out, non_blocking=True)
            out.record_stream(down)
            d2h += out.numel() * 2
    main.wait_stream(up)
    main.wait_stream(down)
    return h2d, d2h


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while alive."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz, self._stop_evt = index, [], set(), None, threading.Event()

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(vis.split(",")[self.index]) if vis and vis.split(",")[self.index].isdigit() else self.index
            h = nv.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {
                getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
                getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
                getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
                getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
            }
            while not self._stop_evt.is_set():
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
                time.sleep(0.05)
        except Exception as exc:     # clocks are evidence, not a dependency of the measurement
            self.reasons.add(f"nvml_unavailable:{type(exc).__name__}")

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1400.0, "source": "fallback"}


def run_ours(args):
    import torch.distributed as dist
    from VAR_Q import _cabi
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    lib = _cabi.lib()
    inputs, host_inputs = make_inputs(device, seed=rank, pin_host=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up; the first warm-up step is probed to find the kernel that dominates
    tot = {}
    def probe_all(kind, si):
        ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        tot.setdefault((kind, si), []).append(ev)
        return ev
    n_warm = max(args.warmup, 3)
    for w in range(n_warm):
        hot_path_step(inputs, probe_all if w == n_warm - 1 else None)   # the first steps pay one-off set-up costs
    torch.cuda.synchronize()
    share = {k: sum(a.elapsed_time(b) for a, b in v) for k, v in tot.items()}
    top = max(share, key=share.get)

    # ---- the step's launches are static, so they are captured once in a CUDA graph and replayed
    graph, launches_per_step = None, None
    if not args.no_graph:
        n0 = lib.varq_launch_count()
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            hot_path_step(inputs)                      # allocator warm-up on the capture stream
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize()
        n0 = lib.varq_launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            graph_out = hot_path_step(inputs)
        launches_per_step = lib.varq_launch_count() - n0
        for _ in range(2):
            graph.replay()
        torch.cuda.synchronize()

    # ---- timed region: K steps, events on the launching stream, clocks sampled alongside
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    n0 = lib.varq_launch_count()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        if graph is not None:
            graph.replay()
        else:
            hot_path_step(inputs)
    t1.record()
    barrier()
    launches = launches_per_step * args.steps if graph is not None else lib.varq_launch_count() - n0
    clocks = sampler.stop()
    ms = t0.elapsed_time(t1)

    # ---- the dominant kernel alone: back-to-back launches on the state it sees in the step, so that
    # the CUDA events measure the kernel and not the Python between launches
    from VAR_Q.attention import attend_cached
    kind, si = top
    kq, vq = new_quantizers()[0]
    for rec in inputs[:si]:
        kq.append(rec["k"]); vq.append(rec["v"])
    rec = inputs[si]
    if kind == "attn":
        kq.append(rec["k"]); vq.append(rec["v"])
        launch = lambda: attend_cached(rec["q"], kq, vq, 1.0, out_dtype=torch.bfloat16)
    elif kind == "quant_k":
        launch = lambda: kq.quant(rec["k"])          # re-quantizes the pending step in place
    else:
        launch = lambda: vq.quant(rec["v"])
    reps = 20
    for _ in range(3):
        launch()
    torch.cuda.synchronize()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for _ in range(reps):
        launch()
    k1.record()
    torch.cuda.synchronize()
    top_ms = k0.elapsed_time(k1) / reps

    # ---- end to end with host buffers
    dev_bufs = [{"q": torch.empty_like(r["q"]), "k": torch.empty_like(r["k"]), "v16": torch.empty_like(r["v"], memory_format=torch.contiguous_format)}
                for r in inputs]
    host_out = [torch.empty((B2, l, HEADS, HEAD_DIM), dtype=torch.bfloat16).pin_memory() for l in STEPS_L]
    e2e_steps = max(1, min(args.steps, 2))
    side = (torch.cuda.Stream(device), torch.cuda.Stream(device))
    e2e_step(host_inputs, device, dev_bufs, host_out, side)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        h2d, d2h = e2e_step(host_inputs, device, dev_bufs, host_out, side)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)

    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()

    if rank == 0:
        peaks = load_peaks()
        kind, si = top
        lq, lk = STEPS_L[si], sum(STEPS_L[:si + 1])
        if kind == "attn":
            nbytes = algorithmic_bytes_attn(lq, lk)
            flops = 4 * B2 * HEADS * lq * lk * HEAD_DIM
            tensor_bound = flops / nbytes > peaks["tflops"] * 1e12 / (peaks["hbm_gbs"] * 1e9)
        else:
            nbytes, flops, tensor_bound = algorithmic_bytes_quant(lq, 4 if kind == "quant_k" else 2), 0, False
        if tensor_bound:
            ach = flops / (top_ms * 1e-3) / 1e12
            roof = {"bound": "tensor", "achieved": ach, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": ach / peaks["tflops"]}
        else:
            ach = nbytes / (top_ms * 1e-3) / 1e9
            roof = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"]}
        # DRAM bytes per launch from one ncu capture of this kernel at a quarter of the batch
        # (profiles/attn_tc_kernel_var_d16_last_scale.md: 39.2 MB read + 0.03 MB written; traffic scales with batch)
        traffic = 4 * (39217664 + 33792) if (kind, si) == ("attn", len(STEPS_L) - 1) else None
        roof.update({"traffic": traffic, "kernel": f"{kind}[scale {si}: l={lq}, cached={lk}]", "launch_ms": top_ms,
                     "share_of_step": share[top] / sum(share.values()), "peak_source": peaks["source"],
                     "timing": "CUDA events around 20 back-to-back launches of this kernel on the step's own state",
                     "algorithmic_bytes": nbytes, "algorithmic_flops": flops})
        value = world * IMAGES * args.steps / (ms * 1e-3)
        line = {
            "metric": "kv_hot_path_images_per_sec", "value": value, "unit": "images/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 codes, fp32 accumulate",
            "data": "synthetic", "impl": "ours",
            "config": {"workload": WORKLOAD, "images_per_gpu": IMAGES, "tokens": L_TOTAL,
                       "l2": "per-step inputs total 624 MB > 126 MB L2, no explicit flush",
                       "launch": "eager" if graph is None else "CUDA graph of one step, replayed"},
            "clocks": clocks, "gpu_launches": int(launches),
            "e2e": {"value": world * IMAGES * e2e_steps / (e2e_ms * 1e-3), "unit": "images/s",
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": e2e_steps},
            "roofline": roof,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(sample_blocks=12)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------- CPU arm
def cpu_blocks(host_inputs, blocks):
    """The reference algorithm (CPU restatement) for `blocks` blocks of the workload."""
    from oracle import varq_oracle as O
    out = None
    for _ in range(blocks):
        kq, vq = O.OracleVARQ(8, "BLHc", "G_TOKEN_HEAD"), O.OracleVARQ(8, "BLHc", "G_TOKEN_HEAD")
        for rec in host_inputs:
            k = kq.use_var_q(rec["k"])
            v = vq.use_var_q(rec["qkv16"][:, :, 2])
            out = O.attention(rec["q"], k, v, "BLHc", 1.0)
    return out


def cpu_baseline(sample_blocks=1, host_inputs=None):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    host_inputs = host_inputs or make_inputs(None, seed=0)
    t0 = time.perf_counter()
    cpu_blocks(host_inputs, sample_blocks)
    dt = time.perf_counter() - t0
    return {"value": IMAGES / (dt * DEPTH / sample_blocks), "unit": "images/s", "cores": cores, "kind": "port",
            "sample": f"{sample_blocks} of {DEPTH} blocks of the same workload ({dt:.1f} s), scaled by {DEPTH}/{sample_blocks}"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    host_inputs = make_inputs(None, seed=0)
    blocks = 1
    for _ in range(min(args.warmup, 3)):
        cpu_blocks(host_inputs, blocks)
    steps = max(1, min(args.steps, 60))          # one block is about a second of all host cores
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_blocks(host_inputs, blocks)
    dt = (time.perf_counter() - t0) / steps
    value = IMAGES / (dt * DEPTH / blocks)
    sample = f"each step = {blocks} of {DEPTH} blocks of the workload on {cores} host threads, scaled by {DEPTH}/{blocks}; {steps} steps timed"
    print(json.dumps({
        "impl": "reference", "metric": "kv_hot_path_images_per_sec", "value": value, "unit": "images/s",
        "n_gpus": world, "steps": steps, "warmup": min(args.warmup, 3), "ms_per_step": dt * DEPTH / blocks * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "CPU restatement of the reference algorithm (the reference is Python and cannot travel to the GPU box)"},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def run_case(name):
    """One kernel on a small, larger-than-L2 case, a few launches: the command ncu captures."""
    from VAR_Q.attention import attend_cached
    from VAR_Q.quant import VAR_Q
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    if name == "attn":        # the step's last scale at a quarter of the batch: 512 CTAs of the tensor-core kernel
        B, lq, lk = 16, STEPS_L[-1], L_TOTAL
        kq = VAR_Q(8, "BLHc", "G_TOKEN_HEAD", max_tokens=lk)
        vq = VAR_Q(8, "BLHc", "G_TOKEN_HEAD", max_tokens=lk)
        kq.append(torch.nn.functional.normalize(torch.randn((B, lk, HEADS, HEAD_DIM), generator=g, device=dev), dim=-1))
        vq.append(torch.randn((B, lk, HEADS, HEAD_DIM), generator=g, device=dev).to(torch.bfloat16))
        q = torch.nn.functional.normalize(torch.randn((B, lq, HEADS, HEAD_DIM), generator=g, device=dev), dim=-1) * Q_GAIN
        fn = lambda: attend_cached(q, kq, vq, 1.0, out_dtype=torch.bfloat16)
        nbytes = None
    else:                     # "quant": 252 MB of fp32 K, per-head INT8, batch-shared groups; "quant2": per-dim groups (two passes)
        x = torch.randn((128, 256, 30, 64), generator=g, device=dev)
        qz = VAR_Q(8, "BLHc", "G_TOKEN_HEAD" if name == "quant" else "G_SCALE_HEAD_DIM", max_tokens=256)
        fn = lambda: qz.quant(x)
        nbytes = x.numel() * 5
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(); fn(); e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    print(json.dumps({"case": name, "ms": ms, "GB/s": None if nbytes is None else nbytes / ms / 1e6}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from Python instead of replaying a CUDA graph")
    ap.add_argument("--case", choices=("attn", "quant", "quant2"), help="run one kernel on a small case and exit (profiling aid)")
    args = ap.parse_args()
    if args.case:
        return run_case(args.case)
    if args.impl == "reference":
        run_reference(args)
    else:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device (the library has no CPU path; use --impl reference for the CPU arm)")
        run_ours(args)


if __name__ == "__main__":
    main()
