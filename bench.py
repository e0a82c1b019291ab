#!/usr/bin/env python
"""Benchmark of the fused forward (the headline), with training legs reported beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the fused forward kernel over one batch of 65,536 synthetic 28x28 fp32
images (benchmark configuration 2) per GPU.  At N > 1 (launched by torch.distributed.run, one rank per GPU)
every rank runs the same per-GPU batch on its own shard of the synthetic stream with no
communication (inference shards by image; weak scaling), and the time is the max over ranks.

Keys of the JSON line (rank 0 prints exactly one line on stdout):
  value     images/s with inputs resident in HBM, CUDA-event timed
  e2e       images/s through cnn_forward_batched_host with pinned HOST buffers: H2D of the images,
            the kernel and D2H of sigmoids + argmax all inside the timed region
  roofline  dominant kernel (k_fused_forward) against the measured HBM copy bandwidth, from the
            algorithmic 3,180 B / image
  cpu_baseline  the CPU oracle (a C restatement of the reference's kernels; the reference has no
            CPU implementation of this net) on the host cores, bounded sample
  train_*   fwd+bwd throughput of the minibatch and per-sample SGD kernels (extra, N-aware)

``--impl reference`` times the reference path on the host cores (the oracle port with all host
threads) on the same workload, plus -- when a GPU and the prebuilt unmodified reference kernels are
present -- the reference's own per-sample CUDA launch sequence as an extra key.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402

BATCH = 65536                 # benchmark configuration 2
BYTES_PER_IMAGE = 3136 + 40 + 4
FLOP_PER_IMAGE = 184032
N_ROTATING = 4                # distinct input buffers (4 x 205.5 MB >> 126 MB L2)
METRIC = "images/sec forward (fused conv-sigmoid-subsample-sigmoid-FC-sigmoid, 28x28 fp32)"


SIGMOID_NAMES = {0: "reference expression (expf + IEEE divide)", 1: "ex2/rcp approx (~1e-6 rel)",
                 2: "reduced-argument ex2 + refined rcp (~1e-7 rel)"}


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock, power and clock-event reasons of one GPU through NVML (read-only) every
    20 ms on a background thread."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting",
               0x10: "sync_boost"}

    def __init__(self, torch_device_index: int):
        self.samples = []
        self.ok = False
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(torch_device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode() if hasattr(uuid, "encode") else uuid)
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception as e:  # pragma: no cover - depends on the box
            self.err = repr(e)

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                sm = int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    reasons = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    reasons = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                try:
                    power = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                except Exception:
                    power = None
                self.samples.append((time.perf_counter(), sm, reasons, power))
            except Exception:
                pass
            self._stop.wait(0.02)

    def start(self):
        if self.ok:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=2)

    def summary(self, t0: float, t1: float) -> dict:
        if not self.ok:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "note": "NVML unavailable: " + getattr(self, "err", "")}
        sel = [s for s in self.samples if t0 <= s[0] <= t1]
        if not sel:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "samples": 0}
        bits = 0
        for s in sel:
            bits |= s[2]
        reasons = sorted(name for bit, name in self.REASONS.items() if bits & bit)
        powers = [s[3] for s in sel if s[3] is not None]
        return {"sm_mhz": float(np.median([s[1] for s in sel])), "sm_max_mhz": self.sm_max,
                "sm_min_mhz": int(min(s[1] for s in sel)), "reasons": reasons, "samples": len(sel),
                "power_w_max": max(powers) if powers else None,
                "sampled_over": "timed steps plus an identical untimed continuation of the same launches"}


def dist_env():
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


# --------------------------------------------------------------------------------------------------
# CPU legs (the oracle port; only these functions touch oracle/)
# --------------------------------------------------------------------------------------------------
def cpu_forward_rate(pkg, params, budget_s: float, threads: int):
    """images/s of the oracle's batched forward on `threads` host threads over a bounded sample."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_binding as ob
    probe, _ = pkg.synth.synth_images(1, 1024)
    ob.forward_batch(params, probe[:64], threads=threads)          # warm up the thread pool
    t = time.perf_counter()
    ob.forward_batch(params, probe, threads=threads)
    rate = 1024 / max(time.perf_counter() - t, 1e-9)
    n = int(min(BATCH, max(1024, rate * budget_s)))
    images, _ = pkg.synth.synth_images(1, n)
    t = time.perf_counter()
    ob.forward_batch(params, images, threads=threads)
    dt = time.perf_counter() - t
    return n / dt, n, dt


def run_reference_arm(args):
    """The reference path on the host cores: the oracle port (the reference ships no CPU code for
    this net; CNN.py is a different network), all host threads, bounded sample per step."""
    rank, local_rank, world = dist_env()
    if rank != 0:
        return
    pkg = entry.load_package()
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_binding as ob
    params = pkg.synth.synth_params(0)
    threads = os.cpu_count() or 1
    probe, _ = pkg.synth.synth_images(1, 2048)
    ob.forward_batch(params, probe[:256], threads=threads)
    t = time.perf_counter()
    ob.forward_batch(params, probe, threads=threads)
    rate = 2048 / max(time.perf_counter() - t, 1e-9)
    total_steps = max(args.steps + args.warmup, 1)
    per_step_budget = min(10.0, 120.0 / total_steps)
    n = int(min(BATCH, max(2048, rate * per_step_budget)))
    images, _ = pkg.synth.synth_images(1, n)
    for _ in range(args.warmup):
        ob.forward_batch(params, images, threads=threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ob.forward_batch(params, images, threads=threads)
    dt = time.perf_counter() - t0
    value = n * args.steps / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "images/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / max(args.steps, 1),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "benchmark configuration 2: fused forward over 65,536 synthetic 28x28 fp32 images",
                   "sample_images_per_step": n},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": threads, "kind": "port",
                         "sample": "%d images per step (of 65,536), OpenMP over images on all host threads" % n},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    # Extra: the reference's own per-sample CUDA launch sequence (unmodified layer.cu), when possible.
    try:
        import torch
        if torch.cuda.is_available() and ob.reference_available():
            timg, tlab = pkg.synth.synth_images(0, 3000)
            ref = ob.Reference(0)
            ref.set_params(params)
            ref.time_classify(timg[:200])
            sec_i, _ = ref.time_classify(timg[:2000])
            ref.set_params(params)
            ref.time_train(timg[:200], tlab[:200])
            ref.set_params(params)
            sec_t, mean_err = ref.time_train(timg, tlab)
            ref.close()
            line["reference_cuda_path"] = {
                "what": "unmodified reference kernels, per-sample launch sequence of main.cu (wall clock, device-synchronised)",
                "infer_images_per_s": 2000 / sec_i, "train_images_per_s": 3000 / sec_t,
                "train_mean_err": mean_err, "infer_sample": 2000, "train_sample": 3000}
    except Exception as e:  # pragma: no cover
        line["reference_cuda_path"] = {"unavailable": repr(e)[:200]}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------
_REAL_STDOUT_FD = None


def quiet_stdout():
    """stdout carries exactly one JSON line: everything else that libraries print on fd 1 (NCCL's
    version banner, for one) is sent to stderr; emit() writes to the saved descriptor."""
    global _REAL_STDOUT_FD
    if _REAL_STDOUT_FD is None:
        sys.stdout.flush()
        _REAL_STDOUT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _REAL_STDOUT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_REAL_STDOUT_FD, data)


def finish(world: int) -> None:
    """Leave without hanging in library teardown: synchronise, give the process group ten seconds to
    shut down cleanly, then exit hard (a CUDA graph that holds NCCL kernels made
    destroy_process_group block on an 8-GPU run)."""
    import torch
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    if world > 1:
        import torch.distributed as dist
        t = threading.Thread(target=dist.destroy_process_group, daemon=True)
        t.start()
        t.join(timeout=10.0)
    os._exit(0)


def run_ours(args):
    import torch
    import torch.distributed as dist

    quiet_stdout()

    rank, local_rank, world = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        # stdout carries exactly one JSON line: keep NCCL's version banner off it
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if local_rank == 0:
        entry.build()
    if world > 1:
        dist.barrier()
    pkg = entry.load_package()
    pkg.load_library()
    from hpcnn_b200 import parallel

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    params = pkg.synth.synth_params(0)
    net = pkg.Net(0)
    net.set_params(params)
    net.set_fast_sigmoid(args.fast_sigmoid)
    net.set_option("fw_variant", args.fw_variant)
    stream = torch.cuda.current_stream()

    # Each rank owns a contiguous shard of the synthetic stream (seed 1), generated on the device.
    lo, _ = parallel.shard_range(world * N_ROTATING * BATCH, rank, world)
    bufs = []
    for r in range(N_ROTATING):
        b = torch.empty((BATCH, 28, 28), dtype=torch.float32, device="cuda")
        pkg.synth_images_device(1, lo + r * BATCH, BATCH, b, None, stream)
        bufs.append(b)
    d_out = torch.empty((BATCH, 10), dtype=torch.float32, device="cuda")
    d_arg = torch.empty((BATCH,), dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()

    def step(i):
        net.forward(bufs[i % N_ROTATING], BATCH, d_out, d_arg, stream)

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()
    events = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    t_clock0 = time.perf_counter()
    events[0].record(stream)
    for i in range(args.steps):
        step(i)
        events[i + 1].record(stream)
    barrier()
    total_ms = events[0].elapsed_time(events[-1])
    per_launch_ms = [events[i].elapsed_time(events[i + 1]) for i in range(args.steps)]
    # identical untimed continuation so that the 20 ms clock sampler sees the kernel under load
    t_end = time.perf_counter() + (0.0 if args.only_forward else 1.0)
    i = 0
    while time.perf_counter() < t_end:
        for _ in range(50):
            step(i)
            i += 1
        torch.cuda.synchronize()
    t_clock1 = time.perf_counter()
    clocks = sampler.summary(t_clock0, t_clock1)
    assert net.status() == 0

    total_ms = max_over_ranks(total_ms)
    value = world * BATCH * args.steps / (total_ms * 1e-3)
    kernel_ms = float(np.mean(per_launch_ms))
    peak, peak_kind = measured_peak_gbs()
    achieved = BYTES_PER_IMAGE * BATCH / (kernel_ms * 1e-3) / 1e9
    sm_clock_ghz = (clocks.get("sm_mhz") or 1965.0) / 1e3
    n_sm = torch.cuda.get_device_properties(local_rank).multi_processor_count
    fp32_peak = n_sm * 128 * 2 * sm_clock_ghz * 1e9

    def run_wide_leg(modes=((0, "fp32_simt"), (2, "tf32x3_tcgen05"), (1, "tf32_tcgen05")), steps=5):
        """benchmark configuration 5: widened net (56x56 input, 64 maps), batch 1,024 per GPU, fwd+bwd+update."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        wide_batch = 1024
        wnet = pkg.WideNet(56, 64)
        rng = np.random.default_rng(4)
        wp = rng.uniform(-0.5, 0.5, wnet.n_params).astype(np.float32)
        wp[64 * 25 + 64 + 17: 64 * 25 + 64 + 17 + 10 * 10816] *= np.float32(6.0 / np.sqrt(10816.0))
        d_wimg = (torch.rand((wide_batch, 56, 56), device="cuda", generator=torch.Generator("cuda").manual_seed(4 + rank))
                  * (torch.rand((wide_batch, 56, 56), device="cuda") < 0.2)).contiguous()
        d_wlab = torch.randint(0, 10, (wide_batch,), dtype=torch.int32, device="cuda")
        d_wgrad = torch.zeros(wnet.n_padded, dtype=torch.float32, device="cuda")
        wide = {}
        for mode, name in modes:
            wnet.set_params(wp)
            wnet.set_option("conv", mode)

            def wstep():
                wnet.grad_batch(d_wimg, d_wlab, wide_batch, d_wgrad, stream)
                if world > 1:
                    dist.all_reduce(d_wgrad)
                wnet.apply_update(d_wgrad, 0.1 / (wide_batch * world), stream)

            wstep()
            barrier()
            e0.record(stream)
            for _ in range(steps):
                wstep()
            e1.record(stream)
            barrier()
            ms = max_over_ranks(e0.elapsed_time(e1)) / steps
            wide[name] = {"images_per_s": wide_batch * world / (ms * 1e-3), "ms_per_step": ms,
                          "tflops": 18992896.0 * wide_batch * world / (ms * 1e-3) / 1e12}
        assert wnet.status() == 0
        return {"what": "benchmark configuration 5: 56x56 input, 64 maps, batch 1,024 per GPU, "
                                            "fwd+bwd+update" + (", NCCL all-reduce of 109,856 floats" if world > 1 else ""),
                                    "conv": wide}

    if args.only_wide:
        res = run_wide_leg(modes=((args.only_wide - 1, "conv_mode_%d" % (args.only_wide - 1)),), steps=args.steps)
        sampler.stop()
        if rank == 0:
            emit({"only_wide": True, "train_wide_cfg5": res})
        finish(world)

    if args.only_forward:
        # profiling mode: the forward launches only (used under ncu); prints a reduced line
        sampler.stop()
        if rank == 0:
            emit({"metric": METRIC, "value": value, "unit": "images/s", "n_gpus": world,
                  "steps": args.steps, "kernel_ms": kernel_ms, "only_forward": True})
        finish(world)

    e2e_value = e2e_u8_value = None
    e2e_steps = 0
    if not args.only_train:
        # ---- e2e: host buffers through the C ABI ----------------------------------------------------
        h_img = torch.empty((BATCH, 28, 28), dtype=torch.float32).pin_memory()
        h_img.copy_(bufs[0])
        h_out = torch.empty((BATCH, 10), dtype=torch.float32).pin_memory()
        h_arg = torch.empty((BATCH,), dtype=torch.int32).pin_memory()
        e2e_steps = max(3, min(args.steps, 20))
        for _ in range(2):
            net.forward_host(h_img, BATCH, h_out, h_arg)
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            net.forward_host(h_img, BATCH, h_out, h_arg)
        torch.cuda.synchronize()
        e2e_s = max_over_ranks(time.perf_counter() - t0)
        e2e_value = world * BATCH * e2e_steps / e2e_s
        barrier()
        # the same call on uint8 pixels (the IDX storage the reference's loader reads): a quarter of the bytes
        h_pix = torch.from_numpy(pkg.synth.synth_pixels_u8(1, 4096)).repeat(BATCH // 4096, 1, 1).contiguous().pin_memory()
        for _ in range(2):
            net.forward_u8_host(h_pix, BATCH, h_out, h_arg)
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            net.forward_u8_host(h_pix, BATCH, h_out, h_arg)
        torch.cuda.synchronize()
        e2e_u8_value = world * BATCH * e2e_steps / max_over_ranks(time.perf_counter() - t0)
        barrier()

    # ---- extra: training legs -------------------------------------------------------------------
    train = {}
    try:
        n_train = 60000
        per_gpu_batch = 256
        lo_t, hi_t = parallel.shard_range(n_train, 0, 1)
        d_timg = torch.empty((n_train, 28, 28), dtype=torch.float32, device="cuda")
        d_tlab = torch.empty((n_train,), dtype=torch.int32, device="cuda")
        pkg.synth_images_device(3, 0, n_train, d_timg, d_tlab, stream)
        tnet = pkg.Net(0)
        tnet.set_params(params)
        d_grad = torch.zeros(2368, dtype=torch.float32, device="cuda")
        gb = per_gpu_batch * world

        def grad_fn(a, b, out):
            tnet.grad_batch(d_timg[a:], d_tlab[a:], b - a, out, stream)

        trainer = parallel.DataParallelTrainer(
            rank, world, grad_fn, lambda g, s: tnet.apply_update(g, s, stream),
            (lambda t: dist.all_reduce(t)) if world > 1 else None, d_grad, dt=0.1)
        trainer.epoch(min(n_train, 20 * gb), gb)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # One epoch = one CUDA graph (gradient kernel, row reduction, all-reduce, update per step):
        # the step is a few microseconds of GPU work, so launch latency would otherwise dominate.
        graph_note = "epoch captured in one CUDA graph"
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                cap_stream = torch.cuda.current_stream()
                trainer.grad_fn = lambda a, b, out: tnet.grad_batch(d_timg[a:], d_tlab[a:], b - a, out, cap_stream)
                trainer.update_fn = lambda g, s: tnet.apply_update(g, s, cap_stream)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    steps_t = trainer.epoch(n_train, gb)
            torch.cuda.current_stream().wait_stream(side)
            graph.replay()
            barrier()
            e0.record(stream)
            graph.replay()
            e1.record(stream)
        except Exception as ge:  # pragma: no cover
            graph_note = "eager launches (graph capture failed: %s)" % repr(ge)[:120]
            trainer.grad_fn = grad_fn
            trainer.update_fn = lambda g, s: tnet.apply_update(g, s, stream)
            torch.cuda.synchronize()
            e0.record(stream)
            steps_t = trainer.epoch(n_train, gb)
            e1.record(stream)
        barrier()
        ms = max_over_ranks(e0.elapsed_time(e1))
        graph = None   # drop the captured epoch (it holds NCCL kernels) before anything else runs
        train["train_minibatch"] = {
            "images_per_s": n_train / (ms * 1e-3), "global_batch": gb, "steps": steps_t,
            "us_per_step": 1e3 * ms / steps_t, "images": n_train, "launch": graph_note,
            "what": "benchmark configuration 4, one epoch: fused fwd+bwd gradient kernel, %s, update"
                    % ("NCCL all-reduce of 2,368 floats" if world > 1 else "single GPU (no collective)"),
            "frac_of_hbm_roofline": (3140 * n_train / (ms * 1e-3) / 1e9) / (peak * world)}
        if rank == 0:
            # large-batch fwd+bwd throughput (compute-bound shape of the same kernel)
            big = 57344
            tnet.grad_batch(d_timg, d_tlab, big, d_grad, stream)
            torch.cuda.synchronize()
            e0.record(stream)
            for _ in range(5):
                tnet.grad_batch(d_timg, d_tlab, big, d_grad, stream)
            e1.record(stream)
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 5
            train["train_grad_large_batch"] = {"images_per_s": big / (ms * 1e-3), "batch": big,
                                               "frac_of_hbm_roofline": (3140 * big / (ms * 1e-3) / 1e9) / peak}
            # per-sample SGD, benchmark configuration 1: 10,000 images, one epoch, one persistent six-CTA cluster
            pnet = pkg.Net(0)
            pnet.set_params(params)
            pnet.train_sgd_persample(d_timg, d_tlab, 500, 1)
            pnet.set_params(params)
            t0 = time.perf_counter()
            ran, mean_err = pnet.train_sgd_persample(d_timg, d_tlab, 10000, 1)
            sec = time.perf_counter() - t0
            train["train_persample"] = {"images_per_s": 10000 / sec, "images": 10000, "epochs": ran,
                                        "mean_err": float(mean_err[0]),
                                        "what": "benchmark configuration 1: per-sample SGD in file order, one persistent cluster of six CTAs (does not shard)"}
            # the same through the option that selects the variant with eight outputs per thread and a
            # service warp (cnn_net_set_option "persample_cluster" = 3)
            pnet.set_option("persample_cluster", 3)
            pnet.set_params(params)
            pnet.train_sgd_persample(d_timg, d_tlab, 500, 1)
            pnet.set_params(params)
            t0 = time.perf_counter()
            ran, mean_err = pnet.train_sgd_persample(d_timg, d_tlab, 10000, 1)
            sec = time.perf_counter() - t0
            train["train_persample_option3"] = {"images_per_s": 10000 / sec, "images": 10000, "epochs": ran,
                                                "mean_err": float(mean_err[0]),
                                                "what": "the same with option persample_cluster = 3 (eight conv outputs per thread, service warp)"}
        barrier()
        if not args.only_train:
            train["train_wide_cfg5"] = run_wide_leg()
        barrier()
    except Exception as e:  # pragma: no cover
        train["train_error"] = repr(e)[:300]

    sampler.stop()

    if args.only_train:
        if rank == 0:
            emit({"only_train": True, **train})
        finish(world)

    if rank != 0:
        finish(world)

    cpu = None
    if world == 1:
        threads = os.cpu_count() or 1
        rate, n_s, dt = cpu_forward_rate(pkg, params, 12.0, threads)
        cpu = {"value": rate, "unit": "images/s", "cores": threads, "kind": "port",
               "sample": "%d of 65,536 images, %.1f s, OpenMP over images (C restatement of layer.cu; "
                         "the reference has no CPU code for this net)" % (n_s, dt)}

    line = {
        "metric": METRIC, "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "benchmark configuration 2: fused forward, 65,536 synthetic 28x28 fp32 images per GPU per step",
                   "images_per_gpu_per_step": BATCH, "global_images_per_step": BATCH * world,
                   "l2": "inputs rotate over %d distinct 205.5 MB buffers (> 126 MB L2)" % N_ROTATING,
                   "sigmoid": SIGMOID_NAMES[args.fast_sigmoid],
                   "fw_variant": args.fw_variant, "parallelism": "shard by image, no collective"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": TRAFFIC_BYTES_PER_LAUNCH,
                     "peak_kind": "of " + peak_kind, "kernel": "k_fused_forward",
                     "kernel_ms": kernel_ms, "algorithmic_bytes_per_image": BYTES_PER_IMAGE,
                     "binding_limit": "fp32 FMA + MUFU pipes, not HBM (58 FLOP/B)",
                     "fp32_fma_frac": FLOP_PER_IMAGE * BATCH / (kernel_ms * 1e-3) / fp32_peak},
        "e2e": {"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": BATCH * 3136,
                "d2h_bytes_per_step": BATCH * 44, "steps": e2e_steps,
                "api": "cnn_forward_batched_host (pinned host buffers, 8,192-image chunks on two streams)"},
        "e2e_u8": {"value": e2e_u8_value, "unit": "images/s", "h2d_bytes_per_step": BATCH * 784,
                   "d2h_bytes_per_step": BATCH * 44, "api": "cnn_forward_batched_u8_host (uint8 pixels, "
                   "pixel/255.0 applied in the kernel; bit-identical results)"},
        "gpu_launches": args.steps * world,
        "clocks": clocks,
    }
    if cpu:
        line["cpu_baseline"] = cpu
    line.update(train)
    emit(line)
    finish(world)


# dram__bytes_read.sum + dram__bytes_write.sum of one k_fused_forward launch over 65,536 images,
# from the ncu capture summarised in profiles/k_fused_forward_cfg2_65536_images.md.
TRAFFIC_BYTES_PER_LAUNCH = 211743488


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--fast-sigmoid", type=int, default=2)
    ap.add_argument("--fw-variant", type=int, default=0)
    ap.add_argument("--only-train", type=int, default=0,
                    help="run only the training legs of the reference net (for ncu launch lists)")
    ap.add_argument("--only-wide", type=int, default=0,
                    help="run only the config-5 leg with conv mode N-1 (1: fp32 SIMT, 2: tf32, 3: 3 x tf32); for ncu")
    ap.add_argument("--only-forward", type=int, default=0,
                    help="run only the forward launches (small, for ncu captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
