#!/usr/bin/env python
"""Benchmark of the fused forward (the headline), with the other benchmark configurations beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the fused forward kernel over one batch of 65,536 synthetic 28x28 fp32
images (benchmark configuration 2) per GPU.  At N > 1 (launched by torch.distributed.run, one rank per
GPU) every rank runs the same per-GPU batch on its own shard of the synthetic stream with no
communication (inference shards by image; weak scaling), and the time is the max over ranks.

Keys of the JSON line (rank 0 prints exactly one line on stdout):
  value          images/s with inputs resident in HBM, CUDA-event timed (exact-fp32 kernel)
  e2e / e2e_u8   images/s through cnn_forward_batched[_u8]_host with pinned HOST buffers: H2D of the
                 images, the kernel and D2H of sigmoids + argmax all inside the timed region
  roofline       dominant kernel against the measured HBM copy bandwidth, from the algorithmic
                 3,180 B / image
  forward_paths  the same launch through the tensor-core forward kernels (option "forward_path")
  config1        per-sample SGD, 10,000 images, one epoch, then 2,000 test images (rank 0)
  config3        16,777,216 images generated on the device, split over the ranks (strong scaling)
  config4        minibatch SGD, batch 256 per GPU, 60,000 images, ten epochs, gradient exchange fused
                 into the update kernel (peer stores over NVLink); NCCL timing of the same step beside
                 it; at N > 1 a parity check (ranks bit-identical, oracle, single-GPU run)
  config5        widened net, batch 1,024 per GPU, forward + backward + update
  cpu_baseline   the CPU oracle (a C restatement of the reference's kernels; the reference has no CPU
                 implementation of this net) on the host cores, bounded samples (N = 1 only)

``--impl reference`` times the reference path on the host cores (the oracle port with all host
threads) on the same workload, plus -- when a GPU and the prebuilt unmodified reference kernels are
present -- the reference's own per-sample CUDA launch sequence on configuration 1.
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
CONFIG3_IMAGES = 16777216
CONFIG1_TRAIN, CONFIG1_TEST = 10000, 2000
CONFIG4_IMAGES, CONFIG4_PER_GPU, CONFIG4_EPOCHS = 60000, 256, 10

SIGMOID_NAMES = {0: "reference expression (expf + IEEE divide)",
                 1: "short form: ex2.approx + rcp.approx (~1e-6 rel per evaluation)"}

# dram__bytes_read.sum + dram__bytes_write.sum of one launch over 65,536 images, per forward path,
# from the ncu captures summarised under profiles/ (k_fused_forward_*, k_forward_tc_*).
TRAFFIC_BYTES_PER_LAUNCH = {0: 210611456, 1: 211582976, 2: 211068160}


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def measured_bf16_tflops():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"])
    except Exception:
        return 1590.0


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
# CPU legs (the oracle port; only the functions of this section touch oracle/)
# --------------------------------------------------------------------------------------------------
def _oracle():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_binding as ob
    return ob


def cpu_forward_rate(pkg, params, budget_s: float, threads: int):
    """images/s of the oracle's batched forward on `threads` host threads over a bounded sample."""
    ob = _oracle()
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


def cpu_config1(pkg, params):
    """Benchmark configuration 1 on the CPU oracle, single thread (per-sample SGD is a strict chain):
    one epoch over 10,000 images, then the 2,000 test images."""
    ob = _oracle()
    images, labels = pkg.synth.synth_images(0, CONFIG1_TRAIN + CONFIG1_TEST)
    t = time.perf_counter()
    p, mean_err, _ = ob.train_persample(params, images[:CONFIG1_TRAIN], labels[:CONFIG1_TRAIN], 1)
    sec = time.perf_counter() - t
    _, arg = ob.forward_batch(p, images[CONFIG1_TRAIN:], threads=1)
    acc = float((arg == labels[CONFIG1_TRAIN:].astype(np.int32)).mean())
    return {"train_images_per_s": CONFIG1_TRAIN / sec, "cores": 1, "mean_err": float(mean_err[0]),
            "test_accuracy": acc, "images": CONFIG1_TRAIN, "test_images": CONFIG1_TEST}, p


def cpu_config4_one_epoch(pkg, params, global_batch: int, world: int, images=None, labels=None):
    """One epoch of benchmark configuration 4 on the CPU oracle (OpenMP over the images of a batch): the timed
    CPU baseline of minibatch training, and the checker of the data-parallel GPU run."""
    ob = _oracle()
    if images is None:
        images, labels = pkg.synth.synth_images(3, CONFIG4_IMAGES)
    t = time.perf_counter()
    p, me = ob.train_minibatch(params, images, labels, global_batch, 1, world=world)
    sec = time.perf_counter() - t
    return p, float(me[0]), sec


def run_reference_arm(args):
    """The reference path on the host cores: the oracle port (the reference ships no CPU code for
    this net; CNN.py is a different network), all host threads, bounded sample per step."""
    rank, local_rank, world = dist_env()
    if rank != 0:
        return
    pkg = entry.load_package()
    ob = _oracle()
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
        "config": {"workload": "benchmark configuration 2: fused forward, 65,536 synthetic 28x28 fp32 images per GPU per step",
                   "sample_images_per_step": n},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": threads, "kind": "port",
                         "sample": "%d images per step (of 65,536), OpenMP over images on all host threads" % n},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    # Extra: benchmark configuration 1 on the CPU port and on the reference's own per-sample CUDA launch sequence
    # (unmodified layer.cu), the denominator of the per-sample training speed-up.
    try:
        c1, _ = cpu_config1(pkg, params)
        line["config1_cpu_port"] = c1
    except Exception as e:  # pragma: no cover
        line["config1_cpu_port"] = {"unavailable": repr(e)[:200]}
    try:
        import torch
        if torch.cuda.is_available() and ob.reference_available():
            timg, tlab = pkg.synth.synth_images(0, CONFIG1_TRAIN + CONFIG1_TEST)
            ref = ob.Reference(0)
            ref.set_params(params)
            ref.time_train(timg[:200], tlab[:200])
            ref.time_classify(timg[:200])
            ref.set_params(params)
            sec_t, mean_err = ref.time_train(timg[:CONFIG1_TRAIN], tlab[:CONFIG1_TRAIN])
            sec_i, preds = ref.time_classify(timg[CONFIG1_TRAIN:])
            acc = float((preds.astype(np.int64) == tlab[CONFIG1_TRAIN:].astype(np.int64)).mean())
            ref.close()
            line["reference_cuda_path"] = {
                "what": "benchmark configuration 1 on the unmodified reference kernels, per-sample launch sequence of "
                        "main.cu (wall clock, device-synchronised): one epoch over 10,000 images, then 2,000 test images",
                "train_images_per_s": CONFIG1_TRAIN / sec_t, "infer_images_per_s": CONFIG1_TEST / sec_i,
                "mean_err": mean_err, "test_accuracy": acc, "images": CONFIG1_TRAIN, "test_images": CONFIG1_TEST}
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


def shutdown(world: int) -> None:
    """Orderly end of a rank: everything queued on the device has finished, no CUDA graph is alive,
    the process group is destroyed, and the interpreter then exits the normal way (exit handlers
    run).  A watchdog ends the process with a non-zero code if the teardown has not finished after a
    minute, so a stuck rank cannot hang the job."""
    import gc
    import torch
    gc.collect()
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    if world > 1:
        import torch.distributed as dist
        watchdog = threading.Timer(60.0, lambda: os._exit(3))
        watchdog.daemon = True
        watchdog.start()
        dist.barrier()
        torch.cuda.synchronize()
        dist.destroy_process_group()
        watchdog.cancel()


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
    net.set_option("forward_path", args.forward_path)
    # -1 = the library's default: the three-pass tensor-core kernel from 6,144 images per call on
    eff_path = args.forward_path if args.forward_path >= 0 else (1 if (args.fast_sigmoid and BATCH >= 6144) else 0)
    stream = torch.cuda.current_stream()
    peak, peak_kind = measured_peak_gbs()
    n_sm = torch.cuda.get_device_properties(local_rank).multi_processor_count

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

    def time_forward(fnet, steps, warmup):
        """(total ms over `steps` launches, mean ms per launch) with CUDA events on the launching stream."""
        for i in range(max(warmup, 3)):
            fnet.forward(bufs[i % N_ROTATING], BATCH, d_out, d_arg, stream)
        barrier()
        events = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        events[0].record(stream)
        for i in range(steps):
            fnet.forward(bufs[i % N_ROTATING], BATCH, d_out, d_arg, stream)
            events[i + 1].record(stream)
        barrier()
        total = events[0].elapsed_time(events[-1])
        return total, float(np.mean([events[i].elapsed_time(events[i + 1]) for i in range(steps)]))

    t_clock0 = time.perf_counter()
    total_ms, kernel_ms = time_forward(net, args.steps, args.warmup)
    # identical untimed continuation so that the 20 ms clock sampler sees the kernel under load
    t_end = time.perf_counter() + (0.0 if args.only_forward else 1.0)
    i = 0
    while time.perf_counter() < t_end:
        for _ in range(50):
            net.forward(bufs[i % N_ROTATING], BATCH, d_out, d_arg, stream)
            i += 1
        torch.cuda.synchronize()
    t_clock1 = time.perf_counter()
    clocks = sampler.summary(t_clock0, t_clock1)
    assert net.status() == 0

    total_ms = max_over_ranks(total_ms)
    value = world * BATCH * args.steps / (total_ms * 1e-3)
    achieved = BYTES_PER_IMAGE * BATCH / (kernel_ms * 1e-3) / 1e9
    sm_clock_ghz = (clocks.get("sm_mhz") or 1965.0) / 1e3
    fp32_peak = n_sm * 128 * 2 * sm_clock_ghz * 1e9

    if args.only_forward:
        # profiling mode: the forward launches only (used under ncu); prints a reduced line
        sampler.stop()
        if rank == 0:
            emit({"metric": METRIC, "value": value, "unit": "images/s", "n_gpus": world,
                  "steps": args.steps, "kernel_ms": kernel_ms, "only_forward": True,
                  "forward_path": eff_path})
        shutdown(world)
        return

    extra = {}

    # ---- the same launch through the other forward kernels --------------------------------------------
    def forward_paths_leg():
        names = {0: "exact fp32 on the CUDA cores (k_fused_forward)",
                 1: "conv on tcgen05, three tf32 passes (k_forward_tc<1>), 1e-5 parity",
                 2: "conv on tcgen05, one tf32 pass + tanh.approx sigmoid (k_forward_tc<2>), reduced precision"}
        res = {}
        for path in (0, 1, 2):
            fnet = pkg.Net(0)
            fnet.set_params(params)
            fnet.set_fast_sigmoid(args.fast_sigmoid)
            fnet.set_option("forward_path", path)
            tot, per = time_forward(fnet, 20, 3)
            tot = max_over_ranks(tot)
            assert fnet.status() == 0
            res["path%d" % path] = {
                "what": names[path], "images_per_s": world * BATCH * 20 / (tot * 1e-3), "kernel_ms": per,
                "frac_of_hbm_roofline": BYTES_PER_IMAGE * BATCH / (per * 1e-3) / 1e9 / peak}
        return res

    # ---- benchmark configuration 3: 16,777,216 images split over the ranks -------------------------------------
    def config3_leg():
        lo3, hi3 = parallel.shard_range(CONFIG3_IMAGES, rank, world)
        cnt = hi3 - lo3
        d_img3 = torch.empty((cnt, 28, 28), dtype=torch.float32, device="cuda")
        d_out3 = torch.empty((cnt, 10), dtype=torch.float32, device="cuda")
        d_arg3 = torch.empty((cnt,), dtype=torch.int32, device="cuda")
        pkg.synth_images_device(2, lo3, cnt, d_img3, None, stream)
        torch.cuda.synchronize()
        res = {}
        for path in (0, 1, 2):
            fnet = pkg.Net(0)
            fnet.set_params(params)
            fnet.set_option("forward_path", path)
            fnet.forward(d_img3, min(cnt, 4 * BATCH), d_out3, d_arg3, stream)      # warm-up on a slice
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            fnet.forward(d_img3, cnt, d_out3, d_arg3, stream)
            e1.record(stream)
            barrier()
            ms = max_over_ranks(e0.elapsed_time(e1))
            assert fnet.status() == 0
            hist = torch.bincount(d_arg3.long(), minlength=10)
            if world > 1:
                dist.all_reduce(hist)
            res["path%d" % path] = {"images_per_s": CONFIG3_IMAGES / (ms * 1e-3), "ms": ms,
                                    "frac_of_hbm_roofline": BYTES_PER_IMAGE * CONFIG3_IMAGES / (ms * 1e-3) / 1e9 / (peak * world),
                                    "argmax_histogram": [int(x) for x in hist.tolist()]}
        del d_img3, d_out3, d_arg3
        torch.cuda.empty_cache()
        return {"what": "benchmark configuration 3: 16,777,216 synthetic images of seed 2 generated on the device, contiguous "
                        "index ranges over the ranks, no communication; aggregate = images / max-over-ranks time",
                "images": CONFIG3_IMAGES, "images_per_gpu": cnt, "scaling": "strong", "gpus": world, **res}

    # ---- benchmark configuration 1: per-sample SGD (does not shard: rank 0 only) -------------------------------
    def config1_leg():
        d_img1 = torch.empty((CONFIG1_TRAIN + CONFIG1_TEST, 28, 28), dtype=torch.float32, device="cuda")
        d_lab1 = torch.empty((CONFIG1_TRAIN + CONFIG1_TEST,), dtype=torch.int32, device="cuda")
        pkg.synth_images_device(0, 0, CONFIG1_TRAIN + CONFIG1_TEST, d_img1, d_lab1, stream)
        pnet = pkg.Net(0)
        pnet.set_params(params)
        pnet.train_sgd_persample(d_img1, d_lab1, 500, 1)
        best = None
        for _ in range(3):
            pnet.set_params(params)
            t0 = time.perf_counter()
            ran, mean_err = pnet.train_sgd_persample(d_img1, d_lab1, CONFIG1_TRAIN, 1)
            sec = time.perf_counter() - t0
            best = sec if best is None else min(best, sec)
        d_arg1 = torch.empty((CONFIG1_TEST,), dtype=torch.int32, device="cuda")
        pnet.forward(d_img1[CONFIG1_TRAIN:], CONFIG1_TEST, None, d_arg1, stream)
        torch.cuda.synchronize()
        acc = float((d_arg1 == d_lab1[CONFIG1_TRAIN:]).float().mean().item())
        phases = pkg.persample_phase_clocks()      # None unless the library was built with CNN_PHASE_CLOCKS
        if phases is not None:
            rel = phases / CONFIG1_TRAIN
            rel = rel - rel[0, 0]
            extra_phase = {"phase_clocks": {"note": "mean SM clock of each warp of CTA 0 at each stamp, cycles after warp 0 "
                                                     "reaches the top of the loop; the stamps slow the kernel down",
                                            "stamps": list(pkg.PHASE_CLOCK_STAMPS),
                                            "warps": [[round(float(v), 1) for v in rel[w, :len(pkg.PHASE_CLOCK_STAMPS)]]
                                                      for w in range(4)]}}
        else:
            extra_phase = {}
        return {**extra_phase, "what": "benchmark configuration 1: per-sample SGD in file order over 10,000 images (one persistent cluster of "
                        "six CTAs; does not shard), then argmax over 2,000 test images; labels are uniform random, so "
                        "accuracy is chance level for every arm",
                "train_images_per_s": CONFIG1_TRAIN / best, "us_per_sample": 1e6 * best / CONFIG1_TRAIN,
                "mean_err": float(mean_err[0]), "test_accuracy": acc, "epochs": ran,
                "images": CONFIG1_TRAIN, "test_images": CONFIG1_TEST}, pnet.get_params()

    # ---- benchmark configuration 4: minibatch SGD, data parallel -----------------------------------------------
    def config4_leg(oracle_check):
        n_train, gb = CONFIG4_IMAGES, CONFIG4_PER_GPU * world
        d_timg = torch.empty((n_train, 28, 28), dtype=torch.float32, device="cuda")
        d_tlab = torch.empty((n_train,), dtype=torch.int32, device="cuda")
        pkg.synth_images_device(3, 0, n_train, d_timg, d_tlab, stream)
        tnet = pkg.Net(0)
        tnet.set_params(params)
        dp = pkg.DataParallel(tnet, rank, world, parallel.handle_exchange(dist) if world > 1 else None)
        d_me = torch.zeros(1, dtype=torch.float32, device="cuda")
        dp.train_minibatch(d_timg, d_tlab, min(n_train, 8 * gb), gb, 1, 0.1, d_me, stream)      # warm-up
        torch.cuda.synchronize()
        if tnet.status() != 0:      # a bounded wait of the exchange ran out: report it instead of timing failed steps
            raise RuntimeError("data-parallel exchange timed out during warm-up (rank %d of %d)" % (rank, world))
        barrier()
        res = {"global_batch": gb, "images": n_train, "epochs": CONFIG4_EPOCHS,
               "what": "benchmark configuration 4: fused fwd+bwd gradient kernel, then one kernel that reduces the rows, "
                       "exchanges the 2,368-float vector by peer stores over NVLink, adds the ranks in fixed order "
                       "and applies the update" if world > 1 else
                       "benchmark configuration 4: fused fwd+bwd gradient kernel, then one reduce + update kernel (single GPU)"}
        # One epoch = one CUDA graph (two kernels per step): a step is a few microseconds of GPU work.
        tnet.set_params(params)
        graph = None
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    dp.train_minibatch(d_timg, d_tlab, n_train, gb, 1, 0.1, d_me, torch.cuda.current_stream())
            torch.cuda.current_stream().wait_stream(side)
            res["launch"] = "each epoch replayed as one CUDA graph"

            def run_epoch():
                graph.replay()
        except Exception as ge:  # pragma: no cover
            graph = None
            res["launch"] = "eager launches (graph capture failed: %s)" % repr(ge)[:120]

            def run_epoch():
                dp.train_minibatch(d_timg, d_tlab, n_train, gb, 1, 0.1, d_me, stream)

        # parity: one epoch from the initial parameters
        barrier()
        tnet.set_params(params)
        run_epoch()
        torch.cuda.synchronize()
        assert tnet.status() == 0
        p1 = torch.from_numpy(tnet.get_params()).cuda()
        if world > 1:
            allp = [torch.empty_like(p1) for _ in range(world)]
            dist.all_gather(allp, p1)
            identical = all(torch.equal(allp[0], a) for a in allp)
        else:
            identical = True
        check = {"ranks_bit_identical_after_one_epoch": bool(identical)}
        if rank == 0 and oracle_check is not None:
            p_or, me_or = oracle_check
            scale = float(np.max(np.abs(p_or)))
            check["vs_oracle_params"] = float(np.max(np.abs(p1.cpu().numpy() - p_or)) / scale)
            check["mean_err_epoch1"] = float(d_me.item())
            check["oracle_mean_err_epoch1"] = me_or
            check["within_2e-5_of_oracle"] = bool(check["vs_oracle_params"] < 2e-5)
        if rank == 0 and world > 1:
            single = pkg.Net(0)
            single.set_params(params)
            single.train_minibatch(d_timg, d_tlab, n_train, gb, 1, 0.1, None, stream)
            torch.cuda.synchronize()
            p_s = single.get_params()
            check["vs_single_gpu_same_global_batch"] = float(np.max(np.abs(p1.cpu().numpy() - p_s)) / float(np.max(np.abs(p_s))))
        res["parity"] = check
        assert identical, "data-parallel ranks diverged"

        # timing: ten epochs from the initial parameters
        tnet.set_params(params)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        me_hist = torch.zeros(CONFIG4_EPOCHS, dtype=torch.float32, device="cuda")
        e0.record(stream)
        for ep in range(CONFIG4_EPOCHS):
            run_epoch()
            me_hist[ep:ep + 1].copy_(d_me)
        e1.record(stream)
        barrier()
        ms = max_over_ranks(e0.elapsed_time(e1))
        assert tnet.status() == 0
        steps_per_epoch = (n_train + gb - 1) // gb
        d_targ = torch.empty((CONFIG1_TEST,), dtype=torch.int32, device="cuda")
        tnet.forward(d_timg, CONFIG1_TEST, None, d_targ, stream)
        torch.cuda.synchronize()
        res.update({"images_per_s": CONFIG4_EPOCHS * n_train / (ms * 1e-3), "ms": ms,
                    "us_per_step": 1e3 * ms / (CONFIG4_EPOCHS * steps_per_epoch), "steps_per_epoch": steps_per_epoch,
                    "mean_err_per_epoch": [float(x) for x in me_hist.cpu().tolist()],
                    "train_accuracy_first_2000": float((d_targ == d_tlab[:CONFIG1_TEST]).float().mean().item()),
                    "frac_of_hbm_roofline": (3140 * CONFIG4_EPOCHS * n_train / (ms * 1e-3) / 1e9) / (peak * world)})
        graph = None     # nothing captured stays alive past this leg
        dp.close()

        # the portable fallback beside it: the same step with NCCL's all-reduce (eager launches)
        if world > 1:
            fnet = pkg.Net(0)
            fnet.set_params(params)
            d_grad = torch.zeros(2368, dtype=torch.float32, device="cuda")
            trainer = parallel.DataParallelTrainer(
                rank, world, lambda a, b, out: fnet.grad_batch(d_timg[a:], d_tlab[a:], b - a, out, stream),
                lambda g, s: fnet.apply_update(g, s, stream), lambda t: dist.all_reduce(t), d_grad, dt=0.1)
            trainer.epoch(8 * gb, gb)
            barrier()
            e0.record(stream)
            steps_n = trainer.epoch(n_train, gb)
            e1.record(stream)
            barrier()
            ms_n = max_over_ranks(e0.elapsed_time(e1))
            res["nccl_fallback"] = {"images_per_s": n_train / (ms_n * 1e-3), "us_per_step": 1e3 * ms_n / steps_n,
                                    "what": "gradient kernel, row reduction, NCCL all-reduce of 2,368 floats, update; eager launches, one epoch"}
        if rank == 0:
            big = 57344
            fnet = pkg.Net(0)
            fnet.set_params(params)
            d_grad = torch.zeros(2368, dtype=torch.float32, device="cuda")
            fnet.grad_batch(d_timg, d_tlab, big, d_grad, stream)
            torch.cuda.synchronize()
            e0.record(stream)
            for _ in range(5):
                fnet.grad_batch(d_timg, d_tlab, big, d_grad, stream)
            e1.record(stream)
            torch.cuda.synchronize()
            msb = e0.elapsed_time(e1) / 5
            res["grad_large_batch"] = {"images_per_s": big / (msb * 1e-3), "batch": big,
                                       "frac_of_hbm_roofline": (3140 * big / (msb * 1e-3) / 1e9) / peak}
        return res

    def config5_leg(modes=((0, "fp32_simt"), (2, "tf32x3_tcgen05"), (1, "tf32_tcgen05")), steps=5):
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
        return {"what": "benchmark configuration 5: 56x56 input, 64 maps, batch 1,024 per GPU, fwd+bwd+update"
                        + (", NCCL all-reduce of 109,856 floats" if world > 1 else ""), "conv": wide}

    if args.only_wide:
        res = config5_leg(modes=((args.only_wide - 1, "conv_mode_%d" % (args.only_wide - 1)),), steps=args.steps)
        sampler.stop()
        if rank == 0:
            emit({"only_wide": True, "config5": res})
        shutdown(world)
        return

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
        del h_img, h_pix

    # ---- CPU legs first where a GPU leg is checked against them (rank 0) ---------------------------------
    cpu = None
    oracle_check = None
    cpu_extra = {}
    if rank == 0 and not args.only_train:
        try:
            threads = os.cpu_count() or 1
            if world == 1:
                rate, n_s, dt = cpu_forward_rate(pkg, params, 6.0, threads)
                cpu = {"value": rate, "unit": "images/s", "cores": threads, "kind": "port",
                       "sample": "%d of 65,536 images, %.1f s, OpenMP over images (C restatement of layer.cu; "
                                 "the reference has no CPU code for this net)" % (n_s, dt)}
                r1, n1, dt1 = cpu_forward_rate(pkg, params, 2.0, 1)
                cpu["forward_single_thread"] = {"images_per_s": r1, "cores": 1, "sample": "%d images, %.1f s" % (n1, dt1)}
                c1, _ = cpu_config1(pkg, params)
                cpu["config1_persample_sgd"] = c1
            p_or, me_or, sec = cpu_config4_one_epoch(pkg, params, CONFIG4_PER_GPU * world, world)
            oracle_check = (p_or, me_or)
            cpu_extra = {"images_per_s": CONFIG4_IMAGES / sec, "cores": threads, "mean_err_epoch1": me_or,
                         "sample": "one epoch of 60,000 images, global batch %d, OpenMP over the images of a batch, %.1f s"
                                   % (CONFIG4_PER_GPU * world, sec)}
            if cpu is not None:
                cpu["config4_minibatch"] = cpu_extra
        except Exception as e:  # pragma: no cover
            extra["cpu_legs_error"] = repr(e)[:300]
    barrier()

    for name, leg in (("forward_paths", forward_paths_leg), ("config3", config3_leg)):
        if args.only_train:
            continue
        try:
            extra[name] = leg()
        except Exception as e:  # pragma: no cover
            extra[name] = {"error": repr(e)[:300]}
        barrier()
    if rank == 0:
        try:
            extra["config1"], _ = config1_leg()
        except Exception as e:  # pragma: no cover
            extra["config1"] = {"error": repr(e)[:300]}
    barrier()
    try:
        extra["config4"] = config4_leg(oracle_check)
        if world > 1 and cpu_extra:
            extra["config4"]["cpu_port_one_epoch"] = cpu_extra
    except Exception as e:  # pragma: no cover
        extra["config4"] = {"error": repr(e)[:300]}
    barrier()
    if not args.only_train:
        try:
            extra["config5"] = config5_leg()
        except Exception as e:  # pragma: no cover
            extra["config5"] = {"error": repr(e)[:300]}
        barrier()

    sampler.stop()

    if args.only_train:
        if rank == 0:
            emit({"only_train": True, **extra})
        shutdown(world)
        return

    if rank == 0:
        kernel_names = {0: "k_fused_forward", 1: "k_forward_tc<1,1>", 2: "k_forward_tc<2,2>"}
        limits = {0: "fp32 FMA + MUFU pipes and instruction issue, not HBM (58 FLOP/B)",
                  1: "tensor pipe: 60 tf32 MMAs of 128x80x8 per 128 stacked image rows (three passes), then MUFU; not HBM",
                  2: "MUFU pipe (one tanh per conv output) and shared-memory bandwidth; not HBM"}
        roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": TRAFFIC_BYTES_PER_LAUNCH.get(eff_path),
                "peak_kind": "of " + peak_kind, "kernel": kernel_names[eff_path],
                "kernel_ms": kernel_ms, "algorithmic_bytes_per_image": BYTES_PER_IMAGE,
                "binding_limit": limits[eff_path]}
        if eff_path == 0:
            roof["fp32_fma_frac"] = FLOP_PER_IMAGE * BATCH / (kernel_ms * 1e-3) / fp32_peak
        if eff_path in (1, 2):
            # tensor work actually issued (zeros of the banded operand included): MMAs per tile x 2*128*80*8 flop,
            # one tile = 128 stacked rows = 128/28 images; tf32 peak taken as half the measured bf16 burst peak
            mma_flop_per_image = (60 if eff_path == 1 else 20) * 2 * 128 * 80 * 8 / (128.0 / 28.0)
            tf32_peak = 0.5 * measured_bf16_tflops() * 1e12
            roof["tensor_tflops_issued"] = mma_flop_per_image * BATCH / (kernel_ms * 1e-3) / 1e12
            roof["tensor_frac_of_tf32_peak"] = roof["tensor_tflops_issued"] * 1e12 / tf32_peak
            roof["tf32_peak_kind"] = "half of the measured bf16 burst peak"
        line = {
            "metric": METRIC, "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "benchmark configuration 2: fused forward, 65,536 synthetic 28x28 fp32 images per GPU per step",
                       "images_per_gpu_per_step": BATCH, "global_images_per_step": BATCH * world,
                       "l2": "inputs rotate over %d distinct 205.5 MB buffers (> 126 MB L2)" % N_ROTATING,
                       "sigmoid": SIGMOID_NAMES[1 if args.fast_sigmoid else 0],
                       "forward_path": eff_path, "parallelism": "shard by image, no collective"},
            "roofline": roof,
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
        line.update(extra)
        emit(line)
    shutdown(world)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--fast-sigmoid", type=int, default=1)
    ap.add_argument("--forward-path", type=int, default=-1,
                    help="kernel of the headline: -1 the library's default (1 at this batch size), 0 exact fp32 SIMT, "
                         "1 tcgen05 three tf32 passes (1e-5 parity), 2 tcgen05 one pass + tanh (reduced precision)")
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
