"""Data-parallel host logic on CPU ranks: world_size-2 gloo processes run the package's
DataParallelTrainer with the oracle standing in for the GPU gradient kernel, and must end with
bit-identical parameters on both ranks that match a single-rank run to fp32 rounding."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, n, batch, epochs, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import __graft_entry__ as entry
    import oracle_binding as ob
    pkg = entry.load_package()
    from hpcnn_b200 import parallel
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    images, labels = pkg.synth.synth_images(3, n)
    state = {"p": pkg.synth.synth_params(0)}

    def grad_fn(lo, hi, out):
        if hi > lo:
            g, err = ob.grad_batch(state["p"], images[lo:hi], labels[lo:hi], threads=1)
        else:
            g, err = np.zeros(2343, dtype=np.float32), 0.0
        out.zero_()
        out[:2343] = torch.from_numpy(g)
        out[2344] = err

    def update_fn(grad, scale):
        state["p"] = ob.apply_update(state["p"], grad[:2343].numpy(), scale, 1.0)

    trainer = parallel.DataParallelTrainer(rank, world, grad_fn, update_fn,
                                           (lambda t: dist.all_reduce(t)) if world > 1 else None,
                                           torch.zeros(2368, dtype=torch.float32), dt=0.1)
    for _ in range(epochs):
        trainer.epoch(n, batch)
    np.save(os.path.join(out_dir, "params_%d_of_%d.npy" % (rank, world)), state["p"])
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_gloo_ranks_match_single_rank(tmp_path):
    n, batch, epochs = 96, 32, 2
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, n, batch, epochs, str(tmp_path)), nprocs=2, join=True)
    mp.spawn(_worker, args=(1, port + 1, n, batch, epochs, str(tmp_path)), nprocs=1, join=True)
    p0 = np.load(tmp_path / "params_0_of_2.npy")
    p1 = np.load(tmp_path / "params_1_of_2.npy")
    ps = np.load(tmp_path / "params_0_of_1.npy")
    assert np.array_equal(p0, p1), "ranks diverged"
    assert np.max(np.abs(p0 - ps)) / np.max(np.abs(ps)) < 1e-5
    # and the single-rank driver equals the oracle's own minibatch loop
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import __graft_entry__ as entry
    import oracle_binding as ob
    pkg = entry.load_package()
    images, labels = pkg.synth.synth_images(3, n)
    pref, _ = ob.train_minibatch(pkg.synth.synth_params(0), images, labels, batch, epochs)
    assert np.max(np.abs(ps - pref)) / np.max(np.abs(pref)) < 1e-6


def _infer_worker(rank, world, port, n, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import __graft_entry__ as entry
    import oracle_binding as ob
    pkg = entry.load_package()
    from hpcnn_b200 import parallel
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lo, hi = parallel.shard_range(n, rank, world)
    # every rank generates only its own shard of the stream (as bench.py does on the device)
    images, _ = pkg.synth.synth_images(2, hi - lo, first_index=lo)
    out, arg = ob.forward_batch(pkg.synth.synth_params(0), images, threads=1)
    np.savez(os.path.join(out_dir, "shard_%d.npz" % rank), lo=lo, hi=hi, out=out, arg=arg)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_sharded_inference_tiles_the_stream_without_communication(tmp_path):
    """Inference shards by image: the ranks' contiguous shards, concatenated in rank order, are the
    single-rank result (no collective on the data path)."""
    n, world = 103, 2
    port = 31500 + (os.getpid() % 2000)
    mp.spawn(_infer_worker, args=(world, port, n, str(tmp_path)), nprocs=world, join=True)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import __graft_entry__ as entry
    import oracle_binding as ob
    pkg = entry.load_package()
    images, _ = pkg.synth.synth_images(2, n)
    ref_out, ref_arg = ob.forward_batch(pkg.synth.synth_params(0), images, threads=1)
    parts = [np.load(tmp_path / ("shard_%d.npz" % r)) for r in range(world)]
    assert parts[0]["lo"] == 0 and parts[-1]["hi"] == n and parts[0]["hi"] == parts[1]["lo"]
    assert np.array_equal(np.concatenate([p["out"] for p in parts]), ref_out)
    assert np.array_equal(np.concatenate([p["arg"] for p in parts]), ref_arg)
