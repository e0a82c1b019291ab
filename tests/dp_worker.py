"""One rank of the multi-GPU data-parallel check (started by tests/test_gpu_dp.py through
``python -m torch.distributed.run``; one process per GPU, gloo for the host-side plumbing, the
library's own peer-store exchange for the gradients -- no NCCL involved).

Checks, and prints one JSON line on rank 0:
  * after two epochs of minibatch SGD all ranks' parameter arenas are bit-identical;
  * they agree with the oracle's minibatch run of the same global batch within 2e-5 of the largest
    parameter, and with the single-GPU kernel run of the same global batch;
  * a step in which one rank sends nothing (host-side fault injection, short wait limit) makes every
    rank's bounded wait run out: the kernels return, every rank reports CNN_ERR_TIMEOUT, parameters
    are left untouched, and the following step works again.
"""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import __graft_entry__ as entry  # noqa: E402


def main():
    rank, local_rank, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    torch.cuda.set_device(local_rank)
    pkg = entry.load_package()
    pkg.load_library()
    from hpcnn_b200 import parallel

    n, per_gpu, epochs = 2048 + 100, 64, 2
    gb = per_gpu * world
    images, labels = pkg.synth.synth_images(3, n)
    params = pkg.synth.synth_params(0)
    d_img = torch.from_numpy(images).cuda()
    d_lab = torch.from_numpy(labels.astype(np.int32)).cuda()
    net = pkg.Net(0)
    net.set_params(params)
    dp = pkg.DataParallel(net, rank, world, parallel.handle_exchange(dist))
    d_me = torch.zeros(epochs, dtype=torch.float32, device="cuda")
    dp.train_minibatch(d_img, d_lab, n, gb, epochs, 0.1, d_me)
    torch.cuda.synchronize()
    assert net.status() == 0
    mine = torch.from_numpy(net.get_params())
    everyone = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine)
    me_all = [torch.empty(epochs) for _ in range(world)]
    dist.all_gather(me_all, d_me.cpu())
    result = {"world": world, "global_batch": gb, "images": n, "epochs": epochs}
    if rank == 0:
        import oracle_binding as ob
        for r in range(1, world):
            assert torch.equal(everyone[0], everyone[r]), "rank %d diverged from rank 0" % r
            assert torch.equal(me_all[0], me_all[r])
        p_or, me_or = ob.train_minibatch(params, images, labels, gb, epochs, world=world)
        scale = float(np.max(np.abs(p_or)))
        result["ranks_bit_identical"] = True
        result["vs_oracle"] = float(np.max(np.abs(mine.numpy() - p_or)) / scale)
        assert result["vs_oracle"] < 2e-5, result
        assert np.allclose(me_all[0].numpy(), me_or, rtol=1e-5)
        single = pkg.Net(0)
        single.set_params(params)
        single.train_minibatch(d_img, d_lab, n, gb, epochs, 0.1, None)
        torch.cuda.synchronize()
        result["vs_single_gpu"] = float(np.max(np.abs(mine.numpy() - single.get_params())) / scale)
        assert result["vs_single_gpu"] < 2e-5, result
    dist.barrier()

    # ---- a rank that sends nothing: bounded waits run out everywhere, nothing hangs -----------------
    before = net.get_params()
    dp.set_option("wait_limit_ms", 300)
    if rank == world - 1:
        dp.set_option("drop_next_send", 1)
    dp.step(d_img, d_lab, per_gpu, 0.1 / gb)
    torch.cuda.synchronize()
    timed_out = False
    try:
        net.status()
    except pkg.CnnError as e:
        timed_out = e.code == -3
    assert timed_out, "rank %d: the dropped exchange was not reported" % rank
    assert np.array_equal(net.get_params(), before), "a failed step must not touch the parameters"
    dist.barrier()          # every rank has left the failed step before anyone starts the next
    dp.set_option("wait_limit_ms", 2000)
    dp.step(d_img, d_lab, per_gpu, 0.1 / gb)
    torch.cuda.synchronize()
    assert net.status() == 0
    after = torch.from_numpy(net.get_params())
    everyone = [torch.empty_like(after) for _ in range(world)]
    dist.all_gather(everyone, after)
    assert all(torch.equal(everyone[0], e) for e in everyone) and not torch.equal(after, torch.from_numpy(before))
    result["timeout_reported_and_recovered"] = True
    dist.barrier()
    dp.close()
    if rank == 0:
        print(json.dumps(result), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
