"""Data-parallel minibatch training with the fused peer-store gradient exchange (GPU)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_single_rank_exchange_equals_minibatch_kernel(cuda, pkg, params0):
    """world = 1: the exchange kernel (own slot, own flags, step counters in device memory) must
    reproduce cnn_train_minibatch bit for bit, replayed steps included."""
    n, batch, epochs = 1000, 96, 3
    images, labels = pkg.synth.synth_images(81, n)
    d_img = cuda.from_numpy(images).cuda()
    d_lab = cuda.from_numpy(labels.astype(np.int32)).cuda()
    a = pkg.Net(0); a.set_params(params0)
    b = pkg.Net(0); b.set_params(params0)
    me_a = cuda.zeros(epochs, dtype=cuda.float32, device="cuda")
    me_b = cuda.zeros(epochs, dtype=cuda.float32, device="cuda")
    a.train_minibatch(d_img, d_lab, n, batch, epochs, 0.1, me_a)
    dp = pkg.DataParallel(b)
    dp.train_minibatch(d_img, d_lab, n, batch, epochs, 0.1, me_b)
    cuda.cuda.synchronize()
    assert a.status() == 0 and b.status() == 0
    assert np.array_equal(a.get_params(), b.get_params()) and cuda.equal(me_a, me_b)
    # the all-rank gradient sum of a step is the gradient of cnn_grad_batch
    g1 = cuda.zeros(2368, dtype=cuda.float32, device="cuda")
    g2 = cuda.zeros(2368, dtype=cuda.float32, device="cuda")
    a.grad_batch(d_img, d_lab, 200, g1)
    dp.step(d_img, d_lab, 200, 0.0, g2)
    cuda.cuda.synchronize()
    assert cuda.equal(g1[:2343], g2[:2343]) and float(g1[2344]) == float(g2[2344])
    assert np.array_equal(a.get_params(), b.get_params())
    dp.close()


def test_dp_rejects_bad_arguments(cuda, pkg):
    net = pkg.Net(0)
    with pytest.raises(pkg.CnnError):
        pkg.DataParallel(net, 3, 2, lambda h: [h, h])
    with pytest.raises(pkg.CnnError):
        pkg.DataParallel(net, 0, 9, lambda h: [h] * 9)
    dp = pkg.DataParallel(net)
    with pytest.raises(pkg.CnnError):
        dp.set_option("no_such_option", 1)
    dp.close()


@pytest.mark.parametrize("world", [2, 4])
def test_ranks_stay_bit_identical_and_match_oracle(cuda, built, world):
    """One process per GPU (needs `world` GPUs): see tests/dp_worker.py for what each rank checks."""
    if cuda.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    env = dict(os.environ)
    env.setdefault("NCCL_NVLS_ENABLE", "0")
    port = 29700 + (os.getpid() % 1000) + world
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "dp_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1]
    res = json.loads(line)
    print(res)
    assert res["ranks_bit_identical"] and res["timeout_reported_and_recovered"]
    assert res["vs_oracle"] < 2e-5 and res["vs_single_gpu"] < 2e-5
