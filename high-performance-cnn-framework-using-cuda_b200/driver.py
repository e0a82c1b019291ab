"""The reference program's main() on top of the fused kernels: loaddata -> learn -> test
(main.cu:28-52, 125-170, 195-208), printing the same lines.

    python driver.py <directory containing data/*.idx*-ubyte>

Differences from the reference binary are the ones the fused kernels make: one persistent kernel
for the whole training run instead of ~42 driver calls per image, one fused launch for the test
set, and the per-epoch time printed is measured around the GPU work (the reference brackets
asynchronous launches with a host clock and never synchronises, main.cu:72-91).
"""
from __future__ import annotations

import os
import sys
import time


def learn_and_test(directory: str, epochs: int = 5, dt: float = 0.1, threshold: float = 0.01, out=print,
                   seed: int = 0):
    """Returns (mean_err per epoch, accuracy percent).  Device buffers come from torch."""
    import numpy as np
    import torch

    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.dirname(here))
    import __graft_entry__ as entry
    pkg = entry.load_package()
    from hpcnn_b200 import idx

    d = os.path.join(directory, "data")
    rc_a, train_px, train_lab = idx.read_idx_pair(os.path.join(d, "train-images.idx3-ubyte"),
                                                  os.path.join(d, "train-labels.idx1-ubyte"))
    rc_b, test_px, test_lab = idx.read_idx_pair(os.path.join(d, "t10k-images.idx3-ubyte"),
                                                os.path.join(d, "t10k-labels.idx1-ubyte"))
    if rc_a or rc_b:
        raise RuntimeError("mnist_load codes %d / %d" % (rc_a, rc_b))
    net = pkg.Net(seed)
    d_img = torch.from_numpy(pkg.synth.u8_to_float(train_px)).cuda()
    d_lab = torch.from_numpy(train_lab.astype(np.int32)).cuda()
    out("Learning")
    t0 = time.perf_counter()
    ran, mean_err = net.train_sgd_persample(d_img, d_lab, train_px.shape[0], epochs, dt, threshold)
    sec = time.perf_counter() - t0
    for j in range(ran):
        out("%d: error: %g, time_on_gpu: %g" % (j + 1, float(mean_err[j]), sec * (j + 1) / ran))
    if ran and float(mean_err[ran - 1]) < threshold:
        out("Training complete, error less than threshold\n")
    out("\n Time - %g" % sec)
    n_test = test_px.shape[0]
    h_arg = np.empty(n_test, dtype=np.int32)
    net.forward_u8_host(np.ascontiguousarray(test_px), n_test, None, h_arg)
    errors = int((h_arg.astype(np.uint32) != test_lab).sum())
    acc = (1.0 - errors / float(n_test)) * 100.0
    out("Accuracy: %g%%" % acc)
    return mean_err, acc


if __name__ == "__main__":
    learn_and_test(sys.argv[1] if len(sys.argv) > 1 else ".")
