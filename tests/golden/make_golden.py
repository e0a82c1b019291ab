"""Records golden vectors from the reference's OWN CUDA kernels (the unmodified layer.cu behind
oracle/_ref/libref_cnn.so) on seeded synthetic inputs.  Needs a GPU:

    python tests/golden/make_golden.py <output-dir>

writes reference_cuda_seed<k>.npz holding the inputs, every Layer buffer after the reference's
forward launch sequence, every buffer and the parameters after one training step from identical
state, a short per-sample trajectory, and the reference's own srand(0) initial parameters.  The
CPU test-suite checks the oracle against these files (tests/test_oracle.py)."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import __graft_entry__ as entry  # noqa: E402
import oracle_binding as ob  # noqa: E402

FWD = [("c1", "preact"), ("c1", "output"), ("s1", "preact"), ("s1", "output"), ("f", "preact"), ("f", "output")]
BWD = [("f", "d_preact"), ("f", "d_weight"), ("s1", "d_output"), ("s1", "d_preact"), ("s1", "d_weight"),
       ("c1", "d_output"), ("c1", "d_preact"), ("c1", "d_weight")]


def record(seed: int, n_fwd: int, n_step: int, n_traj: int, out_dir: str) -> str:
    pkg = entry.load_package()
    params = pkg.synth.synth_params(seed)
    images, labels = pkg.synth.synth_images(1000 + seed, max(n_fwd, n_step, n_traj))
    ref = ob.Reference(0)
    rand_init = ref.get_params()
    data = {"params": params, "images": images[:max(n_fwd, n_traj)], "labels": labels[:max(n_fwd, n_traj)],
            "rand_init_params": rand_init}
    fwd = {"fwd_%s_%s" % lb: [] for lb in FWD}
    for i in range(n_fwd):
        ref.set_params(params)
        ref.forward(images[i])
        for lb in FWD:
            fwd["fwd_%s_%s" % lb].append(ref.read(*lb))
    data.update({k: np.stack(v) for k, v in fwd.items()})
    step = {"step_%s_%s" % lb: [] for lb in BWD}
    after, errs = [], []
    for i in range(n_step):
        ref.set_params(params)
        errs.append(ref.train_step(images[i], int(labels[i])))
        for lb in BWD:
            step["step_%s_%s" % lb].append(ref.read(*lb))
        after.append(ref.get_params())
    data.update({k: np.stack(v) for k, v in step.items()})
    data["step_params_after"] = np.stack(after)
    data["step_err"] = np.array(errs, dtype=np.float32)
    ref.set_params(params)
    sec, mean_err = ref.time_train(images[:n_traj], labels[:n_traj])
    data["traj_params"] = ref.get_params()
    data["traj_mean_err"] = np.float32(mean_err)
    data["traj_n"] = np.int64(n_traj)
    ref.close()
    path = os.path.join(out_dir, "reference_cuda_seed%d.npz" % seed)
    np.savez_compressed(path, **data)
    return path


if __name__ == "__main__":
    out = sys.argv[1] if len(sys.argv) > 1 else HERE
    os.makedirs(out, exist_ok=True)
    for s in (0, 1):
        print(record(s, n_fwd=4, n_step=3, n_traj=40, out_dir=out))
