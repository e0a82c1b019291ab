"""Parameter checkpoint files: the Python reader/writer on CPU, and (GPU) the C ABI's save/load."""
import numpy as np
import pytest


def test_checkpoint_roundtrip_and_rejections(pkg, tmp_path, params0):
    ck = pkg.checkpoint
    path = str(tmp_path / "net.ckpt")
    ck.write_checkpoint(path, params0, seed=7)
    got = ck.read_checkpoint(path)
    assert np.array_equal(got["params"], params0) and got["seed"] == 7
    assert (got["kind"], got["H"], got["F"]) == (0, 28, 6)
    data = bytearray(open(path, "rb").read())
    assert len(data) == 32 + 4 * 2343 + 8 and data[:8] == b"CNNB200P"
    # one flipped payload bit, a truncated file, a wrong magic and a wrong parameter count are refused
    bad = bytearray(data); bad[100] ^= 1
    for blob in (bytes(bad), bytes(data[:-3]), b"XXXXXXXX" + bytes(data[8:])):
        open(path, "wb").write(blob)
        with pytest.raises(ck.CheckpointError):
            ck.read_checkpoint(path)
    with pytest.raises(ck.CheckpointError):
        ck.write_checkpoint(path, params0[:100])
    wide = np.arange(ck.param_count(56, 64), dtype=np.float32)
    ck.write_checkpoint(path, wide, kind=1, H=56, F=64)
    got = ck.read_checkpoint(path)
    assert np.array_equal(got["params"], wide) and got["kind"] == 1 and got["F"] == 64


@pytest.mark.gpu
def test_saved_net_reproduces_outputs_bit_for_bit(cuda, pkg, tmp_path, params0):
    n = 777
    images, labels = pkg.synth.synth_images(71, n)
    d_img = cuda.from_numpy(images).cuda()
    d_lab = cuda.from_numpy(labels.astype(np.int32)).cuda()
    a = pkg.Net(3)
    a.set_params(params0)
    a.train_minibatch(d_img, d_lab, n, 32, 1, 0.1, None)     # asynchronous: save must wait for it
    path = str(tmp_path / "trained.ckpt")
    a.save(path)
    out_a = cuda.empty((n, 10), dtype=cuda.float32, device="cuda")
    a.forward(d_img, n, out_a, None)
    b = pkg.Net(0)
    b.load(path)
    out_b = cuda.empty((n, 10), dtype=cuda.float32, device="cuda")
    b.forward(d_img, n, out_b, None)
    cuda.cuda.synchronize()
    assert np.array_equal(a.get_params(), b.get_params()) and cuda.equal(out_a, out_b)
    # the Python reader sees the same bytes, and a file written by Python loads
    got = pkg.checkpoint.read_checkpoint(path)
    assert np.array_equal(got["params"], a.get_params()) and got["seed"] == 3
    pkg.checkpoint.write_checkpoint(path, params0, seed=9)
    b.load(path)
    assert np.array_equal(b.get_params(), params0)
    # shape mismatch and corruption are refused and leave the net untouched
    w = pkg.WideNet(28, 16)
    wp = np.random.default_rng(0).uniform(-0.5, 0.5, w.n_params).astype(np.float32)
    w.set_params(wp)
    wpath = str(tmp_path / "wide.ckpt")
    w.save(wpath)
    with pytest.raises(pkg.CnnError):
        b.load(wpath)
    assert np.array_equal(b.get_params(), params0)
    w2 = pkg.WideNet(28, 16)
    w2.load(wpath)
    assert np.array_equal(w2.get_params(), wp)
    blob = bytearray(open(wpath, "rb").read()); blob[40] ^= 4
    open(wpath, "wb").write(bytes(blob))
    with pytest.raises(pkg.CnnError) as e:
        w2.load(wpath)
    assert "checksum" in str(e.value)
