"""IDX reader/writer (CPU): round trip and the loader's error codes (mnist.h:79-160)."""
import struct

import numpy as np


def test_round_trip_and_codes(pkg, tmp_path):
    from hpcnn_b200 import idx
    pix = pkg.synth.synth_pixels_u8(3, 50)
    lab = pkg.synth.synth_labels(3, 50)
    ip, lp = str(tmp_path / "i.idx3"), str(tmp_path / "l.idx1")
    idx.write_idx_pair(ip, lp, pix, lab)
    raw = open(ip, "rb").read()
    assert struct.unpack(">IIII", raw[:16]) == (2051, 50, 28, 28) and len(raw) == 16 + 50 * 784
    assert struct.unpack(">II", open(lp, "rb").read()[:8]) == (2049, 50)
    code, p2, l2 = idx.read_idx_pair(ip, lp)
    assert code == 0 and np.array_equal(p2, pix) and np.array_equal(l2, lab)
    assert idx.read_idx_pair(str(tmp_path / "missing"), lp)[0] == -1
    assert idx.read_idx_pair(lp, lp)[0] == -2           # label file where the image file should be
    assert idx.read_idx_pair(ip, ip)[0] == -3
    idx.write_idx_pair(str(tmp_path / "i2"), str(tmp_path / "l2"), pix[:10], lab[:10])
    assert idx.read_idx_pair(ip, str(tmp_path / "l2"))[0] == -4


def test_reference_data_dir_layout(pkg, tmp_path):
    from hpcnn_b200 import idx
    tr = (pkg.synth.synth_pixels_u8(0, 20), pkg.synth.synth_labels(0, 20))
    te = (pkg.synth.synth_pixels_u8(0, 8, first_index=20), pkg.synth.synth_labels(0, 8, first_index=20))
    idx.write_reference_data_dir(str(tmp_path), tr, te)
    for name in ("train-images.idx3-ubyte", "train-labels.idx1-ubyte", "t10k-images.idx3-ubyte",
                 "t10k-labels.idx1-ubyte"):
        assert (tmp_path / "data" / name).exists()
