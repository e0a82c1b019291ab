"""Fused batched forward (GPU) against the oracle, the reference kernels and itself."""
import numpy as np
import pytest

from conftest import rel_err

pytestmark = pytest.mark.gpu


def run_forward(torch, net, images, want_out=True, want_arg=True, offset_elems=0):
    n = images.shape[0]
    flat = torch.zeros(n * 784 + offset_elems + 4, dtype=torch.float32, device="cuda")
    d_img = flat[offset_elems:offset_elems + n * 784]
    if n:
        d_img.copy_(torch.from_numpy(np.ascontiguousarray(images).reshape(-1)))
    d_out = torch.full((n, 10), -1.0, dtype=torch.float32, device="cuda") if want_out else None
    d_arg = torch.full((n,), -1, dtype=torch.int32, device="cuda") if want_arg else None
    net.forward(d_img, n, d_out, d_arg)
    torch.cuda.synchronize()
    assert net.status() == 0
    return (d_out.cpu().numpy() if want_out else None), (d_arg.cpu().numpy() if want_arg else None)


def clear_margin(out, tol=1e-5):
    top2 = np.sort(out, axis=1)
    return (top2[:, -1] - top2[:, -2]) > tol * top2[:, -1]


def check_argmax(arg, ref_arg, ref_out, what, tol=1e-5, max_masked_frac=1e-3):
    """argmax must equal the oracle's on every row whose top-two margin exceeds ``tol`` relative
    (below that the reference's own run-to-run atomics order decides the winner); the number of rows
    excused that way is printed and must be tiny."""
    ok = clear_margin(ref_out, tol)
    masked = int((~ok).sum())
    mism = int((arg != ref_arg).sum())
    print("%s: %d rows, %d below the %.0e margin, %d argmax differences in all (%d on clear rows)"
          % (what, len(arg), masked, tol, mism, int((arg[ok] != ref_arg[ok]).sum())))
    assert np.array_equal(arg[ok], ref_arg[ok])
    assert masked <= max(1, int(max_masked_frac * len(arg)))


@pytest.mark.parametrize("fast", [0, 1])
@pytest.mark.parametrize("n", [1, 7, 8, 9, 100, 2368 + 5, 4099])
def test_forward_matches_oracle(cuda, pkg, ob, params0, n, fast):
    images, _ = pkg.synth.synth_images(21, n)
    net = pkg.Net(0)
    net.set_params(params0)
    net.set_fast_sigmoid(fast)
    out, arg = run_forward(cuda, net, images)
    ref_out, ref_arg = ob.forward_batch(params0, images)
    assert rel_err(out, ref_out) < 1e-5       # the 1e-5 relative bar on activations
    check_argmax(arg, ref_arg, ref_out, "n=%d flavour %d" % (n, fast))
    # the argmax written by the kernel is the lowest-index maximum of the row it wrote
    assert np.array_equal(arg, np.argmax(out, axis=1).astype(np.int32))


@pytest.mark.parametrize("path", [-1, 0])
@pytest.mark.parametrize("fast", [0, 1])
def test_full_size_forward_matches_oracle(cuda, pkg, ob, params0, fast, path):
    """Benchmark configuration 2 at its full size: 65,536 images of seed 1 against the oracle --
    every sigmoid within 1e-5 relative, argmax equal on every clear-margin row; the number of rows
    below the margin and the number of differing rows are printed (both are expected to be zero or a
    handful out of 65,536).  Run with the default kernel choice (at this size and with the short sigmoid
    form: the three-pass tensor-core kernel) and with the CUDA-core kernel forced."""
    n = 65536
    images, _ = pkg.synth.synth_images(1, n)
    net = pkg.Net(0)
    net.set_params(params0)
    net.set_fast_sigmoid(fast)
    net.set_option("forward_path", path)
    out, arg = run_forward(cuda, net, images)
    ref_out, ref_arg = ob.forward_batch(params0, images, threads=0)
    err = rel_err(out, ref_out)
    print("full size, flavour %d, forward_path %d: max relative error of the sigmoids %.3e" % (fast, path, err))
    assert err < 1e-5
    check_argmax(arg, ref_arg, ref_out, "65,536 images flavour %d path %d" % (fast, path))
    assert np.array_equal(arg, np.argmax(out, axis=1).astype(np.int32))


def test_forward_empty_and_optional_outputs(cuda, pkg, ob, params0):
    net = pkg.Net(0)
    net.set_params(params0)
    net.forward(None, 0, None, None)
    images, _ = pkg.synth.synth_images(22, 50)
    out, _ = run_forward(cuda, net, images, want_arg=False)
    _, arg = run_forward(cuda, net, images, want_out=False)
    assert np.array_equal(arg, np.argmax(out, axis=1))


def test_forward_rejects_bad_arguments(cuda, pkg, params0):
    net = pkg.Net(0)
    d = cuda.zeros(784 * 4 + 8, dtype=cuda.float32, device="cuda")
    with pytest.raises(pkg.CnnError) as e:
        net.forward(d[1:], 2, None, None)   # 4-byte offset: not 16-byte aligned
    assert e.value.code == -1 and "16-byte" in str(e.value)
    with pytest.raises(pkg.CnnError):
        net.forward(d, -1, None, None)
    with pytest.raises(pkg.CnnError):
        net.forward(None, 3, None, None)
    # a 16-byte (4-float) offset is fine
    net.forward(d[4:], 2, None, None)
    cuda.cuda.synchronize()


def test_forward_is_deterministic_and_tie_breaks_low(cuda, pkg, params0):
    images, _ = pkg.synth.synth_images(23, 1000)
    net = pkg.Net(0)
    net.set_params(params0)
    a = run_forward(cuda, net, images)
    b = run_forward(cuda, net, images)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    # all-zero FC weights and equal biases: every output equal, index 0 must win
    p = params0.copy()
    p[173:2333] = 0
    p[2333:] = 0.25
    net.set_params(p)
    out, arg = run_forward(cuda, net, images[:20])
    assert np.all(out == out[0, 0]) and np.all(arg == 0)


def test_forward_host_pipeline(cuda, pkg, ob, params0):
    n = 8192 * 2 + 123          # spans three staging chunks
    images, _ = pkg.synth.synth_images(24, n)
    net = pkg.Net(0)
    net.set_params(params0)
    h_img = cuda.from_numpy(images).pin_memory()
    h_out = cuda.empty((n, 10), dtype=cuda.float32).pin_memory()
    h_arg = cuda.empty((n,), dtype=cuda.int32).pin_memory()
    net.forward_host(h_img, n, h_out, h_arg)
    d_out, d_arg = run_forward(cuda, net, images)
    bad = np.nonzero((h_out.numpy() != d_out).any(axis=1))[0]
    assert bad.size == 0, "rows differing between host pipeline and device call: %s ... (%d)" % (bad[:8], bad.size)
    assert np.array_equal(h_arg.numpy(), d_arg)
    # pageable host memory works too
    out2 = np.empty((n, 10), dtype=np.float32)
    net.forward_host(images, n, out2, None)
    assert np.array_equal(out2, d_out)


def test_forward_against_reference_kernels(cuda, pkg, ob, params0):
    if not ob.reference_available():
        pytest.skip("reference kernels not built")
    images, _ = pkg.synth.synth_images(25, 96)
    net = pkg.Net(0)
    net.set_params(params0)
    out, arg = run_forward(cuda, net, images)
    ref = ob.Reference(0)
    ref.set_params(params0)
    ref_out = np.zeros((96, 10), dtype=np.float32)
    ref_arg = np.zeros(96, dtype=np.int32)
    for i in range(96):
        ref_arg[i] = ref.classify(images[i])
        ref_out[i] = ref.read("f", "output")
    ref.close()
    assert rel_err(out, ref_out) < 1e-5
    check_argmax(arg, ref_arg, ref_out, "96 images against the reference kernels", max_masked_frac=0.05)


@pytest.mark.parametrize("path", [-1, 0])
def test_full_size_property_linearity_in_batch(cuda, pkg, params0, path):
    """benchmark configuration 2 size (65,536 images): results of a batch do not depend on where an image
    sits in it -- the full batch equals the concatenation of two half batches, bit for bit, and the
    device generator fills the same images as the host generator.  Holds for the default kernel choice
    (tensor cores at these sizes) and for the CUDA-core kernel."""
    n = 65536
    net = pkg.Net(0)
    net.set_params(params0)
    net.set_option("forward_path", path)
    d_img = cuda.empty((n, 28, 28), dtype=cuda.float32, device="cuda")
    pkg.synth_images_device(1, 0, n, d_img)
    d_out = cuda.empty((n, 10), dtype=cuda.float32, device="cuda")
    d_arg = cuda.empty((n,), dtype=cuda.int32, device="cuda")
    net.forward(d_img, n, d_out, d_arg)
    o2 = cuda.empty_like(d_out)
    a2 = cuda.empty_like(d_arg)
    half = n // 2 + 3 * 8       # keeps the second half on a tile boundary multiple
    net.forward(d_img, half, o2, a2)
    net.forward(d_img[half:], n - half, o2[half:], a2[half:])
    cuda.cuda.synchronize()
    assert cuda.equal(d_out, o2) and cuda.equal(d_arg, a2)
    host, _ = pkg.synth.synth_images(1, 2048, first_index=30000)
    assert np.array_equal(d_img[30000:32048].cpu().numpy(), host)


def test_device_generator_matches_host(cuda, pkg):
    n = 3000
    d_img = cuda.empty((n, 28, 28), dtype=cuda.float32, device="cuda")
    d_lab = cuda.empty((n,), dtype=cuda.int32, device="cuda")
    pkg.synth_images_device(9, 12345, n, d_img, d_lab)
    cuda.cuda.synchronize()
    h_img, h_lab = pkg.synth.synth_images(9, n, first_index=12345)
    assert np.array_equal(d_img.cpu().numpy(), h_img)
    assert np.array_equal(d_lab.cpu().numpy().astype(np.uint32), h_lab)


@pytest.mark.parametrize("n", [1, 9, 1000, 8192 + 77])
def test_uint8_input_is_bit_identical_to_fp32(cuda, pkg, params0, n):
    """uint8 pixels through the in-kernel pixel/255.0 table == fp32 images through the fp32 kernel
    (the CUDA-core kernel, which is the one that has the uint8 ingest)."""
    pix = pkg.synth.synth_pixels_u8(26, n)
    images = pkg.synth.u8_to_float(pix)
    net = pkg.Net(0)
    net.set_params(params0)
    net.set_option("forward_path", 0)
    out_f, arg_f = run_forward(cuda, net, images)
    d_pix = cuda.from_numpy(pix).cuda()
    d_out = cuda.empty((n, 10), dtype=cuda.float32, device="cuda")
    d_arg = cuda.empty((n,), dtype=cuda.int32, device="cuda")
    net.forward_u8(d_pix, n, d_out, d_arg)
    cuda.cuda.synchronize()
    assert net.status() == 0
    assert np.array_equal(d_out.cpu().numpy(), out_f) and np.array_equal(d_arg.cpu().numpy(), arg_f)
    h_out = np.empty((n, 10), dtype=np.float32)
    h_arg = np.empty((n,), dtype=np.int32)
    net.forward_u8_host(pix, n, h_out, h_arg)
    assert np.array_equal(h_out, out_f) and np.array_equal(h_arg, arg_f)


def test_sigmoid_flavours_agree(cuda, pkg, ob, params0):
    """The default (short) sigmoid form against the reference expression on the full benchmark batch:
    maximum relative difference of the ten outputs between the two, and the distance of each from the
    fp64 oracle, beside the fp32 oracle's own distance from it."""
    n = 65536
    images, _ = pkg.synth.synth_images(1, n)
    d_img = cuda.from_numpy(images).cuda()
    ref64, _ = ob.forward_batch(params0, images, threads=0, dtype=np.float64)
    ref32, _ = ob.forward_batch(params0, images, threads=0)
    outs = {}
    for fl in (0, 1):
        net = pkg.Net(0)
        net.set_params(params0)
        net.set_fast_sigmoid(fl)
        net.set_option("forward_path", 0)      # the same kernel for both forms
        o = cuda.empty((n, 10), dtype=cuda.float32, device="cuda")
        net.forward(d_img, n, o, None)
        cuda.cuda.synchronize()
        outs[fl] = o.cpu().numpy().astype(np.float64)
    d = float(np.max(np.abs(outs[1] - outs[0]) / outs[0]))
    e0, e1, eo = rel_err(outs[0], ref64), rel_err(outs[1], ref64), rel_err(ref32, ref64)
    print("short form vs reference expression: %.3e; against the fp64 oracle: reference expression %.3e, "
          "short form %.3e, fp32 oracle %.3e" % (d, e0, e1, eo))
    assert d < 5e-6 and e1 < max(5e-6, 1.5 * e0)


def test_forward_host_is_ordered_behind_legacy_stream_work(cuda, pkg, params0):
    """A host-buffer forward issued right after an asynchronous parameter update on the legacy
    stream (no synchronisation in between) must see the updated parameters."""
    n = 4096
    images, labels = pkg.synth.synth_images(27, n)
    d_img = cuda.from_numpy(images).cuda()
    d_lab = cuda.from_numpy(labels.astype(np.int32)).cuda()
    h_img = cuda.from_numpy(images).pin_memory()
    outs = []
    for sync_between in (True, False):
        net = pkg.Net(0)
        net.set_params(params0)
        net.forward_host(h_img, 8, None, None)          # staging buffers and streams exist
        cuda.cuda.synchronize()
        h_out = cuda.empty((n, 10), dtype=cuda.float32).pin_memory()
        net.train_minibatch(d_img, d_lab, n, 64, 3, 0.1, None, None)   # asynchronous, stream NULL
        if sync_between:
            cuda.cuda.synchronize()
        net.forward_host(h_img, n, h_out, None)
        outs.append(h_out.numpy().copy())
    assert np.array_equal(outs[0], outs[1])
    assert not np.array_equal(outs[0][:8], 0 * outs[0][:8])


# ---- the convolution on the tensor cores (option "forward_path") ------------------------------------
@pytest.mark.parametrize("fast", [0, 1])
@pytest.mark.parametrize("n", [1, 5, 16, 17, 100, 2368 + 5, 4099])
def test_tensor_core_forward_three_passes_matches_oracle(cuda, pkg, ob, params0, n, fast):
    """forward_path = 1: tcgen05 convolution in three tf32 passes keeps the 1e-5 bar of the fp32 path."""
    images, _ = pkg.synth.synth_images(21, n)
    net = pkg.Net(0)
    net.set_params(params0)
    net.set_fast_sigmoid(fast)
    net.set_option("forward_path", 1)
    out, arg = run_forward(cuda, net, images)
    ref_out, ref_arg = ob.forward_batch(params0, images)
    assert rel_err(out, ref_out) < 1e-5
    check_argmax(arg, ref_arg, ref_out, "tensor cores, three passes, n=%d flavour %d" % (n, fast))
    assert np.array_equal(arg, np.argmax(out, axis=1).astype(np.int32))


def test_tensor_core_forward_full_size(cuda, pkg, ob, params0):
    """Benchmark configuration 2 at full size on both tensor-core paths.  Path 1 (three passes): 1e-5
    on every sigmoid, argmax on every clear-margin row.  Path 2 (one tf32 pass, tanh.approx sigmoid) is
    a reduced-precision mode: its bar is 5e-3 absolute on the sigmoids and argmax equality on every
    row whose top-two margin is clear of that error (1e-2 relative); both counts are printed."""
    n = 65536
    images, _ = pkg.synth.synth_images(1, n)
    ref_out, ref_arg = ob.forward_batch(params0, images, threads=0)
    net = pkg.Net(0)
    net.set_params(params0)
    net.set_option("forward_path", 1)
    out, arg = run_forward(cuda, net, images)
    err = rel_err(out, ref_out)
    print("three passes: max relative error of the sigmoids %.3e" % err)
    assert err < 1e-5
    check_argmax(arg, ref_arg, ref_out, "65,536 images, tensor cores, three passes")
    # bit-repeatable, and independent of where an image sits in the batch
    out2, arg2 = run_forward(cuda, net, images[1000:3000])
    assert np.array_equal(out2, out[1000:3000]) and np.array_equal(arg2, arg[1000:3000])
    net.set_option("forward_path", 2)
    out, arg = run_forward(cuda, net, images)
    abs_err = float(np.max(np.abs(out.astype(np.float64) - ref_out)))
    print("one pass + tanh: max absolute error of the sigmoids %.3e, mean %.3e"
          % (abs_err, float(np.mean(np.abs(out.astype(np.float64) - ref_out)))))
    assert abs_err < 5e-3
    check_argmax(arg, ref_arg, ref_out, "65,536 images, tensor cores, one pass + tanh", tol=1e-2,
                 max_masked_frac=0.05)
    assert np.array_equal(arg, np.argmax(out, axis=1).astype(np.int32))


def test_tensor_core_forward_optional_outputs_and_host_pipeline(cuda, pkg, params0):
    n = 8192 + 300
    images, _ = pkg.synth.synth_images(28, n)
    net = pkg.Net(0)
    net.set_params(params0)
    net.set_option("forward_path", 1)
    out, arg = run_forward(cuda, net, images)
    o2, _ = run_forward(cuda, net, images, want_arg=False)
    _, a2 = run_forward(cuda, net, images, want_out=False)
    assert np.array_equal(o2, out) and np.array_equal(a2, arg)
    h_out = np.empty((n, 10), dtype=np.float32)
    h_arg = np.empty((n,), dtype=np.int32)
    net.forward_host(images, n, h_out, h_arg)
    assert np.array_equal(h_out, out) and np.array_equal(h_arg, arg)


def test_default_kernel_choice_follows_batch_size(cuda, pkg, params0):
    """forward_path = -1 (the default): below 6,144 images per call the CUDA-core kernel answers, from
    6,144 on the three-pass tensor-core kernel -- bit for bit in both cases; with the reference's
    sigmoid expression selected the default stays on the CUDA-core kernel at every size."""
    images, _ = pkg.synth.synth_images(29, 6144)
    outs = {}
    for path in (-1, 0, 1):
        net = pkg.Net(0)
        net.set_params(params0)
        net.set_option("forward_path", path)
        outs[path] = (run_forward(cuda, net, images[:6143]), run_forward(cuda, net, images))
    assert np.array_equal(outs[-1][0][0], outs[0][0][0]) and np.array_equal(outs[-1][0][1], outs[0][0][1])
    assert np.array_equal(outs[-1][1][0], outs[1][1][0]) and np.array_equal(outs[-1][1][1], outs[1][1][1])
    assert not np.array_equal(outs[0][1][0], outs[1][1][0])     # the two kernels do differ in the last bits
    ref = {}
    for path in (-1, 0):
        net = pkg.Net(0)
        net.set_params(params0)
        net.set_fast_sigmoid(0)
        net.set_option("forward_path", path)
        ref[path] = run_forward(cuda, net, images)
    assert np.array_equal(ref[-1][0], ref[0][0])
