"""The allocation-free gradient entry point (GPU), collected last.

``cnn_grad_batch_noalloc`` serves callers that are not allowed to allocate device memory when they
need a gradient (plug-ins working inside buffers handed to them, services with pre-carved memory
pools, latency-critical loops).  It must give what ``cnn_grad_batch`` gives, on every call, although
all its calls share one fixed scratch array that still holds the previous call's contents."""
import numpy as np
import pytest

from conftest import scaled_err

pytestmark = pytest.mark.gpu


def _both(torch, pkg, params, seed, n, stream=None):
    images, labels = pkg.synth.synth_images(seed, n)
    d_img = torch.from_numpy(images).cuda()
    d_lab = torch.from_numpy(labels.astype(np.int32)).cuda()
    d_par = torch.from_numpy(params).cuda()
    net = pkg.Net(0)
    net.set_params(params)
    net.set_fast_sigmoid(0)     # the allocation-free call always uses the reference expression
    g_ref = torch.full((2368,), 5.0, dtype=torch.float32, device="cuda")
    net.grad_batch(d_img, d_lab, n, g_ref)
    g_new = torch.full((2368,), -5.0, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    pkg.grad_batch_noalloc(d_par, d_img, d_lab, n, g_new, stream)
    pkg.grad_batch_noalloc_status(stream)       # waits for the stream; raises if a wait ran out
    torch.cuda.synchronize()
    return g_new.cpu().numpy(), g_ref.cpu().numpy(), images, labels


def test_noalloc_gradient_matches_on_calls_in_a_row(cuda, pkg, ob, params0):
    """Four calls in a row over the shared array: a large batch, a small one that leaves most rows of
    the first call stale, a larger one again (rows grow back over stale ones), and one on a side
    stream.  With the same sigmoid both entry points run the same kernel over the same number of
    blocks, so the results must be bit-identical; the oracle is the independent check."""
    side = cuda.cuda.Stream()
    for seed, n, stream in ((51, 1000, None), (52, 37, None), (53, 400, None), (54, 90, side)):
        got, want, images, labels = _both(cuda, pkg, params0, seed, n, stream)
        assert np.array_equal(got, want), "call with n=%d differs from cnn_grad_batch" % n
        G, err = ob.grad_batch(params0, images, labels)
        assert scaled_err(got[:2343], G) < 1e-5
        assert abs(got[2344] - err) <= 1e-5 * max(err, 1.0)
        assert got[2343] == 0 and not got[2345:].any()


def test_noalloc_limits_and_arguments(cuda, pkg, params0):
    d_par = cuda.from_numpy(params0).cuda()
    d_g = cuda.full((2368,), 1.0, dtype=cuda.float32, device="cuda")
    pkg.grad_batch_noalloc(d_par, None, None, 0, d_g)
    cuda.cuda.synchronize()
    assert not d_g.cpu().numpy().any()
    d_img = cuda.zeros((4, 28, 28), dtype=cuda.float32, device="cuda")
    d_lab = cuda.zeros((4,), dtype=cuda.int32, device="cuda")
    with pytest.raises(pkg.CnnError) as e:
        pkg.grad_batch_noalloc(d_par, d_img, d_lab, 65537, d_g)
    assert e.value.code == -1 and "65536" in str(e.value)
    with pytest.raises(pkg.CnnError):
        pkg.grad_batch_noalloc(None, d_img, d_lab, 4, d_g)
    # an empty call after non-empty ones leaves nothing behind and the status stays clear
    pkg.grad_batch_noalloc(d_par, d_img, d_lab, 4, d_g)
    pkg.grad_batch_noalloc(d_par, None, None, 0, d_g)
    pkg.grad_batch_noalloc_status()
    assert not d_g.cpu().numpy().any()
