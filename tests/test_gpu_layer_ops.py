"""Per-operator parity (GPU): every C-ABI launcher against the oracle's trace, and against the
reference's own kernel of the same name run with its stock <<<64,64>>> and with odd launch shapes."""
import numpy as np
import pytest

from conftest import rel_err, scaled_err

pytestmark = pytest.mark.gpu


class Net4:
    """The reference's four Layer objects (main.cu:17-20) through the mirror API."""

    def __init__(self, pkg, params):
        self.pkg = pkg
        self.input = pkg.Layer(0, 0, 28 * 28)
        self.c1 = pkg.Layer(5 * 5, 6, 24 * 24 * 6)
        self.s1 = pkg.Layer(4 * 4, 1, 6 * 6 * 6)
        self.f = pkg.Layer(6 * 6 * 6, 10, 10)
        self.c1.write("weight", params[0:150]); self.c1.write("bias", params[150:156])
        self.s1.write("weight", params[156:172]); self.s1.write("bias", params[172:173])
        self.f.write("weight", params[173:2333]); self.f.write("bias", params[2333:2343])

    def params(self):
        return np.concatenate([self.c1.read("weight"), self.c1.read("bias"), self.s1.read("weight"),
                               self.s1.read("bias"), self.f.read("weight"), self.f.read("bias")])

    def forward_pass(self, image):
        """main.cu:67-88 with the mirror API."""
        p = self.pkg
        for l in (self.input, self.c1, self.s1, self.f):
            l.clear()
        self.input.setOutput(image)
        p.fp_preact_c1(self.input.output, self.c1.preact, self.c1.weight)
        p.fp_bias_c1(self.c1.preact, self.c1.bias)
        p.apply_step_function(self.c1.preact, self.c1.output, self.c1.O)
        p.fp_preact_s1(self.c1.output, self.s1.preact, self.s1.weight)
        p.fp_bias_s1(self.s1.preact, self.s1.bias)
        p.apply_step_function(self.s1.preact, self.s1.output, self.s1.O)
        p.fp_preact_f(self.s1.output, self.f.preact, self.f.weight)
        p.fp_bias_f(self.f.preact, self.f.bias)
        p.apply_step_function(self.f.preact, self.f.output, self.f.O)

    def back_pass(self, label):
        """main.cu:147-152 and 99-119."""
        p = self.pkg
        for l in (self.f, self.s1, self.c1):
            l.bp_clear()
        p.makeError(self.f.d_preact, self.f.output, label, 10)
        p.bp_weight_f(self.f.d_weight, self.f.d_preact, self.s1.output)
        p.bp_bias_f(self.f.bias, self.f.d_preact)
        p.bp_output_s1(self.s1.d_output, self.f.weight, self.f.d_preact)
        p.bp_preact_s1(self.s1.d_preact, self.s1.d_output, self.s1.preact)
        p.bp_weight_s1(self.s1.d_weight, self.s1.d_preact, self.c1.output)
        p.bp_bias_s1(self.s1.bias, self.s1.d_preact)
        p.bp_output_c1(self.c1.d_output, self.s1.weight, self.s1.d_preact)
        p.bp_preact_c1(self.c1.d_preact, self.c1.d_output, self.c1.preact)
        p.bp_weight_c1(self.c1.d_weight, self.c1.d_preact, self.input.output)
        p.bp_bias_c1(self.c1.bias, self.c1.d_preact)
        p.apply_grad(self.f.weight, self.f.d_weight, self.f.M * self.f.N)
        p.apply_grad(self.s1.weight, self.s1.d_weight, self.s1.M * self.s1.N)
        p.apply_grad(self.c1.weight, self.c1.d_weight, self.c1.M * self.c1.N)


TRACE_TO_LAYER = {
    "c1_preact": ("c1", "preact"), "c1_output": ("c1", "output"), "s1_preact": ("s1", "preact"),
    "s1_output": ("s1", "output"), "f_preact": ("f", "preact"), "f_output": ("f", "output"),
    "f_d_preact": ("f", "d_preact"), "f_d_weight": ("f", "d_weight"), "s1_d_output": ("s1", "d_output"),
    "s1_d_preact": ("s1", "d_preact"), "s1_d_weight": ("s1", "d_weight"), "c1_d_output": ("c1", "d_output"),
    "c1_d_preact": ("c1", "d_preact"), "c1_d_weight": ("c1", "d_weight"),
}


def check_buffers(get, trace, names):
    for name in names:
        layer, buf = TRACE_TO_LAYER[name]
        got = get(layer, buf)
        if buf == "output":
            assert rel_err(got, trace[name]) < 1e-5, name
        else:
            assert scaled_err(got, trace[name]) < 1e-5, name


def test_layer_object_contract(cuda, pkg):
    l = pkg.Layer(25, 6, 3456)
    assert (l.M, l.N, l.O) == (25, 6, 3456)
    w, b = l.read("weight"), l.read("bias")
    assert w.shape == (150,) and np.all(np.abs(w) <= 0.5) and np.all(np.abs(b) <= 0.5)
    l.write("output", np.ones(3456)); l.write("preact", np.ones(3456))
    l.write("d_output", np.ones(3456)); l.write("d_preact", np.ones(3456)); l.write("d_weight", np.ones(150))
    l.clear()
    assert not l.read("output").any() and not l.read("preact").any() and l.read("d_output").all()
    l.bp_clear()
    assert not l.read("d_output").any() and not l.read("d_preact").any() and not l.read("d_weight").any()
    assert np.array_equal(l.read("weight"), w)
    x = np.arange(3456, dtype=np.float32)
    l.setOutput(x)
    assert np.array_equal(l.read("output"), x)
    with pytest.raises(ValueError):
        l.setOutput(np.zeros(5))
    empty = pkg.Layer(0, 0, 784)
    assert empty.read("weight").size == 0
    empty.clear(); empty.bp_clear()


def test_layer_init_reproduces_reference_draw_order(cuda, pkg):
    """Net(seed) and three Layer(...) constructions after srand(seed) draw the same parameters."""
    import ctypes
    libc = ctypes.CDLL("libc.so.6")
    libc.srand(0)
    c1 = pkg.Layer(25, 6, 3456); s1 = pkg.Layer(16, 1, 216); f = pkg.Layer(216, 10, 10)
    net = pkg.Net(0)
    p = net.get_params()
    assert np.array_equal(p[0:150], c1.read("weight")) and np.array_equal(p[150:156], c1.read("bias"))
    assert np.array_equal(p[156:172], s1.read("weight")) and np.array_equal(p[172:173], s1.read("bias"))
    assert np.array_equal(p[173:2333], f.read("weight")) and np.array_equal(p[2333:], f.read("bias"))
    libc.srand(0)
    first = np.float32(0.5) - np.float32(libc.rand()) / np.float32(2147483647)
    assert p[150] == first  # the first draw is c1.bias[0]


def test_operator_sequence_matches_oracle(cuda, pkg, ob, params0, data64):
    images, labels = data64
    for i in (0, 5, 17):
        net = Net4(pkg, params0)
        net.forward_pass(images[i])
        p1, err, tr = ob.sgd_step(params0, images[i], int(labels[i]))
        check_buffers(lambda l, b: getattr(net, l).read(b), tr,
                      ["c1_preact", "c1_output", "s1_preact", "s1_output", "f_preact", "f_output"])
        net.back_pass(int(labels[i]))
        check_buffers(lambda l, b: getattr(net, l).read(b), tr,
                      ["f_d_preact", "f_d_weight", "s1_d_output", "s1_d_preact", "s1_d_weight",
                       "c1_d_output", "c1_d_preact", "c1_d_weight"])
        assert scaled_err(net.params(), p1) < 1e-5
        assert scaled_err(net.params() - params0, p1 - params0) < 1e-4


def test_operators_accumulate_like_the_reference(cuda, pkg, params0, data64):
    """Operators the reference implements with atomicAdd add INTO their destination."""
    images, _ = data64
    net = Net4(pkg, params0)
    net.forward_pass(images[1])
    base = net.c1.read("preact")
    net.input.setOutput(images[1])
    net.c1.write("preact", np.full(3456, 2.0))
    pkg.fp_preact_c1(net.input.output, net.c1.preact, net.c1.weight)
    pkg.fp_bias_c1(net.c1.preact, net.c1.bias)
    assert scaled_err(net.c1.read("preact") - 2.0, base) < 1e-5
    before = net.f.read("bias")
    net.f.write("d_preact", np.arange(10))
    pkg.bp_bias_f(net.f.bias, net.f.d_preact)
    assert np.allclose(net.f.read("bias"), before + 0.1 * np.arange(10), rtol=1e-6, atol=1e-7)


def test_operators_are_deterministic(cuda, pkg, params0, data64):
    images, labels = data64
    runs = []
    for _ in range(2):
        net = Net4(pkg, params0)
        net.forward_pass(images[2]); net.back_pass(int(labels[2]))
        runs.append(net.params())
    assert np.array_equal(runs[0], runs[1])


# The reference kernels compute N * thread_index in int, so with N = 86,400 they are only valid for
# launches of fewer than 24,855 threads; (96, 256) is the largest shape tried.
@pytest.mark.parametrize("shape", [(64, 64), (1, 32), (96, 256), (3, 7), (10, 1)])
def test_against_reference_kernels(cuda, pkg, ob, params0, data64, shape):
    """Same inputs through the reference's own CUDA kernels (unmodified layer.cu)."""
    if not ob.reference_available():
        pytest.skip("reference kernels not built")
    images, labels = data64
    ref = ob.Reference(0)
    ref.set_params(params0)
    g, b = shape
    for i in (0, 9):
        ref.set_params(params0)
        err_ref = ref.train_step(images[i], int(labels[i]), g, b)
        net = Net4(pkg, params0)
        net.forward_pass(images[i]); net.back_pass(int(labels[i]))
        for name, (layer, buf) in TRACE_TO_LAYER.items():
            got, want = getattr(net, layer).read(buf), ref.read(layer, buf)
            if buf == "output":
                assert rel_err(got, want) < 1e-5, (name, shape)
            else:
                assert scaled_err(got, want) < 1e-5, (name, shape)
        assert scaled_err(net.params(), ref.get_params()) < 1e-5
        assert scaled_err(net.params() - params0, ref.get_params() - params0) < 1e-4
        d = net.f.read("d_preact")
        assert abs(float(np.sqrt((d.astype(np.float64) ** 2).sum())) - err_ref) < 1e-5
    ref.close()


def test_reference_own_init_matches_net_seed0(cuda, pkg, ob):
    if not ob.reference_available():
        pytest.skip("reference kernels not built")
    ref = ob.Reference(0)
    assert np.array_equal(ref.get_params(), pkg.Net(0).get_params())
    ref.close()
