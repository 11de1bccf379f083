"""frelu, fsoftmax, fpool, fconv2d, ftranspose, fslice: the oracle against the targets the reference's own
tests write out (tests/integration/operations/{ReLU,Softmax,Pool2D,Conv2D}Operation.cpp),
and the CUDA builtins against the oracle."""
import numpy as np
import pytest

# inputs and literal targets of the reference tests (file:line in the reference project)
RELU = (np.array([-1, 1], np.float32), np.array([0, 1], np.float32))                     # ReLUOperation.cpp:22-23
SOFTMAX = (np.array([1, 2, 3, 4], np.float32),
           np.array([0.0320586, 0.08714432, 0.23688282, 0.64391426], np.float32))        # SoftmaxOperation.cpp:36-37
POOL = (np.array([1, 0, 2, 3, 4, 6, 6, 8, 3, 1, 1, 0, 1, 2, 2, 4], np.float32).reshape(4, 4),
        np.array([6, 8, 3, 4], np.float32))                                               # Pool2DOperation.cpp:36-37
CONV = (np.ones((4, 4), np.float32), np.full((3, 3), 0.1, np.float32),
        np.full(4, 0.9, np.float32))                                                      # Conv2DOperation.cpp:36-38


def ulps(a, b):
    ia = np.ascontiguousarray(a, np.float32).ravel().view(np.int32).astype(np.int64)
    ib = np.ascontiguousarray(b, np.float32).ravel().view(np.int32).astype(np.int64)
    return int(np.max(np.abs(ia - ib)))


def check_reference_targets(impl):
    assert np.array_equal(impl.frelu(RELU[0]), RELU[1])
    assert ulps(impl.fsoftmax(SOFTMAX[0]), SOFTMAX[1]) <= 4          # EXPECT_FLOAT_EQ's bound
    assert np.array_equal(impl.fpool(POOL[0], (2, 2), (2, 2)).ravel(), POOL[1])
    assert ulps(impl.fconv2d(CONV[0], CONV[1]).ravel(), CONV[2]) <= 4


def test_oracle_meets_the_reference_targets(oracle):
    check_reference_targets(oracle)
    # softmax is over the whole tensor and does not subtract the maximum
    x = np.array([[0.5, -1.0], [2.0, 0.0]], np.float32)
    e = np.exp(x.astype(np.float64))
    assert np.allclose(oracle.fsoftmax(x), e / e.sum(), rtol=1e-6)
    # pooling never returns less than -10e5
    assert oracle.fpool(np.full((2, 2), -5e6, np.float32), (2, 2), (1, 1))[0, 0] == np.float32(-10e5)
    assert oracle.frelu(np.array([np.nan, -0.0, 3.0], np.float32)).tolist() == [0.0, 0.0, 3.0]


def test_oracle_transpose_and_slice_are_what_numpy_says(oracle):
    # the reference holds no vector for these two (it names the builtins and leaves the kernels
    # empty), so the restatement is checked against the definitions themselves
    rng = np.random.default_rng(5)
    a = rng.standard_normal((37, 53)).astype(np.float32)
    a[0, 0], a[1, 2] = np.nan, -0.0
    assert np.array_equal(oracle.ftranspose(a).view(np.uint32), np.ascontiguousarray(a.T).view(np.uint32))
    t = rng.standard_normal((5, 7, 3)).astype(np.float32)
    for i in (0, 2, 4):
        assert np.array_equal(oracle.fslice(t, i), t[i])


@pytest.fixture(scope="module")
def gpu():
    import __graft_entry__ as ge
    ge.load_package()
    from polarai_framework_b200.device_builtins import HostBuiltins
    return HostBuiltins("cuda:0")


@pytest.mark.gpu
def test_cuda_meets_the_reference_targets(gpu):
    check_reference_targets(gpu)


@pytest.mark.gpu
def test_cuda_against_oracle_on_seeded_inputs(gpu, oracle):
    rng = np.random.default_rng(11)
    x = rng.uniform(-3, 3, 100_003).astype(np.float32)
    x[:3] = [np.nan, -0.0, 0.0]
    assert np.array_equal(gpu.frelu(x).view(np.uint32), oracle.frelu(x).view(np.uint32))
    s = rng.uniform(-4, 4, 50_001).astype(np.float32)
    got, want = gpu.fsoftmax(s), oracle.fsoftmax(s)
    assert np.max(np.abs(got - want) / want) <= 1e-5
    assert abs(float(got.astype(np.float64).sum()) - 1.0) <= 1e-5
    img = rng.uniform(-1, 1, (67, 131)).astype(np.float32)
    for window, stride in (((2, 2), (2, 2)), ((3, 5), (2, 1)), ((67, 131), (1, 1)), ((1, 1), (3, 4))):
        assert np.array_equal(gpu.fpool(img, window, stride), oracle.fpool(img, window, stride))
    for kshape in ((3, 3), (5, 1), (1, 7), (67, 131)):
        ker = rng.uniform(-1, 1, kshape).astype(np.float32)
        assert np.array_equal(gpu.fconv2d(img, ker).view(np.uint32), oracle.fconv2d(img, ker).view(np.uint32))


@pytest.mark.gpu
def test_transpose_and_slice_against_oracle(gpu, oracle):
    rng = np.random.default_rng(6)
    for shape in ((1, 1), (32, 32), (33, 31), (1, 1000), (1000, 1), (257, 4099), (4096, 10)):
        a = rng.standard_normal(shape).astype(np.float32)
        a.ravel()[:2] = [np.nan, -0.0][:a.size]
        assert np.array_equal(gpu.ftranspose(a).view(np.uint32), oracle.ftranspose(a).view(np.uint32)), shape
    t = rng.standard_normal((6, 17, 5)).astype(np.float32)
    for i in (0, 3, 5):
        assert np.array_equal(gpu.fslice(t, i).view(np.uint32), oracle.fslice(t, i).view(np.uint32))
    v = rng.standard_normal((9,)).astype(np.float32)          # a vector slices into scalars
    assert gpu.fslice(v, 4).reshape(()) == v[4]
    import torch
    from polarai_framework_b200.capi import PolarB200Error
    with pytest.raises(PolarB200Error):
        gpu.d.fslice(torch.zeros((3, 4), device="cuda"), 3, torch.zeros(4, device="cuda"))   # index out of range


@pytest.mark.gpu
def test_bad_shapes_are_statuses(gpu):
    import torch
    from polarai_framework_b200.capi import PolarB200Error
    a = torch.zeros((4, 4), device="cuda")
    k = torch.zeros((2, 2), device="cuda")
    out = torch.zeros((3, 3), device="cuda")
    with pytest.raises(PolarB200Error):
        gpu.d.fconv2d(a, k, out)                       # even kernel extents: not what the reference computes
    with pytest.raises(PolarB200Error):
        gpu.d.fpool(a, (5, 1), (1, 1), out)            # window larger than the input
