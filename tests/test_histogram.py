"""The 256-bin byte histogram (the reference repository's second task, pmpp_v2/histogram_py).

CPU: the checker (the reference's own ``torch.bincount`` call) against an operator-free restatement,
hand-written answers and the committed fixture.  GPU: the kernel through the C ABI against the
checker, bit-exact (integer work), on the task's own test and benchmark sizes and contentions, on
ragged sizes, unaligned starts and degenerate inputs."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import histogram_oracle as HO

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "histogram.npz")


def test_checker_known_answers():
    data = torch.tensor([0, 0, 255, 7, 7, 7, 200], dtype=torch.uint8)
    want = np.zeros(256, dtype=np.int64)
    want[0], want[255], want[7], want[200] = 2, 1, 3, 1
    assert np.array_equal(HO.ref_histogram(data).numpy(), want)
    assert np.array_equal(HO.count_bytes(data), want)
    empty = torch.zeros(0, dtype=torch.uint8)
    assert int(HO.ref_histogram(empty).sum()) == 0 and HO.ref_histogram(empty).shape == (256,)


@pytest.mark.parametrize("size,seed,contention", HO.REFERENCE_TESTS)
def test_checker_agrees_with_its_restatement(size, seed, contention):
    data, out = HO.generate_input(size, contention, seed)
    h = HO.ref_histogram(data)
    assert h.dtype == torch.int64 and int(h.sum()) == size
    assert np.array_equal(h.numpy(), HO.count_bytes(data))
    # the generator's "evil" value really dominates at high contention
    if contention >= 90:
        assert int(h.max()) > 0.85 * size
    assert out.shape == (256,) and out.dtype == torch.int64


def test_checker_reproduces_the_committed_fixture():
    z = np.load(GOLDEN)
    for i in range(int(z["cases"])):
        size, seed, contention = (int(v) for v in z[f"c{i}_spec"])
        data, _ = HO.generate_input(size, contention, seed)
        assert np.array_equal(data.numpy(), z[f"c{i}_data"])
        assert np.array_equal(HO.ref_histogram(data).numpy(), z[f"c{i}_hist"])


def _run(data_gpu):
    from gpu_mode_kernels_b200.histogram import custom_kernel

    out = torch.full((256,), -5, dtype=torch.int64, device=data_gpu.device)  # stale content must be overwritten
    got = custom_kernel((data_gpu, out))
    torch.cuda.synchronize()
    assert got is out
    return out.cpu()


@pytest.mark.gpu
@pytest.mark.parametrize("size,seed,contention", HO.REFERENCE_TESTS + HO.REFERENCE_BENCHMARKS)
def test_reference_task_cases(size, seed, contention):
    data, _ = HO.generate_input(size, contention, seed)
    assert torch.equal(_run(data.to("cuda:0")), HO.ref_histogram(data))


@pytest.mark.gpu
def test_committed_fixture_on_the_gpu():
    z = np.load(GOLDEN)
    for i in range(int(z["cases"])):
        data = torch.from_numpy(z[f"c{i}_data"].copy())
        assert np.array_equal(_run(data.to("cuda:0")).numpy(), z[f"c{i}_hist"])


@pytest.mark.gpu
@pytest.mark.parametrize("size", [0, 1, 15, 16, 17, 31, 33, 4095, 4097, 1 << 20])
@pytest.mark.parametrize("offset", [0, 1, 7])
def test_ragged_sizes_and_unaligned_starts(size, offset):
    g = torch.Generator().manual_seed(size * 8 + offset)
    base = torch.randint(0, 256, (size + offset,), dtype=torch.uint8, generator=g)
    data = base.to("cuda:0")[offset:]  # starts `offset` bytes past an aligned allocation
    assert torch.equal(_run(data.contiguous() if offset == 0 else data), HO.ref_histogram(base[offset:]))


@pytest.mark.gpu
def test_degenerate_inputs_and_two_calls_in_a_row():
    same = torch.full((1 << 22,), 200, dtype=torch.uint8)
    h = _run(same.to("cuda:0"))
    assert int(h[200]) == 1 << 22 and int(h.sum()) == 1 << 22
    ramp = (torch.arange(1 << 16) % 256).to(torch.uint8)
    assert torch.equal(_run(ramp.to("cuda:0")), torch.full((256,), 256, dtype=torch.int64))


@pytest.mark.gpu
def test_arguments_are_checked():
    from gpu_mode_kernels_b200 import _lib
    from gpu_mode_kernels_b200.histogram import histogram256

    data = torch.zeros(64, dtype=torch.uint8, device="cuda:0")
    out = torch.zeros(256, dtype=torch.int64, device="cuda:0")
    for bad in ((data.to(torch.int32), out), (data, out.to(torch.int32)), (data, out[:100]), (data.cpu(), out)):
        with pytest.raises(_lib.A2AError):
            histogram256(*bad)
    lib = _lib.load()
    assert lib.a2a_histogram256(None, 16, C.c_void_p(out.data_ptr()), None) == _lib.A2A_ERR_CONFIG
    assert lib.a2a_histogram256(C.c_void_p(data.data_ptr()), 16, None, None) == _lib.A2A_ERR_CONFIG
