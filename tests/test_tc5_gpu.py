"""Known-answer tests of the tcgen05 building blocks (tensor-memory allocation, shared-memory / instruction descriptors,
MMA issue + commit, tensor-memory loads and stores) through fr_tc5_selftest of the test-only library libflagrot_tc5test.so: D[128][N] = A[128][K] B[N][K]^T against
torch on the same operands.  FP16 products with fp32 accumulation are compared with a float64 product (tolerance 1e-3 of
the result scale); the u8 x s8 product must be exact."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L():
    from pathlib import Path
    path = Path(__file__).resolve().parents[1] / "flagrot_releaser_b200" / "lib" / "libflagrot_tc5test.so"
    assert path.exists(), f"{path} missing: run python -m flagrot_releaser_b200._build"
    lib = ctypes.CDLL(str(path))
    lib.fr_tc5_selftest.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                    ctypes.c_void_p]
    lib.fr_tc5_selftest.restype = ctypes.c_int
    return lib


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("N,K", [(64, 128), (128, 64), (16, 64), (128, 256), (32, 192)])
def test_f16(L, mode, N, K):
    g = torch.Generator().manual_seed(N + K + mode)
    A = torch.randn(128, K, generator=g).half().cuda()
    B = torch.randn(N, K, generator=g).half().cuda()
    D = torch.full((128, N), float("nan"), dtype=torch.float32, device="cuda")
    rc = L.fr_tc5_selftest(mode, A.data_ptr(), B.data_ptr(), D.data_ptr(), N, K, None)
    assert rc == 0, rc
    ref = A.double() @ B.double().T
    assert torch.allclose(D.double(), ref, rtol=0, atol=1e-3 * float(ref.abs().max())), float((D.double() - ref).abs().max())


@pytest.mark.parametrize("N,K", [(16, 32), (32, 128), (128, 512), (64, 64)])
def test_i8(L, N, K):
    g = torch.Generator().manual_seed(N + K)
    A = torch.randint(0, 256, (128, K), generator=g, dtype=torch.uint8).cuda()
    B = torch.randint(-128, 128, (N, K), generator=g, dtype=torch.int8).cuda()
    D = torch.full((128, N), -7, dtype=torch.int32, device="cuda")
    rc = L.fr_tc5_selftest(2, A.data_ptr(), B.data_ptr(), D.data_ptr(), N, K, None)
    assert rc == 0, rc
    ref = (A.cpu().long() @ B.cpu().long().T).int()
    assert torch.equal(D.cpu(), ref)


def test_shapes_refused(L):
    assert L.fr_tc5_selftest(0, None, None, None, 24, 64, None) == -3
    assert L.fr_tc5_selftest(2, None, None, None, 16, 48, None) == -3
    assert L.fr_tc5_selftest(5, None, None, None, 16, 64, None) == -3
