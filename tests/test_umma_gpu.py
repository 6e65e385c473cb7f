"""tcgen05 building blocks: shared-memory descriptors for the three operand-layout combinations,
the swizzled tile layout and the tensor-memory readback, checked against torch matmul."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("N,kred", [(128, 128), (64, 128), (128, 64), (64, 64)])
def test_umma_tile_product(mode, N, kred):
    from hattention_b200 import _lib
    lib = _lib.lib()
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(mode * 10 + N + kred)
    a_shape = (kred, 128) if mode == 2 else (128, kred)
    b_shape = (N, kred) if mode == 0 else (kred, N)
    A = torch.randn(a_shape, generator=gen).bfloat16().to(dev)
    B = torch.randn(b_shape, generator=gen).bfloat16().to(dev)
    D = torch.zeros(128, N, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = lib.llattn_selftest_umma(A.data_ptr(), B.data_ptr(), D.data_ptr(), N, kred, mode, err.data_ptr(),
                                  torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert err.item() == 0, "tensor core completion was not signalled"
    Af, Bf = A.float(), B.float()
    want = Af @ Bf.T if mode == 0 else (Af @ Bf if mode == 1 else Af.T @ Bf)
    assert torch.allclose(D, want, rtol=1e-3, atol=1e-2), (D - want).abs().max().item()
