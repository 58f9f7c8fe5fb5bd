"""Kernel-based host -> device staging (rxmet_stage_from_pinned_host): byte-exact copies of pinned host
tensors, sizes that are no multiple of 16 bytes, side streams, and the argument checks."""
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    return torch


@pytest.mark.parametrize("numel,dtype_name", [(1, "float32"), (3, "float32"), (4, "float32"), (1027, "float32"),
                                              (100 * 256 * 40, "float32"), (5, "uint8"), (4099, "uint8"), (33, "int32")])
def test_staging_copies_exactly(torch_cuda, numel, dtype_name):
    torch = torch_cuda
    from rx_met_b200.staging import stage_from_pinned_host
    dtype = getattr(torch, dtype_name)
    gen = torch.Generator().manual_seed(numel)
    src = (torch.randn(numel, generator=gen) * 100).to(dtype).pin_memory()
    dst = torch.full((numel + 8,), 7, dtype=dtype, device="cuda")
    side = torch.cuda.Stream()
    for ctas, stream in ((1, None), (4, side), (64, side)):
        dst.fill_(7)
        if stream is not None:
            stream.wait_stream(torch.cuda.current_stream())
        stage_from_pinned_host(dst[:numel], src, ctas=ctas, stream=stream)
        if stream is not None:
            torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        assert torch.equal(dst[:numel].cpu(), src)
        assert bool((dst[numel:] == 7).all())  # nothing beyond the requested bytes is written


def test_staging_argument_checks(torch_cuda):
    torch = torch_cuda
    from rx_met_b200.staging import stage_from_pinned_host
    dst = torch.empty(16, device="cuda")
    with pytest.raises(RuntimeError):
        stage_from_pinned_host(dst, torch.zeros(16))  # pageable source
    with pytest.raises(RuntimeError):
        stage_from_pinned_host(dst, torch.zeros(8).pin_memory())  # size mismatch
    with pytest.raises(RuntimeError):
        stage_from_pinned_host(torch.empty(16), torch.zeros(16).pin_memory())  # host destination
