"""fp8 block-scaled quantisation kernels against their fp32 PyTorch restatement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols", [(1, 128), (17, 7168), (128, 7168), (333, 2048)])
def test_quant_1x128_matches_reference(rows, cols):
    from dlslime_b200.ops import quant

    torch.manual_seed(0)
    x = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    x[0, :128] = 0  # an all-zero group exercises the amax floor
    q, s = quant.fp8_quant_1x128(x)
    q_ref, s_ref = quant.ref_quant_1x128(x)
    torch.cuda.synchronize()
    assert torch.equal(s, s_ref)
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))
    y = quant.fp8_dequant_1x128(q, s)
    y_ref = quant.ref_dequant_1x128(q_ref, s_ref).to(torch.bfloat16)
    assert torch.equal(y, y_ref)
    # round trip error is bounded by half an fp8 ulp of the group maximum (2^-4 relative)
    err = (y.float() - x.float()).abs().reshape(rows, -1, 128).amax(-1)
    bound = x.float().abs().reshape(rows, -1, 128).amax(-1).clamp_min(1e-4) * 2 ** -4 + 1e-6
    assert (err <= bound).all()


@pytest.mark.parametrize("rows,cols", [(128, 128), (256, 7168), (200, 328)])
def test_quant_128x128_matches_reference(rows, cols):
    from dlslime_b200.ops import quant

    torch.manual_seed(1)
    w = (torch.randn(rows, cols, device="cuda") * 0.02).to(torch.bfloat16)
    q, s = quant.fp8_quant_128x128(w)
    q_ref, s_ref = quant.ref_quant_128x128(w)
    torch.cuda.synchronize()
    assert torch.equal(s, s_ref)
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))


def test_quant_1x128_strided_rows():
    """Rows that are slices of a wider matrix (pitch != cols) take the kernels' general addressing path."""
    from dlslime_b200.ops import quant

    torch.manual_seed(2)
    wide = torch.randn(45, 1024, device="cuda", dtype=torch.bfloat16)
    x = wide[:, 256:768]
    q_wide = torch.zeros(45, 1024, device="cuda", dtype=torch.uint8).view(torch.float8_e4m3fn)
    q, s = quant.fp8_quant_1x128(x, out=q_wide[:, 128:640])
    q_ref, s_ref = quant.ref_quant_1x128(x.contiguous())
    torch.cuda.synchronize()
    assert torch.equal(s, s_ref)
    assert torch.equal(q.contiguous().view(torch.uint8), q_ref.view(torch.uint8))
    assert q_wide.view(torch.uint8)[:, :128].eq(0).all() and q_wide.view(torch.uint8)[:, 640:].eq(0).all()
    y_wide = torch.zeros(45, 1024, device="cuda", dtype=torch.bfloat16)
    y = quant.fp8_dequant_1x128(q, s, out=y_wide[:, 512:])
    assert torch.equal(y, quant.ref_dequant_1x128(q_ref, s_ref).to(torch.bfloat16))
    assert y_wide[:, :512].eq(0).all()
