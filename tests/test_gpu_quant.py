"""GPU numerics of the quantised serving kernels against the PyTorch fp32 oracles."""

import pytest
import torch

from triune_b200 import ops
from triune_b200.ops import quant_cuda, reference as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")


def test_fp8_act_quantiser_matches_oracle():
    torch.manual_seed(0)
    x = (torch.randn(300, 384, device="cuda") * 3).bfloat16()
    q, s = quant_cuda.fp8_quantize_act(x)
    q_ref, s_ref = ref.fp8_block_quantize_act(x)
    assert torch.allclose(s, s_ref, rtol=1e-6, atol=0)
    deq, deq_ref = q.float() * s.repeat_interleave(128, 1), q_ref.float() * s_ref.repeat_interleave(128, 1)
    # one E4M3 ulp at most where the division rounds differently
    assert (deq - deq_ref).abs().max() <= 0.07 * deq_ref.abs().max()
    assert (q.view(torch.uint8) != q_ref.view(torch.uint8)).float().mean() < 0.01


@pytest.mark.parametrize("M,N,K", [(256, 256, 384), (1000, 1536, 384), (4096, 384, 1536), (130, 200, 272)])
def test_fp8_block_gemm_matches_dequant_oracle(M, N, K):
    torch.manual_seed(1)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda") * 0.05
    wq, ws = ref.fp8_block_quantize_weight(w)
    xq, xs = quant_cuda.fp8_quantize_act(x)
    y = quant_cuda.fp8_block_gemm(xq, xs, wq, ws).float()
    want = ref.fp8_block_gemm(xq, xs, wq, ws, 128, torch.float32)
    err = (y - want).abs().max() / want.abs().max()
    assert err < 1e-2, err  # bf16 output rounding only: the operands are identical
    full = x.float() @ w.t()
    assert torch.nn.functional.cosine_similarity(y.flatten(), full.flatten(), dim=0) > 0.995


@pytest.mark.parametrize("hadamard", [False, True])
def test_nvfp4_quantise_and_dequant(hadamard):
    torch.manual_seed(2)
    w = torch.randn(192, 256, device="cuda") * 0.1
    p, s, t = quant_cuda.nvfp4_quantize(w, hadamard)
    wr = ref.fwht16(w) if hadamard else w
    p_ref, s_ref, t_ref = ref.nvfp4_quantize(wr)
    assert torch.allclose(t, t_ref, rtol=1e-6)
    assert (s.view(torch.uint8) != s_ref.view(torch.uint8)).float().mean() < 0.01
    assert (p != p_ref).float().mean() < 0.02
    deq = quant_cuda.nvfp4_dequant(p, s, t).float()
    assert torch.equal(deq, ref.nvfp4_dequantize(p, s, t, torch.bfloat16).float())
    assert torch.nn.functional.cosine_similarity(deq.flatten(), wr.flatten(), dim=0) > 0.98
    # bf16 block scales (the reference's legacy layout) decode through the same kernel
    p2, s2, t2 = ref.nvfp4_quantize(wr, torch.bfloat16)
    assert torch.equal(quant_cuda.nvfp4_dequant(p2, s2, t2).float(), ref.nvfp4_dequantize(p2, s2, t2, torch.bfloat16).float())


@pytest.mark.parametrize("M", [1, 3, 8, 64])
def test_nvfp4_linear_paths(M):
    torch.manual_seed(3)
    w = torch.randn(512, 384, device="cuda") * 0.05
    x = torch.randn(M, 384, device="cuda").bfloat16()
    p, s, t = quant_cuda.nvfp4_quantize(w)
    y = ops.nvfp4_linear(x, p, s, t).float()
    want = x.float() @ ref.nvfp4_dequantize(p, s, t, torch.float32).t()
    assert (y - want).abs().max() <= 2e-2 * want.abs().max()


@pytest.mark.parametrize("hadamard", [False, True])
def test_nvfp4_activation_quantiser_matches_oracle(hadamard):
    torch.manual_seed(5)
    x = (torch.randn(200, 384, device="cuda") * 1.5).bfloat16()
    p, sf = quant_cuda.nvfp4_quantize_act(x, hadamard)
    p_ref, s_ref = ref.nvfp4_quantize_act(x, hadamard)
    s = ref.nvfp4_unblock_scales(sf, 200, 384)
    assert (s.view(torch.uint8) != s_ref.view(torch.uint8)).float().mean() < 0.01
    assert (p != p_ref).float().mean() < 0.02
    # the blocked layout: re-blocking the oracle's scales gives the kernel's buffer wherever the scales agree
    same = (s.view(torch.uint8) == s_ref.view(torch.uint8)).all()
    if same:
        assert torch.equal(ref.nvfp4_block_scales(s_ref, 384), sf)
    # weight scales through the layout kernel
    w_s = ref.nvfp4_quantize(torch.randn(136, 384, device="cuda"))[1]
    assert torch.equal(quant_cuda.nvfp4_block_scales(w_s, 384), ref.nvfp4_block_scales(w_s, 384))


@pytest.mark.parametrize("tile_n", [128, 256])
@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (256, 384, 512), (200, 136, 384), (1000, 1536, 2048), (4096, 512, 1056)])
def test_nvfp4_block_scaled_gemm_matches_decoded_product(M, N, K, tile_n):
    """E2M1 x E2M1 with both scale sets applied by the tensor core == the fp32 product of the decoded operands."""
    torch.manual_seed(6)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda") * 0.05
    wp, ws, wt = quant_cuda.nvfp4_quantize(w)
    a_p, a_sf = quant_cuda.nvfp4_quantize_act(x, False)
    y, status = quant_cuda._ext.ext().nvfp4_gemm(a_p, a_sf, wp, quant_cuda.nvfp4_block_scales(ws, K), float(wt), tile_n)
    assert int(status.item()) == 0
    a = ref.nvfp4_dequantize(a_p, ref.nvfp4_unblock_scales(a_sf, M, K), 1.0, torch.float32)
    want = a @ ref.nvfp4_dequantize(wp, ws, wt, torch.float32).t()
    err = (y.float() - want).abs().max() / want.abs().max()
    assert err < 1e-2, err  # bf16 output rounding only: the operands are identical and the products exact in fp32
    full = x.float() @ w.t()
    assert torch.nn.functional.cosine_similarity(y.float().flatten(), full.flatten(), dim=0) > 0.97


def test_nvfp4_module_takes_the_block_scaled_path_for_prefill():
    from triune_b200.models.quant_linear import NVFP4Linear

    torch.manual_seed(7)
    lin = torch.nn.Linear(512, 384, bias=True).cuda().bfloat16()
    x = torch.randn(3, 50, 512, device="cuda").bfloat16()
    want = lin(x).float()
    for hadamard in (False, True):
        m = NVFP4Linear.from_linear(lin, hadamard=hadamard)
        assert m._w4a4_ready(x.reshape(-1, 512))
        with torch.no_grad():
            y = m(x).float()
            oracle = ref.nvfp4_w4a4_linear(x.reshape(-1, 512), m.packed_weight, m.block_scales, m.tensor_scale, hadamard)
        assert int(quant_cuda.last_gemm_status.item()) == 0
        oracle = oracle.reshape(3, 50, 384) + lin.bias.float()
        assert (y - oracle).abs().max() <= 3e-2 * oracle.abs().max()  # differs only where a scale or code rounds the other way
        assert torch.nn.functional.cosine_similarity(y.flatten(), want.flatten(), dim=0) > 0.97
        m.w4a4 = False
        with torch.no_grad():
            y16 = m(x).float()
        assert torch.nn.functional.cosine_similarity(y16.flatten(), want.flatten(), dim=0) > 0.98


def test_mxfp8_quantiser_matches_oracle():
    torch.manual_seed(8)
    x = (torch.randn(200, 384, device="cuda") * torch.logspace(-3, 2, 384, device="cuda")).bfloat16()
    x[5] = 0
    q, sf = quant_cuda.mxfp8_quantize(x)
    q_ref, e_ref = ref.mxfp8_quantize(x)
    e = ref.mxfp8_unblock_scales(sf, 200, 384)
    assert torch.equal(e, e_ref)  # exponents are exact integer arithmetic
    assert torch.equal(ref.mxfp8_block_scales(e_ref, 384), sf)
    assert (q.view(torch.uint8) != q_ref.view(torch.uint8)).float().mean() < 1e-3
    deq = ref.mxfp8_dequantize(q, e)
    assert (deq - x.float()).abs().max() <= 0.0625 * x.float().abs().max()  # half an E4M3 ulp (3 mantissa bits)
    assert torch.nn.functional.cosine_similarity(deq.flatten(), x.float().flatten(), dim=0) > 0.999


@pytest.mark.parametrize("tile_n", [128, 256])
@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 512), (200, 136, 416), (1000, 1536, 2048), (4096, 512, 1056)])
def test_mxfp8_block_scaled_gemm_matches_decoded_product(M, N, K, tile_n):
    """E4M3 x E4M3 with 1x32 power-of-two scales applied by the tensor core == the fp32 product of the decoded operands."""
    torch.manual_seed(9)
    x = (torch.randn(M, K, device="cuda") * torch.logspace(-1, 1, K, device="cuda")).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    xq, x_sf = quant_cuda.mxfp8_quantize(x)
    wq, w_sf = quant_cuda.mxfp8_quantize(w)
    y = quant_cuda.mxfp8_gemm(xq, x_sf, wq, w_sf, 1.0, tile_n)
    assert int(quant_cuda.last_gemm_status.item()) == 0
    a = ref.mxfp8_dequantize(xq, ref.mxfp8_unblock_scales(x_sf, M, K))
    b = ref.mxfp8_dequantize(wq, ref.mxfp8_unblock_scales(w_sf, N, K))
    want = a @ b.t()
    err = (y.float() - want).abs().max() / want.abs().max()
    assert err < 1e-2, err  # bf16 output rounding only
    full = x.float() @ w.float().t()
    assert torch.nn.functional.cosine_similarity(y.float().flatten(), full.flatten(), dim=0) > 0.998


def test_fp8_module_takes_the_block_scaled_path():
    from triune_b200.models.quant_linear import FP8Linear

    torch.manual_seed(10)
    lin = torch.nn.Linear(512, 384, bias=True).cuda().bfloat16()
    x = torch.randn(3, 50, 512, device="cuda").bfloat16()
    want = lin(x).float()
    m = FP8Linear.from_linear(lin).eval()
    with torch.no_grad():
        y_mx = m(x).float()
        m.mx = False
        y_blk = m(x).float()
    oracle = ref.mxfp8_linear(x.reshape(-1, 512), lin.weight).reshape(3, 50, 384) + lin.bias.float()
    assert (y_mx - oracle).abs().max() <= 2e-2 * oracle.abs().max()
    cos = torch.nn.functional.cosine_similarity
    assert cos(y_mx.flatten(), want.flatten(), dim=0) > 0.998
    assert cos(y_mx.flatten(), want.flatten(), dim=0) >= cos(y_blk.flatten(), want.flatten(), dim=0) - 1e-3  # finer scales


def test_block_scaled_gemm_bias_and_gelu_epilogues():
    """Bias and tanh-GELU inside the block-scaled GEMM epilogues == the same applied to the plain GEMM's output."""
    from triune_b200.models.quant_linear import FP8Linear, NVFP4Linear

    torch.manual_seed(11)
    lin = torch.nn.Linear(512, 384, bias=True).cuda().bfloat16()
    with torch.no_grad():
        lin.bias.mul_(20.0)  # a bias large enough to matter
    x = torch.randn(300, 512, device="cuda").bfloat16()
    for mod in (FP8Linear.from_linear(lin).eval(), NVFP4Linear.from_linear(lin)):
        with torch.no_grad():
            plain = mod(x).float()
            fused = mod(x, gelu=True).float()
            mod_nobias = type(mod).from_linear(torch.nn.Linear(512, 384, bias=False).cuda().bfloat16())
        want = torch.nn.functional.gelu(plain, approximate="tanh")
        assert (fused - want).abs().max() <= 2e-2 * want.abs().max().clamp_min(1.0), type(mod).__name__
        assert int(quant_cuda.last_gemm_status.item()) == 0
        # the bias really is in: remove it and the outputs move by the bias
        if isinstance(mod, FP8Linear):
            mod_nobias.weight.data.copy_(lin.weight)
            with torch.no_grad():
                nb = mod_nobias.eval()(x).float()
            assert (plain - nb - lin.bias.float()).abs().max() <= 3e-2 * plain.abs().max()


def test_fwht16_kernel():
    x = torch.randn(64, 128, device="cuda").bfloat16()
    y = quant_cuda.fwht16(x)
    assert torch.allclose(y.float(), ref.fwht16(x.float()), atol=2e-2, rtol=2e-2)
    assert torch.allclose(quant_cuda.fwht16(y).float(), x.float(), atol=3e-2, rtol=3e-2)  # involution


def test_quantised_modules_on_gpu():
    from triune_b200.models.quant_linear import FP8Linear, NVFP4Linear

    torch.manual_seed(4)
    lin = torch.nn.Linear(384, 512, bias=True).cuda().bfloat16()
    x = torch.randn(2, 40, 384, device="cuda").bfloat16()
    want = lin(x).float()
    for m in (FP8Linear.from_linear(lin).eval(), NVFP4Linear.from_linear(lin), NVFP4Linear.from_linear(lin, hadamard=True)):
        with torch.no_grad():
            y = m(x).float()
        assert torch.nn.functional.cosine_similarity(y.flatten(), want.flatten(), dim=0) > 0.98, type(m).__name__
