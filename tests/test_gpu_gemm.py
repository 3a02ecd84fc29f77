"""The tcgen05 GEMM against a plain fp32 torch reference, through the C ABI."""
from __future__ import annotations

import pytest
import torch

from oracle import packed_oracle as O

pytestmark = pytest.mark.gpu

# (M, N, K): every projection shape of the base / large / 1B models, plus ragged M
SHAPES = [
    (128, 256, 64), (1, 768, 768), (127, 768, 768), (129, 2304, 768), (1000, 768, 1152),
    (4097, 2304, 768), (300, 3072, 1024), (300, 1024, 2624), (300, 5248, 1024),
    (200, 5376, 1792), (200, 1792, 3840), (200, 7680, 1792), (77, 8, 8), (513, 72, 200),
]


def _inputs(m, n, k, device, seed=0):
    gen = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=gen).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=gen) * 0.05).to(torch.bfloat16)
    return a, w, a.to(device), w.to(device)


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_gemm_matches_fp32_reference(pe, cuda_device, m, n, k):
    from flash_modernbert_b200 import ops

    a, w, a_d, w_d = _inputs(m, n, k, cuda_device)
    out = ops._linear(a_d, w_d)
    ops.check_status(cuda_device)
    ref = a_d.float() @ w_d.float().t()           # fp32 reference of the same op
    got = out.float()
    # bf16 output of an fp32 accumulation: half a bf16 step of the result plus fp32 summation-order noise
    tol = ref.abs() * 2 ** -8 + 1e-3 * (k ** 0.5) * 0.05
    assert bool(((got - ref).abs() <= tol).all()), float((got - ref).abs().max())
    # tolerance of the reference's own GEMM test (tests/test_matmul.py:49-55)
    torch.testing.assert_close(out, torch.nn.functional.linear(a_d, w_d), rtol=1e-2, atol=1.0)


def test_gemm_is_deterministic_and_handles_empty(pe, cuda_device):
    from flash_modernbert_b200 import ops

    _, _, a_d, w_d = _inputs(2000, 768, 768, cuda_device, seed=1)
    assert torch.equal(ops._linear(a_d, w_d), ops._linear(a_d, w_d))
    empty = ops._linear(a_d[:0], w_d)
    assert empty.shape == (0, 768)
    lead = ops._linear(a_d.view(4, 500, 768), w_d)
    assert lead.shape == (4, 500, 768) and torch.equal(lead.view(2000, 768), ops._linear(a_d, w_d))


def test_gemm_linearity_at_full_size(pe, cuda_device):
    """cfg3-sized M: W (a + b) == W a + W b up to rounding, and row blocks are independent."""
    from flash_modernbert_b200 import ops

    gen = torch.Generator(device=cuda_device).manual_seed(0)
    m = 306851
    a = torch.randn(m, 768, device=cuda_device, generator=gen).to(torch.bfloat16)
    w = (torch.randn(2304, 768, device=cuda_device, generator=gen) * 0.05).to(torch.bfloat16)
    full = ops._linear(a, w)
    ops.check_status(cuda_device)
    rows = torch.randint(0, m, (4096,), device=cuda_device)
    ref = a[rows].float() @ w.float().t()
    assert float((full[rows].float() - ref).abs().max()) < 0.05
    tail = ops._linear(a[m - 1000:], w)
    assert torch.equal(tail, full[m - 1000:])


@pytest.mark.parametrize("m,inter,k", [(129, 1152, 768), (1000, 1152, 768), (300, 2624, 1024), (200, 3840, 1792), (64, 128, 64)])
def test_fused_wi_geglu_equals_two_kernels(pe, cuda_device, m, inter, k):
    from flash_modernbert_b200 import ops

    a, wi, a_d, wi_d = _inputs(m, 2 * inter, k, cuda_device, seed=2)
    fused = ops.linear_geglu(a_d, wi_d)
    two = ops.fused_geglu(ops._linear(a_d, wi_d))
    ops.check_status(cuda_device)
    assert torch.equal(fused, two)                 # same rounding points => same bits
    ref = O.geglu(O.linear(a, wi))
    assert float((fused.cpu().float() - ref).abs().max()) <= 0.02 * float(ref.abs().max()) + 1e-3


@pytest.mark.parametrize("m,n_heads,k", [(129, 12, 768), (1000, 12, 768), (300, 16, 1024), (200, 28, 1792), (77, 4, 256)])
def test_fused_wqkv_rope_equals_two_kernels(pe, cuda_device, m, n_heads, k):
    from flash_modernbert_b200 import ops

    a, w, a_d, w_d = _inputs(m, 3 * n_heads * 64, k, cuda_device, seed=3)
    pos = torch.randint(0, 8192, (m,), generator=torch.Generator().manual_seed(m)).to(cuda_device)
    table = ops.rope_table(10000.0, 8192, cuda_device)
    fused = ops.linear_qkv_rope(a_d, w_d, pos, table, n_heads)
    two = ops.rope_qk_inplace(ops._linear(a_d, w_d), pos, table, n_heads)
    ops.check_status(cuda_device)
    assert torch.equal(fused, two)                 # same rounding points => same bits
    h = n_heads * 64
    assert torch.equal(fused[:, 2 * h:], ops._linear(a_d, w_d)[:, 2 * h:])   # v is not rotated


@pytest.mark.parametrize("m,n,k", [(129, 768, 768), (1000, 768, 1152), (300, 1024, 2624), (200, 1792, 3840), (77, 72, 64)])
def test_fused_residual_equals_two_steps(pe, cuda_device, m, n, k):
    from flash_modernbert_b200 import ops

    a, w, a_d, w_d = _inputs(m, n, k, cuda_device, seed=4)
    res = torch.randn(m, n, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).to(cuda_device)
    expected = res + ops._linear(a_d, w_d)          # bf16 + bf16 with one rounding, as add+LN forms x_new
    fused = ops.linear_residual(a_d, w_d, res)
    assert torch.equal(fused, expected)
    inplace = res.clone()
    assert ops.linear_residual(a_d, w_d, inplace, inplace=True).data_ptr() == inplace.data_ptr()
    ops.check_status(cuda_device)
    assert torch.equal(inplace, expected)


@pytest.mark.parametrize("m,n,k", [(40961, 768, 768), (45000, 768, 1152)])
def test_inplace_residual_with_several_tiles_per_cta(pe, cuda_device, m, n, k):
    """More output tiles than CTAs (321 x 3 or 352 x 3 tiles on 148 SMs): every CTA owns
    several tiles, so the epilogue's chain that fetches the first block of X for the NEXT tile
    while finishing this one is live, and X is overwritten in place while other CTAs still read
    their own blocks. Bit-exact against the two-step form."""
    from flash_modernbert_b200 import ops

    a, w, a_d, w_d = _inputs(m, n, k, cuda_device, seed=11)
    res = torch.randn(m, n, generator=torch.Generator().manual_seed(12)).to(torch.bfloat16).to(cuda_device)
    expected = res + ops._linear(a_d, w_d)
    inplace = res.clone()
    ops.linear_residual(a_d, w_d, inplace, inplace=True)
    ops.check_status(cuda_device)
    assert torch.equal(inplace, expected)
    assert torch.equal(ops.linear_residual(a_d, w_d, res), expected)


@pytest.mark.parametrize("m", [257, 1000, 4097])
def test_cta_pair_and_single_cta_tiles_agree(pe, cuda_device, m):
    """Above 256 rows every GEMM runs on pairs of CTAs sharing 256 x 256 tiles (cta_group::2);
    `pe_set_option(PE_OPT_GEMM_PAIR, 0)` selects the single-CTA 128 x 256 tiles. Same k order and
    the same epilogues: identical bits in every mode, including ragged last tiles."""
    from flash_modernbert_b200 import _lib, ops

    lib = _lib.load()
    a, w, a_d, w_d = _inputs(m, 2304, 768, cuda_device, seed=21)
    _, wo, _, wo_d = _inputs(m, 768, 768, cuda_device, seed=22)
    _, wp, _, wp_d = _inputs(m, 128, 768, cuda_device, seed=23)
    res = torch.randn(m, 768, generator=torch.Generator().manual_seed(24)).to(torch.bfloat16).to(cuda_device)
    pos = torch.randint(0, 512, (m,), generator=torch.Generator().manual_seed(m)).to(cuda_device)
    table = ops.rope_table(160000.0, 512, cuda_device)

    def run_all():
        return [ops._linear(a_d, w_d), ops.linear_geglu(a_d, w_d), ops.linear_qkv_rope(a_d, w_d, pos, table, 12),
                ops.linear_residual(a_d, wo_d, res), ops.linear_residual(a_d, wo_d, res.clone(), inplace=True),
                ops.project_normalize(a_d, wp_d)]

    paired = run_all()
    try:
        assert lib.pe_set_option(_lib.OPT_GEMM_PAIR, 0) == 0
        single = run_all()
    finally:
        lib.pe_set_option(_lib.OPT_GEMM_PAIR, 1)
    ops.check_status(cuda_device)
    for name, x, y in zip(("plain", "geglu", "rope", "residual", "residual in place", "l2norm"), paired, single):
        assert torch.equal(x, y), name


@pytest.mark.parametrize("m,n,k", [(300, 768, 768), (4097, 768, 1152), (129, 1024, 2624), (513, 72, 200)])
def test_residual_by_reduce_add_in_and_out_of_place(pe, cuda_device, m, n, k):
    """The residual GEMM adds its rounded product to what C holds with TMA reduce-adds (the memory
    system performs the bf16 add) and never reads X; out of place X is copied to C first. One add
    with one rounding per element: the same bits as the two-step form, in place and out of place,
    and X is left untouched out of place."""
    from flash_modernbert_b200 import ops

    a, w, a_d, w_d = _inputs(m, n, k, cuda_device, seed=31)
    res = torch.randn(m, n, generator=torch.Generator().manual_seed(32)).to(torch.bfloat16).to(cuda_device)
    keep = res.clone()
    expected = res + ops._linear(a_d, w_d)
    out_of_place = ops.linear_residual(a_d, w_d, res)
    assert torch.equal(res, keep) and out_of_place.data_ptr() != res.data_ptr()
    in_place = ops.linear_residual(a_d, w_d, res, inplace=True)
    ops.check_status(cuda_device)
    assert torch.equal(out_of_place, expected)
    assert torch.equal(in_place, expected) and in_place.data_ptr() == res.data_ptr()
