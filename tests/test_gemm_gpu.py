"""tcgen05 GEMM family vs. a plain PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float().t() if b_mn else b.float()
    return A @ B.t()


def _close(out, ref, k):
    tol = 2e-2 * max(1.0, (k ** 0.5) / 8)
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err <= tol * scale / 4 + 1e-2, f"max err {err} (scale {scale})"
    # the element-wise bound above only catches mis-indexed tiles; a dropped k-slice at large K changes
    # every element a little, which the relative Frobenius error sees (bf16 output rounding alone
    # gives about 1.7e-3)
    fro = ((out.float() - ref).norm() / (ref.norm() + 1e-12)).item()
    assert fro <= 4e-3, f"relative Frobenius error {fro}"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 256, 128), (384, 768, 768), (1000, 264, 200),
                                   (4096, 2304, 768), (2048, 50304, 768)])
def test_gemm_layouts(kernel_lib, a_mn, b_mn, m, n, k):
    from neuralfn_b200.ops import _lib
    from neuralfn_b200.ops.gemm import gemm
    if a_mn and m % 8:
        pytest.skip("MN-major A needs M % 8 == 0")
    torch.manual_seed(0)
    dev = "cuda"
    a = torch.randn((k, m) if a_mn else (m, k), device=dev, dtype=torch.bfloat16)
    b = torch.randn((k, n) if b_mn else (n, k), device=dev, dtype=torch.bfloat16)
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    _lib.assert_status_ok("gemm")
    _close(out, _ref(a, b, a_mn, b_mn), k)


def test_gemm_epilogues(kernel_lib):
    from neuralfn_b200.ops import _lib
    from neuralfn_b200.ops.gemm import gemm
    torch.manual_seed(1)
    m, n, k = 512, 768, 256
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16) * 0.1
    bias = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(m, n, device="cuda", dtype=torch.bfloat16)
    base = x.float() @ w.float().t() + bias.float()

    y = gemm(x, w, bias=bias)
    _close(y, base, k)

    pre = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    y = gemm(x, w, bias=bias, act="gelu_tanh", save_pre=pre)
    _close(pre, base, k)
    _close(y, torch.nn.functional.gelu(base, approximate="tanh"), k)

    y = gemm(x, w, bias=bias, act="gelu_erf")
    _close(y, torch.nn.functional.gelu(base), k)

    y = gemm(x, w, bias=bias, resid=res)
    _close(y, base + res.float(), k)

    # dGELU epilogue: (x @ w.T) * gelu'(pre)
    pre_f = pre.float().requires_grad_(True)
    torch.nn.functional.gelu(pre_f, approximate="tanh").sum().backward()
    y = gemm(x, w, act="gelu_tanh", dact_pre=pre)
    _close(y, (x.float() @ w.float().t()) * pre_f.grad, k)

    # fp32 output with accumulation
    acc = torch.ones(m, n, device="cuda", dtype=torch.float32)
    gemm(x, w, out=acc, accum=True, alpha=0.5)
    _close(acc, 0.5 * (x.float() @ w.float().t()) + 1.0, k)

    # logit soft-cap
    y = gemm(x, w, act="tanh_cap", act_param=30.0)
    _close(y, 30.0 * torch.tanh((x.float() @ w.float().t()) / 30.0), k)
    _lib.assert_status_ok("gemm epilogues")


def test_gemm_strided_views(kernel_lib):
    """Operands that are column slices of a wider buffer (leading dim > width)."""
    from neuralfn_b200.ops import _lib
    from neuralfn_b200.ops.gemm import gemm
    torch.manual_seed(2)
    big = torch.randn(256, 3 * 128, device="cuda", dtype=torch.bfloat16)
    x = big[:, 128:256]
    w = torch.randn(64, 128, device="cuda", dtype=torch.bfloat16)
    outbuf = torch.zeros(256, 256, device="cuda", dtype=torch.bfloat16)
    out = outbuf[:, 64:128]
    gemm(x, w, out=out)
    _lib.assert_status_ok("gemm views")
    _close(out, x.float() @ w.float().t(), 128)
    assert outbuf[:, :64].abs().max().item() == 0 and outbuf[:, 128:].abs().max().item() == 0


@pytest.mark.parametrize("m,n,k", [(16384, 768, 768), (16384, 2304, 768), (8192, 3072, 768), (16384, 768, 3072),
                                   (8192 + 128, 2304 + 64, 768 + 32)])
def test_gemm_cta_pair(kernel_lib, m, n, k):
    """CTA-pair (cta_group::2) kernel: plain product and the fused epilogues against fp32."""
    from neuralfn_b200.ops import _lib
    from neuralfn_b200.ops.gemm import gemm
    L = _lib.load()
    torch.manual_seed(3)
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(m, n, device="cuda", dtype=torch.bfloat16)
    base = x.float() @ w.float().t()
    old = L.nfn_gemm_set_pair_mode(1)
    try:
        y = gemm(x, w)
        _lib.assert_status_ok("gemm pair")
        _close(y, base, k)
        pre = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        y = gemm(x, w, bias=bias, act="gelu_tanh", save_pre=pre)
        _lib.assert_status_ok("gemm pair gelu")
        _close(pre, base + bias.float(), k)
        _close(y, torch.nn.functional.gelu(base + bias.float(), approximate="tanh"), k)
        y = gemm(x, w, bias=bias, resid=res)
        _lib.assert_status_ok("gemm pair resid")
        _close(y, base + bias.float() + res.float(), k)
    finally:
        L.nfn_gemm_set_pair_mode(old)


@pytest.mark.parametrize("m", [1, 2, 3, 4])
@pytest.mark.parametrize("n,k", [(4096, 4096), (1000, 1032), (6144, 14336)])
def test_gemv_small_m_with_epilogues(kernel_lib, m, n, k):
    """Products with at most four rows take the weight-streaming GEMV kernel; same epilogue semantics
    as the tensor-core path (checked against fp32 and against the GEMM path itself)."""
    from neuralfn_b200.ops import _lib
    from neuralfn_b200.ops.gemm import gemm
    torch.manual_seed(m * 7 + n)
    a = (torch.randn(m, k, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
    bias = (torch.randn(n, device="cuda") * 0.1).bfloat16()
    resid = torch.randn(m, n, device="cuda").bfloat16()
    ref = a.float() @ w.float().t()
    _close(gemm(a, w), ref, k)
    out = gemm(a, w, bias=bias, act="gelu_tanh", resid=resid)
    full = torch.nn.functional.gelu(ref + bias.float(), approximate="tanh") + resid.float()
    _close(out, full, k)
    acc = resid.clone()
    gemm(a, w, out=acc, accum=True, alpha=0.5)
    _close(acc, resid.float() + 0.5 * ref, k)
    capped = gemm(a, w, act="tanh_cap", act_param=2.0)
    _close(capped, 2.0 * torch.tanh(ref / 2.0), k)
    # the tensor-core path gives the same numbers
    L = _lib.load()
    old = L.nfn_gemm_set_gemv_mode(0)
    try:
        tc = gemm(a, w, bias=bias, act="gelu_tanh", resid=resid)
    finally:
        L.nfn_gemm_set_gemv_mode(old)
    torch.testing.assert_close(out.float(), tc.float(), atol=3e-2, rtol=3e-2)
    _lib.assert_status_ok("gemv")


@pytest.mark.parametrize("m,n,k", [(16384, 768, 2304), (16384, 3072, 768), (8192 + 128, 768 + 64, 3072 + 32), (1024, 256, 256)])
def test_gemm_cta_pair_mn_major_b(kernel_lib, m, n, k):
    """CTA-pair kernel with an MN-major B operand (input gradients dY W): plain product and the
    dGELU epilogue against fp32; the one-CTA kernel must agree to rounding."""
    from neuralfn_b200.ops import _lib
    from neuralfn_b200.ops.gemm import gemm
    L = _lib.load()
    torch.manual_seed(5)
    dy = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(k, n, device="cuda", dtype=torch.bfloat16) * 0.05      # [K, N]: N contiguous
    pre = torch.randn(m, n, device="cuda", dtype=torch.bfloat16)
    base = dy.float() @ w.float()
    t = pre.float().requires_grad_(True)
    torch.nn.functional.gelu(t, approximate="tanh").sum().backward()
    old = L.nfn_gemm_set_pair_mode(1)
    try:
        y = gemm(dy, w, b_mn=True)
        _lib.assert_status_ok("gemm pair b_mn")
        _close(y, base, k)
        yg = gemm(dy, w, b_mn=True, act="gelu_tanh", dact_pre=pre)
        _lib.assert_status_ok("gemm pair b_mn dgelu")
        _close(yg, base * t.grad, k)
        L.nfn_gemm_set_pair_mode(0)
        y1 = gemm(dy, w, b_mn=True)
        assert (y.float() - y1.float()).abs().max().item() <= 0.02 * base.abs().max().item()
    finally:
        L.nfn_gemm_set_pair_mode(old)


@pytest.mark.parametrize("m", [3, 8, 17, 32, 33, 64])
@pytest.mark.parametrize("n,k", [(6656, 1024), (2304, 6656), (1000, 1056)])
def test_skinny_products_take_the_weight_streaming_mma_kernel(kernel_lib, m, n, k):
    """3 - 64 rows over a large K-major weight matrix: mma.sync with permuted-k fragments, in-CTA split-K, fused epilogue.
    Checked against fp32 and against the tcgen05 split-K path it replaces."""
    from neuralfn_b200.ops import _lib
    from neuralfn_b200.ops.gemm import gemm
    torch.manual_seed(m * 13 + n)
    a = (torch.randn(m, k, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
    bias = (torch.randn(n, device="cuda") * 0.1).bfloat16()
    resid = torch.randn(m, n, device="cuda").bfloat16()
    ws = torch.empty(32 * 1024 * 1024, device="cuda", dtype=torch.float32)
    L = _lib.load()
    forced = L.nfn_gemm_skinny_set_impl(2)                         # every eligible row count (the default stops at 16 rows)
    before = _lib.launch_count()
    ref = a.float() @ w.float().t()
    y = gemm(a, w, workspace=ws)
    assert _lib.launch_count() - before == 1                       # one launch: no separate split-K reduction
    _close(y, ref, k)
    out = gemm(a, w, bias=bias, act="silu", resid=resid, workspace=ws)
    _close(out, torch.nn.functional.silu(ref + bias.float()) + resid.float(), k)
    acc = resid.clone()
    gemm(a, w, out=acc, accum=True, alpha=0.5, workspace=ws)
    _close(acc, resid.float() + 0.5 * ref, k)
    # strided views: rows of a wider buffer in, columns of a wider buffer out
    wide_in = torch.zeros(m, k + 64, device="cuda", dtype=torch.bfloat16)
    wide_in[:, :k] = a
    wide_out = torch.zeros(m, n + 128, device="cuda", dtype=torch.bfloat16)
    gemm(wide_in[:, :k], w, out=wide_out[:, 64:64 + n], workspace=ws)
    _close(wide_out[:, 64:64 + n], ref, k)
    assert float(wide_out[:, :64].abs().max()) == 0.0 and float(wide_out[:, 64 + n:].abs().max()) == 0.0
    L.nfn_gemm_skinny_set_impl(0)
    try:
        tc = gemm(a, w, bias=bias, act="silu", resid=resid, workspace=ws)
    finally:
        L.nfn_gemm_skinny_set_impl(forced)
    torch.testing.assert_close(out.float(), tc.float(), atol=4e-2, rtol=4e-2)
    _lib.assert_status_ok("skinny gemm")


@pytest.mark.parametrize("m,mode", [(17, 3), (24, 3), (32, 3), (5, 3), (16, 3)])
@pytest.mark.parametrize("n,k", [(6656, 1024), (2304, 6656), (1000, 1056), (12288, 6656), (520, 4096)])
def test_skinny_products_with_resident_token_fragments(kernel_lib, m, mode, n, k):
    """The opt-in form for up to 32 rows: token fragments held in registers, K split over a thread-block cluster whose CTAs
    add their strips over distributed shared memory. One launch, the same bits on every call, fp32 and tcgen05 agreement."""
    from neuralfn_b200.ops import _lib
    from neuralfn_b200.ops.gemm import gemm
    torch.manual_seed(m * 7 + n)
    a = (torch.randn(m, k, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
    bias = (torch.randn(n, device="cuda") * 0.1).bfloat16()
    resid = torch.randn(m, n, device="cuda").bfloat16()
    ws = torch.empty(32 * 1024 * 1024, device="cuda", dtype=torch.float32)
    L = _lib.load()
    old = L.nfn_gemm_skinny_set_impl(mode)
    try:
        ref = a.float() @ w.float().t()
        before = _lib.launch_count()
        y = gemm(a, w, workspace=ws)
        assert _lib.launch_count() - before == 1
        _close(y, ref, k)
        assert torch.equal(y, gemm(a, w, workspace=ws))
        out = gemm(a, w, bias=bias, act="gelu_tanh", resid=resid, workspace=ws)
        _close(out, torch.nn.functional.gelu(ref + bias.float(), approximate="tanh") + resid.float(), k)
        acc = resid.clone()
        gemm(a, w, out=acc, accum=True, alpha=0.5, workspace=ws)
        _close(acc, resid.float() + 0.5 * ref, k)
        wide_in = torch.zeros(m, k + 64, device="cuda", dtype=torch.bfloat16)
        wide_in[:, :k] = a
        wide_out = torch.zeros(m, n + 128, device="cuda", dtype=torch.bfloat16)
        gemm(wide_in[:, :k], w, out=wide_out[:, 64:64 + n], workspace=ws)
        _close(wide_out[:, 64:64 + n], ref, k)
        assert float(wide_out[:, :64].abs().max()) == 0.0 and float(wide_out[:, 64 + n:].abs().max()) == 0.0
        L.nfn_gemm_skinny_set_impl(0)
        tc = gemm(a, w, bias=bias, act="gelu_tanh", resid=resid, workspace=ws)
    finally:
        L.nfn_gemm_skinny_set_impl(old)
    torch.testing.assert_close(out.float(), tc.float(), atol=4e-2, rtol=4e-2)
    _lib.assert_status_ok("resident skinny gemm")


@pytest.mark.parametrize("m,n,dtype", [(256, 512, torch.bfloat16), (2048, 1024, torch.bfloat16), (192, 200, torch.float32)])
def test_grouped_contraction_gives_every_experts_weight_gradient(kernel_lib, m, n, dtype):
    """out[g] = a[rows of g]^T b[rows of g] for all groups in one launch: segments padded to 128 rows with zero rows in a, an empty
    group, accumulation on top of an existing gradient."""
    from neuralfn_b200.ops import _lib
    from neuralfn_b200.ops.gemm import gemm_grouped_k
    torch.manual_seed(m + n)
    counts = [300, 0, 128, 77, 1, 513]
    offs = [0]
    for c in counts:
        offs.append(offs[-1] + (c + 127) // 128 * 128)
    rows = offs[-1] + 256                                             # rows past the last group are never read
    a = torch.zeros(rows, m, device="cuda", dtype=torch.bfloat16)
    b = (torch.randn(rows, n, device="cuda") * 0.3).bfloat16()        # padding rows of b are finite, not zero
    for g, c in enumerate(counts):
        a[offs[g]:offs[g] + c] = (torch.randn(c, m, device="cuda") * 0.3).bfloat16()
    a[offs[-1]:] = float("nan")                                       # must not be touched
    group_rows = torch.tensor(offs, device="cuda", dtype=torch.int32)
    out = torch.full((len(counts), m, n), 7.0, device="cuda", dtype=dtype)
    before = _lib.launch_count()
    gemm_grouped_k(a, b, group_rows, out)
    assert _lib.launch_count() - before == 1
    ref = torch.stack([a[offs[g]:offs[g] + c].float().t() @ b[offs[g]:offs[g] + c].float() for g, c in enumerate(counts)])
    assert float(out[1].abs().max()) == 0.0
    tol = 2e-2 * float(ref.abs().max()) + 1e-3
    assert float((out.float() - ref).abs().max()) < tol
    keep = out.clone()
    gemm_grouped_k(a, b, group_rows, out, alpha=0.5, accum=True)
    assert float((out.float() - (keep.float() + 0.5 * ref)).abs().max()) < 2 * tol
    # column views of a wider buffer (the gate / up halves of the hidden gradient)
    wide = torch.zeros(rows, 2 * n, device="cuda", dtype=torch.bfloat16)
    wide[:, n:] = b
    out2 = torch.empty_like(keep)
    gemm_grouped_k(a, wide[:, n:], group_rows, out2)
    assert torch.equal(out2, keep)
    _lib.assert_status_ok("grouped contraction")
