"""Inference-side kernels against fp32 PyTorch / numpy references."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _rope_ref(x, cos, sin, sign):
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat((x1 * cos - sign * x2 * sin, x2 * cos + sign * x1 * sin), dim=-1)


@pytest.mark.parametrize("hd,convention", [(64, "legacy"), (128, "hf")])
def test_rope_inplace_forward_and_inverse(hd, convention):
    from neuralfn_b200.ops import infer
    torch.manual_seed(0)
    B, T, Hq, Hkv = 2, 37, 4, 2
    qkv = torch.randn(B * T, (Hq + 2 * Hkv) * hd, device=_dev()).bfloat16()
    orig = qkv.clone()
    cos, sin = infer.rope_tables(64, hd, 10000.0, device=_dev())
    infer.rope_inplace(qkv, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=hd, cos=cos, sin=sin, convention=convention, q_scale=0.5)
    sign = 1.0 if convention == "hf" else -1.0
    x = orig.float().view(B, T, Hq + 2 * Hkv, hd)
    c, s = cos[:T, None, :], sin[:T, None, :]
    ref = x.clone()
    ref[:, :, :Hq + Hkv] = _rope_ref(x[:, :, :Hq + Hkv], c, s, sign)
    ref[:, :, :Hq] *= 0.5
    torch.testing.assert_close(qkv.float().view(B, T, -1, hd), ref, atol=2e-2, rtol=2e-2)
    assert torch.equal(qkv.view(B, T, -1, hd)[:, :, Hq + Hkv:], orig.view(B, T, -1, hd)[:, :, Hq + Hkv:])  # v untouched
    infer.rope_inplace(qkv, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=hd, cos=cos, sin=sin, convention=convention,
                       q_scale=2.0, backward=True)
    torch.testing.assert_close(qkv.float(), orig.float(), atol=3e-2, rtol=3e-2)


def test_qk_norm_rope_fused_matches_composition():
    from neuralfn_b200.ops import infer
    torch.manual_seed(1)
    T, Hq, Hkv, hd = 19, 4, 1, 128
    qkv = torch.randn(T, (Hq + 2 * Hkv) * hd, device=_dev()).bfloat16()
    qw = (1 + 0.1 * torch.randn(hd, device=_dev())).bfloat16()
    kw = (1 + 0.1 * torch.randn(hd, device=_dev())).bfloat16()
    pos = torch.randint(0, 500, (T,), device=_dev(), dtype=torch.int32)
    cos, sin = infer.rope_tables(512, hd, 500000.0, device=_dev())
    x = qkv.float().view(T, -1, hd)
    got = qkv.clone()
    rstd = torch.empty(T * (Hq + Hkv), device=_dev())
    infer.qk_norm_rope_forward(got, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=hd, cos=cos, sin=sin, convention="hf",
                               q_weight=qw, k_weight=kw, positions=pos, eps=1e-6, q_scale=hd ** -0.5, rstd=rstd)
    r = torch.rsqrt(x[:, :Hq + Hkv].pow(2).mean(-1, keepdim=True) + 1e-6)
    w = torch.cat([qw.float().expand(Hq, hd), kw.float().expand(Hkv, hd)])[None]
    ref = _rope_ref(x[:, :Hq + Hkv] * r * w, cos[pos.long()][:, None], sin[pos.long()][:, None], 1.0)
    ref[:, :Hq] *= hd ** -0.5
    torch.testing.assert_close(got.float().view(T, -1, hd)[:, :Hq + Hkv], ref, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(rstd.view(T, -1), r.squeeze(-1), atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_argmax_rows_ties_and_offsets(dtype):
    from neuralfn_b200.ops import infer
    torch.manual_seed(2)
    logits = torch.randn(32, 50304, device=_dev()).to(dtype)
    logits[3, 100] = logits[3, 40000] = 50.0  # tie -> lowest index
    logits[5, 7] = float("nan")
    idx, val = infer.argmax_rows(logits, index_offset=1000, return_values=True)
    ref = torch.where(torch.isnan(logits), torch.full_like(logits, -1e30), logits).float().argmax(-1)
    ref[3] = 100
    assert torch.equal(idx.long() - 1000, ref)
    assert float(val[3]) == 50.0
    one = infer.argmax_rows(logits[:1, :1000].contiguous())
    assert int(one[0]) == int(logits[0, :1000].float().argmax())


def test_sampling_truncation_and_distribution():
    from neuralfn_b200.ops import infer
    torch.manual_seed(3)
    V, rows = 1000, 2048
    base = torch.randn(V, device=_dev()) * 2.0
    logits = base.expand(rows, V).contiguous()
    # greedy
    assert torch.equal(infer.sample_rows(logits, temperature=0.0).long(), base.argmax().expand(rows))
    # top-k: only the k best may appear, frequencies follow the renormalised softmax
    k = 5
    top = base.topk(k)
    got = infer.sample_rows(logits, temperature=1.0, top_k=k, seed=11)
    assert set(got.tolist()) <= set(top.indices.tolist())
    p = torch.softmax(top.values, 0)
    freq = torch.stack([(got == i).float().mean() for i in top.indices])
    assert float((freq - p).abs().max()) < 0.05
    # top-p: the smallest prefix of the sorted distribution reaching p
    rounded = base.bfloat16().float()
    probs = torch.softmax(rounded / 0.8, 0)
    srt = probs.sort(descending=True)
    n_keep = int((srt.values.cumsum(0) < 0.6).sum()) + 1
    got = infer.sample_rows(rounded.expand(rows, V).contiguous(), temperature=0.8, top_p=0.6, seed=5)
    # everything tied with the last kept value (and the next distinct value, for a
    # cumulative sum that lands on the boundary) may appear
    floor = srt.values[min(n_keep, V - 1)]
    allowed = set(torch.nonzero(probs >= floor).flatten().tolist())
    assert set(got.tolist()) <= allowed and len(set(got.tolist())) >= max(1, n_keep - 1)
    # different offsets give different draws, same offset repeats
    a = infer.sample_rows(logits, temperature=1.0, seed=1, offset=0)
    b = infer.sample_rows(logits, temperature=1.0, seed=1, offset=0)
    c = infer.sample_rows(logits, temperature=1.0, seed=1, offset=1)
    assert torch.equal(a, b) and not torch.equal(a, c)
    # untruncated sampling: chi-square-ish check on the 10 most likely tokens
    full = infer.sample_rows(logits, temperature=1.0, seed=99, return_logprob=True)
    pf = torch.softmax(base, 0)
    for i in pf.topk(10).indices.tolist():
        assert abs(float((full[0] == i).float().mean()) - float(pf[i])) < 0.03
    lp_ref = torch.log_softmax(base, 0)[full[0].long()]
    torch.testing.assert_close(full[1], lp_ref, atol=2e-3, rtol=2e-3)


def _decode_ref(q, kc, vc, lengths, cap, scale):
    B, Hq, hd = q.shape
    Hkv = kc.shape[1]
    out = torch.zeros(B, Hq, hd, device=q.device)
    for b in range(B):
        n = min(int(lengths[b]), cap)
        for h in range(Hq):
            kv = h // (Hq // Hkv)
            s = (kc[b, kv, :n].float() @ q[b, h]) * scale
            out[b, h] = torch.softmax(s, 0) @ vc[b, kv, :n].float()
    return out


@pytest.fixture(params=["mma", "simt"])
def decode_impl(request):
    from neuralfn_b200.ops import infer
    old = infer.decode_attention_set_impl(request.param)
    yield request.param
    infer.decode_attention_set_impl(old)


@pytest.mark.parametrize("hd,Hq,Hkv,cap,ring", [(128, 4, 1, 700, False), (64, 6, 2, 128, True), (128, 8, 8, 300, False), (128, 24, 2, 513, False),
                                                (64, 16, 1, 200, True)])
def test_decode_attention_append_and_attend(hd, Hq, Hkv, cap, ring, decode_impl):
    from neuralfn_b200.ops import infer
    torch.manual_seed(4)
    B = 5
    dev = _dev()
    if ring:
        lengths = torch.tensor([1, 90, 128, 129, 700], dtype=torch.int32, device=dev)
    else:
        lengths = torch.tensor([1, 2, 257, cap, 100], dtype=torch.int32, device=dev)
    kc = torch.randn(B, Hkv, cap, hd, device=dev).bfloat16()
    vc = torch.randn(B, Hkv, cap, hd, device=dev).bfloat16()
    qkv = torch.randn(B, (Hq + 2 * Hkv) * hd, device=dev).bfloat16()
    qw = (1 + 0.1 * torch.randn(hd, device=dev)).bfloat16()
    kw = (1 + 0.1 * torch.randn(hd, device=dev)).bfloat16()
    cos, sin = infer.rope_tables(1024, hd, 10000.0, device=dev)
    ws = infer.DecodeAttentionWorkspace(B, Hq, Hkv, hd, dev)
    # reference: normalise + rotate the new q/k, write k/v into the slot, full softmax
    x = qkv.float().view(B, Hq + 2 * Hkv, hd)
    pos = (lengths - 1).long()
    r = torch.rsqrt(x[:, :Hq + Hkv].pow(2).mean(-1, keepdim=True) + 1e-6)
    w = torch.cat([qw.float().expand(Hq, hd), kw.float().expand(Hkv, hd)])[None]
    qk = _rope_ref(x[:, :Hq + Hkv] * r * w, cos[pos][:, None], sin[pos][:, None], 1.0)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    for b in range(B):
        slot = int(pos[b]) % cap
        kc_ref[b, :, slot] = qk[b, Hq:].bfloat16()
        vc_ref[b, :, slot] = x[b, Hq + Hkv:].bfloat16()
    ref = _decode_ref(qk[:, :Hq], kc_ref, vc_ref, lengths, cap, hd ** -0.5)
    for splits in (0, 3):
        k2, v2 = kc.clone(), vc.clone()
        out = infer.decode_attention(qkv, k2, v2, lengths, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=hd, workspace=ws, cos=cos, sin=sin,
                                     convention="hf", qk_norm=True, q_norm_weight=qw, k_norm_weight=kw, splits=splits)
        torch.testing.assert_close(out.float().view(B, Hq, hd), ref, atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(k2.float(), kc_ref.float(), atol=2e-2, rtol=2e-2)
        assert torch.equal(v2, vc_ref)
    assert int(ws.buf[:256].sum()) == 0  # tickets are back to zero


@pytest.mark.parametrize("name", ["Q4_K", "Q5_K", "Q6_K"])
def test_kquant_dequant_matches_numpy_oracle(name):
    from neuralfn_b200.ops import infer
    from neuralfn_b200.quant import kquant
    t = kquant.GGML_TYPE[name]
    raw = kquant.random_blocks(t, 300, seed=7)
    ref = torch.from_numpy(kquant.dequantize(t, raw.tobytes()))
    got = infer.dequant_kquant(t, torch.from_numpy(raw).to(_dev()).reshape(-1))
    torch.testing.assert_close(got.float().cpu(), ref, atol=2e-2, rtol=1e-2)


def test_nf4_dequant():
    from neuralfn_b200.ops import infer
    from neuralfn_b200.quant import kquant
    w = np.random.default_rng(0).normal(size=64 * 50).astype(np.float32)
    codes, absmax = kquant.nf4_encode(w)
    got = infer.dequant_nf4(torch.from_numpy(codes).to(_dev()), torch.from_numpy(absmax).to(_dev()))
    torch.testing.assert_close(got.float().cpu(), torch.from_numpy(kquant.nf4_decode(codes, absmax)), atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("name,B,N,K,gated", [("Q4_K", 1, 96, 512, False), ("Q4_K", 8, 70, 4096 + 256, True),
                                                ("Q6_K", 3, 33, 768, False), ("Q5_K", 2, 64, 256, True)])
def test_kquant_gemv(name, B, N, K, gated):
    from neuralfn_b200.ops import infer
    from neuralfn_b200.quant import kquant
    t = kquant.GGML_TYPE[name]
    dev = _dev()
    nb = N * K // 256
    raw1, raw2 = kquant.random_blocks(t, nb, seed=1), kquant.random_blocks(t, nb, seed=2)
    w1 = torch.from_numpy(kquant.dequantize(t, raw1.tobytes())).view(N, K).to(dev)
    w2 = torch.from_numpy(kquant.dequantize(t, raw2.tobytes())).view(N, K).to(dev)
    x = (torch.randn(B, K, device=dev) * 0.5).bfloat16()
    bias = torch.randn(N, device=dev).bfloat16()
    resid = torch.randn(B, N, device=dev).bfloat16()
    a = x.float() @ w1.T
    ref = (torch.nn.functional.silu(a) * (x.float() @ w2.T) if gated else a) + bias.float() + resid.float()
    got = infer.kquant_gemv(t, torch.from_numpy(raw1).to(dev).reshape(-1), x, N,
                            w_gate_pair=torch.from_numpy(raw2).to(dev).reshape(-1) if gated else None, bias=bias, resid=resid)
    torch.testing.assert_close(got.float(), ref, atol=0.05 * float(ref.abs().max()), rtol=2e-2)


def _block_attention_ref(qkv, kc, vc, lengths, rows, Hq, Hkv, D, window, causal, n_rows):
    """fp32 oracle: logical key list per sequence = cached positions still in the cache + block rows."""
    B, _, cap, _ = kc.shape
    G = Hq // Hkv
    out = torch.zeros(B * rows, Hq * D, dtype=torch.float32, device=qkv.device)
    q = qkv[:, :Hq * D].float().view(B, rows, Hq, D)
    kb = qkv[:, Hq * D:(Hq + Hkv) * D].float().view(B, rows, Hkv, D)
    vb = qkv[:, (Hq + Hkv) * D:(Hq + 2 * Hkv) * D].float().view(B, rows, Hkv, D)
    for b in range(B):
        pos0, nr = int(lengths[b]), rows if n_rows is None else int(n_rows[b])
        if nr <= 0:
            continue
        first = max(0, pos0 - cap)
        pos = torch.arange(first, pos0, device=qkv.device)
        kk = torch.cat([kc[b, :, pos % cap].float(), kb[b, :nr].transpose(0, 1)], dim=1)  # [Hkv, n, D]
        vv = torch.cat([vc[b, :, pos % cap].float(), vb[b, :nr].transpose(0, 1)], dim=1)
        kpos = torch.cat([pos, pos0 + torch.arange(nr, device=qkv.device)])
        for r in range(nr):
            qp = pos0 + r
            vis = torch.ones_like(kpos, dtype=torch.bool)
            if causal:
                vis &= kpos <= qp
            if window > 0:
                vis &= (kpos > qp - window) | (kpos >= pos0)
            for h in range(Hq):
                s = (kk[h // G] @ q[b, r, h]) * D ** -0.5
                s = s.masked_fill(~vis, float("-inf"))
                out[b * rows + r, h * D:(h + 1) * D] = torch.softmax(s, 0) @ vv[h // G]
    return out


@pytest.mark.parametrize("D,Hq,Hkv,rows,cap,window,causal,splits", [
    (64, 8, 2, 16, 300, 0, True, 1), (64, 8, 2, 16, 300, 0, True, 3), (128, 8, 1, 16, 700, 0, True, 0),
    (128, 4, 2, 5, 256, 256, True, 0), (64, 4, 4, 17, 200, 200, True, 2), (128, 16, 2, 16, 520, 0, False, 0),
    (64, 2, 2, 100, 384, 0, True, 0), (128, 32, 4, 1, 640, 0, True, 0)])
def test_block_attention_matches_fp32(kernel_lib, D, Hq, Hkv, rows, cap, window, causal, splits):
    from neuralfn_b200.ops import _lib
    from neuralfn_b200.ops.infer import BlockAttentionWorkspace, block_attention, kv_commit_layers
    torch.manual_seed(11)
    dev, B = "cuda", 3
    ld = (Hq + 2 * Hkv) * D + 64
    qkv = torch.randn(B * rows, ld, device=dev, dtype=torch.bfloat16)
    kc = torch.randn(B, Hkv, cap, D, device=dev, dtype=torch.bfloat16)
    vc = torch.randn(B, Hkv, cap, D, device=dev, dtype=torch.bfloat16)
    # sequence 0: short (ring not wrapped), 1: wrapped ring / long, 2: empty cache
    lengths = torch.tensor([min(cap, 131), (cap * 2 + 37) if window else cap - rows, 0], dtype=torch.int32, device=dev)
    n_rows = torch.tensor([rows, max(1, rows - 2), rows], dtype=torch.int32, device=dev)
    ws = BlockAttentionWorkspace(B, rows, Hq, Hkv, D, dev)
    sk = torch.zeros(B * rows, Hkv * D, device=dev, dtype=torch.bfloat16)
    sv = torch.zeros_like(sk)
    for _ in range(2):  # second call exercises the self-resetting tickets
        out = block_attention(qkv, kc, vc, lengths, rows=rows, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D, workspace=ws, window=window,
                              causal=causal, n_rows=n_rows, stage_k=sk, stage_v=sv, splits=splits)
    _lib.assert_status_ok("block_attention")
    ref = _block_attention_ref(qkv, kc, vc, lengths.cpu(), rows, Hq, Hkv, D, window, causal, n_rows.cpu())
    for b in range(B):
        nr = int(n_rows[b])
        got = out[b * rows:b * rows + nr].float()
        assert (got - ref[b * rows:b * rows + nr]).abs().max().item() < 3e-2
        assert torch.equal(sk[b * rows:b * rows + nr].view(nr, Hkv, D), qkv[b * rows:b * rows + nr, Hq * D:(Hq + Hkv) * D].view(nr, Hkv, D))
    # commit a prefix and check the ring rows
    accepted = torch.tensor([min(3, rows), 1, min(2, rows)], dtype=torch.int32, device=dev)
    k2, v2 = kc.clone(), vc.clone()
    kv_commit_layers([sk], [sv], [k2], [v2], lengths, accepted, rows=rows)
    for b in range(B):
        for i in range(int(accepted[b])):
            slot = (int(lengths[b]) + i) % cap
            assert torch.equal(k2[b, :, slot], sk[b * rows + i].view(Hkv, D))
            assert torch.equal(v2[b, :, slot], sv[b * rows + i].view(Hkv, D))
    untouched = torch.ones(B, cap, dtype=torch.bool, device=dev)
    for b in range(B):
        for i in range(int(accepted[b])):
            untouched[b, (int(lengths[b]) + i) % cap] = False
    assert torch.equal(k2.transpose(1, 2)[untouched], kc.transpose(1, 2)[untouched])


@pytest.mark.parametrize("name,M,N,K", [("Q4_K", 256, 128, 512), ("Q4_K", 1000, 264, 2048), ("Q5_K", 384, 256, 768), ("Q6_K", 300, 136, 1024),
                                         ("Q6_K", 2048, 512, 6656)])
def test_gemm_with_fused_kquant_dequant(kernel_lib, name, M, N, K):
    from neuralfn_b200.ops import _lib, infer
    from neuralfn_b200.quant import kquant
    t = kquant.GGML_TYPE[name]
    dev = _dev()
    raw = kquant.random_blocks(t, N * K // 256, seed=3)
    w = torch.from_numpy(kquant.dequantize(t, raw.tobytes())).view(N, K).to(dev)
    x = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
    bias = torch.randn(N, device=dev).bfloat16()
    resid = torch.randn(M, N, device=dev).bfloat16()
    wq = torch.from_numpy(raw).to(dev).reshape(-1)
    got = infer.gemm_kquant(t, x, wq, N)
    _lib.assert_status_ok("gemm_kquant")
    ref = x.float() @ w.bfloat16().float().T  # the kernel rounds the decoded weights to bf16, like the two-step path
    torch.testing.assert_close(got.float(), ref, atol=0.02 * float(ref.abs().max()), rtol=2e-2)
    got = infer.gemm_kquant(t, x, wq, N, bias=bias, act="silu", resid=resid)
    _lib.assert_status_ok("gemm_kquant epilogue")
    ref2 = torch.nn.functional.silu(ref + bias.float()) + resid.float()
    torch.testing.assert_close(got.float(), ref2, atol=0.02 * float(ref2.abs().max()), rtol=2e-2)


@pytest.mark.parametrize("M,N,K,r", [(256, 128, 512, 8), (1000, 264, 1024, 16)])
def test_nf4_lora_linear_fused_forward_and_backward(kernel_lib, M, N, K, r):
    from neuralfn_b200.ops import _lib, infer
    from neuralfn_b200.quant import kquant
    dev = _dev()
    rng = np.random.default_rng(4)
    w0 = (rng.normal(size=N * K) * 0.05).astype(np.float32)
    codes, absmax = kquant.nf4_encode(w0)
    w = torch.from_numpy(kquant.nf4_decode(codes, absmax)).view(N, K).to(dev)
    A = (torch.randn(r, K, device=dev) * 0.05).bfloat16()
    B = (torch.randn(N, r, device=dev) * 0.05).bfloat16()
    x = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
    dy = (torch.randn(M, N, device=dev) * 0.1).bfloat16()
    lin = infer.NF4LoRALinear(torch.from_numpy(codes).to(dev), torch.from_numpy(absmax).to(dev), N, K, A, B, alpha=16.0)
    y = lin.forward(x)
    _lib.assert_status_ok("nf4 lora forward")
    s = 16.0 / r
    xf, Af, Bf, wf = x.float(), A.float(), B.float(), w.bfloat16().float()
    ref = xf @ wf.T + s * (xf @ Af.T) @ Bf.T
    torch.testing.assert_close(y.float(), ref, atol=0.02 * float(ref.abs().max()), rtol=2e-2)
    base_only = infer.NF4LoRALinear(lin.codes, lin.absmax, N, K, torch.zeros_like(A), B).forward(x)
    torch.testing.assert_close(base_only.float(), xf @ wf.T, atol=0.02 * float(ref.abs().max()), rtol=2e-2)
    dx, da, db = lin.backward(x, dy)
    _lib.assert_status_ok("nf4 lora backward")
    dyf = dy.float()
    dx_ref = dyf @ wf + s * (dyf @ Bf) @ Af
    da_ref = s * (dyf @ Bf).T @ xf
    db_ref = s * dyf.T @ (xf @ Af.T)
    for got, want in ((dx.float(), dx_ref), (da, da_ref), (db, db_ref)):
        torch.testing.assert_close(got, want, atol=0.03 * float(want.abs().max()), rtol=3e-2)
