"""Non-GEMM sm_100a kernels vs. plain PyTorch fp32 references."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("C", [768, 2048, 4096, 6656])
@pytest.mark.parametrize("mode", ["layer", "rms", "rms_centered"])
def test_norm_fwd_bwd(kernel_lib, C, mode):
    from neuralfn_b200.ops import kernels as K, _lib
    torch.manual_seed(0)
    rows = 300
    x = torch.randn(rows, C, device="cuda", dtype=BF)
    w = (torch.randn(C, device="cuda") * 0.2 + (0.0 if mode == "rms_centered" else 1.0)).to(BF)
    b = (torch.randn(C, device="cuda") * 0.1).to(BF) if mode == "layer" else None
    dy = torch.randn(rows, C, device="cuda", dtype=BF)
    dres = torch.randn(rows, C, device="cuda", dtype=BF)
    eps = 1e-5
    kmode = K.NORM_LAYER if mode == "layer" else K.NORM_RMS
    centered = mode == "rms_centered"
    y, mean, rstd = K.norm_forward(x, w, b, eps=eps, mode=kmode, centered=centered)
    xf = x.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    bf = b.float().requires_grad_(True) if b is not None else None
    if mode == "layer":
        ref = F.layer_norm(xf, (C,), wf, bf, eps)
    else:
        n = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        ref = n * ((1 + wf) if centered else wf)
    assert _rel(y, ref) < 1e-2
    ref.backward(dy.float())
    dx = K.norm_backward_dx(dy, x, w, mean, rstd, mode=kmode, centered=centered, dresid=dres)
    assert _rel(dx, xf.grad + dres.float()) < 1e-2
    scratch = torch.empty(64 * 2 * C, device="cuda", dtype=torch.float32)
    dw = torch.empty(C, device="cuda", dtype=BF)
    db = torch.empty(C, device="cuda", dtype=BF) if b is not None else None
    K.norm_backward_wb(dy, x, mean, rstd, dw, db, scratch, mode=kmode)
    assert _rel(dw, wf.grad) < 1e-2
    if db is not None:
        assert _rel(db, bf.grad) < 1e-2
    # the fused single-pass variant gives the same three results
    scratch2 = torch.empty(K.norm_fused_rows() * 3 * C, device="cuda", dtype=torch.float32)
    dw2 = torch.empty(C, device="cuda", dtype=BF)
    db2 = torch.empty(C, device="cuda", dtype=BF) if b is not None else None
    dcol = torch.empty(C, device="cuda", dtype=BF)
    dx2 = K.norm_backward(dy, x, w, mean, rstd, dw2, db2, scratch2, mode=kmode, centered=centered, dresid=dres, dx_colsum=dcol)
    assert _rel(dcol, dx2.float().sum(0)) < 1e-2
    assert _rel(dx2, xf.grad + dres.float()) < 1e-2 and _rel(dw2, wf.grad) < 1e-2
    if db2 is not None:
        assert _rel(db2, bf.grad) < 1e-2
    _lib.assert_status_ok()


def test_colsum(kernel_lib):
    from neuralfn_b200.ops import kernels as K
    torch.manual_seed(0)
    big = torch.randn(1000, 3 * 768, device="cuda", dtype=BF)
    dy = big[:, 768:1536]
    out = torch.empty(768, device="cuda", dtype=BF)
    scratch = torch.empty(64 * 768, device="cuda", dtype=torch.float32)
    K.colsum(dy, out, scratch)
    assert _rel(out, dy.float().sum(0)) < 1e-2
    K.colsum(dy, out, scratch, accumulate=True)
    assert _rel(out, 2 * dy.float().sum(0)) < 2e-2


@pytest.mark.parametrize("D", [64, 128])
def test_qk_norm(kernel_lib, D):
    from neuralfn_b200.ops import kernels as K
    torch.manual_seed(0)
    tokens, Hq, Hkv = 200, 6, 2
    width = (Hq + 2 * Hkv) * D
    qkv = torch.randn(tokens, width, device="cuda", dtype=BF)
    orig = qkv.clone()
    q_scale = 1.7
    rstd = K.qk_norm_forward(qkv, Hq, Hkv, D, eps=1e-6, q_scale=q_scale)
    xf = orig.float().requires_grad_(True)
    heads = xf[:, : (Hq + Hkv) * D].view(tokens, Hq + Hkv, D)
    normed = heads * torch.rsqrt(heads.pow(2).mean(-1, keepdim=True) + 1e-6)
    scale = torch.cat([torch.full((Hq,), q_scale), torch.ones(Hkv)]).cuda().view(1, -1, 1)
    ref = torch.cat([(normed * scale).reshape(tokens, -1), xf[:, (Hq + Hkv) * D:]], dim=1)
    assert _rel(qkv, ref) < 1e-2
    assert (qkv[:, (Hq + Hkv) * D:] == orig[:, (Hq + Hkv) * D:]).all()
    dy = torch.randn(tokens, width, device="cuda", dtype=BF)
    ref.backward(dy.float())
    dqkv = dy.clone()
    K.qk_norm_backward(dqkv, qkv, rstd, Hq, Hkv, D, q_scale=q_scale)
    assert _rel(dqkv, xf.grad) < 2e-2


def _attn_ref(q, k, v, B, T, Hq, Hkv, D, causal, window, scale):
    qf = q.float().view(B, T, Hq, D).transpose(1, 2)
    kf = k.float().view(B, T, Hkv, D).transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    vf = v.float().view(B, T, Hkv, D).transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    s = (qf @ kf.transpose(-1, -2)) * scale
    qi = torch.arange(T, device=q.device)[:, None]
    ki = torch.arange(T, device=q.device)[None, :]
    mask = torch.ones(T, T, dtype=torch.bool, device=q.device)
    if causal:
        mask &= ki <= qi
        if window > 0:
            mask &= ki > qi - window
    elif window > 0:
        mask &= (ki > qi - window) & (ki < qi + window)
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = (p @ vf).transpose(1, 2).reshape(B * T, Hq * D)
    lse = torch.logsumexp(s, dim=-1)
    return o, lse


@pytest.mark.parametrize("B,T,Hq,Hkv,D,causal,window", [
    (2, 256, 4, 4, 64, True, 0),
    (1, 1024, 3, 3, 64, True, 0),
    (2, 512, 8, 2, 128, True, 0),
    (1, 640, 4, 1, 128, True, 200),
    (1, 384, 2, 2, 64, False, 0),
    (1, 512, 2, 2, 64, False, 100),
    (2, 200, 2, 2, 64, True, 0),
])
def test_attention_fwd_bwd(kernel_lib, B, T, Hq, Hkv, D, causal, window):
    from neuralfn_b200.ops import kernels as K, _lib
    torch.manual_seed(0)
    width = (Hq + 2 * Hkv) * D
    qkv = torch.randn(B * T, width, device="cuda", dtype=BF)
    q = qkv[:, : Hq * D]
    k = qkv[:, Hq * D: (Hq + Hkv) * D]
    v = qkv[:, (Hq + Hkv) * D:]
    scale = 1.0 / math.sqrt(D)
    o, lse = K.attention_forward(q, k, v, B=B, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D,
                                 causal=causal, window=window, scale=scale)
    _lib.assert_status_ok("attention fwd")
    qkv_f = qkv.float().requires_grad_(True)
    qf = qkv_f[:, : Hq * D]
    kf = qkv_f[:, Hq * D: (Hq + Hkv) * D]
    vf = qkv_f[:, (Hq + Hkv) * D:]
    o_ref, lse_ref = _attn_ref(qf, kf, vf, B, T, Hq, Hkv, D, causal, window, scale)
    assert _rel(o, o_ref) < 2e-2, _rel(o, o_ref)
    assert (lse - lse_ref).abs().max().item() < 2e-2
    do = torch.randn(B * T, Hq * D, device="cuda", dtype=BF)
    o_ref.backward(do.float())
    dqkv = torch.zeros_like(qkv)
    K.attention_backward(do, q, k, v, o, lse, B=B, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D,
                         causal=causal, window=window, scale=scale,
                         dq=dqkv[:, : Hq * D], dk=dqkv[:, Hq * D: (Hq + Hkv) * D],
                         dv=dqkv[:, (Hq + Hkv) * D:])
    _lib.assert_status_ok("attention bwd")
    g = qkv_f.grad
    for name, sl in (("dq", slice(0, Hq * D)), ("dk", slice(Hq * D, (Hq + Hkv) * D)),
                     ("dv", slice((Hq + Hkv) * D, width))):
        r = _rel(dqkv[:, sl], g[:, sl])
        assert r < 3e-2, (name, r)


def _attn_ref_ex(q, k, v, B, T, Hq, Hkv, D, causal, window, scale, softcap=0.0, seq_ids=None, gate=None):
    """fp32 oracle with the optional score soft-cap, packed-sequence mask and sigmoid output gate."""
    qf = q.float().view(B, T, Hq, D).transpose(1, 2)
    kf = k.float().view(B, T, Hkv, D).transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    vf = v.float().view(B, T, Hkv, D).transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    s = (qf @ kf.transpose(-1, -2)) * scale
    if softcap > 0:
        s = softcap * torch.tanh(s / softcap)
    qi = torch.arange(T, device=q.device)[:, None]
    ki = torch.arange(T, device=q.device)[None, :]
    mask = torch.ones(T, T, dtype=torch.bool, device=q.device)
    if causal:
        mask &= ki <= qi
        if window > 0:
            mask &= ki > qi - window
    elif window > 0:
        mask &= (ki > qi - window) & (ki < qi + window)
    mask = mask[None, None].expand(B, 1, T, T)
    if seq_ids is not None:
        ids = seq_ids.view(B, T)
        mask = mask & (ids[:, None, :, None] == ids[:, None, None, :])
    s = s.masked_fill(~mask, float("-inf"))
    o = (torch.softmax(s, dim=-1) @ vf).transpose(1, 2).reshape(B * T, Hq * D)
    lse = torch.logsumexp(s, dim=-1)
    if gate is not None:
        o = o * torch.sigmoid(gate.float())
    return o, lse


@pytest.mark.parametrize("B,T,Hq,Hkv,D,causal,window,softcap,packed", [
    (2, 384, 4, 2, 64, True, 0, 0.0, True),      # packed sequences, GQA
    (1, 512, 2, 2, 128, True, 0, 0.0, True),
    (2, 256, 2, 2, 64, True, 0, 20.0, False),    # score soft-cap
    (1, 448, 4, 1, 128, True, 160, 30.0, True),  # window + soft-cap + packed sequences
    (1, 320, 2, 2, 64, False, 0, 15.0, True),    # bidirectional
])
def test_attention_softcap_and_sequence_ids(kernel_lib, B, T, Hq, Hkv, D, causal, window, softcap, packed):
    from neuralfn_b200.ops import kernels as K, _lib
    torch.manual_seed(1)
    width = (Hq + 2 * Hkv) * D
    qkv = torch.randn(B * T, width, device="cuda", dtype=BF) * 1.5
    q, k, v = qkv[:, : Hq * D], qkv[:, Hq * D: (Hq + Hkv) * D], qkv[:, (Hq + Hkv) * D:]
    seq = None
    if packed:  # three documents of uneven length per row of the batch
        cuts = torch.tensor([0, T // 5, T // 2 + 7, T])
        seq = torch.cat([torch.full((int(cuts[i + 1] - cuts[i]),), i) for i in range(3)]).repeat(B).to("cuda", torch.int32)
    scale = 1.0 / math.sqrt(D)
    o, lse = K.attention_forward(q, k, v, B=B, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D, causal=causal,
                                 window=window, scale=scale, softcap=softcap, seq_ids=seq)
    _lib.assert_status_ok("attention fwd (soft-cap / sequence ids)")
    qkv_f = qkv.float().requires_grad_(True)
    qf, kf, vf = qkv_f[:, : Hq * D], qkv_f[:, Hq * D: (Hq + Hkv) * D], qkv_f[:, (Hq + Hkv) * D:]
    o_ref, lse_ref = _attn_ref_ex(qf, kf, vf, B, T, Hq, Hkv, D, causal, window, scale, softcap, seq)
    assert _rel(o, o_ref) < 2e-2, _rel(o, o_ref)
    assert (lse - lse_ref).abs().max().item() < 3e-2
    do = torch.randn(B * T, Hq * D, device="cuda", dtype=BF)
    o_ref.backward(do.float())
    dqkv = torch.zeros_like(qkv)
    K.attention_backward(do, q, k, v, o, lse, B=B, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D, causal=causal,
                         window=window, scale=scale, softcap=softcap, seq_ids=seq,
                         dq=dqkv[:, : Hq * D], dk=dqkv[:, Hq * D: (Hq + Hkv) * D], dv=dqkv[:, (Hq + Hkv) * D:])
    _lib.assert_status_ok("attention bwd (soft-cap / sequence ids)")
    g = qkv_f.grad
    for name, sl in (("dq", slice(0, Hq * D)), ("dk", slice(Hq * D, (Hq + Hkv) * D)), ("dv", slice((Hq + Hkv) * D, width))):
        assert _rel(dqkv[:, sl], g[:, sl]) < 3e-2, (name, _rel(dqkv[:, sl], g[:, sl]))


def test_attention_output_gate(kernel_lib):
    from neuralfn_b200.ops import kernels as K, _lib
    torch.manual_seed(2)
    B, T, Hq, Hkv, D = 2, 256, 4, 1, 128
    q = torch.randn(B * T, Hq * D, device="cuda", dtype=BF)
    k = torch.randn(B * T, Hkv * D, device="cuda", dtype=BF)
    v = torch.randn(B * T, Hkv * D, device="cuda", dtype=BF)
    gate = torch.randn(B * T, Hq * D, device="cuda", dtype=BF)
    o, _ = K.attention_forward(q, k, v, B=B, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D, causal=True, window=64, gate=gate)
    _lib.assert_status_ok("attention fwd (gate)")
    o_ref, _ = _attn_ref_ex(q, k, v, B, T, Hq, Hkv, D, True, 64, D ** -0.5, gate=gate)
    assert _rel(o, o_ref) < 2e-2


def test_attention_first_generation_kernels_still_match(kernel_lib):
    """The first-generation kernels stay selectable (nfn_attention_set_impl(1)); both generations
    must give the same gradients."""
    from neuralfn_b200.ops import kernels as K, _lib
    torch.manual_seed(3)
    B, T, H, D = 1, 512, 2, 64
    qkv = torch.randn(B * T, 3 * H * D, device="cuda", dtype=BF)
    q, k, v = qkv[:, : H * D], qkv[:, H * D: 2 * H * D], qkv[:, 2 * H * D:]
    do = torch.randn(B * T, H * D, device="cuda", dtype=BF)
    outs = []
    for impl in (2, 1):
        old = kernel_lib.nfn_attention_set_impl(impl)
        try:
            o, lse = K.attention_forward(q, k, v, B=B, T=T, n_q_heads=H, n_kv_heads=H, head_dim=D)
            d = torch.zeros_like(qkv)
            K.attention_backward(do, q, k, v, o, lse, B=B, T=T, n_q_heads=H, n_kv_heads=H, head_dim=D,
                                 dq=d[:, : H * D], dk=d[:, H * D: 2 * H * D], dv=d[:, 2 * H * D:],
                                 dq_accum=torch.empty(B * T, H * D, device="cuda"))
            _lib.assert_status_ok(f"attention impl {impl}")
            outs.append((o.float(), d.float()))
        finally:
            kernel_lib.nfn_attention_set_impl(old)
    assert _rel(outs[0][0], outs[1][0]) < 1e-2 and _rel(outs[0][1], outs[1][1]) < 2e-2


@pytest.mark.parametrize("vocab,ld,cap,z", [(50257, 50304, 30.0, 1e-4), (1000, 1024, 0.0, 0.0),
                                            (128256, 128256, 0.0, 1e-4)])
def test_cross_entropy(kernel_lib, vocab, ld, cap, z):
    from neuralfn_b200.ops import kernels as K
    torch.manual_seed(0)
    rows = 64
    raw = torch.randn(rows, ld, device="cuda") * 3
    capped = cap * torch.tanh(raw / cap) if cap > 0 else raw
    logits = capped.to(BF)
    targets = torch.randint(0, vocab, (rows,), device="cuda", dtype=torch.int32)
    targets[5] = -1
    lf = logits.float().requires_grad_(True)
    lse = torch.logsumexp(lf[:, :vocab], dim=-1)
    tv = lf[torch.arange(rows), targets.clamp(min=0).long()]
    per = lse - tv + z * lse * lse
    valid = (targets >= 0).float()
    ref_loss = (per * valid).sum() / rows
    ref_loss.backward()
    ref_grad = lf.grad.clone()
    if cap > 0:
        ref_grad = ref_grad * (1 - (logits.float() / cap) ** 2)
    work = logits.clone()
    mean_loss, row_loss = K.cross_entropy(work, targets, vocab=vocab, cap=cap, z_coef=z,
                                          grad_scale=1.0 / rows, loss_scale=1.0 / rows)
    assert abs(mean_loss.item() - ref_loss.item()) < 2e-3 * max(1.0, abs(ref_loss.item()))
    assert _rel(work[:, :vocab], ref_grad[:, :vocab]) < 2e-2
    assert work[:, vocab:].abs().max().item() == 0 if ld > vocab else True
    assert work[5].abs().max().item() == 0


def test_embedding(kernel_lib):
    from neuralfn_b200.ops import kernels as K
    torch.manual_seed(0)
    B, T, C, V = 3, 64, 768, 1000
    wte = torch.randn(V, C, device="cuda", dtype=BF)
    wpe = torch.randn(T, C, device="cuda", dtype=BF)
    tok = torch.randint(0, V, (B * T,), device="cuda", dtype=torch.int32)
    out = K.embedding_forward(tok, wte, wpe, T=T)
    pos = torch.arange(B * T, device="cuda") % T
    ref = wte.float()[tok.long()] + wpe.float()[pos]
    assert _rel(out, ref) < 1e-2
    dout = torch.randn(B * T, C, device="cuda", dtype=BF)
    dwte = torch.zeros(V, C, device="cuda", dtype=BF)
    dwpe = torch.empty(T, C, device="cuda", dtype=BF)
    K.embedding_backward(dout, tok, dwte, dwpe, B=B, T=T)
    ref_wte = torch.zeros(V, C, device="cuda").index_add_(0, tok.long(), dout.float())
    ref_wpe = dout.float().view(B, T, C).sum(0)
    assert _rel(dwte, ref_wte) < 2e-2
    assert _rel(dwpe, ref_wpe) < 1e-2


@pytest.mark.parametrize("C", [768, 100])
def test_embedding_gradient_is_reproducible_on_skewed_tokens(kernel_lib, C):
    """Runs of equal tokens from one to thousands of rows (and an out-of-range id, which is skipped): every call gives the same
    bits, on top of what the tied head's weight gradient left in the buffer, and the sum agrees with an fp32 index_add."""
    from neuralfn_b200.ops import kernels as K
    g = torch.Generator(device="cuda").manual_seed(4)
    B, T, V = 4, 1024, 3000
    tok = (torch.rand(B * T, device="cuda", generator=g) ** 6 * V).int().clamp_(0, V - 1)
    tok[17] = V + 5
    dout = (torch.randn(B * T, C, device="cuda", generator=g) * 0.05).to(BF)
    base = (torch.randn(V, C, device="cuda", generator=g) * 0.05).to(BF)
    assert int(torch.bincount(tok.long().clamp(max=V - 1)).max()) > 500
    outs = []
    for _ in range(3):
        dwte = base.clone()
        K.embedding_backward(dout, tok, dwte, None, B=B, T=T)
        outs.append(dwte)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    ok = tok < V
    ref = base.float().index_add_(0, tok[ok].long(), dout[ok].float())
    assert _rel(outs[0], ref) < 1e-2


def test_adamw_and_clip(kernel_lib):
    from neuralfn_b200.ops import kernels as K
    torch.manual_seed(0)
    n, n_decay = 8 * 5000, 8 * 3000
    master = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    grad = (torch.randn(n, device="cuda") * 3).to(BF)
    param = torch.empty(n, device="cuda", dtype=BF)
    lr, b1, b2, eps, wd, step, max_norm, gscale = 1e-2, 0.9, 0.95, 1e-8, 0.1, 1, 1.0, 0.5
    hyper = torch.zeros(K.HYPER_SIZE, device="cuda")
    hyper[:9] = torch.tensor([lr, b1, b2, eps, wd, 1 - b1 ** step, 1 - b2 ** step, gscale, max_norm])
    partial = torch.empty(K.optim_max_partials(), device="cuda")
    clip = torch.empty(2, device="cuda")
    K.grad_clip_scale(grad, partial, hyper, clip)
    g = grad.float() * gscale
    norm = g.norm()
    assert abs(clip[1].item() - norm.item()) < 1e-3 * norm.item()
    c = min(1.0, max_norm / (norm.item() + 1e-6))
    assert abs(clip[0].item() - c) < 1e-4
    ref_w = master.clone()
    gg = g * c
    rm = (1 - b1) * gg
    rv = (1 - b2) * gg * gg
    wdv = torch.zeros(n, device="cuda")
    wdv[:n_decay] = wd
    ref_w = ref_w - lr * ((rm / (1 - b1)) / ((rv / (1 - b2)).sqrt() + eps) + wdv * ref_w)
    K.adamw_flat(master, m, v, grad, param, n_decay, hyper, clip)
    assert _rel(master, ref_w) < 1e-5
    assert _rel(param, ref_w) < 1e-2
    assert _rel(m, rm) < 1e-5 and _rel(v, rv) < 1e-5


def test_dp_emulated_ranks(kernel_lib):
    """Sharded reduce + AdamW for W emulated ranks on one GPU: every phase runs for all
    ranks before the next phase starts, so no launch ever waits on a later launch."""
    from neuralfn_b200.ops import kernels as K, _lib
    torch.manual_seed(0)
    W, n = 4, 8 * 4096
    n_decay = 8 * 1000
    shard = n // W
    grads = [(torch.randn(n, device="cuda")).to(BF) for _ in range(W)]
    params = [torch.zeros(n, device="cuda", dtype=BF) for _ in range(W)]
    master0 = torch.randn(n, device="cuda")
    masters = [master0[r * shard:(r + 1) * shard].clone() for r in range(W)]
    ms = [torch.zeros(shard, device="cuda") for _ in range(W)]
    vs = [torch.zeros(shard, device="cuda") for _ in range(W)]
    gsh = [torch.empty(shard, device="cuda") for _ in range(W)]
    parts = [torch.empty(K.optim_max_partials(), device="cuda") for _ in range(W)]
    slots = [torch.zeros(16, device="cuda", dtype=torch.int64) for _ in range(W)]
    flags = [torch.zeros(4 * W, device="cuda", dtype=torch.int32) for _ in range(W)]
    clips = [torch.empty(2, device="cuda") for _ in range(W)]
    lr, b1, b2, eps, wd, max_norm = 1e-2, 0.9, 0.95, 1e-8, 0.1, 1.0
    hyper = torch.zeros(K.HYPER_SIZE, device="cuda")
    hyper[:9] = torch.tensor([lr, b1, b2, eps, wd, 1 - b1, 1 - b2, 1.0 / W, max_norm])
    gp = [g.data_ptr() for g in grads]
    pp = [p.data_ptr() for p in params]
    sp = [s.data_ptr() for s in slots]
    fp = [f.data_ptr() for f in flags]
    epoch = 1
    for r in range(W):
        K.peer_arrive(fp, r, W, 0, epoch)
    for r in range(W):
        K.peer_wait(fp[r], W, 0, epoch, timeout_s=0.5)
    for r in range(W):
        K.dp_reduce(gp, r, W, r * shard, shard, gsh[r], parts[r])
    for r in range(W):
        K.dp_norm_publish(parts[r], shard, sp, r, W, epoch)
    for r in range(W):
        K.dp_norm_collect(sp[r], W, epoch, hyper, clips[r], timeout_s=0.5)
    for r in range(W):
        K.dp_adamw(masters[r], ms[r], vs[r], gsh[r], pp, r, W, r * shard, shard, n_decay, hyper, clips[r])
    _lib.assert_status_ok("dp emulated")
    gsum = sum(g.float() for g in grads) / W
    norm = gsum.norm().item()
    c = min(1.0, max_norm / (norm + 1e-6))
    for r in range(W):
        assert abs(clips[r][1].item() - norm) < 1e-3 * norm
    gg = gsum * c
    wdv = torch.zeros(n, device="cuda")
    wdv[:n_decay] = wd
    ref = master0 - lr * (gg / (gg.abs() + eps) + wdv * master0)
    got = torch.cat(masters)
    assert _rel(got, ref) < 1e-4
    for r in range(W):
        assert _rel(params[r], ref) < 1e-2


def test_peer_wait_times_out_cleanly(kernel_lib):
    """A flag nobody sets: the bounded wait gives up, reports through the status word,
    and the context stays usable."""
    from neuralfn_b200.ops import kernels as K, _lib
    flags = torch.zeros(8, device="cuda", dtype=torch.int32)
    K.peer_wait(flags.data_ptr(), 2, 0, 1, timeout_s=0.2)
    assert _lib.status_read_reset() == 5
    assert _lib.status_read_reset() == 0
    x = torch.ones(4, device="cuda")
    assert x.sum().item() == 4


@pytest.mark.parametrize("D", [64, 128])
def test_differential_glue_kernels(kernel_lib, D):
    """q expand / collapse, the differential combine and its backward against fp32 autograd."""
    from neuralfn_b200.ops import _lib
    from neuralfn_b200.ops import kernels as K
    torch.manual_seed(0)
    N, H = 300, 3                                      # a ragged last warp of (token, head) groups
    qkv = torch.randn(N, 3 * H * D, device="cuda", dtype=torch.bfloat16)
    q2 = torch.empty(N, 2 * H * D, device="cuda", dtype=torch.bfloat16)
    K.diff_q_expand(qkv[:, :H * D], q2, H, D)
    q = qkv[:, :H * D].view(N, H, D)
    ref = torch.zeros(N, H, 2, D, device="cuda", dtype=torch.bfloat16)
    ref[:, :, 0, :D // 2] = q[..., :D // 2]
    ref[:, :, 1, D // 2:] = q[..., D // 2:]
    assert torch.equal(q2.view(N, H, 2, D), ref)
    dq = torch.zeros(N, 3 * H * D, device="cuda", dtype=torch.bfloat16)
    g2 = torch.randn_like(q2)
    K.diff_q_collapse(g2, dq[:, :H * D], H, D)
    want = torch.cat([g2.view(N, H, 2, D)[:, :, 0, :D // 2], g2.view(N, H, 2, D)[:, :, 1, D // 2:]], dim=-1)
    assert torch.equal(dq[:, :H * D].view(N, H, D), want) and dq[:, H * D:].abs().max() == 0

    a = torch.randn(N, 2 * H * D, device="cuda", dtype=torch.bfloat16)
    lam = torch.zeros(8, device="cuda", dtype=torch.bfloat16)
    lam[0] = 0.6875
    out = torch.empty(N, H * D, device="cuda", dtype=torch.bfloat16)
    rstd = torch.empty(N * H, device="cuda", dtype=torch.float32)
    K.diff_combine(a, lam, 0.2, 1e-5, out, rstd, H, D)
    af = a.float().view(N, H, 2, D).requires_grad_(True)
    lf = lam[0].float().clone().requires_grad_(True)
    x = af[:, :, 0] - lf * af[:, :, 1]
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * 0.2
    torch.testing.assert_close(out.float().view(N, H, D), y, atol=2e-3, rtol=2e-2)
    dout = torch.randn(N, H * D, device="cuda", dtype=torch.bfloat16)
    y.backward(dout.float().view(N, H, D))
    da = torch.empty_like(a)
    dlam = torch.full((8,), 7.0, device="cuda", dtype=torch.bfloat16)
    partial = torch.empty(K.diff_partials(), device="cuda", dtype=torch.float32)
    K.diff_combine_backward(dout, a, lam, 0.2, rstd, da, partial, dlam, H, D)
    _lib.assert_status_ok("differential glue")
    torch.testing.assert_close(da.float().view(N, H, 2, D), af.grad, atol=3e-3, rtol=3e-2)
    assert abs(float(dlam[0]) - float(lf.grad)) <= 2e-2 * abs(float(lf.grad)) + 1e-2
    assert dlam[1:].abs().max() == 0
