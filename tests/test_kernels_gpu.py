"""Numerics of the sm_100a kernels against plain PyTorch fp32 references of the same op."""

import pytest
import torch
import torch.nn.functional as F

from scaling_b200.ops import functional as K

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(64, 768), (37, 4096), (5, 8192), (300, 64)])
@pytest.mark.parametrize("rms", [True, False])
def test_norm(dtype, shape, rms):
    torch.manual_seed(0)
    x = torch.randn(*shape, device=DEV, dtype=dtype, requires_grad=True)
    w = (torch.rand(shape[1], device=DEV) + 0.5).to(dtype).requires_grad_()
    b = None if rms else (torch.randn(shape[1], device=DEV) * 0.1).to(dtype).requires_grad_()
    y = K.rms_norm(x, w, 1e-5) if rms else K.layer_norm(x, w, b, 1e-5)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    br = None if rms else b.detach().float().requires_grad_()
    if rms:
        yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    else:
        yr = F.layer_norm(xr, (shape[1],), wr, br, 1e-5)
    yr.backward(dy.float())
    tol = 2e-2 if dtype != torch.float32 else 1e-5
    assert _rel(y, yr) < tol
    assert _rel(x.grad, xr.grad) < tol
    assert _rel(w.grad, wr.grad) < tol
    if not rms:
        assert _rel(b.grad, br.grad) < tol


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_swiglu_gelu(dtype):
    torch.manual_seed(1)
    M, Fd = 333, 1024
    ag = torch.randn(M, 2 * Fd, device=DEV, dtype=dtype, requires_grad=True)
    a, g = ag[:, :Fd], ag[:, Fd:]
    y = K.swiglu(a, g)
    dy = torch.randn_like(y)
    y.backward(dy)
    agr = ag.detach().float().requires_grad_()
    yr = F.silu(agr[:, :Fd]) * agr[:, Fd:]
    yr.backward(dy.float())
    tol = 2e-2 if dtype != torch.float32 else 1e-5
    assert _rel(y, yr) < tol and _rel(ag.grad, agr.grad) < tol
    x = torch.randn(1000, 77, device=DEV, dtype=dtype, requires_grad=True)
    y = K.gelu(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    yr = F.gelu(xr)
    yr.backward(dy.float())
    assert _rel(y, yr) < tol and _rel(x.grad, xr.grad) < tol


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("rot", [64, 32])
def test_rope(interleaved, rot):
    torch.manual_seed(2)
    T, H, D = 257, 12, 64
    x = torch.randn(T, H, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    pos = torch.randint(0, 4096, (T,), device=DEV)
    y = K.rope(x, pos, rot, 10000.0, interleaved)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().cpu().requires_grad_()
    yr = K.rope_reference(xr, pos.cpu(), rot, 10000.0, interleaved)
    yr.backward(dy.float().cpu())
    assert _rel(y.cpu(), yr) < 1e-2
    assert _rel(x.grad.cpu(), xr.grad) < 1e-2
    # strided view (q slice of a fused qkv buffer)
    qkv = torch.randn(T, H, 3 * D, device=DEV, dtype=torch.bfloat16)
    q = qkv[:, :, :D]
    yq = K.rope(q, pos, rot, 10000.0, interleaved)
    yq_ref = K.rope_reference(q.float().cpu(), pos.cpu(), rot, 10000.0, interleaved)
    assert _rel(yq.cpu(), yq_ref) < 1e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_masked_softmax(dtype):
    torch.manual_seed(3)
    b, h, sq, sk = 2, 3, 65, 130
    x = torch.randn(b, h, sq, sk, device=DEV, dtype=dtype, requires_grad=True)
    mask = torch.rand(b, 1, sq, sk, device=DEV) > 0.7
    y = K.masked_softmax(x, mask, 0.37)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    yr = torch.softmax((xr * 0.37).masked_fill(mask, -10000.0), -1)
    yr.backward(dy.float())
    tol = 2e-2 if dtype != torch.float32 else 1e-5
    assert _rel(y, yr) < tol and _rel(x.grad, xr.grad) < tol


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("V", [32768, 1000])
def test_cross_entropy(dtype, V):
    torch.manual_seed(4)
    N = 129
    logits = (torch.randn(N, V, device=DEV) * 3).to(dtype)
    tg = torch.randint(0, V, (N,), device=DEV)
    w = torch.rand(N, device=DEV)
    ref_l = logits.float().requires_grad_()
    per = F.cross_entropy(ref_l, tg, reduction="none")
    (per * w).sum().backward()
    # two "ranks": split vocab in halves and combine statistics by hand
    half = V // 2
    parts = [logits[:, :half], logits[:, half:]]
    stats = [K.ce_stats(p, tg, vocab_start=i * half) for i, p in enumerate(parts)]
    gmax = torch.maximum(stats[0][0], stats[1][0])
    gsum = sum(s[1] * torch.exp(s[0] - gmax) for s in stats)
    gtgt = stats[0][2] + stats[1][2]
    losses = []
    grads = []
    for i, p in enumerate(parts):
        loss, dl = K.ce_finalize(p.clone(), tg, gmax, gsum, gtgt, w, vocab_start=i * half)
        losses.append(loss)
        grads.append(dl)
    tol = 2e-2 if dtype != torch.float32 else 1e-5
    assert _rel(losses[0], per) < 1e-3 if dtype != torch.float32 else 1e-5
    assert torch.equal(losses[0], losses[1])
    assert _rel(torch.cat(grads, 1), ref_l.grad) < tol
    am = torch.where(stats[0][3] >= stats[1][3], stats[0][4], stats[1][4])
    assert (am == logits.float().argmax(-1)).float().mean() > 0.99


def test_embedding():
    torch.manual_seed(5)
    V, H = 1000, 256
    W = torch.randn(V, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, 2 * V, (4, 300), device=DEV)
    out = K.embedding(ids, W, vocab_start=500)
    dy = torch.randn_like(out)
    out.backward(dy)
    Wr = W.detach().float().requires_grad_()
    loc = ids - 500
    oob = (loc < 0) | (loc >= V)
    ref = F.embedding(loc.masked_fill(oob, 0), Wr).masked_fill(oob[..., None], 0)
    ref.backward(dy.float())
    assert torch.equal(out.float(), ref.detach().to(torch.bfloat16).float())
    assert _rel(W.grad, Wr.grad) < 1e-2
    # deterministic
    W2 = W.detach().clone().requires_grad_()
    K.embedding(ids, W2, vocab_start=500).backward(dy)
    assert torch.equal(W.grad, W2.grad)


@pytest.mark.parametrize("gdtype", [torch.bfloat16, torch.float32])
def test_adamw_and_sumsq(gdtype):
    torch.manual_seed(6)
    n = 1_000_003
    p = torch.randn(n, device=DEV)
    pr = p.clone().requires_grad_()
    m = torch.zeros_like(p)
    v = torch.zeros_like(p)
    lp = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    opt = torch.optim.AdamW([pr], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ctrl = torch.tensor([0.5, 0.0], device=DEV)
    for step in range(1, 4):
        g = torch.randn(n, device=DEV).to(gdtype)
        pr.grad = g.float() * 0.5
        opt.step()
        K.adamw_step(p, m, v, g, lp, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, ctrl)
    assert _rel(p, pr.detach()) < 1e-5
    assert torch.equal(lp, p.to(torch.bfloat16))
    # skip flag leaves state untouched
    before = p.clone()
    K.adamw_step(p, m, v, g, lp, 1e-2, 0.9, 0.95, 1e-8, 0.1, 4, torch.tensor([1.0, 1.0], device=DEV))
    assert torch.equal(before, p)
    out = torch.zeros(1, device=DEV)
    flag = torch.zeros(1, device=DEV, dtype=torch.int32)
    K.sumsq_(g, out, flag, 1.0, True)
    assert abs(out.item() - (g.float() ** 2).sum().item()) / out.item() < 1e-4
    assert flag.item() == 0
    g[12345] = float("inf")
    K.sumsq_(g, out, flag, 1.0, False)
    assert flag.item() == 1


GEMM_SHAPES = [(128, 256, 64), (256, 512, 128), (300, 264, 200), (2048, 2304, 768), (1000, 768, 3072), (64, 32, 1024),
               (4096, 136, 72),
               # few output tiles with a long reduction: these take the split-K path
               (256, 384, 8192), (640, 768, 4096), (136, 200, 2048)]


@pytest.mark.parametrize("M,N,K_", GEMM_SHAPES)
@pytest.mark.parametrize("mode", ["nt", "nn", "tn"])
@pytest.mark.parametrize("bn", [0, 128, 256, 512])
def test_gemm(M, N, K_, mode, bn):
    torch.manual_seed(7)
    dt = torch.bfloat16
    if mode == "nt":  # forward: a [M,K], b [N,K]
        a = torch.randn(M, K_, device=DEV, dtype=dt)
        b = torch.randn(N, K_, device=DEV, dtype=dt)
        ref = a.float() @ b.float().t()
        c = K.gemm(a, b, bn=bn)
    elif mode == "nn":  # dgrad: a [M,K], b [K,N]
        a = torch.randn(M, K_, device=DEV, dtype=dt)
        b = torch.randn(K_, N, device=DEV, dtype=dt)
        ref = a.float() @ b.float()
        c = K.gemm(a, b, b_mn=True, bn=bn)
    else:  # wgrad: a [K,M], b [K,N]
        a = torch.randn(K_, M, device=DEV, dtype=dt)
        b = torch.randn(K_, N, device=DEV, dtype=dt)
        ref = a.float().t() @ b.float()
        c = K.gemm(a, b, a_mn=True, b_mn=True, bn=bn)
    K.check_status()
    assert c.shape == (M, N)
    assert _rel(c, ref) < 1e-2, f"rel err {_rel(c, ref)}"


def test_gemm_epilogues():
    torch.manual_seed(8)
    M, N, K_ = 512, 1024, 256
    a = torch.randn(M, K_, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K_, device=DEV, dtype=torch.bfloat16) * 0.1
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    pre = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    c = K.gemm(a, b, bias=bias, act="gelu", pre_act_out=pre)
    ref_pre = a.float() @ b.float().t() + bias.float()
    assert _rel(pre, ref_pre) < 1e-2
    assert _rel(c, F.gelu(ref_pre)) < 1e-2
    acc = torch.randn(M, N, device=DEV, dtype=torch.float32)
    acc0 = acc.clone()
    K.gemm(a, b, out=acc, accumulate=True)
    assert _rel(acc, acc0 + a.float() @ b.float().t()) < 1e-2
    K.check_status()


def test_gemm_split_k_epilogues_and_determinism():
    """Long-K problems with few tiles are split; bias, accumulation and fp32 / fp16 outputs go through the same
    finishing code, and the result is bitwise reproducible."""
    torch.manual_seed(18)
    M, N, K_ = 384, 768, 8192
    a = torch.randn(K_, M, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(K_, N, device=DEV, dtype=torch.bfloat16)
    ref = a.float().t() @ b.float()
    base = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    out = base.clone()
    K.gemm(a, b, a_mn=True, b_mn=True, out=out, accumulate=True)
    assert _rel(out, ref + base.float()) < 1e-2
    out2 = base.clone()
    K.gemm(a, b, a_mn=True, b_mn=True, out=out2, accumulate=True)
    assert torch.equal(out, out2)
    c32 = K.gemm(a, b, a_mn=True, b_mn=True, out_dtype=torch.float32)
    assert _rel(c32, ref) < 1e-2
    for shape, split in ((512, 1), (512, 2), (512, 5), (256, 3), (128, 4)):  # CTA pairs and single CTAs, split or not
        c = K.gemm(a, b, a_mn=True, b_mn=True, bn=shape, split=split)
        assert _rel(c, ref) < 1e-2, (shape, split, _rel(c, ref))
    x = torch.randn(M, K_, device=DEV, dtype=torch.float16) * 0.1
    w = torch.randn(N, K_, device=DEV, dtype=torch.float16) * 0.1
    bias = torch.randn(N, device=DEV, dtype=torch.float16)
    pre = torch.empty(M, N, device=DEV, dtype=torch.float16)
    y = K.gemm(x, w, bias=bias, act="gelu", pre_act_out=pre)
    ref_pre = x.float() @ w.float().t() + bias.float()
    assert _rel(pre, ref_pre) < 1e-2
    assert _rel(y, F.gelu(ref_pre)) < 1e-2
    K.check_status()


def test_linear_autograd():
    torch.manual_seed(9)
    x = torch.randn(4, 100, 768, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(2304, 768, device=DEV) * 0.02).to(torch.bfloat16).requires_grad_()
    b = torch.randn(2304, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = K.linear(x, w, b, act="gelu")
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = F.gelu(F.linear(xr, wr, br))
    yr.backward(dy.float())
    K.check_status()
    assert _rel(y, yr) < 1e-2
    assert _rel(x.grad, xr.grad) < 2e-2
    assert _rel(w.grad, wr.grad) < 2e-2
    assert _rel(b.grad, br.grad) < 2e-2


@pytest.mark.parametrize("M,N", [(16384, 768), (1000, 3072), (77, 40), (5, 8)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_column_sum(M, N, dtype):
    torch.manual_seed(5)
    x = torch.randn(M, N, device=DEV, dtype=dtype)
    ref = x.double().sum(0)
    out = K.column_sum(x)
    assert _rel(out, ref) < (1e-2 if dtype == torch.bfloat16 else 1e-5)
    base = torch.randn(N, device=DEV, dtype=dtype)
    acc = base.clone()
    K.column_sum(x, out=acc, accumulate=True)
    assert _rel(acc, ref + base.double()) < (1e-2 if dtype == torch.bfloat16 else 1e-5)
    assert torch.equal(K.column_sum(x), out)  # deterministic


def test_fused_gradient_accumulation_matches_autograd():
    """Parameters flagged for in-kernel accumulation receive the same gradients as through autograd."""
    torch.manual_seed(6)
    M, Kd, N = 512, 256, 384
    x = torch.randn(M, Kd, device=DEV, dtype=torch.bfloat16)
    dy = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    w0 = torch.randn(N, Kd, device=DEV, dtype=torch.bfloat16) * 0.05
    b0 = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    results = []
    for fused in (False, True):
        w = torch.nn.Parameter(w0.clone())
        b = torch.nn.Parameter(b0.clone())
        g = torch.nn.Parameter(torch.ones(N, device=DEV, dtype=torch.bfloat16))
        gb = torch.nn.Parameter(torch.zeros(N, device=DEV, dtype=torch.bfloat16))
        params = (w, b, g, gb)
        for p in params:
            p.grad = torch.zeros_like(p)
            if fused:
                p.fused_grad_accumulation = True
        for _ in range(2):  # two micro batches accumulate
            xin = x.clone().requires_grad_()
            y = K.layer_norm(K.linear(xin, w, b, act="gelu"), g, gb, 1e-5)
            y.backward(dy)
        K.check_status()
        results.append([p.grad.clone() for p in params] + [xin.grad.clone()])
    for a, b_ in zip(*results):
        assert _rel(a, b_) < 1e-2, _rel(a, b_)


FA_CASES = [
    # T, Hq, Hkv, D, cu_seqlens, causal, window
    (256, 2, 2, 64, [0, 256], True, None),
    (384, 4, 2, 64, [0, 100, 101, 300, 384], True, None),
    (300, 2, 1, 128, [0, 37, 300], True, None),
    (512, 4, 4, 64, [0, 512], False, None),
    (512, 2, 2, 64, [0, 200, 512], True, 64),
    (1024, 8, 2, 128, [0, 1024], True, None),
    (333, 3, 3, 64, [0, 333], False, 50),
]


@pytest.mark.parametrize("T,Hq,Hkv,D,cu,causal,window", FA_CASES)
def test_flash_attention(T, Hq, Hkv, D, cu, causal, window):
    from scaling_b200.ops.attention import attention_reference, flash_attention

    torch.manual_seed(10)
    q = torch.randn(T, Hq, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(T, Hkv, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(T, Hkv, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    cu_t = torch.tensor(cu, device=DEV, dtype=torch.int32)
    scale = D ** -0.5
    out = flash_attention(q, k, v, cu_t, None, causal=causal, scale=scale, window=window)
    do = torch.randn_like(out)
    out.backward(do)
    K.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = attention_reference(qr, kr, vr, cu_t, None, causal, scale, window)
    ref.backward(do.float())
    assert _rel(out, ref) < 2e-2, _rel(out, ref)
    assert _rel(q.grad, qr.grad) < 3e-2, _rel(q.grad, qr.grad)
    assert _rel(k.grad, kr.grad) < 3e-2, _rel(k.grad, kr.grad)
    assert _rel(v.grad, vr.grad) < 3e-2, _rel(v.grad, vr.grad)
    # deterministic backward: bitwise equal on a second run
    q2, k2, v2 = (t.detach().clone().requires_grad_() for t in (q, k, v))
    flash_attention(q2, k2, v2, cu_t, None, causal=causal, scale=scale, window=window).backward(do)
    assert torch.equal(q.grad, q2.grad) and torch.equal(k.grad, k2.grad) and torch.equal(v.grad, v2.grad)


@pytest.mark.parametrize("T,H,D,cu,window,rot,interleaved", [
    (384, 4, 64, [0, 100, 384], None, 64, False),
    (300, 2, 128, [0, 300], None, 64, True),
    (4352, 12, 64, [0, 2048, 4352], None, 64, False),   # enough heads x tiles to take the split dK/dV path
    (512, 3, 64, [0, 512], 100, None, False),
])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_packed_qkv_attention(T, H, D, cu, window, rot, interleaved, dtype):
    """Fused rotary + attention on a packed [T, H, 3D] projection against rope + attention on separate tensors."""
    from scaling_b200.ops.attention import attention_reference
    from scaling_b200.ops.attention_kernel import packed_qkv_attention, packed_qkv_supported

    torch.manual_seed(12)
    src = torch.randn(T, H, 3 * D, device=DEV, dtype=dtype)
    cu_t = torch.tensor(cu, device=DEV, dtype=torch.int32)
    pos = torch.cat([torch.arange(b - a, device=DEV, dtype=torch.int32) for a, b in zip(cu[:-1], cu[1:])])
    scale = D ** -0.5
    rotary = None if rot is None else (rot, 10000.0, interleaved)

    x = src.clone().requires_grad_()
    qkv = x * 1.0  # the fused op consumes its input, as it does the projection's output inside the model
    assert packed_qkv_supported(qkv)
    out = packed_qkv_attention(qkv, pos, rotary, cu_t, True, scale, window)
    do = torch.randn_like(out)
    out.backward(do)
    K.check_status()

    xr = src.detach().float().requires_grad_()
    q, k, v = xr[..., :D], xr[..., D:2 * D], xr[..., 2 * D:]
    if rotary is not None:
        q = K.rope_reference(q, pos, rot, 10000.0, interleaved)
        k = K.rope_reference(k, pos, rot, 10000.0, interleaved)
    ref = attention_reference(q, k, v, cu_t, None, True, scale, window)
    ref.backward(do.float())
    assert _rel(out, ref) < 2e-2, _rel(out, ref)
    for sl in (slice(0, D), slice(D, 2 * D), slice(2 * D, 3 * D)):
        assert _rel(x.grad[..., sl], xr.grad[..., sl]) < 3e-2, _rel(x.grad[..., sl], xr.grad[..., sl])
    x2 = src.clone().requires_grad_()
    packed_qkv_attention(x2 * 1.0, pos, rotary, cu_t, True, scale, window).backward(do)
    assert torch.equal(x.grad, x2.grad)


def test_flash_attention_strided_qkv():
    from scaling_b200.ops.attention import attention_reference, flash_attention

    torch.manual_seed(11)
    T, H, D = 256, 4, 64
    qkv = torch.randn(T, H, 3 * D, device=DEV, dtype=torch.bfloat16)
    q, k, v = qkv[..., :D], qkv[..., D:2 * D], qkv[..., 2 * D:]
    cu = torch.tensor([0, 128, 256], device=DEV, dtype=torch.int32)
    out = flash_attention(q, k, v, cu, None, causal=True, scale=D ** -0.5)
    ref = attention_reference(q.float(), k.float(), v.float(), cu, None, True, D ** -0.5)
    K.check_status()
    assert _rel(out, ref) < 2e-2


def test_peer_barrier_wait_runs_out_and_reports_timeout():
    """A flag that nobody sets: the bounded wait gives up, the host sees CommTimeout, the context stays usable."""
    import ctypes
    import time

    from scaling_b200.ops import _lib
    from scaling_b200.ops._lib import CommTimeout, lib

    mine = torch.zeros(16, dtype=torch.int32, device=DEV)    # this rank's flag words
    peer = torch.zeros(16, dtype=torch.int32, device=DEV)    # stands in for a peer that never arrives
    rounds = torch.zeros(1, dtype=torch.int32, device=DEV)
    ptrs = (ctypes.c_void_p * 2)(mine.data_ptr(), peer.data_ptr())
    K.check_status()
    t0 = time.time()
    rc = lib().sb200_p2p_barrier(ptrs, rounds.data_ptr(), 0, 2, K.status_word().data_ptr(), 0.05, _lib.stream())
    assert rc == 0
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    assert peer[0].item() == 1 and mine[0].item() == 1 and mine[1].item() == 0  # signalled both, heard from itself only
    with pytest.raises(CommTimeout):
        K.check_status()
    K.check_status()  # the status word was cleared
    x = torch.randn(64, 64, device=DEV, dtype=torch.bfloat16)
    assert torch.isfinite(K.gemm(x, x).float()).all()  # kernels still run
    # a complete round: both "ranks" set each other's flags
    peer.zero_(); mine.zero_(); rounds.zero_()
    mine[1] = 1
    rc = lib().sb200_p2p_barrier(ptrs, rounds.data_ptr(), 0, 2, K.status_word().data_ptr(), 0.05, _lib.stream())
    torch.cuda.synchronize()
    K.check_status()


# ---------------------------------------------------------------------------------------------- dropout kernels
def _rng_state(seed=1234):
    from scaling_b200.parallel.rng_tracker import KernelDropoutState

    st = KernelDropoutState(seed, torch.device(DEV))
    st.begin_step()
    return st


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n", [8 * 1000 + 3, 4096 * 6])
def test_dropout_residual_kernel(dtype, n):
    """y = dropout(x) * xs + r * rs against the same expression on the exported mask; the backward pass rebuilds the
    mask; masks depend on (step, call, element) only, so token shards of a tensor see their part of the full mask."""
    torch.manual_seed(3)
    p = 0.25
    st = _rng_state()
    x = torch.randn(n, device=DEV, dtype=dtype, requires_grad=True)
    r = torch.randn(n, device=DEV, dtype=dtype, requires_grad=True)
    y = K.dropout_add(x, r, p, st, True, x_scale=0.5, r_scale=2.0)       # call 0
    mask = K.dropout_mask((n,), p, st, 0)
    kept = (mask > 0).float().mean().item()
    assert abs(kept - (1 - p)) < 0.02
    assert all(v == 0.0 or abs(v - 1 / (1 - p)) < 1e-6 for v in mask.unique().tolist())
    ref = (x.detach().float() * mask * 0.5 + r.detach().float() * 2.0).to(dtype)
    assert _rel(y, ref) < (1e-3 if dtype == torch.bfloat16 else 1e-6)
    assert ((y.float() - r.detach().float() * 2.0).abs() < 1e-2 * (1 + r.detach().float().abs())).logical_or(mask > 0).all()
    dy = torch.randn_like(y)
    y.backward(dy)
    assert _rel(x.grad, dy.float() * mask * 0.5) < 1e-2 and ((x.grad == 0) == (mask == 0)).all()
    assert torch.equal(r.grad.float(), (dy.float() * 2.0).to(dtype).float())
    # another call index and another step give other masks; the same triple gives the same mask
    assert not torch.equal(K.dropout_mask((n,), p, st, 1), mask)
    assert torch.equal(K.dropout_mask((n,), p, st, 0), mask)
    st.begin_step()
    assert not torch.equal(K.dropout_mask((n,), p, st, 0), mask)
    # shards: elements [a, b) of the tensor, processed on their own with elem_offset = a
    a = (n // 3) // 4 * 4
    full = K.dropout_mask((n,), p, st, 0)
    assert torch.equal(K.dropout_mask((n - a,), p, st, 0, elem_offset=a), full[a:])
    # p = 0: a plain scaled add, no random numbers
    z = K.dropout_add(x.detach(), r.detach(), 0.0, None, True, x_scale=1.0, r_scale=1.0)
    assert torch.equal(z, x.detach() + r.detach())


def test_dropout_is_replayed_by_activation_checkpointing():
    from scaling_b200.core.nn.parallel_module.activation_checkpointing import checkpoint
    from scaling_b200.parallel import Topology, TopologyConfig

    topo = Topology(TopologyConfig.from_dict({"world_size": 1, "model_parallel_size": 1, "pipe_parallel_size": 1,
                                              "global_rank": 0, "local_slot": 0, "micro_batch_size": 1,
                                              "gradient_accumulation_steps": 1}))
    st = topo.kernel_rng
    st.begin_step()
    w = torch.randn(512, device=DEV, requires_grad=True)

    def block(x):
        return K.dropout_add(x * w, None, 0.5, st, True) + K.dropout_add(x, x, 0.3, st, True)

    x = torch.randn(512, device=DEV)
    plain = block(x)
    plain.sum().backward()
    g_plain, w.grad = w.grad.clone(), None
    st.call_index = 0
    ck = checkpoint(block, topo, x)
    after = st.call_index
    ck.sum().backward()
    assert torch.equal(ck, plain) and torch.equal(w.grad, g_plain) and st.call_index == after == 2


@pytest.mark.parametrize("T,Hq,Hkv,D,cu,causal", [
    (256, 2, 2, 64, [0, 256], True),
    (384, 4, 2, 64, [0, 100, 384], True),
    (320, 2, 1, 128, [0, 320], True),
    (256, 2, 2, 128, [0, 256], False),
])
def test_flash_attention_dropout(T, Hq, Hkv, D, cu, causal):
    """Attention dropout inside the kernels against the dense expression with the kernels' own mask (read back by
    `attention_dropout_mask`): forward, and the three gradients of the backward kernels, which rebuild the mask."""
    from scaling_b200.ops.attention import attention_reference, flash_attention
    from scaling_b200.ops.attention_kernel import attention_dropout_mask

    torch.manual_seed(21)
    p = 0.2
    st = _rng_state(77)
    q = torch.randn(T, Hq, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(T, Hkv, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(T, Hkv, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    cu_t = torch.tensor(cu, device=DEV, dtype=torch.int32)
    scale = D ** -0.5
    out = flash_attention(q, k, v, cu_t, None, causal=causal, scale=scale, dropout_p=p, rng_state=st)  # call 0
    do = torch.randn_like(out)
    out.backward(do)
    K.check_status()
    p_eff = round(p * 256) / 256
    raw = attention_dropout_mask(T, Hq, p, st, 0)
    mask = (raw > 0).float() / (1 - p_eff)
    assert abs((raw > 0).float().mean().item() - (1 - p_eff)) < 0.01
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = attention_reference(qr, kr, vr, cu_t, None, causal, scale, None, dropout_mask=mask)
    ref.backward(do.float())
    assert _rel(out, ref) < 2e-2, _rel(out, ref)
    assert _rel(q.grad, qr.grad) < 3e-2, _rel(q.grad, qr.grad)
    assert _rel(k.grad, kr.grad) < 3e-2, _rel(k.grad, kr.grad)
    assert _rel(v.grad, vr.grad) < 3e-2, _rel(v.grad, vr.grad)
    # without dropout the result differs, with the same call index again it is reproduced bit for bit
    st.call_index = 0
    q2, k2, v2 = (t.detach().clone().requires_grad_() for t in (q, k, v))
    out2 = flash_attention(q2, k2, v2, cu_t, None, causal=causal, scale=scale, dropout_p=p, rng_state=st)
    out2.backward(do)
    assert torch.equal(out, out2) and torch.equal(q.grad, q2.grad) and torch.equal(k.grad, k2.grad)
    assert _rel(out, flash_attention(q, k, v, cu_t, None, causal=causal, scale=scale)) > 0.05


# ---------------------------------------------------------------------------------------------- fp8 GEMM
@pytest.mark.parametrize("M,N,K_", [(256, 256, 128), (300, 520, 1040), (4096, 768, 3072), (128, 128, 16), (2000, 3072, 768)])
@pytest.mark.parametrize("fa,fb", [(torch.float8_e4m3fn, torch.float8_e4m3fn), (torch.float8_e5m2, torch.float8_e4m3fn),
                                   (torch.float8_e4m3fn, torch.float8_e5m2)])
def test_gemm_fp8(M, N, K_, fa, fb):
    """fp8 operands on the tensor cores against the fp32 product of the same (exactly representable) values."""
    torch.manual_seed(5)
    a = (torch.randn(M, K_, device=DEV) * 0.5).to(fa)
    b = (torch.randn(N, K_, device=DEV) * 0.5).to(fb)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    out32 = K.gemm_fp8(a, b, out_dtype=torch.float32)
    assert _rel(out32, ref) < 1e-5, _rel(out32, ref)
    row = ((out32 - ref).abs().amax(-1) / ref.abs().amax(-1).clamp_min(1e-3)).max().item()
    assert row < 1e-4, row
    out16 = K.gemm_fp8(a, b, bias=bias)
    assert out16.dtype == torch.bfloat16 and _rel(out16, ref + bias.float()) < 4e-3
    K.check_status()


def test_fp8_linear_on_the_tensor_cores_matches_the_widened_product():
    from scaling_b200.core.fp8.fp8_linear import fp8_linear

    torch.manual_seed(6)
    e4, e5 = torch.float8_e4m3fn, torch.float8_e5m2
    x = torch.randn(4, 96, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(512, 256, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_()
    y = fp8_linear(x, w, None, dtypes_forward=(e4, e4), dtypes_grad_input=(e5, e4), dtypes_grad_weight=(e4, e5))
    dy = torch.randn_like(y)
    y.backward(dy)
    xq, wq = x.detach().to(e4).float(), w.detach().to(e4).float()
    assert _rel(y.reshape(-1, 512), xq.reshape(-1, 256) @ wq.t()) < 4e-3
    dyq5, dyq5b = dy.to(e5).float().reshape(-1, 512), dy.to(e5).float().reshape(-1, 512)
    assert _rel(x.grad.reshape(-1, 256), dyq5 @ wq) < 4e-3
    assert _rel(w.grad, dyq5b.t() @ xq.reshape(-1, 256)) < 4e-3


@pytest.mark.parametrize("M,N", [(16384, 3072), (517, 264), (64, 8)])
def test_gelu_backward_with_bias_gradient_in_one_pass(M, N):
    torch.manual_seed(9)
    dy = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    x = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    grad = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    before = grad.clone()
    dx = K.gelu_backward_with_bias_grad(dy, x, grad, accumulate=True)
    ref = K.gelu_backward(dy, x)
    assert torch.equal(dx, ref)
    want = before.float() + ref.float().sum(0)
    assert _rel(grad, want) < 1e-2 and ((grad.float() - want).abs() < 0.02 * (1 + want.abs())).all()
    again = before.clone()
    K.gelu_backward_with_bias_grad(dy, x, again, accumulate=True)
    assert torch.equal(again, grad)  # fixed summation order


# ---------------------------------------------------------------------------------------------- edges and canaries
def _rows_close(got, ref, tol):
    """Largest absolute error of every row relative to that row's largest reference value: a wrong tile edge, a
    dropped row or two swapped columns show up here even when the norm over the whole tensor hides them."""
    got, ref = got.float(), ref.float()
    err = (got - ref).abs().amax(dim=-1) / ref.abs().amax(dim=-1).clamp_min(1e-3)
    return err.max().item() < tol, err.max().item()


@pytest.mark.parametrize("M,N,K_", [(1, 8, 8), (127, 8, 72), (128, 128, 8), (129, 136, 72), (255, 264, 64), (257, 520, 136),
                                    (384, 256, 8), (2312, 1288, 72)])
@pytest.mark.parametrize("mode", ["nt", "nn", "tn"])
def test_gemm_tile_edges_and_canaries(M, N, K_, mode):
    """One tile, one row / column more or less than a tile, reductions shorter than a k-block; the result goes into
    the middle of a buffer whose border must come back untouched."""
    torch.manual_seed(17)
    dt = torch.bfloat16
    if mode == "nt":
        a, b = torch.randn(M, K_, device=DEV, dtype=dt), torch.randn(N, K_, device=DEV, dtype=dt)
        ref, kw = a.float() @ b.float().t(), {}
    elif mode == "nn":
        a, b = torch.randn(M, K_, device=DEV, dtype=dt), torch.randn(K_, N, device=DEV, dtype=dt)
        ref, kw = a.float() @ b.float(), {"b_mn": True}
    else:
        if M % 8:  # a transposed A operand needs rows of a multiple of 16 bytes
            pytest.skip("M is the leading dimension of the transposed operand")
        a, b = torch.randn(K_, M, device=DEV, dtype=dt), torch.randn(K_, N, device=DEV, dtype=dt)
        ref, kw = a.float().t() @ b.float(), {"a_mn": True, "b_mn": True}
    sentinel = -1234.0
    buf = torch.full((M + 2, N + 16), sentinel, device=DEV, dtype=dt)
    out = buf[1:M + 1, 8:N + 8]
    K.gemm(a, b, out=out, **kw)
    K.check_status()
    ok, worst = _rows_close(out, ref, 2e-2)
    assert ok, worst
    border = buf.clone()
    border[1:M + 1, 8:N + 8] = sentinel
    assert (border == sentinel).all(), "the kernel wrote outside its output"
    K.gemm(a, b, out=out, accumulate=True, **kw)  # the accumulating form adds into memory through the same boxes
    K.check_status()
    ok, worst = _rows_close(out, 2 * ref, 3e-2)
    assert ok, worst
    border = buf.clone()
    border[1:M + 1, 8:N + 8] = sentinel
    assert (border == sentinel).all(), "the accumulating kernel wrote outside its output"


@pytest.mark.parametrize("T", [1, 127, 128, 129, 257])
@pytest.mark.parametrize("D", [64, 128])
def test_flash_attention_tile_edges(T, D):
    """Sequences of one token, one less, exactly and one more than a tile, alone and split into single-token and
    odd-length documents; every row is checked on its own."""
    from scaling_b200.ops.attention import attention_reference, flash_attention

    torch.manual_seed(23)
    cuts = sorted({0, T} | {c for c in (1, 2, T // 2, T - 1) if 0 < c < T})
    for cu in ([0, T], cuts):
        q = torch.randn(T, 2, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        k = torch.randn(T, 1, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        v = torch.randn(T, 1, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        cu_t = torch.tensor(cu, device=DEV, dtype=torch.int32)
        out = flash_attention(q, k, v, cu_t, None, causal=True, scale=D ** -0.5)
        do = torch.randn_like(out)
        out.backward(do)
        K.check_status()
        qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
        ref = attention_reference(qr, kr, vr, cu_t, None, True, D ** -0.5)
        ref.backward(do.float())
        for got, want, tol in ((out, ref, 3e-2), (q.grad, qr.grad, 5e-2), (k.grad, kr.grad, 5e-2), (v.grad, vr.grad, 5e-2)):
            ok, worst = _rows_close(got.reshape(T, -1), want.reshape(T, -1), tol)
            assert ok, (cu, worst)


@pytest.mark.parametrize("D", [32, 80, 96])
def test_flash_attention_head_sizes_between_the_native_ones(D):
    """Head sizes other than 64 and 128 run on the same kernels, padded with zero columns."""
    from scaling_b200.ops.attention import attention_reference, flash_attention

    torch.manual_seed(31)
    T = 384
    cu = torch.tensor([0, 100, 384], device=DEV, dtype=torch.int32)
    q = torch.randn(T, 4, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(T, 2, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(T, 2, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    out = flash_attention(q, k, v, cu, None, causal=True)
    assert out.shape == q.shape
    do = torch.randn_like(out)
    out.backward(do)
    K.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = attention_reference(qr, kr, vr, cu, None, True, D ** -0.5)
    ref.backward(do.float())
    for got, want, tol in ((out, ref, 3e-2), (q.grad, qr.grad, 5e-2), (k.grad, kr.grad, 5e-2), (v.grad, vr.grad, 5e-2)):
        ok, worst = _rows_close(got.reshape(T, -1), want.reshape(T, -1), tol)
        assert ok, (D, worst)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal,window", [(True, None), (True, 100), (False, None), (False, 37)])
def test_attention_of_few_queries_against_a_long_cache(D, causal, window):
    """Queries shorter than the keys of their document (decoding with a KV cache): the streaming kernel against the
    dense fp32 expression, with a document whose query sees a single key and one with as many queries as keys."""
    from scaling_b200.ops.attention import attention_reference, flash_attention

    torch.manual_seed(41)
    cu_q = torch.tensor([0, 1, 4, 5, 37], device=DEV, dtype=torch.int32)
    cu_k = torch.tensor([0, 700, 1500, 1501, 1533], device=DEV, dtype=torch.int32)
    tq, tk = 37, 1533
    q = torch.randn(tq, 8, D, device=DEV, dtype=torch.bfloat16)
    cache = torch.randn(tk, 2, 2, D, device=DEV, dtype=torch.bfloat16)  # k and v interleaved: strided rows
    k, v = cache[:, 0], cache[:, 1]
    with torch.no_grad():
        out = flash_attention(q, k, v, cu_q, cu_k, causal=causal, window=window)
    K.check_status()
    ref = attention_reference(q.float(), k.float(), v.float(), cu_q, cu_k, causal, D ** -0.5, window)
    ok, worst = _rows_close(out.reshape(tq, -1), ref.reshape(tq, -1), 2e-2)
    assert ok, worst


def test_loss_overwrites_logits_only_when_their_producer_allows_it():
    """The gradient of the loss is written over the logits only if their producer marked them as read by nobody
    else; logits that the caller holds come back unchanged, with the same loss and gradient either way."""
    from scaling_b200.transformer.model.losses.cross_entropy import vocab_parallel_cross_entropy

    torch.manual_seed(3)
    n, v = 64, 512
    held = torch.randn(n, v, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    before = held.detach().clone()
    targets = torch.randint(0, v, (n,), device=DEV)
    weights = torch.ones(n, device=DEV)
    loss, _ = vocab_parallel_cross_entropy(held, targets, weights, None, False)
    loss.backward()
    assert torch.equal(held.detach(), before)  # a leaf the caller still reads
    ref = F.cross_entropy(before.float(), targets)
    assert abs(loss.item() - ref.item()) < 2e-2

    base = before.clone().requires_grad_()
    temporary = base * 1.0
    temporary._sb200_loss_may_overwrite = True
    loss2, _ = vocab_parallel_cross_entropy(temporary, targets, weights, None, False)
    loss2.backward()
    assert loss2.item() == loss.item()
    assert _rel(base.grad, held.grad) < 1e-3
    assert not torch.equal(temporary.detach(), before)  # its storage now holds the gradient


@pytest.mark.parametrize("D", [64, 128])
def test_flash_attention_in_fp16_keeps_fp16_precision(D):
    """Half-precision inputs run on half-precision tensor-core operands (P and dS are packed as halves), so the
    result is as close to the fp32 expression as an fp16 kernel's: within 1e-3 on unit-scale outputs, which the same
    inputs rounded to bf16 miss."""
    from scaling_b200.ops.attention import attention_reference, flash_attention

    torch.manual_seed(7)
    T = 512
    cu = torch.tensor([0, 200, 512], device=DEV, dtype=torch.int32)
    q = torch.randn(T, 4, D, device=DEV, dtype=torch.float16, requires_grad=True)
    k = torch.randn(T, 2, D, device=DEV, dtype=torch.float16, requires_grad=True)
    v = torch.randn(T, 2, D, device=DEV, dtype=torch.float16, requires_grad=True)
    out = flash_attention(q, k, v, cu, None, causal=True)
    assert out.dtype == torch.float16
    do = torch.randn_like(out)
    out.backward(do)
    K.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = attention_reference(qr, kr, vr, cu, None, True, D ** -0.5)
    ref.backward(do.float())
    assert (out.float() - ref).abs().max().item() < 2e-3
    for got, want in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        ok, worst = _rows_close(got.reshape(T, -1), want.reshape(T, -1), 1e-2)
        assert ok, worst
    as_bf16 = flash_attention(q.detach().bfloat16(), k.detach().bfloat16(), v.detach().bfloat16(), cu, None, causal=True)
    assert (as_bf16.float() - ref).abs().max().item() > (out.float() - ref).abs().max().item()
