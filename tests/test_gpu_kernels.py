"""Numerics of the non-GEMM sm_100a kernels against the fp32 reference path of the same ops (CPU tensors)."""
import math

import pytest
import torch

from rustral_b200 import ops
from rustral_b200.ops import norm as norm_ops
from rustral_b200.ops import attention as attn_ops

pytestmark = pytest.mark.gpu


def _bf(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16)


def _close(out, ref, tol=2e-2, what=""):
    out, ref = out.float().cpu(), ref.float().cpu()
    err = (out - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err <= tol * scale, f"{what}: max abs err {err:.4g} vs scale {scale:.4g}"


@pytest.mark.parametrize("rows,n", [(7, 64), (33, 768), (128, 1000), (5, 2048), (9, 4096), (3, 8192), (1024, 768)])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_fwd_bwd(rows, n, rms, cuda_status):
    x, g, b, dy, dres = _bf((rows, n), 1), _bf((n,), 2) + 1, _bf((n,), 3), _bf((rows, n), 4), _bf((rows, n), 5)
    beta = None if rms else b
    yc, mc, rc = norm_ops.norm_forward(x, g, beta, 1e-5, rms)
    yg, mg, rg = norm_ops.norm_forward(x.cuda(), g.cuda(), None if rms else b.cuda(), 1e-5, rms)
    _close(yg, yc, what="y")
    _close(rg, rc, tol=1e-3, what="rstd")
    dxc, dgc, dbc = norm_ops.norm_backward(dy, x, g, mc, rc, rms, dres=dres)
    dxg, dgg, dbg = norm_ops.norm_backward(dy.cuda(), x.cuda(), g.cuda(), mg, rg, rms, dres=dres.cuda())
    _close(dxg, dxc, what="dx")
    _close(dgg, dgc, tol=1e-2, what="dgamma")
    if not rms:
        _close(dbg, dbc, tol=1e-2, what="dbeta")
    # run-twice determinism of the parameter gradients
    _, dgg2, _ = norm_ops.norm_backward(dy.cuda(), x.cuda(), g.cuda(), mg, rg, rms, dres=dres.cuda())
    assert torch.equal(dgg, dgg2)


@pytest.mark.parametrize("rows,n_valid,n_pad", [(5, 10, 16), (64, 1000, 1000), (16, 50257, 50304), (3, 37, 37)])
def test_cross_entropy(rows, n_valid, n_pad, cuda_status):
    logits = _bf((rows, n_pad), 1, 2.0)
    t = torch.randint(0, n_valid, (rows,), generator=torch.Generator().manual_seed(2))
    t[0] = -100
    lc, lsec, gc = ops.cross_entropy_fwd_bwd(logits, t, n_valid, 0.25)
    lg, lseg, gg = ops.cross_entropy_fwd_bwd(logits.cuda(), t.cuda(), n_valid, 0.25)
    _close(lg, lc, tol=1e-3, what="loss")
    _close(lseg, lsec, tol=1e-3, what="lse")
    _close(gg, gc, tol=2e-2, what="dlogits")
    assert gg[:, n_valid:].abs().sum().item() == 0
    # in-place variant
    l2 = logits.cuda().clone()
    loss_inplace, lse_inplace, _ = ops.cross_entropy_fwd_bwd(l2, t.cuda(), n_valid, 0.25, dlogits=l2)
    assert torch.equal(l2, gg)
    # the loss of the in-place call is the out-of-place loss bit for bit: the target logit is read before any
    # thread of the row's block overwrites it with a gradient
    assert torch.equal(loss_inplace, lg) and torch.equal(lse_inplace, lseg)


def test_cross_entropy_in_place_loss_is_exact_on_many_wide_rows(cuda_status):
    """Wide rows (several chunks per thread) and targets near the start of the row, where the first gradient stores
    land: the per-row loss of the in-place form equals the out-of-place form exactly, on every repetition."""
    rows, n = 512, 50304
    g = torch.Generator().manual_seed(11)
    logits = (torch.randn(rows, n, generator=g) * 3).to(torch.bfloat16).cuda()
    t = torch.randint(0, 64, (rows,), generator=g).cuda()
    want, _, _ = ops.cross_entropy_fwd_bwd(logits, t, 50257, 1.0)
    for _ in range(3):
        l2 = logits.clone()
        got, _, _ = ops.cross_entropy_fwd_bwd(l2, t, 50257, 1.0, dlogits=l2)
        assert torch.equal(got, want)


def test_softmax_rows(cuda_status):
    x = torch.randn(17, 333)
    for fn in (ops.softmax, ops.log_softmax):
        xc = x.clone().requires_grad_()
        xg = x.cuda().requires_grad_()
        yc, yg = fn(xc), fn(xg)
        _close(yg, yc, tol=1e-5, what=fn.__name__)
        w = torch.randn(17, 333)
        (yc * w).sum().backward()
        (yg * w.cuda()).sum().backward()
        _close(xg.grad, xc.grad, tol=1e-4, what=fn.__name__ + " grad")


@pytest.mark.parametrize("B,S,H,Hk,D,causal", [(2, 128, 4, 4, 64, True), (1, 200, 3, 3, 64, True),
                                               (2, 96, 4, 2, 64, False), (1, 256, 4, 1, 128, True),
                                               (1, 77, 2, 2, 128, False), (2, 1024, 2, 2, 64, True)])
def test_flash_attention_fwd_bwd(B, S, H, Hk, D, causal, cuda_status):
    q, k, v = _bf((B, S, H, D), 1), _bf((B, S, Hk, D), 2), _bf((B, S, Hk, D), 3)
    do = _bf((B, S, H, D), 4)
    qc, kc, vc = (t.float().requires_grad_() for t in (q, k, v))
    oc = attn_ops.attention_reference(qc, kc, vc, causal)
    (oc * do.float()).sum().backward()
    qg, kg, vg = (t.cuda().requires_grad_() for t in (q, k, v))
    og = ops.flash_attention(qg, kg, vg, causal)
    (og.float() * do.cuda().float()).sum().backward()
    _close(og, oc, what="o")
    _close(qg.grad, qc.grad, tol=3e-2, what="dq")
    _close(kg.grad, kc.grad, tol=3e-2, what="dk")
    _close(vg.grad, vc.grad, tol=3e-2, what="dv")


def test_flash_attention_packed_qkv(cuda_status):
    # q, k, v as strided views of one [B, S, 3*H*D] projection output, gradients written packed
    B, S, H, D = 2, 192, 3, 64
    qkv = _bf((B, S, 3 * H * D), 7).cuda()
    q, k, v = (qkv[:, :, i * H * D:(i + 1) * H * D].view(B, S, H, D) for i in range(3))
    o, lse = attn_ops.attention_forward(q, k, v, True, 1 / math.sqrt(D))
    ref = attn_ops.attention_reference(q.cpu(), k.cpu(), v.cpu(), True)
    _close(o, ref, what="o packed")
    do = _bf((B, S, H, D), 8).cuda()
    dqkv = torch.zeros_like(qkv)
    dq, dk, dv = (dqkv[:, :, i * H * D:(i + 1) * H * D].view(B, S, H, D) for i in range(3))
    attn_ops.attention_backward(do, q, k, v, o, lse, True, 1 / math.sqrt(D), dq=dq, dk=dk, dv=dv)
    qc, kc, vc = (t.cpu().float().requires_grad_() for t in (q, k, v))
    (attn_ops.attention_reference(qc, kc, vc, True) * do.cpu().float()).sum().backward()
    _close(dq, qc.grad, tol=3e-2, what="dq packed")
    _close(dk, kc.grad, tol=3e-2, what="dk packed")
    _close(dv, vc.grad, tol=3e-2, what="dv packed")


def test_embedding_fwd_bwd(cuda_status):
    V, Dm, B, S = 1000, 64, 4, 32
    wte, wpe = _bf((V, Dm), 1), _bf((S, Dm), 2)
    ids = torch.randint(0, 50, (B * S,), generator=torch.Generator().manual_seed(3))   # many duplicates
    yc = ops.embedding_forward(ids, wte, wpe, S)
    yg = ops.embedding_forward(ids.cuda(), wte.cuda(), wpe.cuda(), S)
    _close(yg, yc, tol=1e-2)
    dy = _bf((B * S, Dm), 4)
    dwc, dpc = torch.zeros(V, Dm), torch.zeros(S, Dm)
    ops.embedding_backward(ids, dy, dwc, dpc, S)
    dwg, dpg = torch.zeros(V, Dm, device="cuda"), torch.zeros(S, Dm, device="cuda")
    ops.embedding_backward(ids.cuda(), dy.cuda(), dwg, dpg, S)
    _close(dwg, dwc, tol=1e-4, what="dwte")
    _close(dpg, dpc, tol=1e-4, what="dwpe")
    dwg2 = torch.zeros(V, Dm, device="cuda")
    ops.embedding_backward(ids.cuda(), dy.cuda(), dwg2, None, S)
    assert torch.equal(dwg, dwg2)


def test_adam_and_sgd(cuda_status):
    n = 10007
    torch.manual_seed(0)
    p, g = torch.randn(n), torch.randn(n)
    for decoupled in (True, False):
        pc, mc, vc = p.clone(), torch.zeros(n), torch.zeros(n)
        pg, mg, vg = p.cuda(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
        lowp = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        for step in (1, 2, 3):
            kw = dict(lr=1e-2, weight_decay=0.1, step=step, decoupled=decoupled, grad_scale=0.5)
            ops.adam_step(pc, mc, vc, g, **kw)
            ops.adam_step(pg, mg, vg, g.cuda(), p_lowp=lowp, **kw)
        _close(pg, pc, tol=1e-5, what="adam p")
        _close(lowp, pc, tol=1e-2, what="adam bf16 copy")
    # clipping and overflow skip decided on the device
    pg = p.cuda()
    gn = ops.optim.sqrt_scalar(ops.sumsq(g.cuda()))
    _close(gn, g.norm(), tol=1e-5)
    inf = torch.ones((), dtype=torch.int32, device="cuda")
    before = pg.clone()
    ops.adam_step(pg, torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda"), g.cuda(), lr=1e-2, step=1,
                  found_inf=inf)
    assert torch.equal(pg, before)
    pc2, pg2 = p.clone(), p.cuda()
    ops.sgd_step(pc2, g, lr=0.1, momentum=0.9, weight_decay=0.01, mom=torch.zeros(n))
    ops.sgd_step(pg2, g.cuda(), lr=0.1, momentum=0.9, weight_decay=0.01, mom=torch.zeros(n, device="cuda"))
    _close(pg2, pc2, tol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_elementwise_family(dtype, cuda_status):
    torch.manual_seed(1)
    a = (torch.rand(37, 53) + 0.5).to(dtype)
    b = (torch.rand(37, 53) + 0.5).to(dtype)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for op in ("add", "mul", "sub", "div", "maximum"):
        _close(ops.binary(op, a.cuda(), b.cuda()), ops.binary(op, a, b), tol, op)
    for op in ("relu", "sigmoid", "tanh", "exp", "log", "sqrt", "neg", "gelu", "silu"):
        _close(ops.unary(op, (a - 1).cuda() if op in ("relu", "gelu", "silu", "tanh") else a.cuda()),
               ops.unary(op, (a - 1) if op in ("relu", "gelu", "silu", "tanh") else a), tol, op)
    for op in ("add_scalar", "mul_scalar", "gt_scalar", "fill"):
        _close(ops.scalar_op(op, a.cuda(), 0.75), ops.scalar_op(op, a, 0.75), tol, op)
    for op in ("relu", "gelu", "silu", "sigmoid", "tanh"):
        _close(ops.unary_bwd(op, (a - 1).cuda(), b.cuda()), ops.unary_bwd(op, a - 1, b), tol, "d" + op)
    _close(ops.add_row_vector(a.cuda(), b[0].cuda()), ops.add_row_vector(a, b[0]), tol)
    _close(ops.sum_dim0(a.cuda()), ops.sum_dim0(a), 1e-4)
    _close(ops.sum_all(a.cuda()), ops.sum_all(a), 1e-4)
    _close(ops.transpose2d(a.cuda()), a.t(), 0)
    idx = torch.tensor([3, 0, 36, 3])
    _close(ops.gather_rows(a.cuda(), idx.cuda()), a[idx], 0)
    out = torch.zeros(40, 53, dtype=dtype, device="cuda")
    ops.scatter_rows(a[:3].cuda(), torch.tensor([5, 7, 9]).cuda(), out)
    assert torch.equal(out[[5, 7, 9]].cpu(), a[:3])
    _close(ops.broadcast_to(a[:1].cuda(), 6, 53), a[:1].expand(6, 53), 0)
    _close(ops.apply_mask(a.cuda(), (b > 1).to(dtype).cuda(), -1e9), torch.where(b > 1, a, torch.full_like(a, -1e9)), 0)
    assert torch.equal(ops.argmax_rows(a.cuda()).cpu(), a.float().argmax(-1))
    big = torch.randn(3000, 40).to(dtype)
    _close(ops.sum_dim0(big.cuda()), big.float().sum(0), 1e-3)


def test_dropout(cuda_status):
    x = torch.ones(100000)
    y, mask = ops.dropout(x.cuda(), 0.3, True, seed=5, return_mask=True)
    keep = mask.float().mean().item()
    assert abs(keep - 0.7) < 0.01
    assert torch.allclose(y[mask.bool()], torch.full_like(y[mask.bool()], 1 / 0.7))
    y2 = ops.dropout(x.cuda(), 0.3, True, seed=5)
    assert torch.equal(y, y2)
    # PCG-hash generator: identical keep mask on host and device
    yp, mp = ops.dropout(x.cuda(), 0.25, True, seed=123, rng="pcg", return_mask=True)
    from rustral_b200.ops.elementwise import dropout_mask_reference
    assert torch.equal(mp.bool().cpu(), dropout_mask_reference(100000, 0.25, 123))


@pytest.mark.parametrize("H,Hk,D", [(4, 4, 64), (8, 2, 128), (32, 8, 128), (12, 1, 64), (40, 2, 64)])
def test_paged_attention_and_kv_append(H, Hk, D, cuda_status):
    from rustral_b200.ops import paged
    torch.manual_seed(0)
    nb, bs, B = 64, 16, 5
    ctx = torch.tensor([1, 16, 17, 100, 333], dtype=torch.int32)
    kc = torch.zeros(nb, bs, Hk, D, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    perm = torch.randperm(nb)
    max_blocks = 21
    bt = torch.zeros(B, max_blocks, dtype=torch.int32)
    used = 0
    for b in range(B):
        n = (int(ctx[b]) + bs - 1) // bs
        bt[b, :n] = perm[used:used + n].to(torch.int32)
        used += n
    # fill the caches through kv_append (CPU reference and CUDA kernel) from random packed K/V rows
    kcg, vcg = kc.cuda(), vc.cuda()
    for b in range(B):
        n = int(ctx[b])
        kv = _bf((n, 2 * Hk * D), 10 + b)
        toks = torch.arange(n)
        slots = bt[b, toks // bs].long() * bs + toks % bs
        paged.kv_append(kv[:, :Hk * D], kv[:, Hk * D:], kc, vc, slots)
        kvg = kv.cuda()
        paged.kv_append(kvg[:, :Hk * D], kvg[:, Hk * D:], kcg, vcg, slots.cuda())
    assert torch.equal(kcg.cpu(), kc) and torch.equal(vcg.cpu(), vc)
    q = _bf((B, H * D), 3)
    ref = paged.paged_attention_decode(q, kc, vc, bt, ctx)
    out = paged.paged_attention_decode(q.cuda(), kcg, vcg, bt.cuda(), ctx.cuda())
    _close(out, ref, what="paged decode")


def test_rope_and_swiglu(cuda_status):
    from rustral_b200.ops import rotary
    B, S, H, D = 2, 48, 6, 64
    x = _bf((B * S, H * D + 32), 1)
    for inverse in (False, True):
        xc, xg = x.clone(), x.cuda().clone()
        rotary.rope_(xc, H, D, S, theta=500000.0, inverse=inverse)
        rotary.rope_(xg, H, D, S, theta=500000.0, inverse=inverse)
        _close(xg, xc, what="rope")
        assert torch.equal(xg[:, H * D:].cpu(), x[:, H * D:])        # columns past the heads are untouched
    pos = torch.randint(0, 4000, (B * S,))
    xc, xg = x.clone(), x.cuda().clone()
    rotary.rope_(xc, H, D, positions=pos, theta=10000.0)
    rotary.rope_(xg, H, D, positions=pos.cuda(), theta=10000.0)
    _close(xg, xc, what="rope positions")
    gu, dh = _bf((70, 256), 2), _bf((70, 128), 3)
    _close(rotary.swiglu_forward(gu.cuda()), rotary.swiglu_forward(gu), what="swiglu")
    _close(rotary.swiglu_backward(dh.cuda(), gu.cuda()), rotary.swiglu_backward(dh, gu), what="swiglu bwd")


@pytest.mark.parametrize("kind", ["swiglu", "gelu"])
def test_moe_layer_fwd_bwd(kind, cuda_status):
    from rustral_b200.ops import moe
    torch.manual_seed(0)
    T, d, F, E, k = 700, 128, 192, 8, 2
    f1 = 2 * F if kind == "swiglu" else F
    x, rw = _bf((T, d), 1), _bf((E, d), 2, 0.5)
    w1, w2 = _bf((E, f1, d), 3, 0.1), _bf((E, d, F), 4, 0.1)
    res = []
    for dev in ("cpu", "cuda"):
        ts = [t.detach().clone().to(dev).requires_grad_() for t in (x, rw, w1, w2)]
        y, aux = moe.moe_mlp(*ts, k, kind)
        (y.float().sum() + 0.5 * aux).backward()
        res.append((y, aux, *[t.grad for t in ts]))
    names = ["y", "aux", "dx", "drouter", "dw1", "dw2"]
    for n, a, b in zip(names, res[1], res[0]):
        _close(a, b, tol=4e-2, what=f"moe {kind} {n}")


def test_moe_plan_is_deterministic_and_padded(cuda_status):
    from rustral_b200.ops import moe
    g = torch.Generator().manual_seed(5)
    idx = torch.stack([torch.randperm(8, generator=g)[:2] for _ in range(1000)]).to(torch.int32)
    pc, pg = moe.plan(idx, 8), moe.plan(idx.cuda(), 8)
    for a in ("counts", "offsets", "slot_pos", "row_slot", "tile_expert", "num_tiles"):
        assert torch.equal(getattr(pg, a).cpu(), getattr(pc, a)), a
    assert all(int(o) % 128 == 0 for o in pc.offsets)


@pytest.mark.parametrize("B,Sq,Sk,H,Hk,D,causal", [(2, 128, 128, 4, 4, 64, True), (1, 200, 200, 3, 3, 64, True),
                                                  (2, 96, 96, 4, 2, 64, False), (1, 256, 256, 4, 1, 128, True),
                                                  (1, 77, 77, 2, 2, 128, False), (2, 1024, 1024, 2, 2, 64, True),
                                                  (1, 64, 320, 2, 2, 64, True), (1, 384, 384, 2, 2, 128, True)])
def test_flash_attention_forward_tcgen05(B, Sq, Sk, H, Hk, D, causal, cuda_status):
    q, k, v = _bf((B, Sq, H, D), 1), _bf((B, Sk, Hk, D), 2), _bf((B, Sk, Hk, D), 3)
    ref = attn_ops.attention_reference(q, k, v, causal)
    scale = 1 / math.sqrt(D)
    o_tc, lse_tc = attn_ops.attention_forward(q.cuda(), k.cuda(), v.cuda(), causal, scale, impl="tc")
    o_mma, lse_mma = attn_ops.attention_forward(q.cuda(), k.cuda(), v.cuda(), causal, scale, impl="mma")
    _close(o_tc, ref, what="tc o")
    _close(lse_tc, lse_mma, tol=1e-3, what="tc lse")
    # packed QKV views (strided heads) go through the 4-D tensor maps unchanged
    if Sq == Sk and H == Hk:
        qkv = torch.cat([q.reshape(B, Sq, -1), k.reshape(B, Sq, -1), v.reshape(B, Sq, -1)], -1).cuda()
        qs, ks, vs = (qkv[:, :, i * H * D:(i + 1) * H * D].view(B, Sq, H, D) for i in range(3))
        o2, _ = attn_ops.attention_forward(qs, ks, vs, causal, scale, impl="tc")
        assert torch.equal(o2, o_tc)


@pytest.mark.parametrize("B,Sq,Sk,H,Hk,D,causal", [(1, 128, 128, 1, 1, 64, True), (2, 128, 128, 4, 4, 64, True), (1, 200, 200, 3, 3, 64, True),
                                                  (2, 96, 96, 4, 2, 64, False), (1, 256, 256, 4, 1, 128, True),
                                                  (1, 77, 77, 2, 2, 128, False), (2, 1024, 1024, 2, 2, 64, True),
                                                  (1, 64, 320, 2, 2, 64, True), (1, 384, 384, 2, 2, 128, True),
                                                  (1, 640, 640, 2, 2, 64, True), (1, 512, 512, 2, 1, 128, False)])
@pytest.mark.parametrize("poly", [0, 4])
def test_flash_attention_forward_two_tile_kernel(B, Sq, Sk, H, Hk, D, causal, poly, cuda_status):
    """The ping-pong kernel (P in TMEM, output accumulated in TMEM with lazy rescaling) against the fp32 reference and
    the log-sum-exp of the mma.sync kernel; odd sizes exercise a missing second query tile and partial tiles."""
    q, k, v = _bf((B, Sq, H, D), 1), _bf((B, Sk, Hk, D), 2), _bf((B, Sk, Hk, D), 3)
    ref = attn_ops.attention_reference(q, k, v, causal)
    scale = 1 / math.sqrt(D)
    o2, lse2 = attn_ops.attention_forward(q.cuda(), k.cuda(), v.cuda(), causal, scale, impl=f"tc2:{poly}")
    _, lse_mma = attn_ops.attention_forward(q.cuda(), k.cuda(), v.cuda(), causal, scale, impl="mma")
    _close(o2, ref, what="tc2 o")
    _close(lse2, lse_mma, tol=1e-3, what="tc2 lse")
    o3, lse3 = attn_ops.attention_forward(q.cuda(), k.cuda(), v.cuda(), causal, scale, impl=f"tc2:{poly}")
    assert torch.equal(o2, o3) and torch.equal(lse2, lse3)          # run-twice determinism
    if Sq == Sk and H == Hk:                                        # packed QKV views through the 4-D tensor maps
        qkv = torch.cat([q.reshape(B, Sq, -1), k.reshape(B, Sq, -1), v.reshape(B, Sq, -1)], -1).cuda()
        qs, ks, vs = (qkv[:, :, i * H * D:(i + 1) * H * D].view(B, Sq, H, D) for i in range(3))
        o4, _ = attn_ops.attention_forward(qs, ks, vs, causal, scale, impl=f"tc2:{poly}")
        assert torch.equal(o4, o2)


def test_flash_attention_two_tile_kernel_rescales_sharp_rows(cuda_status):
    """Scores with a large spread move the running maximum by more than the lazy-rescale threshold again and again:
    the accumulator in TMEM is rescaled in place and the result still matches the reference."""
    B, S, H, D = 1, 1024, 2, 64
    q, k, v = _bf((B, S, H, D), 1, 4.0), _bf((B, S, H, D), 2, 4.0), _bf((B, S, H, D), 3)
    ref = attn_ops.attention_reference(q, k, v, True)
    o, _ = attn_ops.attention_forward(q.cuda(), k.cuda(), v.cuda(), True, 1 / math.sqrt(D), impl="tc2:0")
    _close(o, ref, tol=2e-2, what="sharp rows")


@pytest.mark.parametrize("B,Sq,Sk,H,Hk,D,causal", [
    (2, 256, 256, 4, 4, 64, True), (1, 384, 384, 2, 2, 128, True), (2, 200, 200, 4, 2, 64, True),
    (1, 128, 320, 4, 1, 64, True), (2, 160, 288, 2, 2, 128, False), (1, 512, 512, 3, 3, 64, False),
    (1, 1024, 1024, 2, 2, 64, True), (1, 640, 640, 4, 2, 128, True),
])
@pytest.mark.parametrize("impl", ["tc", "tc2"])
def test_flash_attention_backward_tcgen05(B, Sq, Sk, H, Hk, D, causal, impl, cuda_status):
    q, k, v = _bf((B, Sq, H, D), 1), _bf((B, Sk, Hk, D), 2), _bf((B, Sk, Hk, D), 3)
    do = _bf((B, Sq, H, D), 4)
    qc, kc, vc = (t.float().requires_grad_() for t in (q, k, v))
    (attn_ops.attention_reference(qc, kc, vc, causal) * do.float()).sum().backward()
    scale = 1 / math.sqrt(D)
    qg, kg, vg, dog = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    o, lse = attn_ops.attention_forward(qg, kg, vg, causal, scale, impl="tc")
    dq, dk, dv = attn_ops.attention_backward(dog, qg, kg, vg, o, lse, causal, scale, impl=impl)
    _close(dq, qc.grad, tol=3e-2, what="tc dq")
    _close(dk, kc.grad, tol=3e-2, what="tc dk")
    _close(dv, vc.grad, tol=3e-2, what="tc dv")
    # bit-reproducible: no atomics anywhere in the backward pass
    dq2, dk2, dv2 = attn_ops.attention_backward(dog, qg, kg, vg, o, lse, causal, scale, impl=impl)
    assert torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)
    # the mma.sync path gives the same gradients within rounding
    dq3, dk3, dv3 = attn_ops.attention_backward(dog, qg, kg, vg, o, lse, causal, scale, impl="mma")
    _close(dq, dq3, tol=3e-2, what="tc vs mma dq")
    _close(dk, dk3, tol=3e-2, what="tc vs mma dk")
    _close(dv, dv3, tol=3e-2, what="tc vs mma dv")


@pytest.mark.parametrize("B,S,H,Hk,D,causal,lens", [
    (3, 256, 2, 2, 64, False, [256, 100, 1]), (2, 384, 4, 2, 128, True, [384, 130]), (2, 200, 2, 2, 64, False, [200, 0]),
])
def test_flash_attention_key_padding_lengths(B, S, H, Hk, D, causal, lens, cuda_status):
    """Per-sequence key counts (a key-padding mask): keys at or past a sequence's length get no weight and no gradient;
    a sequence of length 0 yields zero output and zero gradients."""
    q, k, v, do = _bf((B, S, H, D), 1), _bf((B, S, Hk, D), 2), _bf((B, S, Hk, D), 3), _bf((B, S, H, D), 4)
    L = torch.tensor(lens, dtype=torch.int32)
    qc, kc, vc = (t.float().requires_grad_() for t in (q, k, v))
    ref = attn_ops.attention_reference(qc, kc, vc, causal, None, L)
    (ref * do.float()).sum().backward()
    scale = 1 / math.sqrt(D)
    qg, kg, vg, dog, Lg = q.cuda(), k.cuda(), v.cuda(), do.cuda(), L.cuda()
    o, lse = attn_ops.attention_forward(qg, kg, vg, causal, scale, kv_lens=Lg)
    _close(o, ref, tol=2e-2, what="kv_lens o")
    dq, dk, dv = attn_ops.attention_backward(dog, qg, kg, vg, o, lse, causal, scale, kv_lens=Lg)
    _close(dq, qc.grad, tol=3e-2, what="kv_lens dq")
    _close(dk, kc.grad, tol=3e-2, what="kv_lens dk")
    _close(dv, vc.grad, tol=3e-2, what="kv_lens dv")
    for b, n in enumerate(lens):
        assert not dk[b, n:].any() and not dv[b, n:].any(), "padded keys received a gradient"


def test_bounded_wait_expires_and_reports_without_losing_the_context():
    """A flag that nothing ever sets: the wait kernel gives up after its limit, records the timeout in the device
    status word, and the context keeps working (this is what a rank sees when a peer never signals)."""
    import time
    from rustral_b200 import _native as N
    from rustral_b200.parallel import symm  # noqa: F401  (declares rb_wait_all)
    lib = N.kernels()
    lib.rb_init()
    N.read_status(clear=True)
    pad = torch.zeros(1024, dtype=torch.int32, device="cuda")          # a private "signal pad": nobody writes to it
    t0 = time.perf_counter()
    N.check(lib.rb_wait_all(pad.data_ptr(), 2, 0, 1, 50, N.stream_ptr()), "rb_wait_all")     # 50 ms limit
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    bits, where = N.read_status(clear=True)
    assert bits != 0 and where == 100, (bits, where)                 # timeout bit set, raised by the channel-0 wait
    assert 0.03 < waited < 2.0, waited
    with pytest.raises(N.NativeError):
        N.check(lib.rb_wait_all(pad.data_ptr(), 2, 0, 1, 20, N.stream_ptr()), "rb_wait_all")
        N.raise_on_status()
    # the context is intact: a GEMM runs and is correct, and the status word is clean again
    a, b = _bf((128, 64), 1).cuda(), _bf((64, 64), 2).cuda()
    out = ops.gemm(a, b)
    _close(out, a.float().cpu() @ b.float().cpu().t(), tol=2e-2, what="gemm after timeout")
    assert N.read_status(clear=True)[0] == 0
    # a flag that IS set lets the wait through at once
    pad[:2] = 1
    N.check(lib.rb_wait_all(pad.data_ptr(), 2, 0, 1, 50, N.stream_ptr()), "rb_wait_all")
    torch.cuda.synchronize()
    assert N.read_status(clear=True)[0] == 0


def test_autotuner_tunes_real_kernels_and_feeds_gemm(tmp_path, cuda_status):
    """The tuner times the tcgen05 GEMM's tile plans and both attention implementations with CUDA events, caches the
    winners, and the applied table changes nothing about the result of a GEMM it serves."""
    from rustral_b200.ops import matmul
    from rustral_b200.tune import (AutoTuner, ConfigCache, GemmKernel, GemmTuningTable, TunerConfig, tune_attention, tune_gemm)
    cfg = TunerConfig.fast()
    cfg.max_evals, cfg.max_tuning_time_s, cfg.min_improvement_pct = 6, 20.0, 0.0
    tuner = AutoTuner(cfg, ConfigCache(str(tmp_path / "tune.json"), cfg.device_id or torch.cuda.get_device_name(0)))
    r = tune_gemm(2048, 1536, 512, tuner)
    assert r.time_us > 0 and r.evaluated >= 1 and set(r.config) == {"block_n", "splits", "group_m"}
    again = tune_gemm(2048, 1536, 512, tuner)
    assert again.from_cache and again.config == r.config
    ra = tune_attention(2, 512, 4, 2, 64, tuner)
    assert ra.config["impl"] in (0, 1) and ra.time_us > 0
    a = _bf((2048, 512), 1).cuda()
    b = _bf((1536, 512), 2).cuda()
    ref = matmul.gemm(a, b)
    table = GemmTuningTable(tuner.cache, device_id=tuner.config.device_id)
    try:
        table.apply()
        out = matmul.gemm(a, b)
    finally:
        GemmTuningTable.remove()
    _close(out, ref, what="gemm under a tuned plan")
    assert table.hits + table.misses == 1


@pytest.mark.parametrize("N,C,H,W,O,k,stride,nopad", [(4, 1, 28, 28, 8, 3, 1, False), (2, 3, 33, 47, 13, 3, 2, False),
                                                       (1, 3, 64, 64, 16, 5, 1, True), (3, 2, 9, 7, 5, 1, 1, False)])
def test_direct_conv2d_matches_fp32_convolution(N, C, H, W, O, k, stride, nopad, cuda_status):
    """The direct kernel (inference path of Conv2d) against an fp32 PyTorch convolution, and against the im2col +
    GEMM path that the same layer takes when gradients are needed."""
    import torch.nn.functional as F
    from rustral_b200.core import B200Backend, ForwardCtx
    from rustral_b200.nn import Conv2d, Conv2dConfig
    be = B200Backend()
    conv = Conv2d.new(be, Conv2dConfig(O, k, k, stride=stride, no_padding=nopad, in_channels=C), seed=3)
    conv.bias.tensor.data.copy_(_bf((O,), 9).cuda())
    x = _bf((N, C, H, W), 4).cuda()
    y = conv(x, ForwardCtx.inference(be))
    pad = 0 if nopad else k // 2
    ref = F.conv2d(x.float(), conv.weight.tensor.float(), conv.bias.tensor.float(), stride=stride, padding=pad)
    assert y.shape == ref.shape and y.dtype == torch.bfloat16 and not y.requires_grad
    _close(y, ref, what="direct conv2d")
    y_train = conv(x, ForwardCtx.train(be))
    assert y_train.requires_grad
    _close(y_train, ref, what="im2col conv2d")


@pytest.mark.parametrize("T,B,I,H", [(12, 1, 128, 128), (7, 5, 40, 64)])
def test_lstm_inference_sequence_matches_fp32_recurrence(T, B, I, H, cuda_status):
    """The GPU inference path of LstmCell (one input-projection GEMM, then per step one GEMM + the fused gate kernel)
    against the recurrence evaluated in fp32 PyTorch, and against the generic per-step path."""
    from rustral_b200.core import B200Backend, ForwardCtx
    from rustral_b200.nn import LstmCell
    be = B200Backend()
    cell = LstmCell.new(be, I, H, seed=5)
    cell.b.tensor.data.copy_(_bf((4 * H,), 8, 0.1).cuda())
    xs = _bf((T, B, I), 6).cuda()
    outs, (h, c) = cell.forward_sequence(xs, ForwardCtx.inference(be))
    wx, wh, b = cell.wx.tensor.float().cpu(), cell.wh.tensor.float().cpu(), cell.b.tensor.float().cpu()
    hr, cr, ref = torch.zeros(B, H), torch.zeros(B, H), []
    for t in range(T):
        g = xs[t].float().cpu() @ wx.t() + hr @ wh.t() + b
        i, f, o, gg = torch.sigmoid(g[:, :H]), torch.sigmoid(g[:, H:2 * H]), torch.sigmoid(g[:, 2 * H:3 * H]), torch.tanh(g[:, 3 * H:])
        cr = f * cr + i * gg
        hr = o * torch.tanh(cr)
        ref.append(hr)
    ref = torch.stack(ref)
    assert outs.shape == (T, B, H) and not outs.requires_grad
    _close(outs, ref, tol=3e-2, what="lstm outputs")
    _close(c, cr, tol=3e-2, what="lstm cell state")
    assert torch.equal(h, outs[-1])
    slow, _ = super(LstmCell, cell).forward_sequence(xs, ForwardCtx.inference(be))
    _close(outs, slow, tol=3e-2, what="fast vs generic lstm path")
    # second call captures the sequence into a CUDA graph, the third and fourth replay it (new inputs, new initial state)
    outs2, (h2, c2) = cell.forward_sequence(xs, ForwardCtx.inference(be))
    outs3, (h3, c3) = cell.forward_sequence(xs, ForwardCtx.inference(be))
    assert torch.equal(outs2, outs) and torch.equal(outs3, outs) and torch.equal(c3, c) and torch.equal(h3, h)
    xs_b = _bf((T, B, I), 16).cuda()
    st = (_bf((B, H), 17, 0.3).cuda(), _bf((B, H), 18, 0.3).cuda())
    got, (hg, cg) = cell.forward_sequence(xs_b, ForwardCtx.inference(be), st)
    want, (hw, cw) = cell._sequence_body(xs_b, st[0].contiguous(), st[1].contiguous().clone())
    assert torch.equal(got, want) and torch.equal(cg, cw) and torch.equal(st[1], _bf((B, H), 18, 0.3).cuda())


@pytest.mark.parametrize("T,B,I,H", [(12, 1, 128, 128), (7, 5, 40, 64)])
def test_gru_inference_sequence_matches_fp32_recurrence_and_replays_from_a_graph(T, B, I, H, cuda_status):
    """GruCell's GPU inference path (one input-projection GEMM, then per step the hidden projection and the fused gate
    kernel writing into the output sequence) against the recurrence in fp32 PyTorch; the second call captures a CUDA graph,
    later calls replay it with new inputs and a new initial state."""
    from rustral_b200.core import B200Backend, ForwardCtx
    from rustral_b200.nn import GruCell
    be = B200Backend()
    cell = GruCell.new(be, I, H, seed=5)
    cell.b.tensor.data.copy_(_bf((3 * H,), 8, 0.1).cuda())
    xs = _bf((T, B, I), 6).cuda()
    ctx = ForwardCtx.inference(be)
    outs, h = cell.forward_sequence(xs, ctx)
    wx, wh, b = cell.wx.tensor.float().cpu(), cell.wh.tensor.float().cpu(), cell.b.tensor.float().cpu()
    hr, ref = torch.zeros(B, H), []
    for t in range(T):
        gx, gh = xs[t].float().cpu() @ wx.t() + b, hr @ wh.t()
        r, z = torch.sigmoid(gx[:, :H] + gh[:, :H]), torch.sigmoid(gx[:, H:2 * H] + gh[:, H:2 * H])
        n = torch.tanh(gx[:, 2 * H:] + r * gh[:, 2 * H:])
        hr = (1 - z) * n + z * hr
        ref.append(hr)
    ref = torch.stack(ref)
    assert outs.shape == (T, B, H) and not outs.requires_grad and torch.equal(h, outs[-1])
    _close(outs, ref, tol=3e-2, what="gru outputs")
    outs2, _ = cell.forward_sequence(xs, ctx)                 # captures
    outs3, h3 = cell.forward_sequence(xs, ctx)                # replays
    assert torch.equal(outs2, outs) and torch.equal(outs3, outs) and torch.equal(h3, h)
    xs_b, h0 = _bf((T, B, I), 16).cuda(), _bf((B, H), 17, 0.3).cuda()
    got, hg = cell.forward_sequence(xs_b, ctx, h0)
    want, hw = cell._sequence_body(xs_b, h0.contiguous())
    assert torch.equal(got, want) and torch.equal(hg, hw) and torch.equal(h0, _bf((B, H), 17, 0.3).cuda())
