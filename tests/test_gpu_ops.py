"""Kernel-vs-oracle checks: every sm_100a op against its plain-PyTorch fp32 statement."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def relerr(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda")


def _bf(*shape, scale=1.0, dev="cuda"):
    return (torch.randn(*shape, device=dev) * scale).to(torch.bfloat16)


def _sync_status():
    from moe_b200.ops import gemm as G

    torch.cuda.synchronize()
    G.check_status()


@pytest.fixture(params=["pair", "single"])
def tile_kind(request, monkeypatch):
    """Run a GEMM test on the pair-tile (`cta_group::2`) kernels and on the one-CTA kernels."""
    monkeypatch.setenv("MOE_B200_GEMM_PAIR", "1" if request.param == "pair" else "0")
    return request.param


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (1000, 520, 264), (2048, 1024, 1024), (300, 48, 512),
                                   (257, 136, 72), (513, 264, 1032), (4096, 384, 128)])
def test_gemm_nt(dev, tile_kind, M, N, K):
    from moe_b200.ops import gemm as G

    torch.manual_seed(0)
    a, b = _bf(M, K), _bf(N, K)
    c = G.gemm_nt(a, b)
    _sync_status()
    assert relerr(c, a.float() @ b.float().T) < 5e-3
    c32 = G.gemm_nt(a, b, out_dtype=torch.float32)
    _sync_status()
    assert relerr(c32, a.float() @ b.float().T) < 1e-5


@pytest.mark.parametrize("M,N,K", [(384, 512, 192), (1000, 264, 520), (256, 128, 16), (776, 1032, 328)])
def test_gemm_nn_and_tn(dev, tile_kind, M, N, K):
    from moe_b200.ops import gemm as G

    torch.manual_seed(1)
    a, b = _bf(M, K), _bf(K, N)
    assert relerr(G.gemm_nn(a, b), a.float() @ b.float()) < 5e-3
    at, bt = _bf(K, M), _bf(K, N)
    out = torch.randn(M, N, device=dev)
    ref = out + at.float().T @ bt.float()
    G.gemm_tn(at, bt, out, beta=1)
    _sync_status()
    assert relerr(out, ref) < 1e-5
    G.gemm_tn(at, bt, out, beta=0)
    _sync_status()
    assert relerr(out, at.float().T @ bt.float()) < 1e-5


@pytest.mark.parametrize("Kc,M,N", [(8192, 16, 1024), (4096, 128, 512), (12288, 8, 264)])
def test_gemm_tn_short_wide_output_is_split_along_the_contraction(dev, Kc, M, N):
    """The router's weight-gradient shape: partial products per contraction segment, summed in a fixed order."""
    from moe_b200.ops import gemm as G

    torch.manual_seed(2)
    at, bt = _bf(Kc, M), _bf(Kc, N)
    assert G._split_k_segments(Kc, at.device) is not None
    out = torch.randn(M, N, device=dev)
    ref = out + at.float().T @ bt.float()
    G.gemm_tn(at, bt, out, beta=1)
    _sync_status()
    assert relerr(out, ref) < 1e-5
    G.gemm_tn(at, bt, out, beta=0)
    again = torch.empty_like(out)
    G.gemm_tn(at, bt, again, beta=0)
    _sync_status()
    assert relerr(out, at.float().T @ bt.float()) < 1e-5 and torch.equal(out, again)


@pytest.mark.parametrize("B,S,nh,nkv,H", [(2, 128, 4, 2, 256), (1, 384, 16, 8, 1024), (3, 256, 3, 1, 512)])
def test_qkv_projection_with_norm_and_rope_in_the_epilogue(dev, B, S, nh, nkv, H):
    """The fused QKV epilogue against the GEMM followed by the stand-alone QK-norm + RoPE kernel (same arithmetic),
    then through autograd against the fp32 statement, with attention reading the slices in place."""
    from moe_b200 import ops
    from moe_b200.ops import functional as F
    from moe_b200.ops import gemm as G

    torch.manual_seed(7)
    hd, T, N = 128, B * S, (nh + 2 * nkv) * 128
    assert G.qkv_rope_supported(T, N, H, hd)
    x, w = _bf(T, H), _bf(N, H, scale=0.05)
    qw, kw = 1 + 0.1 * torch.randn(hd, device=dev), 1 + 0.1 * torch.randn(hd, device=dev)
    cs = F.rope_table(S, hd, 1e6, x.device)
    raw, rot, rstd = G.gemm_nt_qkrope(x, w, cs, qw, kw, S, nh, nkv, 1e-6)
    ref_raw = G.gemm_nt(x, w)
    q, k, v = F.qk_norm_rope(ref_raw.view(B, S, N), qw, kw, B, S, nh, nkv, hd, 1e6, 1e-6)
    _sync_status()
    assert torch.equal(raw, ref_raw)
    got = rot.view(B, S, nh + 2 * nkv, hd)
    assert torch.equal(got[:, :, nh + nkv:], v)
    assert relerr(got[:, :, :nh], q) < 4e-3 and relerr(got[:, :, nh:nh + nkv], k) < 4e-3
    # module-level: projection + norm + rope + attention, kernels against the oracle
    xs = _bf(B, S, H).requires_grad_()
    ws = [(_bf(n, H, scale=0.05)).float().requires_grad_() for n in (nh * hd, nkv * hd, nkv * hd)]
    nq, nk = qw.clone().requires_grad_(), kw.clone().requires_grad_()

    def run(xi, wi, a, b):
        qq, kk, vv = ops.qkv_proj_norm_rope(xi, *wi, None, a, b, B, S, nh, nkv, hd, 1e6, 1e-6)
        return ops.attention(qq, kk, vv) if (nh // nkv) % 2 == 0 else torch.cat(
            [qq.reshape(B, S, -1), kk.reshape(B, S, -1), vv.reshape(B, S, -1)], -1)

    out = run(xs, ws, nq, nk)
    g = torch.randn_like(out.float()).to(out.dtype)
    out.backward(g)
    xo = xs.detach().float().requires_grad_()
    wo = [t.detach().bfloat16().float().requires_grad_() for t in ws]
    ao, bo = nq.detach().clone().requires_grad_(), nk.detach().clone().requires_grad_()
    with ops.force_oracle():
        out2 = run(xo, wo, ao, bo)
    out2.backward(g.float())
    _sync_status()
    assert relerr(out, out2) < 2e-2
    assert relerr(xs.grad, xo.grad) < 4e-2
    for a_, b_ in zip(ws + [nq, nk], wo + [ao, bo]):
        assert relerr(a_.grad, b_.grad) < 4e-2


def test_rmsnorm_fwd_bwd(dev):
    from moe_b200.ops import functional as F, oracle

    torch.manual_seed(2)
    for H in (128, 1024, 2048):
        x = _bf(300, H).requires_grad_()
        r = _bf(300, H).requires_grad_()
        w = (1 + 0.1 * torch.randn(H, device=dev)).requires_grad_()
        h, y = F.add_rmsnorm(x, r, w, 1e-6)
        gy, gh = _bf(300, H), _bf(300, H)
        (y.float() * gy.float()).sum().add((h.float() * gh.float()).sum()).backward()
        x2, r2, w2 = x.detach().float().requires_grad_(), r.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
        h2 = (x2 + r2)
        y2 = oracle.rmsnorm(h2.bfloat16().float(), w2, 1e-6)
        (y2 * gy.float()).sum().add((h2 * gh.float()).sum()).backward()
        assert relerr(y, y2) < 1e-2
        assert relerr(x.grad, x2.grad) < 2e-2
        assert relerr(r.grad, r2.grad) < 2e-2
        assert relerr(w.grad, w2.grad) < 2e-2


@pytest.mark.parametrize("hd,nh,nkv", [(32, 4, 2), (64, 4, 2), (128, 4, 2), (32, 6, 3), (64, 5, 5), (128, 3, 1)])
def test_qknorm_rope(dev, hd, nh, nkv):
    """Head counts that do not fill the last warp pass are included (several heads share a warp)."""
    from moe_b200.ops import functional as F, oracle

    torch.manual_seed(3)
    B, S = 2, 64
    qkv = _bf(B, S, (nh + 2 * nkv) * hd).requires_grad_()
    qw = (1 + 0.1 * torch.randn(hd, device=dev)).requires_grad_()
    kw = (1 + 0.1 * torch.randn(hd, device=dev)).requires_grad_()
    q, k, v = F.qk_norm_rope(qkv, qw, kw, B, S, nh, nkv, hd, 1e6, 1e-6)
    gq, gk, gv = _bf(*q.shape), _bf(*k.shape), _bf(*v.shape)
    ((q.float() * gq.float()).sum() + (k.float() * gk.float()).sum() + (v.float() * gv.float()).sum()).backward()
    x2 = qkv.detach().float().requires_grad_()
    qw2, kw2 = qw.detach().clone().requires_grad_(), kw.detach().clone().requires_grad_()
    q2, k2, v2 = x2.view(B, S, nh + 2 * nkv, hd).split([nh, nkv, nkv], dim=2)
    cos, sin = oracle.rope_tables(S, hd, 1e6, device=dev)
    q2, k2 = oracle.qk_norm_rope(q2, k2, qw2, kw2, cos, sin, 1e-6)
    ((q2 * gq.float()).sum() + (k2 * gk.float()).sum() + (v2 * gv.float()).sum()).backward()
    assert relerr(q, q2) < 1e-2 and relerr(k, k2) < 1e-2 and relerr(v, v2) < 1e-6
    assert relerr(qkv.grad, x2.grad) < 2e-2
    assert relerr(qw.grad, qw2.grad) < 2e-2 and relerr(kw.grad, kw2.grad) < 2e-2


@pytest.mark.parametrize("mode,E,K,groups", [("softmax", 16, 4, None), ("softmax", 128, 8, None),
                                             ("sigmoid", 64, 4, None), ("sigmoid", 64, 4, (8, 4)),
                                             ("sigmoid", 256, 8, (8, 4))])
def test_router(dev, mode, E, K, groups):
    from moe_b200 import ops
    from moe_b200.ops import oracle

    torch.manual_seed(4)
    T, H = 500, 256
    x = _bf(T, H)
    w = (torch.randn(E, H, device=dev) * 0.05)
    bias = torch.randn(E, device=dev) * 0.01 if mode == "sigmoid" else None
    ng, gt = groups if groups else (None, None)
    sf = 2.5 if mode == "sigmoid" else None
    xk = x.clone().requires_grad_()
    wk = w.clone().requires_grad_()
    s, tw, ti = ops.router(xk, wk, bias, top_k=K, score_fn=mode, norm_topk_prob=True, scaling_factor=sf,
                           num_groups=ng, group_topk=gt)
    xo = x.float().requires_grad_()
    wo = w.bfloat16().float().requires_grad_()
    with ops.force_oracle():
        s2, tw2, ti2 = ops.router(xo, wo, bias, top_k=K, score_fn=mode, norm_topk_prob=True, scaling_factor=sf,
                                  num_groups=ng, group_topk=gt)
    assert relerr(s, s2) < 1e-3
    same = (ti.long().sort(-1).values == ti2.sort(-1).values).all(-1)
    assert same.float().mean() > 0.98  # near-ties may flip between bf16-GEMM and fp32 logits
    order = ti.long().argsort(-1), ti2.argsort(-1)
    a = tw.gather(1, order[0])[same]
    b = tw2.gather(1, order[1])[same]
    assert relerr(a, b) < 1e-2
    # backward: same upstream gradients, compare on the rows with identical selection
    gs, gw = torch.randn_like(s) * 0.1, torch.randn_like(tw)
    gw2 = torch.zeros_like(gw).scatter_(1, order[1], gw.gather(1, order[0]))
    mask = same.float()[:, None]
    ((s * gs * mask).sum() + (tw * gw * mask).sum()).backward()
    ((s2 * gs * mask).sum() + (tw2 * gw2 * mask).sum()).backward()
    assert relerr(xk.grad, xo.grad) < 5e-2
    assert relerr(wk.grad, wo.grad) < 5e-2


@pytest.mark.parametrize("T,H,I,E,K", [(300, 256, 192, 8, 2), (1024, 512, 256, 16, 4), (64, 128, 64, 32, 8),
                                       (2000, 256, 320, 4, 2)])
@pytest.mark.parametrize("mode", ["plain", "fold", "gather"])
def test_moe_experts(dev, tile_kind, monkeypatch, mode, T, H, I, E, K):
    """plain: weighted combine kernel; fold: routing weight applied in the GEMM epilogues (default where the
    pair-tile kernels apply); gather: token rows fetched by index inside the GEMMs on top of that."""
    from moe_b200 import ops

    monkeypatch.setenv("MOE_B200_MOE_FOLD", "0" if mode == "plain" else "1")
    monkeypatch.setenv("MOE_B200_MOE_GATHER", "1" if mode == "gather" else "0")
    torch.manual_seed(5)
    x = _bf(T, H)
    gu = torch.randn(E, 2 * I, H, device=dev) * 0.05
    dn = torch.randn(E, H, I, device=dev) * 0.05
    idx = torch.stack([torch.randperm(E, device=dev)[:K] for _ in range(T)]).int()
    w = torch.rand(T, K, device=dev)
    w = w / w.sum(-1, keepdim=True)
    xk, guk, dnk, wk = x.clone().requires_grad_(), gu.clone().requires_grad_(), dn.clone().requires_grad_(), w.clone().requires_grad_()
    out = ops.moe_experts(xk, idx, wk, guk, dnk)
    g = _bf(T, H)
    (out.float() * g.float()).sum().backward()
    xo = x.float().requires_grad_()
    guo, dno, wo = gu.bfloat16().float().requires_grad_(), dn.bfloat16().float().requires_grad_(), w.clone().requires_grad_()
    with ops.force_oracle():
        out2 = ops.moe_experts(xo, idx, wo, guo, dno)
    (out2 * g.float()).sum().backward()
    _sync_status()
    assert relerr(out, out2) < 2e-2
    assert relerr(xk.grad, xo.grad) < 3e-2
    assert relerr(guk.grad, guo.grad) < 3e-2
    assert relerr(dnk.grad, dno.grad) < 3e-2
    assert relerr(wk.grad, wo.grad) < 3e-2


def test_moe_plan_is_stable_sort(dev):
    from moe_b200.ops.functional import MoEPlan

    torch.manual_seed(6)
    T, K, E = 777, 4, 16
    idx = torch.randint(0, E, (T, K), device=dev, dtype=torch.int32)
    plan = MoEPlan(idx, E)
    torch.cuda.synchronize()
    counts = torch.bincount(idx.view(-1).long(), minlength=E)
    assert torch.equal(plan.counts.long(), counts)
    seg = plan.seg_off.long().cpu()
    flat = idx.view(-1).long().cpu()
    pos = plan.pos.long().cpu()
    for e in range(E):
        slots = (flat == e).nonzero().view(-1)
        assert torch.equal(pos[slots], seg[e] + torch.arange(len(slots)))  # token order kept inside an expert
        assert (seg[e + 1] - seg[e]) == (counts[e].item() + 127) // 128 * 128
    assert plan.num_m_tiles.item() == seg[E].item() // 128
    # pair tiles: every 128-row tile of every expert exactly once, never two experts in one pair
    npair = plan.num_pair_tiles.item()
    pt = plan.pair_tiles[:npair].cpu()
    te = plan.tile_expert[:plan.num_m_tiles.item()].cpu()
    seen = []
    for m0, info in pt.tolist():
        e, halves = info & 0xffff, info >> 16
        assert m0 % 128 == 0 and halves in (1, 2)
        for h in range(halves):
            assert te[m0 // 128 + h].item() == e
            seen.append(m0 // 128 + h)
    assert sorted(seen) == list(range(plan.num_m_tiles.item()))


@pytest.mark.parametrize("T,H,V,chunk", [(512, 256, 1000, 4096), (300, 128, 4096, 4096), (700, 256, 2048, 256)])
def test_linear_cross_entropy(dev, monkeypatch, T, H, V, chunk):
    """`chunk` < T: several token chunks share the logits scratch (the last one partial) and the
    weight gradient is accumulated over them."""
    from moe_b200 import ops
    from moe_b200.ops import functional as F

    monkeypatch.setattr(F, "LCE_CHUNK_ROWS", chunk)
    torch.manual_seed(7)
    V = V // 8 * 8
    h = _bf(T, H)
    w = torch.randn(V, H, device=dev) * 0.05
    labels = torch.randint(0, V, (T,), device=dev)
    labels[::7] = -100
    hk, wk = h.clone().requires_grad_(), w.clone().requires_grad_()
    loss = ops.linear_cross_entropy(hk, wk, labels)
    loss.backward()
    ho, wo = h.float().requires_grad_(), w.bfloat16().float().requires_grad_()
    with ops.force_oracle():
        loss2 = ops.linear_cross_entropy(ho, wo, labels)
    loss2.backward()
    _sync_status()
    assert abs(loss.item() - loss2.item()) < 2e-2 * abs(loss2.item())
    assert relerr(hk.grad, ho.grad) < 3e-2
    assert relerr(wk.grad, wo.grad) < 3e-2
    # fixed-order loss reduction: the same bits on a second run
    hk2, wk2 = h.clone().requires_grad_(), w.clone().requires_grad_()
    assert ops.linear_cross_entropy(hk2, wk2, labels).item() == loss.item()


@pytest.mark.parametrize("n_tok", [400, 20000])
def test_embedding(dev, n_tok):
    """Gather, and the sorted segmented-sum backward (20000 tokens: past the built-in key sort); ids repeat
    many times, and two runs must give the same bits."""
    from moe_b200 import ops

    torch.manual_seed(8)
    V, H = 1000, 256
    w = torch.randn(V, H, device=dev)
    ids = torch.randint(0, V, (4, n_tok // 4), device=dev)
    ids[0, :50] = 7  # a long run of one id
    g = _bf(4, n_tok // 4, H)
    grads = []
    for _ in range(2):
        wk = w.clone().requires_grad_()
        out = ops.embedding(ids, wk)
        (out.float() * g.float()).sum().backward()
        grads.append(wk.grad.clone())
    wo = w.bfloat16().float().requires_grad_()
    out2 = torch.nn.functional.embedding(ids, wo)
    (out2 * g.float()).sum().backward()
    assert relerr(out, out2) < 1e-6
    assert relerr(grads[0], wo.grad) < 1e-5
    assert torch.equal(grads[0], grads[1])


@pytest.mark.parametrize("mtype,E,K,groups,B,S", [("softmax", 16, 4, None, 4, 128), ("sigmoid", 64, 4, (8, 4), 2, 256),
                                                   ("sigmoid", 32, 2, None, 3, 96), ("softmax", 16, 4, None, 2, 100)])
def test_router_statistics_and_balance_losses(dev, mtype, E, K, groups, B, S):
    """The router kernels' statistics against the plain-PyTorch losses: counts, Switch loss, sequence-level
    loss, margins, and the gradient both losses send into the router weight."""
    from moe_b200 import ops
    from moe_b200.models.load_balancing import load_balancing_loss_func, seq_load_balancing_loss_func
    from moe_b200.ops import functional as F
    from moe_b200.ops.oracle import topk_lowest_index

    torch.manual_seed(11)
    T, H, L = B * S, 128, 2
    ng, gt = groups if groups else (None, None)
    bias = [torch.randn(E, device=dev) * 0.05 if mtype == "sigmoid" else None for _ in range(L)]
    xs = [_bf(T, H) for _ in range(L)]
    ws = [(torch.randn(E, H, device=dev) * 0.2).bfloat16().float() for _ in range(L)]
    holder = F.MoeStatsHolder(L, B, S, E, K, dev, separate_unb=mtype == "sigmoid")
    holder.begin()
    acc = [torch.zeros(E, device=dev) for _ in range(L)]
    wk = [w.clone().requires_grad_() for w in ws]
    outs = [ops.router(xs[l], wk[l], bias[l], top_k=K, score_fn=mtype, norm_topk_prob=True, scaling_factor=None,
                       num_groups=ng, group_topk=gt, site=holder.sites[l], tokens_acc=acc[l]) for l in range(L)]
    scores = tuple(o[0] for o in outs)
    aux, seq = ops.moe_aux_losses(holder, scores, seq_on=True)
    (0.7 * aux + 0.3 * seq).backward()
    _sync_status()
    # plain PyTorch on the kernel's own scores and selections (so near-ties cannot differ)
    wo = [w.clone().requires_grad_() for w in ws]
    sc2 = []
    for l in range(L):
        logit = xs[l].float() @ wo[l].T
        sc2.append(torch.softmax(logit, -1) if mtype == "softmax" else torch.sigmoid(logit))
    sel = tuple(o[2].long() for o in outs)
    unb = tuple(topk_lowest_index(s.detach(), K)[1] for s in scores)
    aux2 = load_balancing_loss_func(tuple(sc2), E, K, selected_experts=unb)
    seq2 = seq_load_balancing_loss_func(tuple(sc2), E, K, batch_size=B, selected_experts=sel)
    (0.7 * aux2 + 0.3 * seq2).backward()
    assert abs(aux.item() - aux2.item()) < 1e-3 * abs(aux2.item())
    assert abs(seq.item() - seq2.item()) < 1e-3 * abs(seq2.item())
    for l in range(L):
        cnt_sel = torch.bincount(sel[l].reshape(-1), minlength=E)
        assert torch.equal(holder.cnt_sel[l].sum(0).long(), cnt_sel)
        assert torch.equal(acc[l].long(), cnt_sel)
        assert torch.equal(holder.cnt_unb[l].sum(0).long(), torch.bincount(unb[l].reshape(-1), minlength=E))
        per_seq = torch.stack([torch.bincount(sel[l][b * S:(b + 1) * S].reshape(-1), minlength=E) for b in range(B)])
        assert torch.equal(holder.cnt_sel[l].long(), per_seq)
        top = topk_lowest_index(scores[l].detach(), K + 1)[0]
        assert torch.allclose(holder.margin[l], top[:, K - 1] - top[:, K], atol=1e-6)
        assert relerr(wk[l].grad, wo[l].grad) < 3e-2, (l, relerr(wk[l].grad, wo[l].grad))


def test_dense_swiglu_mlp(dev, tile_kind):
    from moe_b200 import ops

    torch.manual_seed(12)
    T, H, I = 600, 256, 384
    x = _bf(T, H)
    wg, wu, wd = (torch.randn(I, H, device=dev) * 0.05, torch.randn(I, H, device=dev) * 0.05,
                  torch.randn(H, I, device=dev) * 0.05)
    ks = [t.clone().requires_grad_() for t in (x, wg, wu, wd)]
    y = ops.swiglu_mlp(*ks)
    g = _bf(T, H)
    (y.float() * g.float()).sum().backward()
    os_ = [x.float().requires_grad_()] + [t.bfloat16().float().requires_grad_() for t in (wg, wu, wd)]
    with ops.force_oracle():
        y2 = ops.swiglu_mlp(*os_)
    (y2 * g.float()).sum().backward()
    _sync_status()
    assert relerr(y, y2) < 2e-2
    for a, b in zip(ks, os_):
        assert relerr(a.grad, b.grad) < 3e-2


def test_adamw_and_norm(dev):
    from moe_b200.ops import _ext, oracle

    e = _ext.load()
    torch.manual_seed(9)
    n = 1_000_003 // 64 * 64
    p = torch.randn(n, device=dev)
    g = torch.randn(n, device=dev)
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    p16 = torch.empty(n, device=dev, dtype=torch.bfloat16)
    p2, m2, v2 = p.clone(), m.clone(), v.clone()
    ss = torch.zeros(1, device=dev)
    coef = torch.zeros(2, device=dev)
    scratch = torch.empty(e.sumsq_blocks(n), device=dev)
    for step in (1, 2, 3):
        e.sumsq(g, scratch, ss, False)
        e.clip_coef(ss, 1.0, coef)
        hyper = torch.tensor([1e-3, 1 - 0.9 ** step, 1 - 0.95 ** step], device=dev)
        e.adamw(p, g, m, v, p16, hyper, 0.9, 0.95, 1e-8, 0.1, coef)
        c = min(1.0, 1.0 / (g.norm().item() + 1e-6))
        oracle.adamw_step_(p2, g, m2, v2, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step,
                           grad_scale=c)
    assert abs(coef[1].item() - g.norm().item()) < 1e-3 * g.norm().item()
    assert relerr(p, p2) < 1e-6 and relerr(m, m2) < 1e-5 and relerr(v, v2) < 1e-5
    assert relerr(p16, p2) < 5e-3


@pytest.mark.parametrize("bwd", ["library", "own"])
@pytest.mark.parametrize("hd", [128, 64])
@pytest.mark.parametrize("B,S,nh,nkv,spread", [(1, 128, 2, 1, 1.0), (2, 384, 4, 2, 1.0), (1, 1024, 8, 1, 1.0),
                                               (2, 512, 4, 2, 6.0)])
def test_flash_attention_forward_and_grads(dev, monkeypatch, B, S, nh, nkv, spread, bwd, hd):
    """Own tcgen05 forward (output and log-sum-exp) and the gradients of `ops.attention` against the fp32
    statement; `spread` widens the score range so that the lazy accumulator rescale in TMEM is exercised."""
    from moe_b200.ops import _ext, oracle
    from moe_b200.ops import functional as F
    from moe_b200.ops import gemm as G

    q, k, v = _bf(B, S, nh, hd, scale=spread), _bf(B, S, nkv, hd, scale=spread), _bf(B, S, nkv, hd)
    assert F.flash_supported(q, k)
    o = torch.empty_like(q)
    lse2 = torch.empty(B, nh, S, device=dev)
    _ext.load().flash_fwd(q, k, v, o, lse2, 1 / math.sqrt(hd), G.status_word(dev))
    _sync_status()
    qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
    ref = oracle.causal_gqa_attention(qf, kf, vf)
    assert relerr(o, ref) < 1.5e-2
    kk = kf.detach().repeat_interleave(nh // nkv, 2)
    sc = torch.einsum("bqhd,bkhd->bhqk", qf.detach(), kk) / math.sqrt(hd)
    sc = sc.masked_fill(torch.ones(S, S, dtype=torch.bool, device=dev).triu(1), float("-inf"))
    assert (lse2 * math.log(2) - torch.logsumexp(sc, -1)).abs().max() < 2e-3
    # through autograd: own forward, then the library's or the own backward kernels
    monkeypatch.setenv("MOE_B200_ATTN_BWD", bwd)
    do = _bf(B, S, nh, hd)
    q2, k2, v2 = (t.clone().requires_grad_() for t in (q, k, v))
    out = F.attention(q2, k2, v2)
    assert torch.equal(out, o)
    out.backward(do)
    ref.backward(do.float())
    _sync_status()
    for a, b in ((q2.grad, qf.grad), (k2.grad, kf.grad), (v2.grad, vf.grad)):
        assert relerr(a, b) < 2e-2
