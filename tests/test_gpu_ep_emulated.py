"""Expert parallelism with the ranks emulated on ONE GPU: every rank's buffers live on the same device, the
flag words are pre-set so that every wait is already satisfied, and the phases of the protocol run for all
ranks one after the other (count exchange twice, so that every rank finally sees every peer's counts).  This
drives the same kernels as the multi-GPU path - `ep_exchange`, `ep_dispatch`, the GEMM producer that waits for
the senders' flags, the scatter epilogue that stores result rows into the token owners' buffers, the
flag-waiting combine - and checks each rank's output against the plain expert computation on the whole bank.
A second test lets the GEMM producer's wait run out (a flag nobody sets) and reads the status word."""
import pytest
import torch

pytestmark = pytest.mark.gpu

CH_COUNTS, CH_DISPATCH, CH_RETURN = 0, 1, 2
MAXR = 8


def _bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def relerr(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("use_pair", [True, False])
@pytest.mark.parametrize("W,T,H,I,E,K", [(2, 300, 256, 128, 8, 2), (4, 512, 128, 256, 16, 4), (8, 64, 128, 64, 32, 2)])
def test_emulated_ranks_forward_matches_whole_bank(W, T, H, I, E, K, use_pair):
    from moe_b200 import ops
    from moe_b200.ops import _ext
    from moe_b200.ops import gemm as G
    from moe_b200.ops.functional import MoEPlan

    e = _ext.load()
    dev = torch.device("cuda")
    torch.manual_seed(21)
    El = E // W
    gu = torch.randn(E, 2 * I, H, device=dev) * 0.05
    dn = torch.randn(E, H, I, device=dev) * 0.05
    gu16, dn16 = gu.bfloat16(), dn.bfloat16()
    xs = [_bf(T, H) for _ in range(W)]
    idx = [torch.stack([torch.randperm(E, device=dev)[:K] for _ in range(T)]).int() for _ in range(W)]
    tw = [torch.rand(T, K, device=dev) for _ in range(W)]
    cap = (W * T * K + El * 128 + 127) // 128 * 128  # worst case: everything lands on one owner
    big = 1 << 20
    flags = [torch.full((3 * MAXR,), big, dtype=torch.int32, device=dev) for _ in range(W)]
    cmat = [torch.zeros(W * E, dtype=torch.int32, device=dev) for _ in range(W)]
    xrecv = [torch.zeros(cap, H, dtype=torch.bfloat16, device=dev) for _ in range(W)]
    meta = [torch.full((cap,), -1, dtype=torch.int32, device=dev) for _ in range(W)]
    yret = [torch.zeros(T * K, H, dtype=torch.bfloat16, device=dev) for _ in range(W)]
    epoch = torch.ones(1, dtype=torch.int32, device=dev)
    status = G.status_word(dev)
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    gcounter = torch.zeros(1, dtype=torch.int32, device=dev)
    ptr = lambda ts: [t.data_ptr() for t in ts]
    plans = [MoEPlan(idx[r], E) for r in range(W)]
    send_base = [torch.empty(E, dtype=torch.int32, device=dev) for _ in range(W)]
    rseg = [torch.empty(El + 1, dtype=torch.int32, device=dev) for _ in range(W)]
    rtile = [torch.zeros(cap // 128, dtype=torch.int32, device=dev) for _ in range(W)]
    rnt = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in range(W)]
    rpair = [torch.zeros((cap // 128 + El + 1) // 2, 2, dtype=torch.int32, device=dev) for _ in range(W)]
    rnp = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in range(W)]
    for _ in range(2):  # second round: every count matrix is complete
        for r in range(W):
            e.ep_exchange(plans[r].counts, ptr(cmat), ptr(flags), epoch, 0, r, W, E, H, send_base[r], rseg[r], rtile[r],
                          rnt[r], xrecv[r], meta[r], status, rpair[r], rnp[r])
    for r in range(W):
        e.ep_dispatch(xs[r], None, idx[r].view(-1), plans[r].pos, plans[r].seg_off, send_base[r], ptr(xrecv), ptr(meta),
                      ptr(flags), epoch, 1, r, W, E, K, cap, counter)
    for r in range(W):  # expert owners: up projection waits on the (satisfied) dispatch flags, down projection scatters
        act = torch.empty(cap, I, dtype=torch.bfloat16, device=dev)
        pre = torch.empty(cap, 2 * I, dtype=torch.bfloat16, device=dev)
        w1, w2 = gu16[r * El:(r + 1) * El].contiguous(), dn16[r * El:(r + 1) * El].contiguous()
        G.grouped_up_swiglu(xrecv[r], w1, rtile[r], rnt[r], act, pre,
                            ep=dict(ep_wait_flags=flags[r][CH_DISPATCH * MAXR:(CH_DISPATCH + 1) * MAXR], ep_wait_n=W,
                                    ep_epoch_base=epoch, ep_wait_epoch_off=1),
                            pair=(rpair[r], rnp[r]) if use_pair else None)
        G.grouped_nt(act, w2, rtile[r], rnt[r], yret[r], scatter=True,
                     ep=dict(ep_scatter_dst=ptr(yret), ep_scatter_meta=meta[r], ep_post_flags=ptr(flags),
                             ep_post_index=CH_RETURN * MAXR + r, ep_post_epoch_off=2, ep_world=W, ep_counter=gcounter,
                             ep_epoch_base=epoch))
    torch.cuda.synchronize()
    G.check_status()
    for r in range(W):
        out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        e.moe_combine(yret[r], None, tw[r], None, out, K, flags[r][CH_RETURN * MAXR:(CH_RETURN + 1) * MAXR], W, epoch, 2,
                      status)
        with ops.force_oracle():
            ref = ops.moe_experts(xs[r].float(), idx[r], tw[r], gu16.float(), dn16.float())
        torch.cuda.synchronize()
        assert relerr(out, ref) < 2e-2, (r, relerr(out, ref))
        # the routing-weight gradient kernel of the backward pass on the same return buffer
        d = _bf(T, H)
        dw = torch.empty(T, K, device=dev)
        e.moe_slot_dot(d, yret[r], K, dw)
        ref_dw = torch.einsum("tkh,th->tk", yret[r].view(T, K, H).float(), d.float())
        assert relerr(dw, ref_dw) < 1e-3
    G.check_status()
    # every posted flag carries the epoch of its phase (the pre-set words were overwritten by real posts)
    for r in range(W):
        assert int(flags[r][CH_DISPATCH * MAXR]) == 2 and int(flags[r][CH_RETURN * MAXR + r]) == 3


def test_gemm_producer_wait_runs_out_and_reports():
    """The senders never post their flag: the producer gives up after its limit, the other warp roles stop with
    it, the status word says 'peer wait', and the context keeps working."""
    import time

    from moe_b200.ops import gemm as G

    dev = torch.device("cuda")
    R, H, I, E = 512, 128, 64, 2
    xs = _bf(R, H)
    w1 = _bf(E, 2 * I, H, scale=0.05)
    act = torch.zeros(R, I, dtype=torch.bfloat16, device=dev)
    pre = torch.zeros(R, 2 * I, dtype=torch.bfloat16, device=dev)
    tile_expert = torch.zeros(R // 128, dtype=torch.int32, device=dev)
    nt = torch.full((1,), R // 128, dtype=torch.int32, device=dev)
    never = torch.zeros(MAXR, dtype=torch.int32, device=dev)
    epoch = torch.ones(1, dtype=torch.int32, device=dev)
    t0 = time.time()
    G.grouped_up_swiglu(xs, w1, tile_expert, nt, act, pre,
                        ep=dict(ep_wait_flags=never, ep_wait_n=2, ep_epoch_base=epoch, ep_wait_epoch_off=0,
                                ep_limit_ns=50_000_000))
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0  # 50 ms limit, and nobody sits out a long barrier wait afterwards
    with pytest.raises(RuntimeError, match="peer wait"):
        G.check_status()
    assert float(act.float().abs().sum()) == 0.0  # gave up before computing anything
    y = torch.ones(4, device=dev) * 3
    assert float(y.sum()) == 12.0
    G.check_status()
