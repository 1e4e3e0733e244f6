"""Every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import math

import numpy as np
import pytest
import torch

from distca_b200.ops import _lib
from distca_b200.ops import attention as A
from distca_b200.ops import elementwise as ew

pytestmark = pytest.mark.gpu


def _bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-9)


# ---------------------------------------------------------------- norm / activation
@pytest.mark.parametrize("T,H", [(7, 256), (1000, 4096), (513, 8192)])
def test_rmsnorm_fwd_bwd(T, H):
    x, g, dy, dres = _bf(T, H), (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16(), _bf(T, H), _bf(T, H)
    y, rstd = ew.rmsnorm_fwd(x, g, 1e-5)
    yr, rr = ew.rmsnorm_fwd(x.cpu().float(), g.cpu().float(), 1e-5)
    assert _rel(y.cpu(), yr) < 1e-2 and _rel(rstd.cpu(), rr) < 1e-4
    dg = torch.zeros(H, dtype=torch.float32, device="cuda")
    dx = ew.rmsnorm_bwd(x, g, rstd, dy, dg, dres=dres, accumulate_dg=False)
    dgr = torch.zeros(H)
    dxr = ew.rmsnorm_bwd(x.cpu().float(), g.cpu().float(), rr, dy.cpu().float(), dgr, dres=dres.cpu().float(),
                         accumulate_dg=False)
    assert _rel(dx.cpu(), dxr) < 1e-2 and _rel(dg.cpu(), dgr) < 1e-2
    _lib.check_status()


def test_swiglu_and_add():
    T, F = 300, 688
    pre, dact = _bf(T, 2 * F), _bf(T, F)
    act = ew.swiglu_fwd(pre)
    assert _rel(act.cpu(), ew.swiglu_fwd(pre.cpu().float())) < 1e-2
    want = ew.swiglu_bwd(pre.cpu().float().clone(), dact.cpu().float(), inplace=False)
    got = ew.swiglu_bwd(pre.clone(), dact, inplace=True)
    assert _rel(got.cpu(), want) < 1e-2
    a, b = _bf(64, 128), _bf(64, 128)
    ref = a.float() + b.float()
    assert _rel(ew.add_(a, b).cpu(), ref.cpu()) < 1e-2


# ---------------------------------------------------------------- rope (+ fused scatter)
def test_rope_fwd_bwd_and_scatter():
    T, Hq, Hkv, D = 200, 4, 2, 128
    qkv = _bf(T, (Hq + 2 * Hkv) * D)
    pos = torch.randint(0, 5000, (T,), device="cuda", dtype=torch.int32)
    table = ew.rope_table(8192, D, 500000.0, "cuda")
    ref = ew.rope_(qkv.cpu().float().clone(), pos.cpu(), table.cpu(), Hq, Hkv, D)
    out = ew.rope_(qkv.clone(), pos, table, Hq, Hkv, D)
    assert _rel(out.cpu(), ref) < 1e-2
    back = ew.rope_(out.clone(), pos, table, Hq, Hkv, D, backward=True)
    assert _rel(back.cpu()[:, :(Hq + Hkv) * D], qkv.cpu().float()[:, :(Hq + Hkv) * D]) < 2e-2
    # scatter: token t's Q row to row perm[t] of Qd; K/V rows to two copies
    perm = torch.randperm(T, device="cuda")
    Qd = torch.zeros(T, Hq * D, dtype=torch.bfloat16, device="cuda")
    Kd = torch.zeros(2 * T, Hkv * D, dtype=torch.bfloat16, device="cuda")
    Vd = torch.zeros(2 * T, Hkv * D, dtype=torch.bfloat16, device="cuda")
    q_dst = Qd.data_ptr() + perm.long() * (Hq * D * 2)
    kv_dst = torch.stack([Kd.data_ptr() + perm.long() * (Hkv * D * 2),
                          Kd.data_ptr() + (T + perm.long()) * (Hkv * D * 2)], dim=1).contiguous()
    kv_dst[::3, 1] = 0  # every third token has a single copy
    src = qkv.clone()
    ew.rope_(src, pos, table, Hq, Hkv, D, q_dst=q_dst, kv_dst=kv_dst, max_copies=2,
             v_off_bytes=Vd.data_ptr() - Kd.data_ptr(), write_inplace=False)
    torch.cuda.synchronize()
    assert torch.equal(src, qkv)  # nothing written back
    assert torch.equal(Qd[perm], out[:, :Hq * D])
    assert torch.equal(Kd[perm], out[:, Hq * D:(Hq + Hkv) * D])
    assert torch.equal(Vd[perm], qkv[:, (Hq + Hkv) * D:])
    two = torch.ones(T, dtype=torch.bool, device="cuda"); two[::3] = False
    assert torch.equal(Kd[T + perm[two]], out[two][:, Hq * D:(Hq + Hkv) * D])
    assert (Kd[T + perm[~two]] == 0).all()


def test_qkv_gemm_with_rope_and_dispatch_epilogue():
    """QKV projection whose epilogue rotates the heads and stores the rows to per-token destinations
    == plain GEMM followed by the RoPE / dispatch kernel (which is checked against fp32 above)."""
    from distca_b200.ops import gemm
    T, K, Hq, Hkv, D = 1000, 512, 4, 2, 128     # 1000 rows: a partial M tile; 8 heads: 4 N tiles
    x = _bf(T, K, scale=1.0)
    w = _bf((Hq + 2 * Hkv) * D, K, scale=0.05)
    pos = torch.randint(0, 5000, (T,), device="cuda", dtype=torch.int32)
    table = ew.rope_table(8192, D, 500000.0, "cuda")
    plain = gemm.linear_fwd(x, w)
    ref = ew.rope_(plain.clone(), pos, table, Hq, Hkv, D)
    out = gemm.linear_qkv_rope(x, w, pos, table, Hq, Hkv)
    torch.cuda.synchronize()
    _lib.check_status()
    assert (out.float() - ref.float()).abs().max().item() <= 2e-2 * ref.float().abs().max().item()
    assert torch.equal(out[:, (Hq + Hkv) * D:], plain[:, (Hq + Hkv) * D:])      # V passes through
    fp32 = ew.rope_((x.float() @ w.float().t()).cpu(), pos.cpu(), table.cpu(), Hq, Hkv, D)
    assert _rel(out.cpu(), fp32) < 1e-2
    # destinations only (nothing written locally), two K/V copies for most tokens
    perm = torch.randperm(T, device="cuda")
    Qd = torch.zeros(T, Hq * D, dtype=torch.bfloat16, device="cuda")
    Kd = torch.zeros(2 * T, Hkv * D, dtype=torch.bfloat16, device="cuda")
    Vd = torch.zeros(2 * T, Hkv * D, dtype=torch.bfloat16, device="cuda")
    q_dst = Qd.data_ptr() + perm.long() * (Hq * D * 2)
    kv_dst = torch.stack([Kd.data_ptr() + perm.long() * (Hkv * D * 2),
                          Kd.data_ptr() + (T + perm.long()) * (Hkv * D * 2)], dim=1).contiguous()
    kv_dst[::3, 1] = 0
    none = gemm.linear_qkv_rope(x, w, pos, table, Hq, Hkv, write_local=False, q_dst=q_dst, kv_dst=kv_dst,
                                max_copies=2, v_off_bytes=Vd.data_ptr() - Kd.data_ptr())
    torch.cuda.synchronize()
    _lib.check_status()
    assert none is None
    assert torch.equal(Qd[perm], out[:, :Hq * D])
    assert torch.equal(Kd[perm], out[:, Hq * D:(Hq + Hkv) * D])
    assert torch.equal(Vd[perm], out[:, (Hq + Hkv) * D:])
    two = torch.ones(T, dtype=torch.bool, device="cuda"); two[::3] = False
    assert torch.equal(Kd[T + perm[two]], out[two][:, Hq * D:(Hq + Hkv) * D])
    assert (Kd[T + perm[~two]] == 0).all() and (Vd[T + perm[~two]] == 0).all()


# ---------------------------------------------------------------- loss / embedding / optimizer
@pytest.mark.parametrize("V,R", [(512, 1), (4096, 2)])
def test_cross_entropy_vocab_parallel(V, R):
    T = 257
    logits = torch.randn(T, V, device="cuda") * 3
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[::7] = -100
    n_valid = int((labels >= 0).sum())
    Vp = V // R
    stats = torch.stack([ew.ce_stats(logits[:, r * Vp:(r + 1) * Vp].contiguous(), labels, r * Vp) for r in range(R)])
    loss_sum, grads = 0.0, []
    for r in range(R):
        loss, g = ew.ce_grad(logits[:, r * Vp:(r + 1) * Vp].contiguous(), labels, stats, 1.0 / n_valid, r * Vp)
        grads.append(g)
        loss_sum = loss.sum().item() / n_valid
    lg = logits.clone().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lg, labels, ignore_index=-100)
    ref.backward()
    assert abs(loss_sum - ref.item()) < 1e-4
    assert _rel(torch.cat(grads, dim=1), lg.grad) < 1e-2
    _lib.check_status()


def test_embedding_fwd_bwd():
    V, H, T = 1000, 256, 5000
    table = _bf(V, H)
    ids = torch.randint(0, V, (T,), device="cuda")
    out = ew.embedding_fwd(ids, table)
    assert torch.equal(out, table[ids])
    half = ew.embedding_fwd(ids, table[500:], vocab_start=500)
    assert torch.equal(half[ids >= 500], table[ids[ids >= 500]]) and (half[ids < 500] == 0).all()
    dout = _bf(T, H)
    dt = torch.zeros(V, H, dtype=torch.float32, device="cuda")
    ew.embedding_bwd(ids, dout, dt)
    ref = torch.zeros(V, H, device="cuda").index_add_(0, ids, dout.float())
    assert _rel(dt, ref) < 1e-5


def test_adam_split_master_matches_fp32_adamw():
    n = 4096 * 3
    w0 = torch.randn(n, device="cuda") * 0.02
    p = w0.to(torch.bfloat16)
    lo = torch.zeros(n, dtype=torch.int16, device="cuda")
    master = p.float().clone()   # exact start: lo = 0
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    mr, vr = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    gs = torch.tensor([0.5], device="cuda")
    for step in range(1, 6):
        g = (torch.randn(n, device="cuda") * 1e-2).to(torch.bfloat16)
        ew.adam_step_(p, lo, g, m, v, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01, step=step, gscale=gs)
        gf = g.float() * 0.5
        mr.mul_(0.9).add_(gf, alpha=0.1)
        vr.mul_(0.95).addcmul_(gf, gf, value=0.05)
        upd = (mr / (1 - 0.9 ** step)) / ((vr / (1 - 0.95 ** step)).sqrt() + 1e-8) + 0.01 * master
        master -= 1e-3 * upd
    got = ew.master_from_split(p, lo)
    assert (got - master).abs().max().item() < 1e-6
    assert torch.equal(p, got.to(torch.bfloat16)) or _rel(p, got) < 1e-2
    acc = torch.zeros(1, device="cuda")
    ew.sumsq_(g, acc)
    assert abs(acc.item() - g.float().pow(2).sum().item()) < 1e-3 * acc.item()


# ---------------------------------------------------------------- attention
TASKSETS = [
    ("one tile", [(0, 128, 0, 128)], 128, 128, 2, 1),
    ("varlen", None, 1836, 1836, 4, 2),
    ("shards", [(0, 1000, 0, 1000), (1000, 1000, 0, 3000), (2000, 700, 3000, 700)], 2700, 3700, 4, 2),
    ("mha odd group", None, 777, 777, 3, 3),
    ("gqa 8", None, 2048, 2048, 8, 1),
]


@pytest.mark.parametrize("name,tasks,Tq,Tk,Hq,Hkv", TASKSETS)
def test_flash_attention_fwd_bwd(name, tasks, Tq, Tk, Hq, Hkv):
    D = 128
    torch.manual_seed(1)
    if tasks is None:
        lens = {1836: [1000, 24, 512, 300], 777: [777], 2048: [2048]}[Tq]
        t = A.AttnTasks.from_doc_lens(lens)
    else:
        t = A.AttnTasks.from_lists(tasks)
    q, k, v, do = _bf(Tq, Hq, D), _bf(Tk, Hkv, D), _bf(Tk, Hkv, D), _bf(Tq, Hq, D)
    mask = torch.zeros(Tq, dtype=torch.bool, device="cuda")
    for qs, ql in zip(t.q_start, t.q_len):
        mask[int(qs):int(qs) + int(ql)] = True
    do[~mask] = 0
    plan = A.AttnPlan(t, "cuda")
    o, lse = A.flash_fwd(q, k, v, plan)
    dq, dk, dv = A.flash_bwd(q, k, v, o, lse, do, plan)
    _lib.check_status()
    oref, lref = A.attention_reference(q.float(), k.float(), v.float(), t)
    assert (o.float() - oref)[mask].abs().max().item() < 3e-2
    assert (lse - lref)[mask].abs().max().item() < 1e-3
    rq, rk, rv = A.attention_backward_reference(q.float(), k.float(), v.float(), do.float(), t)
    for got, want in ((dq.float()[mask], rq[mask]), (dk.float(), rk), (dv.float(), rv)):
        assert (got - want).abs().max().item() < 2e-2 * want.abs().max().item() + 2e-2
    # shipping rowsum(dO o O) instead of O gives the same gradients
    delta = A.attn_delta_rows(o, do)
    dq2, dk2, dv2 = A.flash_bwd(q, k, v, None, lse, do, plan, delta_rows=delta)
    # dK/dV are reduced inside one CTA (bit-reproducible); dQ sums tiles from several CTAs in
    # arrival order, so two runs may differ in the last bit
    assert torch.equal(dk2, dk) and torch.equal(dv2, dv)
    assert (dq2.float() - dq.float())[mask].abs().max().item() <= 1e-2 * dq.float()[mask].abs().max().item()
    # gradient rows stored through per-row destination addresses (the epilogues' store-to-owner path):
    # rows land permuted in other buffers, dV behind dK in one [K | V] row; an address of 0 skips the row
    qperm, kperm = torch.randperm(Tq, device="cuda"), torch.randperm(Tk, device="cuda")
    dq_buf = torch.zeros(Tq, Hq * D, dtype=torch.bfloat16, device="cuda")
    dkv_buf = torch.zeros(Tk, 2 * Hkv * D, dtype=torch.bfloat16, device="cuda")
    q_ptr = dq_buf.data_ptr() + qperm * (Hq * D * 2)
    kv_ptr = dkv_buf.data_ptr() + kperm * (2 * Hkv * D * 2)
    kv_ptr[3] = 0
    A.flash_bwd(q, k, v, None, lse, do, plan, delta_rows=delta, dq_row_ptr=q_ptr, dkv_row_ptr=kv_ptr,
                dv_off_bytes=Hkv * D * 2)
    _lib.check_status()
    got_dq = dq_buf[qperm].unflatten(1, (Hq, D))
    got_kv = dkv_buf[kperm]
    got_dk, got_dv = got_kv[:, :Hkv * D].unflatten(1, (Hkv, D)), got_kv[:, Hkv * D:].unflatten(1, (Hkv, D))
    assert (got_dq.float() - dq.float())[mask].abs().max().item() <= 1e-2 * dq.float()[mask].abs().max().item()
    kmask = torch.zeros(Tk, dtype=torch.bool, device="cuda")
    for ks, kl in zip(t.k_start, t.kv_len):
        kmask[int(ks):int(ks) + int(kl)] = True
    kmask[3] = False
    assert torch.equal(got_dk[kmask], dk[kmask]) and torch.equal(got_dv[kmask], dv[kmask])
    assert got_kv[3].abs().max().item() == 0


# ---------------------------------------------------------------- peer-memory helpers on one GPU
def test_arena_scatter_sum_and_bounded_wait():
    from distca_b200.parallel.p2p import PeerArena, SignalBoard, scatter_rows, sum_slots
    arena = PeerArena(8 << 20, None, "cuda")
    sig = SignalBoard(arena, 2)
    off = arena.alloc(64 * 256 * 2)
    dst = arena.view(off, (64, 256), torch.bfloat16)
    src = _bf(64, 256)
    perm = torch.randperm(64, device="cuda")
    addr = arena.addr(0, off) + perm.long() * 512
    addr[5] = 0
    scatter_rows(src, 512, addr)
    torch.cuda.synchronize()
    keep = torch.ones(64, dtype=torch.bool, device="cuda"); keep[5] = False
    assert torch.equal(dst[perm[keep]], src[keep]) and (dst[perm[5]] == 0).all()
    slots = _bf(3, 40, 64)
    valid = torch.zeros(40, 3, dtype=torch.int32, device="cuda")
    valid[::2, 1:] = -1
    valid[1::2, 2] = -1
    out = torch.empty(40, 64, dtype=torch.bfloat16, device="cuda")
    sum_slots(slots, valid, out)
    ref = slots[0].float().clone()
    ref[1::2] += slots[1, 1::2].float()
    assert _rel(out, ref) < 1e-2
    # a signal that arrives, then a wait on a flag nothing sets: the kernel gives up and reports
    sig.signal(0)
    sig.wait(0)
    torch.cuda.synchronize()
    _lib.check_status()
    sig.wait(1, target=1, max_polls=2000)
    torch.cuda.synchronize()
    with pytest.raises(_lib.KernelError):
        _lib.check_status()
    _lib.check_status()  # reading clears the word; the context is still usable
    arena.close()
