"""The kernels that read or write SEVERAL ranks' buffers (tensor-parallel GEMM fusion, data-parallel gradient
reduce-scatter, Adam with parameter all-gather), on ONE GPU: the "peers" are separate local buffers, which
exercises the same address tables, row-to-peer arithmetic and reductions as peer-mapped memory does, against
plain PyTorch fp32."""
import ctypes

import pytest
import torch

from distca_b200.ops import _lib
from distca_b200.ops import elementwise as ew
from distca_b200.ops import gemm

pytestmark = pytest.mark.gpu


def _bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-9)


def _tp_gemm(A, w, C, T, N, K, lda, a_peers=None, rows_a=0, c_peers=None, rows_c=0):
    ap = (ctypes.c_void_p * len(a_peers))(*[t.data_ptr() for t in a_peers]) if a_peers else None
    cp = (ctypes.c_void_p * len(c_peers))(*[t.data_ptr() for t in c_peers]) if c_peers else None
    rc = _lib.lib().dca_gemm_bf16_tp(
        _lib.ptr(A), _lib.ptr(w), _lib.ptr(C), _lib.c_int(T), _lib.c_int(N), _lib.c_int(K), _lib.c_long(lda),
        _lib.c_long(w.stride(0)), _lib.c_long(N), _lib.c_int(0), ap, _lib.c_int(len(a_peers) if a_peers else 0),
        _lib.c_long(rows_a), cp, _lib.c_int(len(c_peers) if c_peers else 0), _lib.c_long(rows_c),
        _lib.ptr(_lib.status_word("cuda")), _lib.stream_ptr())
    _lib.check_rc(rc, "gemm_tp")


@pytest.mark.parametrize("peers,rows,N,K", [(2, 256, 512, 256), (4, 128, 384, 512), (8, 384, 256, 128)])
def test_gemm_with_all_gather_in_the_operand_load(peers, rows, N, K):
    """A = row-wise concatenation of ``peers`` separate buffers, read tile by tile by the GEMM's TMA producer."""
    torch.manual_seed(0)
    shards = [_bf(rows, K) for _ in range(peers)]
    w = _bf(N, K, scale=0.1)
    out = torch.empty(peers * rows, N, dtype=torch.bfloat16, device="cuda")
    _tp_gemm(None, w, out, peers * rows, N, K, K, a_peers=shards, rows_a=rows)
    _lib.check_status()
    ref = torch.cat(shards).float() @ w.float().t()
    assert _rel(out, ref) < 1e-2


@pytest.mark.parametrize("peers,rows,N,K", [(2, 256, 512, 256), (4, 128, 256, 384)])
def test_gemm_with_reduce_scatter_in_the_epilogue(peers, rows, N, K):
    """Output row r is stored into buffer r // rows at local row r % rows (the scatter half of reduce-scatter);
    summing every "rank's" slot then gives the reduce-scattered result."""
    torch.manual_seed(1)
    T = peers * rows
    w = _bf(N, K, scale=0.1)
    xs = [_bf(T, K) for _ in range(peers)]                       # the activation of each tensor-parallel "rank"
    # slots[owner][source] : what source rank's GEMM stored for owner's rows
    slots = [[torch.zeros(rows, N, dtype=torch.bfloat16, device="cuda") for _ in range(peers)] for _ in range(peers)]
    for src in range(peers):
        _tp_gemm(xs[src], w, None, T, N, K, K, c_peers=[slots[owner][src] for owner in range(peers)], rows_c=rows)
    _lib.check_status()
    from distca_b200.parallel.p2p import sum_slots
    for owner in range(peers):
        got = torch.empty(rows, N, dtype=torch.bfloat16, device="cuda")
        sum_slots(torch.stack(slots[owner]), torch.zeros(rows, peers, dtype=torch.int32, device="cuda"), got)
        ref = sum(x[owner * rows:(owner + 1) * rows].float() @ w.float().t() for x in xs)
        assert _rel(got, ref) < 2e-2


def test_swiglu_gemm_reads_shards_of_several_peers():
    """FC1 with the all-gather in the operand load and SwiGLU in the epilogue."""
    torch.manual_seed(5)
    peers, rows, F, K = 4, 128, 384, 256
    T = peers * rows
    shards = [_bf(rows, K) for _ in range(peers)]
    w = _bf(2 * F, K, scale=0.1)
    act = torch.empty(T, F, dtype=torch.bfloat16, device="cuda")
    pre = torch.empty(T, 2 * F, dtype=torch.bfloat16, device="cuda")
    ap = (ctypes.c_void_p * peers)(*[t.data_ptr() for t in shards])
    rc = _lib.lib().dca_gemm_swiglu_tp(_lib.ptr(w), _lib.ptr(act), _lib.c_int(T), _lib.c_int(2 * F), _lib.c_int(K),
                                       _lib.c_long(K), _lib.c_long(w.stride(0)), _lib.c_long(F), _lib.ptr(pre),
                                       _lib.c_long(2 * F), ap, _lib.c_int(peers), _lib.c_long(rows),
                                       _lib.ptr(_lib.status_word("cuda")), _lib.stream_ptr())
    _lib.check_rc(rc, "gemm_ag_swiglu")
    _lib.check_status()
    ref_pre = torch.cat(shards).float() @ w.float().t()
    ref_act = torch.nn.functional.silu(ref_pre[:, :F]) * ref_pre[:, F:]
    assert _rel(pre, ref_pre) < 1e-2 and _rel(act, ref_act) < 2e-2


def test_qkv_rope_gemm_reads_shards_of_several_peers():
    torch.manual_seed(2)
    peers, rows, Hq, Hkv, D, K = 4, 128, 4, 2, 128, 256
    T, N = peers * rows, (Hq + 2 * Hkv) * D
    shards = [_bf(rows, K) for _ in range(peers)]
    w = _bf(N, K, scale=0.1)
    pos = torch.randint(0, 4000, (T,), device="cuda", dtype=torch.int32)
    table = ew.rope_table(4096, D, 500000.0, "cuda")
    ap = (ctypes.c_void_p * peers)(*[t.data_ptr() for t in shards])
    got = gemm.linear_qkv_rope(None, w, pos, table, Hq, Hkv, a_peers=ap, a_rows_per_peer=rows)
    _lib.check_status()
    ref = (torch.cat(shards).float() @ w.float().t()).to(torch.bfloat16).cpu().float()
    ref = ew.rope_(ref, pos.cpu(), table.cpu(), Hq, Hkv, D)
    assert _rel(got.cpu(), ref) < 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gradient_reduce_scatter_with_norm_partial(dtype):
    torch.manual_seed(3)
    peers, n = 4, 4096 * 8
    bufs = [(torch.randn(peers * n, device="cuda") * 0.1).to(dtype) for _ in range(peers)]
    ref_full = sum(b.float() for b in bufs)
    tbl = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device="cuda")
    L = _lib.lib()
    fn = L.dca_reduce_scatter_sumsq_f32 if dtype == torch.float32 else L.dca_reduce_scatter_sumsq_bf16
    for me in range(peers):
        sumsq = torch.zeros(1, device="cuda")
        before_other = [bufs[me][(p * n):(p + 1) * n].clone() for p in range(peers)]
        rc = fn(_lib.ptr(tbl), _lib.c_int(peers), _lib.c_int(me), _lib.c_long(me * n), _lib.c_long(n), _lib.ptr(sumsq),
                _lib.stream_ptr())
        _lib.check_rc(rc, "reduce_scatter_sumsq")
        want = ref_full[me * n:(me + 1) * n]
        got = bufs[me][me * n:(me + 1) * n]
        assert _rel(got, want) < (1e-2 if dtype == torch.bfloat16 else 1e-5)
        assert abs(sumsq.item() - want.pow(2).sum().item()) <= 1e-2 * want.pow(2).sum().item()
        for p in range(peers):          # only this rank's own shard was written
            if p != me:
                assert torch.equal(bufs[me][p * n:(p + 1) * n], before_other[p])


@pytest.mark.parametrize("gdtype", [torch.bfloat16, torch.float32])
def test_adam_with_parameter_all_gather(gdtype):
    """AdamW on one shard; the new bf16 values must appear at the shard's offset in every "peer's" flat buffer
    and equal the single-buffer kernel's result."""
    torch.manual_seed(4)
    peers, n, lo = 3, 2048 * 8, 1024 * 8
    total = lo + n + 512
    flats = [torch.zeros(total, dtype=torch.bfloat16, device="cuda") for _ in range(peers)]
    p0 = _bf(n, scale=0.05)
    g = (torch.randn(n, device="cuda") * 0.01).to(gdtype)
    hp = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01, step=1)
    # reference: the plain kernel on a private copy
    pr, lor = p0.clone(), torch.zeros(n, dtype=torch.int16, device="cuda")
    mr, vr = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    ew.adam_step_(pr, lor, g, mr, vr, **hp)
    me = 1
    flats[me][lo:lo + n] = p0
    lo16 = torch.zeros(n, dtype=torch.int16, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    tbl = torch.tensor([f.data_ptr() for f in flats], dtype=torch.int64, device="cuda")
    rc = _lib.lib().dca_adam_push(_lib.ptr(flats[me][lo:lo + n]), _lib.ptr(lo16), _lib.ptr(g),
                                  _lib.c_int(1 if gdtype == torch.float32 else 0), _lib.ptr(m), _lib.ptr(v), _lib.c_long(n),
                                  _lib.c_float(hp["lr"]), _lib.c_float(hp["beta1"]), _lib.c_float(hp["beta2"]),
                                  _lib.c_float(hp["eps"]), _lib.c_float(hp["weight_decay"]), _lib.c_int(1), None,
                                  _lib.ptr(tbl), _lib.c_int(peers), _lib.c_long(lo),
                                  _lib.ptr(_lib.status_word("cuda")), _lib.stream_ptr())
    _lib.check_rc(rc, "adam_push")
    _lib.check_status()
    for f in flats:
        assert torch.equal(f[lo:lo + n], pr)
        assert f[:lo].abs().max().item() == 0 and f[lo + n:].abs().max().item() == 0
    assert torch.equal(lo16, lor) and torch.allclose(m, mr) and torch.allclose(v, vr)
    # against fp32 AdamW from PyTorch
    w = p0.float().clone().requires_grad_(True)
    opt = torch.optim.AdamW([w], lr=hp["lr"], betas=(hp["beta1"], hp["beta2"]), eps=hp["eps"], weight_decay=hp["weight_decay"])
    w.grad = g.float()
    opt.step()
    assert _rel(ew.master_from_split(pr, lor), w.detach()) < 1e-5


def test_adam_skips_the_update_when_the_status_word_is_set():
    n = 4096
    p, lo16 = _bf(n), torch.zeros(n, dtype=torch.int16, device="cuda")
    g, m, v = _bf(n), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    before = p.clone()
    st = _lib.status_word("cuda")
    st[0] = 3                      # as left by a failed bounds check earlier in the step
    try:
        ew.adam_step_(p, lo16, g, m, v, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0, step=1)
        torch.cuda.synchronize()
        assert torch.equal(p, before) and m.abs().max().item() == 0
    finally:
        st.zero_()
    ew.adam_step_(p, lo16, g, m, v, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0, step=1)
    assert not torch.equal(p, before)


def test_push_shard_to_every_peer():
    peers, n, lo = 4, 4096, 8192
    flats = [torch.zeros(lo + n + 64, dtype=torch.bfloat16, device="cuda") for _ in range(peers)]
    src = _bf(n)
    tbl = torch.tensor([f.data_ptr() for f in flats], dtype=torch.int64, device="cuda")
    rc = _lib.lib().dca_push_shard(_lib.ptr(src), _lib.ptr(tbl), _lib.c_int(peers), _lib.c_int(2), _lib.c_long(lo * 2),
                                   _lib.c_long(n * 2), _lib.stream_ptr())
    _lib.check_rc(rc, "push_shard")
    for i, f in enumerate(flats):
        if i == 2:
            assert f.abs().max().item() == 0          # the sender's own buffer is not touched
        else:
            assert torch.equal(f[lo:lo + n], src) and f[:lo].abs().max().item() == 0
