"""Each sm_100a kernel against the plain PyTorch fp32 oracle of the same op."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bf(x):
    return x.to(torch.bfloat16).cuda()


def _close(a, b, atol, rtol=2e-2, what=""):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs()
    lim = atol + rtol * b.abs()
    bad = (err > lim).float().mean().item()
    assert bad < 1e-3, f"{what}: {bad * 100:.3f}% elements off, max err {err.max().item():.4g}"


def test_rms_norm_fwd_bwd():
    from wallx_b200.ops import functional as F_, ref

    torch.manual_seed(0)
    for T, C in [(300, 2048), (77, 1280), (5, 256)]:
        x = torch.randn(T, C)
        w = torch.randn(C) * 0.1 + 1.0
        xb, wb = _bf(x).requires_grad_(), _bf(w).requires_grad_()
        y = F_.rms_norm(xb, wb, 1e-6)
        xr, wr = xb.detach().float().cpu().requires_grad_(), wb.detach().float().cpu().requires_grad_()
        yr = ref.rms_norm(xr, wr, 1e-6)
        _close(y, yr, 2e-2, what="rms fwd")
        g = torch.randn(T, C)
        y.backward(_bf(g))
        yr.backward(_bf(g).float().cpu())
        _close(xb.grad, xr.grad, 3e-2, what="rms dx")
        _close(wb.grad, wr.grad, 0.3, 3e-2, what="rms dw")


def test_rms_norm_fused_permute():
    from wallx_b200.ops import functional as F_, ref

    torch.manual_seed(1)
    T, C = 333, 512
    types = (torch.rand(T) < 0.3).long()
    plan = F_.make_route_plan(types.cuda(), 2)
    dest_ref, seg_ref = ref.route_plan(types, 2, 128)
    assert torch.equal(plan.dest.cpu().long(), dest_ref)
    assert plan.seg.cpu()[:, :2].tolist() == seg_ref[:, :2].tolist()
    inv = plan.inv.cpu()
    assert (inv[dest_ref] == torch.arange(T)).all() and (inv >= 0).sum() == T
    x = torch.randn(T, C)
    w = torch.ones(C)
    xb = _bf(x).requires_grad_()
    yp = F_.rms_norm(xb, _bf(w), 1e-6, dest=plan.dest, out_rows=plan.rows)
    yr = ref.permute_rows(ref.rms_norm(xb.detach().float().cpu(), w, 1e-6), dest_ref, plan.rows)
    _close(yp, yr, 2e-2, what="rms+permute")
    g = torch.randn(plan.rows, C)
    yp.backward(_bf(g))
    xr = xb.detach().float().cpu().requires_grad_()
    ref.permute_rows(ref.rms_norm(xr, w, 1e-6), dest_ref, plan.rows).backward(_bf(g).float().cpu())
    _close(xb.grad, xr.grad, 3e-2, what="rms+permute dx")


@pytest.mark.parametrize("layout", ["hf", "wallx_cuda"])
def test_rope_qk(layout):
    from wallx_b200.ops import functional as F_, ref

    torch.manual_seed(2)
    T, hq, hkv, D = 200, 4, 2, 128
    qkv = torch.randn(T, (hq + 2 * hkv) * D)
    pos3 = torch.randint(0, 500, (3, T))
    cos, sin = ref.mrope_cos_sin(pos3, ref.rope_inv_freq(D, 1e6), [16, 24, 24], layout)
    qb = _bf(qkv).requires_grad_()
    out = F_.rope_qk(qb, cos.cuda().contiguous(), sin.cuda().contiguous(), hq + hkv, D)
    qr = qb.detach().float().cpu().requires_grad_()
    outr = F_.rope_qk(qr, cos, sin, hq + hkv, D)
    _close(out, outr, 2e-2, what="rope fwd")
    g = torch.randn_like(qkv)
    out.backward(_bf(g))
    outr.backward(_bf(g).float().cpu())
    _close(qb.grad, qr.grad, 2e-2, what="rope bwd")


def test_gate_up_swiglu_and_linear_grads():
    from wallx_b200.models.layers import SwiGLUFFN

    torch.manual_seed(3)
    ffn = SwiGLUFFN(256, 340, bias=True)
    ffn.reset_parameters(0.05)
    with torch.no_grad():
        ffn.gate_up_bias.normal_(0, 0.1)
        gb, ub = ffn.unpack_gate_up(ffn.gate_up_bias.data)
        ffn.gate_up_bias.copy_(ffn.pack_gate_up(gb, ub))  # keep padding zero
        ffn.down_bias.normal_(0, 0.1)
    import copy

    ffn_c = copy.deepcopy(ffn).cuda().to(torch.bfloat16)
    ffn_r = copy.deepcopy(ffn_c).float().cpu()
    x = torch.randn(150, 256)
    xb = _bf(x).requires_grad_()
    xr = xb.detach().float().cpu().requires_grad_()
    y = ffn_c(xb, residual=xb)
    yr = ffn_r(xr, residual=xr)
    _close(y, yr, 3e-2, what="ffn fwd")
    g = torch.randn_like(x)
    y.backward(_bf(g))
    yr.backward(_bf(g).float().cpu())
    _close(xb.grad, xr.grad, 5e-2, what="ffn dx")
    for (n, pc), (_, pr) in zip(ffn_c.named_parameters(), ffn_r.named_parameters()):
        _close(pc.grad, pr.grad, 0.15, 5e-2, what=f"ffn d{n}")


@pytest.mark.parametrize("frac", [0.0, 0.1, 0.5, 1.0])
def test_moe_ffn_fwd_bwd(frac):
    from wallx_b200.models.layers import SwiGLUFFN
    from wallx_b200.ops import functional as F_
    import copy

    torch.manual_seed(4)
    T, H = 700, 256
    experts = [SwiGLUFFN(H, 512), SwiGLUFFN(H, 192)]
    for e in experts:
        e.reset_parameters(0.05)
    ec = [copy.deepcopy(e).cuda().to(torch.bfloat16) for e in experts]
    er = [copy.deepcopy(e).float().cpu() for e in ec]
    types = (torch.rand(T) < frac).long()
    x = torch.randn(T, H)
    wn = torch.ones(H)

    def run(xin, exps, dev):
        plan = F_.make_route_plan(types.to(dev), 2)
        xp = F_.rms_norm(xin, wn.to(dev, xin.dtype), 1e-6, dest=plan.dest, out_rows=plan.rows)
        return F_.moe_ffn(xp, xin, plan, [e.weights() for e in exps])

    xb = _bf(x).requires_grad_()
    xr = xb.detach().float().cpu().requires_grad_()
    y, yr = run(xb, ec, "cuda"), run(xr, er, "cpu")
    _close(y, yr, 3e-2, what="moe fwd")
    g = torch.randn_like(x)
    y.backward(_bf(g))
    yr.backward(_bf(g).float().cpu())
    _close(xb.grad, xr.grad, 5e-2, what="moe dx")
    for e_c, e_r in zip(ec, er):
        for (n, pc), (_, pr) in zip(e_c.named_parameters(), e_r.named_parameters()):
            gr = pr.grad if pr.grad is not None else torch.zeros_like(pr)
            _close(pc.grad, gr, 0.2, 5e-2, what=f"moe d{n}")
    from wallx_b200.ops import gemm as G
    G.check_status()


def _attn_case(cu, hq, hkv, D, causal, bidir_frac=0.0, seed=0):
    from wallx_b200.ops import functional as F_

    torch.manual_seed(seed)
    T = cu[-1]
    W = (hq + 2 * hkv) * D
    qkv = torch.randn(T, W) * 0.7
    bidir = None
    if bidir_frac > 0:
        bidir = torch.zeros(T, dtype=torch.bool)
        for i in range(len(cu) - 1):
            n = int((cu[i + 1] - cu[i]) * bidir_frac)
            if n:
                bidir[cu[i + 1] - n:cu[i + 1]] = True
    qb = _bf(qkv).requires_grad_()
    qr = qb.detach().float().cpu().requires_grad_()
    mc = F_.AttnMeta(cu, "cuda", causal, bidir.cuda() if bidir is not None else None)
    mr = F_.AttnMeta(cu, "cpu", causal, bidir)
    o = F_.attention_packed(qb, mc, hq, hkv, D)
    orf = F_.attention_packed(qr, mr, hq, hkv, D)
    _close(o, orf, 2e-2, what="attn fwd")
    g = torch.randn(T, hq * D)
    o.backward(_bf(g))
    orf.backward(_bf(g).float().cpu())
    _close(qb.grad[:, : hq * D], qr.grad[:, : hq * D], 3e-2, 3e-2, what="attn dq")
    _close(qb.grad[:, hq * D:(hq + hkv) * D], qr.grad[:, hq * D:(hq + hkv) * D], 4e-2, 3e-2, what="attn dk")
    _close(qb.grad[:, (hq + hkv) * D:], qr.grad[:, (hq + hkv) * D:], 4e-2, 3e-2, what="attn dv")
    from wallx_b200.ops import gemm as G
    G.check_status()


def test_attention_causal_gqa():
    _attn_case([0, 350, 700, 913], 16, 2, 128, True)


def test_attention_causal_bidirectional_block():
    _attn_case([0, 97, 97 + 346, 97 + 346 + 130], 4, 2, 128, True, bidir_frac=0.1)


def test_attention_vit_windows_hd80():
    cu = [0]
    for n in [64, 64, 32, 64, 16, 4, 64, 324, 100]:
        cu.append(cu[-1] + n)
    _attn_case(cu, 4, 4, 80, False)


def test_attention_small_hd64():
    _attn_case([0, 35, 70], 4, 2, 64, True, bidir_frac=0.4)


def test_attention_prefix_cache_rule():
    """Few new queries against a longer key range (bottom-right aligned causal + bidirectional)."""
    from wallx_b200.ops import functional as F_

    torch.manual_seed(5)
    hq, hkv, D = 8, 2, 128
    lens_k, lq = [300, 211], 32
    cu_k, cu_q = [0, 300, 511], [0, 32, 64]
    q = torch.randn(64, hq * D)
    k = torch.randn(511, hkv * D)
    v = torch.randn(511, hkv * D)
    for causal, bid in [(True, False), (True, True), (False, False)]:
        bq = torch.ones(64, dtype=torch.bool) if bid else None
        bk = torch.zeros(511, dtype=torch.bool)
        bk[300 - 32:300] = True
        bk[511 - 32:] = True
        mc = F_.AttnMeta(cu_q, "cuda", causal, bq.cuda() if bid else None, cu_k=cu_k, bidir_k=bk.cuda() if bid else None)
        mr = F_.AttnMeta(cu_q, "cpu", causal, bq, cu_k=cu_k, bidir_k=bk if bid else None)
        o = F_.attention(_bf(q), _bf(k), _bf(v), mc, hq, hkv, D)
        orf = F_.attention(_bf(q).float().cpu(), _bf(k).float().cpu(), _bf(v).float().cpu(), mr, hq, hkv, D)
        _close(o, orf, 2e-2, what=f"prefix attn causal={causal} bidir={bid}")


@pytest.mark.parametrize("V", [5000, 5002])  # 5002: vocabulary size that is not a multiple of 8 (as 153986 is not)
def test_lm_head_ce(V):
    from wallx_b200.ops import functional as F_, ref

    torch.manual_seed(6)
    R, H = 300, 256
    h = torch.randn(R, H)
    w = torch.randn(V, H) * 0.05
    labels = torch.randint(0, V, (R,))
    labels[::7] = -100
    hb, wb = _bf(h).requires_grad_(), _bf(w).requires_grad_()
    loss, pred = F_.lm_head_ce(hb, wb, labels.cuda())
    hr, wr = hb.detach().float().cpu().requires_grad_(), wb.detach().float().cpu().requires_grad_()
    lossr, predr = ref.lm_head_ce(hr, wr, labels)
    _close(loss, lossr, 3e-2, what="ce loss")
    assert (pred.cpu() == predr).float().mean() > 0.97
    loss.sum().backward()
    lossr.sum().backward()
    _close(hb.grad, hr.grad, 2e-2, 5e-2, what="ce dh")
    _close(wb.grad, wr.grad, 2e-2, 5e-2, what="ce dw")


def test_adamw_matches_torch():
    from wallx_b200.ops import _ext

    C = _ext.get()
    torch.manual_seed(7)
    n = 100003
    p = torch.randn(n)
    g = torch.randn(n) * 0.1
    pr = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([pr], lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1)
    p32, m, v = p.clone().cuda(), torch.zeros(n).cuda(), torch.zeros(n).cuda()
    p16 = p32.to(torch.bfloat16)
    for step in range(1, 4):
        gb = _bf(g * step)
        pr.grad = gb.float().cpu()
        opt.step()
        hyper = torch.tensor([1e-3, 0.9, 0.999, 1e-8, 0.1, 1 - 0.9 ** step, 1 - 0.999 ** step, -1.0, 1.0], device="cuda")
        C.adamw_step(p16, p32, m, v, gb, hyper, None)
    assert torch.allclose(p32.cpu(), pr.detach(), atol=2e-5, rtol=1e-4)
    assert torch.equal(p16, p32.to(torch.bfloat16))
    nsq = torch.zeros(1, device="cuda")
    C.sumsq_bf16(_bf(g), nsq)
    assert abs(nsq.item() - (_bf(g).float() ** 2).sum().item()) / nsq.item() < 1e-3


def test_index_kernels_match_python_originals():
    from wallx_b200.ops import index as IX, ref

    IMG, VID, VS = 900, 901, 902
    torch.manual_seed(8)
    grids = [[1, 18, 18], [1, 8, 12], [1, 4, 4], [2, 6, 8]]
    vgrids = [[3, 4, 6]]
    n = lambda g: g[0] * (g[1] // 2) * (g[2] // 2)
    rows = [
        [5, 6, VS] + [IMG] * n(grids[0]) + [7] * 5 + [VS] + [IMG] * n(grids[1]) + [9, 9],
        [11] * 9,
        [VS] + [IMG] * n(grids[2]) + [8, 8, VS] + [VID] * n(vgrids[0]) + [3] + [VS] + [IMG] * n(grids[3]) + [4] * 7,
    ]
    S = max(len(r) for r in rows)
    ids = torch.zeros((3, S), dtype=torch.long)
    am = torch.zeros((3, S), dtype=torch.long)
    for i, r in enumerate(rows):  # left padding
        ids[i, S - len(r):] = torch.tensor(r)
        am[i, S - len(r):] = 1
    ig, vg = torch.tensor(grids), torch.tensor(vgrids)
    spg = torch.tensor([0.5])
    pos_r, d_r = ref.rope_index(ids, ig, vg, spg, am, 2, IMG, VID, VS, 2.0)
    pos_c, d_c = IX.get_rope_index(ids.cuda(), ig.cuda(), vg.cuda(), spg.cuda(), am.cuda(), 2, IMG, VID, VS, 2.0)
    assert torch.equal(pos_c.cpu(), pos_r) and torch.equal(d_c.cpu(), d_r)
    inv = 1.0 / (10000.0 ** (torch.arange(0, 40, 2).float() / 40))
    a_r = ref.rot_pos_emb(inv, grids, 2)
    a_c = IX.rot_pos_emb(inv.cuda(), ig.cuda(), 2)
    assert torch.allclose(a_c.cpu(), a_r, atol=1e-6)
    w_r, cu_r = ref.window_index(grids + [[1, 16, 16]], 112, 2, 14)
    w_c, cu_c = IX.get_window_index(torch.tensor(grids + [[1, 16, 16]]).cuda(), 112, 2, 14)
    assert torch.equal(w_c.cpu(), w_r) and cu_c.cpu().tolist() == cu_r


@pytest.mark.parametrize("R,C", [(1000, 3840), (31, 2560), (70000, 64), (513, 1282), (5, 7)])
def test_column_sum_matches_fp32_and_is_reproducible(R, C):
    """Bias-gradient reduction: 16-byte path (C % 8 == 0) and the generic path, equal bits on repeated calls."""
    from wallx_b200.ops import _ext

    torch.manual_seed(3)
    x = torch.randn(R, C, device="cuda").to(torch.bfloat16)
    a = _ext.get().column_sum(x)
    b = _ext.get().column_sum(x)
    assert torch.equal(a, b)
    ref = x.float().sum(0)
    assert torch.allclose(a.float(), ref, atol=0.02 * (R ** 0.5) + 0.05, rtol=2e-2)
