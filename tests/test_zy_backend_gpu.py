"""The reference-named operator layers on a GPU: the same calls as tests/test_backend_cpu.py, on bf16 CUDA tensors,
against plain fp32 PyTorch."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(shape, seed, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).cuda()


def _rel(out, ref):
    return (out.float() - ref.float()).abs().max().item() / (ref.float().abs().max().item() + 1e-6)


@pytest.mark.parametrize("trans_a", [False, True])
@pytest.mark.parametrize("trans_b", [False, True])
@pytest.mark.parametrize("m1", [72, 0])
def test_dual_gemm_separated_all_layouts(trans_a, trans_b, m1):
    from wallx_b200.ops import backend as BE

    k = 136
    ins, ws, want = [], [], []
    for i, (m, n) in enumerate([(200, 328), (m1, 136)]):
        a, w = _mk((m, k), 2 * i), _mk((k, n), 2 * i + 1, 0.2)
        want.append(a.float() @ w.float())
        ins.append(a.t().contiguous() if trans_a else a)
        ws.append(w.t().contiguous() if trans_b else w)
    o0 = torch.empty(200, 328, device="cuda", dtype=torch.bfloat16)
    r0, r1 = BE.asym_dual_gmm_separated(ins[0], ins[1], ws[0], ws[1], o0, None, trans_a, trans_b)
    assert r0 is o0 and r1.shape == (m1, 136)
    assert _rel(r0, want[0]) < 1e-2
    if m1:
        assert _rel(r1, want[1]) < 1e-2


@pytest.mark.parametrize("trans_b", [False, True])
def test_dual_gemm_autograd_class(trans_b):
    from wall_x.fusions.ops import AsymmetricDualExpertGemm, asym_dual_gmm

    k = 256
    a = [_mk((264, k), 1).requires_grad_(), _mk((40, k), 2).requires_grad_()]
    w = [_mk((512, k) if trans_b else (k, 512), 3, 0.1).requires_grad_(), _mk((128, k) if trans_b else (k, 128), 4, 0.1).requires_grad_()]
    o0, o1 = asym_dual_gmm(a[0], a[1], w[0], w[1], trans_b)
    p0, p1 = AsymmetricDualExpertGemm.apply(a[0], a[1], w[0], w[1], trans_b)
    assert torch.equal(o0, p0) and torch.equal(o1, p1)
    g = [_mk(tuple(o0.shape), 5), _mk(tuple(o1.shape), 6)]
    torch.autograd.backward([o0, o1], g)
    for i in range(2):
        af, wf = a[i].detach().float().requires_grad_(), w[i].detach().float().requires_grad_()
        of = af @ (wf.t() if trans_b else wf)
        of.backward(g[i].float())
        assert _rel((o0, o1)[i], of.detach()) < 1e-2
        assert _rel(a[i].grad, af.grad) < 1e-2 and _rel(w[i].grad, wf.grad) < 1e-2


def test_multimodal_rope_class_forward_backward():
    from wall_x.fusions.ops import MultimodalRoPE, multimodal_rope
    from wallx_b200.ops import ref

    torch.manual_seed(0)
    B, Hq, Hk, S, D, sections = 2, 16, 2, 37, 128, [16, 24, 24]
    pos = torch.randint(0, 400, (3, B, S)).float()
    inv = ref.rope_inv_freq(D, 1e6)
    ang = torch.cat([pos.unsqueeze(-1) * inv, pos.unsqueeze(-1) * inv], dim=-1).cuda()
    cos, sin = ang.cos(), ang.sin()
    q = _mk((B, Hq, S, D), 1).requires_grad_()
    k = _mk((B, Hk, S, D), 2).requires_grad_()
    qo, ko = MultimodalRoPE.apply(q, k, cos, sin, sections)
    ax = ref.mrope_axis_of_channel(D, sections, "wallx_cuda").cuda()
    sel = ax.view(1, 1, 1, D).expand(1, B, S, D)
    c = cos.gather(0, sel).squeeze(0).unsqueeze(1)
    s = sin.gather(0, sel).squeeze(0).unsqueeze(1)

    def plain(x):
        return x * c + torch.cat((-x[..., D // 2:], x[..., : D // 2]), dim=-1) * s

    qf, kf = q.detach().float().requires_grad_(), k.detach().float().requires_grad_()
    qe, ke = plain(qf), plain(kf)
    assert _rel(qo, qe.detach()) < 1e-2 and _rel(ko, ke.detach()) < 1e-2
    gq, gk = _mk(tuple(qo.shape), 3), _mk(tuple(ko.shape), 4)
    torch.autograd.backward([qo, ko], [gq, gk])
    torch.autograd.backward([qe, ke], [gq.float(), gk.float()])
    assert _rel(q.grad, qf.grad) < 1e-2 and _rel(k.grad, kf.grad) < 1e-2
    q2, k2 = multimodal_rope(q.detach(), k.detach(), cos, sin, sections)
    assert torch.equal(q2, qo.detach()) and torch.equal(k2, ko.detach())


@pytest.mark.parametrize("K", [1, 2])
def test_topk_permute_unpermute_on_gpu_matches_cpu(K):
    from wall_x.fusions.ops import permute, unpermute

    torch.manual_seed(K)
    T, C = 301, 256
    x = torch.randn(T, C)
    idx = torch.randint(0, 2, (T, K)) if K > 1 else torch.randint(0, 2, (T,))
    probs = torch.rand(T, K)
    outs = []
    for dev in ("cpu", "cuda"):
        xd = x.clone().to(dev).requires_grad_()
        pd = probs.clone().to(dev).requires_grad_()
        y, m = permute(xd, idx.to(dev))
        o = unpermute(y * 2.0, m, pd)
        o.backward(torch.ones_like(o))
        outs.append((y.detach().cpu(), m.cpu(), o.detach().cpu(), xd.grad.cpu(), pd.grad.cpu()))
    for a, b in zip(*outs):
        assert torch.allclose(a.float(), b.float(), atol=1e-5)


def test_top1_permute_of_bf16_rows_uses_the_row_kernels_and_matches_indexing():
    from wall_x.fusions.ops import permute, unpermute
    from wallx_b200.ops import backend as BE

    torch.manual_seed(0)
    T, C = 1000, 2048
    x = _mk((T, C), 1)
    idx = (torch.rand(T) < 0.2).long().cuda()
    assert BE._row_kernels_apply(x)
    xg = x.clone().requires_grad_()
    y, m = permute(xg, idx)
    want_pos = BE.sorted_rows(idx).reshape(-1)
    want = torch.empty_like(x)
    want[want_pos] = x
    assert m.dtype == torch.int32 and torch.equal(m.long(), want_pos) and torch.equal(y.detach(), want)
    back = unpermute(y, m)
    assert torch.equal(back.detach(), x)
    g = _mk((T, C), 2)
    back.backward(g)
    assert torch.equal(xg.grad, g)  # permutation followed by its inverse


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
def test_gemm_bits_do_not_depend_on_the_tile_schedule(a_mn, b_mn):
    """Race check by replay: every output element accumulates its k blocks in the same order whatever the tile
    width, the CTA pairing or the raster, so all schedules must agree bit for bit (and with themselves)."""
    from wallx_b200.ops import gemm as G

    M, N, K = 1000, 1280, 1176
    a = _mk((K, M) if a_mn else (M, K), 11)
    b = _mk((K, N) if b_mn else (N, K), 12, 0.1)
    outs = [G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, force_bn=bn) for bn in (64, 128, 256, 512, 0, 256)]
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
