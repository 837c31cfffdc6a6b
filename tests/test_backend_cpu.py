"""The reference-named operator layers (wall_x.fusions.ops classes, wall_x.fusions.backend functions) on CPU."""
import pytest
import torch

from wallx_b200.ops import backend as BE
from wallx_b200.ops import compat as C
from wallx_b200.ops import ref


def _naive_permute(x, indices):
    idx = indices.reshape(indices.shape[0], -1)
    T, K = idx.shape
    pairs = sorted(((int(idx[t, k]), t * K + k) for t in range(T) for k in range(K)))
    out = torch.stack([x[i // K] for _, i in pairs])
    row_of = {i: r for r, (_, i) in enumerate(pairs)}
    return out, row_of


@pytest.mark.parametrize("K", [1, 2, 3])
def test_permute_unpermute_topk_values_and_gradients(K):
    torch.manual_seed(K)
    T, Cn, E = 13, 6, 4
    x = torch.randn(T, Cn, dtype=torch.float64, requires_grad=True)
    indices = torch.randint(0, E, (T, K)) if K > 1 else torch.randint(0, E, (T,))
    probs = torch.rand(T, K, dtype=torch.float64, requires_grad=True)
    y, row_id_map = C.permute(x, indices)
    want, row_of = _naive_permute(x.detach(), indices)
    assert torch.equal(y.detach(), want)
    assert row_id_map.dtype == torch.int32 and row_id_map.numel() == T * K
    for t in range(T):
        for k in range(K):
            assert int(row_id_map[k * T + t]) == row_of[t * K + k]
    # expert-wise processing stand-in, then the weighted inverse
    w = torch.randn(Cn, Cn, dtype=torch.float64)
    out = C.unpermute(torch.tanh(y @ w), row_id_map, probs)
    # the same computation with plain indexing
    x2 = x.detach().clone().requires_grad_(True)
    p2 = probs.detach().clone().requires_grad_(True)
    rows = row_id_map.view(K, T).long()
    z = torch.tanh(x2 @ w)  # row-wise op commutes with the permutation
    expect = sum(p2[:, k:k + 1] * z for k in range(K))
    assert torch.allclose(out, expect, rtol=0, atol=1e-12)
    g = torch.randn_like(out)
    out.backward(g)
    expect.backward(g)
    assert torch.allclose(x.grad, x2.grad, rtol=0, atol=1e-10)
    assert torch.allclose(probs.grad, p2.grad, rtol=0, atol=1e-10)
    assert rows.max() == T * K - 1


def test_permute_with_dropped_rows_and_unweighted_inverse():
    torch.manual_seed(0)
    T, Cn = 9, 4
    x = torch.randn(T, Cn)
    indices = torch.tensor([1, 0, 1, 1, 0, 0, 1, 0, 1])
    y, m = BE.permute(x, indices, num_out_tokens=6)
    assert y.shape == (6, Cn)
    back = BE.unpermute(y, m)
    kept = m.long() < 6
    assert torch.equal(back[kept], x[kept]) and back[~kept].abs().sum() == 0
    dx, dp = BE.unpermute_bwd(torch.ones(T, Cn), y, m, None)
    assert dp is None and torch.equal(dx, torch.ones(6, Cn))
    # empty input passes through
    e, none = C.PermuteMoE_topK.apply(torch.empty(0, Cn), torch.empty(0, dtype=torch.long), 0, 0)
    assert e.numel() == 0 and none is None


def _rope_plain(x, cos3, sin3, sections):
    """x [B, H, S, D]; contiguous channel-to-axis rule; plain PyTorch, differentiable."""
    D = x.shape[-1]
    ax = ref.mrope_axis_of_channel(D, sections, "wallx_cuda")
    sel = ax.view(1, 1, 1, D).expand(1, *cos3.shape[1:])
    c = cos3.gather(0, sel).squeeze(0).unsqueeze(1)  # [B, 1, S, D]
    s = sin3.gather(0, sel).squeeze(0).unsqueeze(1)
    h = D // 2
    return x * c + torch.cat((-x[..., h:], x[..., :h]), dim=-1) * s


def test_multimodal_rope_class_matches_plain_forward_and_backward():
    torch.manual_seed(0)
    B, Hq, Hk, S, D, sections = 2, 3, 1, 5, 16, [2, 3, 3]
    pos = torch.randint(0, 30, (3, B, S)).float()
    inv = ref.rope_inv_freq(D, 1e4)
    ang = torch.cat([pos.unsqueeze(-1) * inv, pos.unsqueeze(-1) * inv], dim=-1)  # [3, B, S, D]
    cos, sin = ang.cos(), ang.sin()
    q = torch.randn(B, Hq, S, D, requires_grad=True)
    k = torch.randn(B, Hk, S, D, requires_grad=True)
    qo, ko = C.MultimodalRoPE.apply(q, k, cos, sin, sections)
    q2, k2 = q.detach().clone().requires_grad_(True), k.detach().clone().requires_grad_(True)
    qe, ke = _rope_plain(q2, cos, sin, sections), _rope_plain(k2, cos, sin, sections)
    assert torch.allclose(qo, qe, atol=1e-6) and torch.allclose(ko, ke, atol=1e-6)
    gq, gk = torch.randn_like(qo), torch.randn_like(ko)
    torch.autograd.backward([qo, ko], [gq, gk])
    torch.autograd.backward([qe, ke], [gq, gk])
    assert torch.allclose(q.grad, q2.grad, atol=1e-6) and torch.allclose(k.grad, k2.grad, atol=1e-6)
    # the functional form agrees with the class
    qf, kf = C.multimodal_rope(q.detach(), k.detach(), cos, sin, sections)
    assert torch.allclose(qf, qo.detach(), atol=1e-6) and torch.allclose(kf, ko.detach(), atol=1e-6)
    with pytest.raises(ValueError):
        BE.rope(q.detach(), k.detach(), cos, sin, torch.empty_like(q), torch.empty_like(k), [4, 4, 4])


@pytest.mark.parametrize("trans_a", [False, True])
@pytest.mark.parametrize("trans_b", [False, True])
def test_dual_gemm_separated_layouts_and_caller_outputs(trans_a, trans_b):
    torch.manual_seed(0)
    k, dims = 8, [(5, 7), (0, 3)]  # the second expert is empty
    ins, ws, want = [], [], []
    for m, n in dims:
        a, w = torch.randn(m, k), torch.randn(k, n)
        want.append(a @ w)
        ins.append(a.t().contiguous() if trans_a else a)
        ws.append(w.t().contiguous() if trans_b else w)
    o0 = torch.empty(5, 7)
    r0, r1 = BE.asym_dual_gmm_separated(ins[0], ins[1], ws[0], ws[1], o0, None, trans_a, trans_b)
    assert r0 is o0 and torch.allclose(r0, want[0], atol=1e-5) and r1.shape == (0, 3)
    with pytest.raises(ValueError):
        BE.asym_dual_gmm_separated(ins[0], ins[1], ws[0], ws[1], torch.empty(4, 7), None, trans_a, trans_b)
    if not trans_a:
        f0, f1 = C.asym_dual_gmm(ins[0], ins[1], ws[0], ws[1], trans_b)
        assert torch.allclose(f0, want[0], atol=1e-5) and f1.shape == (0, 3)


def test_index_entry_points_and_reference_module_paths():
    import wall_x.fusions.backend as rb
    import wall_x.fusions.ops as ro

    for name in ("asym_dual_gmm_separated", "permute", "unpermute", "unpermute_bwd", "rope", "rope_bwd", "get_rope_index",
                 "rot_pos_emb", "get_window_index"):
        assert callable(getattr(rb, name)), name
    for name in ("AsymmetricDualExpertGemm", "PermuteMoE_topK", "UnpermuteMoE_topK", "MultimodalRoPE", "asym_dual_gmm",
                 "permute", "unpermute", "multimodal_rope", "get_rope_index", "rot_pos_emb", "get_window_index"):
        assert hasattr(ro, name), name
    grid = torch.tensor([[1, 18, 18], [1, 8, 8]])
    a_idx, a_cu = ro.get_window_index(grid, 112, 2, 14)
    b_idx, b_cu = rb.get_window_index(grid, 2, 112 // 2 // 14, 14, 4)  # backend form: pre-divided window size
    assert torch.equal(a_idx, b_idx) and torch.equal(torch.as_tensor(a_cu), torch.as_tensor(b_cu))
    inv = ref.rope_inv_freq(8, 1e4)
    assert torch.equal(rb.rot_pos_emb(inv, grid, 2), ro.rot_pos_emb(inv, grid, 2))
    ids = torch.randint(5, 100, (2, 9))
    am = torch.ones(2, 9, dtype=torch.long)
    p1, d1 = rb.get_rope_index(ids, None, None, None, am, 2, 900, 901, 902, 2.0)
    p2, d2 = ro.get_rope_index(ids, None, None, None, am, 2, 900, 901, 902, 2.0)
    assert torch.equal(p1, p2) and torch.equal(d1, d2)


def test_inference_kernel_region_needs_both_the_region_and_grad_mode_off():
    """Launches may pick inference-only kernels only inside an ``inference_kernels`` region with autograd off: grad mode
    alone says nothing (autograd functions run forward and backward with it off)."""
    import torch

    from wallx_b200.ops import gemm as G

    assert not G._inference_launch()
    with torch.no_grad():
        assert not G._inference_launch()
        with G.inference_kernels():
            assert G._inference_launch()
            with G.inference_kernels():  # re-entrant
                assert G._inference_launch()
            assert G._inference_launch()
        assert not G._inference_launch()
    with G.inference_kernels():
        assert not G._inference_launch()  # autograd on: a training step

    @G.inference_kernels()
    def f():
        with torch.no_grad():
            return G._inference_launch()

    assert f() and not G._inference_launch()

    # the region belongs to the thread that opened it
    import threading

    seen = []

    def other():
        with torch.no_grad():
            seen.append(G._inference_launch())

    with torch.no_grad(), G.inference_kernels():
        t = threading.Thread(target=other)
        t.start()
        t.join()
    assert seen == [False]


def test_copy_cta_count_for_fused_gathers():
    """Weights of a training engine take the default count; stand-alone sharded weights at least 16, more when the
    multiplication is short against the bytes that must arrive, never more than 32, always even."""
    from wallx_b200.parallel import ag_linear as A
    from wallx_b200.parallel.zero3 import GatheredWeight

    class Spec:
        def __init__(self, M, N, K):
            self.M, self.N, self.K = M, N, K

    def standalone(rows, cols, world):
        w = A.ShardedWeight.__new__(A.ShardedWeight)
        w.rows, w.cols, w.world = rows, cols, world
        return w

    engine_w = GatheredWeight(2048, 2048, 2, 0, [], None, None)
    assert A.auto_pullers([Spec(4096, 2048, 2048)], [engine_w]) == A.DEFAULT_PULLERS
    big = A.auto_pullers([Spec(32768, 22016, 2048)], [standalone(22016, 2048, 8)])
    small = A.auto_pullers([Spec(256, 22016, 2048)], [standalone(22016, 2048, 8)])
    assert big == A.STANDALONE_PULLERS
    assert A.STANDALONE_PULLERS < small <= 32 and small % 2 == 0
    # a mix of engine and stand-alone weights in one launch is an engine launch
    assert A.auto_pullers([Spec(256, 64, 64), Spec(256, 64, 64)], [engine_w, standalone(64, 64, 2)]) == A.DEFAULT_PULLERS
