"""CPU oracle properties (no GPU): routing, rope index, window index, mRoPE, flow maths."""

import pytest
import torch

from wallx_b200.ops import functional as F_
from wallx_b200.ops import index as IX
from wallx_b200.ops import ref


def test_route_plan_is_stable_and_aligned():
    torch.manual_seed(0)
    types = (torch.rand(1000) < 0.2).long()
    dest, seg = ref.route_plan(types, 2, 128)
    assert seg[0, 0] == 0 and seg[1, 0] % 128 == 0 and seg[1, 0] >= seg[0, 1]
    for e in range(2):
        d = dest[types == e]
        assert torch.equal(d, seg[e, 0] + torch.arange(d.numel()))  # stable order inside the expert
    x = torch.randn(1000, 8)
    rows = int(seg[1, 0] + seg[1, 2])
    xp = ref.permute_rows(x, dest, rows)
    assert torch.equal(ref.unpermute_rows(xp, dest), x)
    pad = torch.ones(rows, dtype=torch.bool)
    pad[dest] = False
    assert xp[pad].abs().sum() == 0


def test_interleave_roundtrip():
    g, u = torch.randn(64, 5), torch.randn(64, 5)
    gu = ref.interleave_gate_up(g, u)
    g2, u2 = ref.deinterleave_gate_up(gu)
    assert torch.equal(g, g2) and torch.equal(u, u2)
    x = torch.randn(3, 128)
    gg, uu = ref.deinterleave_gate_up(x, dim=-1)
    assert torch.allclose(ref.swiglu_interleaved(x), torch.nn.functional.silu(gg) * uu)


def _hf_rope_index_one_image(n_text_before, grid, n_text_after, merge=2):
    t, h, w = grid
    gh, gw = h // merge, w // merge
    pos = [list(range(n_text_before)) for _ in range(3)]
    base = n_text_before
    for ti in range(t):
        for hi in range(gh):
            for wi in range(gw):
                pos[0].append(base + 0)
                pos[1].append(base + hi)
                pos[2].append(base + wi)
    nxt = base + max(gh, gw)
    for a in range(3):
        pos[a].extend(range(nxt, nxt + n_text_after))
    return torch.tensor(pos)


@pytest.mark.parametrize("pad_left", [0, 3])
def test_rope_index_image_and_padding(pad_left):
    IMG, VID, VS = 900, 901, 902
    grid = (1, 4, 6)
    n_img = 1 * 2 * 3
    seq = [5, 6, VS] + [IMG] * n_img + [7, 8, 9]
    ids = torch.tensor([[0] * pad_left + seq])
    am = torch.tensor([[0] * pad_left + [1] * len(seq)])
    pos, delta = ref.rope_index(ids, torch.tensor([grid]), None, None, am, 2, IMG, VID, VS, 2.0)
    expect = _hf_rope_index_one_image(3, grid, 3)
    assert torch.equal(pos[:, 0, pad_left:], expect)
    assert (pos[:, 0, :pad_left] == 1).all()
    assert delta.item() == expect.max().item() + 1 - ids.shape[1]


def test_rope_index_text_only_matches_cumsum():
    ids = torch.randint(5, 100, (2, 9))
    am = torch.tensor([[0, 0, 1, 1, 1, 1, 1, 1, 1], [1] * 9])
    pos, delta = ref.rope_index(ids, None, None, None, am, 2, 900, 901, 902, 2.0)
    assert pos[0, 0].tolist() == [1, 1, 0, 1, 2, 3, 4, 5, 6]
    assert delta.reshape(-1).tolist() == [-2, 0]


def test_window_index_is_permutation_with_monotone_seqlens():
    grid = [[1, 18, 18], [1, 8, 8], [2, 6, 10]]
    idx, cu = ref.window_index(grid, 112, 2, 14)
    n = sum(t * (h // 2) * (w // 2) for t, h, w in grid)
    assert sorted(idx.tolist()) == list(range(n))
    assert all(b >= a for a, b in zip(cu[:-1], cu[1:])) and cu[-1] == 4 * n
    # 18x18 patches -> 9x9 merged -> windows of 4: 3x3 windows of sizes 16,16,4 / 16,16,4 / 4,4,1 (x4 patches)
    first = [b - a for a, b in zip(cu[:9], cu[1:10])]
    assert first == [64, 64, 16, 64, 64, 16, 16, 16, 4]
    t_idx, t_cu = IX.get_window_index(torch.tensor(grid), 112, 2, 14)
    assert torch.equal(t_idx, idx) and t_cu.tolist() == cu


def test_rot_pos_emb_matches_direct_formula():
    inv = 1.0 / (10000.0 ** (torch.arange(0, 8, 2).float() / 8))
    grid = [[1, 4, 4]]
    ang = ref.rot_pos_emb(inv, grid, 2)
    ids = ref.rot_pos_ids(grid, 2)
    assert ids[:4].tolist() == [[0, 0], [0, 1], [1, 0], [1, 1]]  # merge-block order
    assert torch.allclose(ang[:, :4], ids[:, 0:1].float() * inv)
    assert torch.allclose(ang[:, 4:], ids[:, 1:2].float() * inv)


@pytest.mark.parametrize("layout", ["hf", "wallx_cuda"])
def test_mrope_layouts(layout):
    D, sections = 32, [4, 6, 6]
    ax = ref.mrope_axis_of_channel(D, sections, layout)
    if layout == "hf":
        assert ax.tolist() == [0] * 4 + [1] * 6 + [2] * 6 + [0] * 4 + [1] * 6 + [2] * 6
        assert torch.equal(ax[:16], ax[16:])
    else:
        assert ax.tolist() == [0] * 8 + [1] * 12 + [2] * 12
    pos3 = torch.randint(0, 50, (3, 11))
    cos, sin = ref.mrope_cos_sin(pos3, ref.rope_inv_freq(D, 1e4), sections, layout)
    x = torch.randn(11, 3, D, dtype=torch.float64)
    y = ref.apply_rope(x, cos.double(), sin.double())
    if layout == "hf":  # a proper rotation preserves norms
        assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-6)
    same = torch.arange(11).view(1, -1).expand(3, -1)
    c1, s1 = ref.mrope_cos_sin(same, ref.rope_inv_freq(D, 1e4), sections, "hf")
    c2, s2 = ref.mrope_cos_sin(same, ref.rope_inv_freq(D, 1e4), sections, "wallx_cuda")
    assert torch.allclose(c1, c2) and torch.allclose(s1, s2)  # text tokens: both layouts agree


def test_attention_rules():
    torch.manual_seed(0)
    T, H, D = 12, 2, 8
    qkv = torch.randn(T, 3 * H * D)
    cu = [0, 5, 12]
    bid = torch.zeros(T, dtype=torch.bool)
    bid[9:12] = True
    o_c = F_.attention_packed(qkv, F_.AttnMeta(cu, "cpu", True), H, H, D)
    o_b = F_.attention_packed(qkv, F_.AttnMeta(cu, "cpu", True, bid), H, H, D)
    o_ref = ref.attention_varlen(qkv[:, :16].view(T, H, D), qkv[:, 16:32].view(T, H, D), qkv[:, 32:].view(T, H, D), cu,
                                 True, bid).reshape(T, -1)
    assert torch.allclose(o_b, o_ref, atol=1e-5)
    assert torch.allclose(o_c[:9], o_b[:9], atol=1e-6)  # only the flagged block changes
    assert not torch.allclose(o_c[9:11], o_b[9:11], atol=1e-4)
    assert torch.allclose(o_c[11], o_b[11], atol=1e-6)  # the last token already saw everything


def test_flow_interpolation_and_euler_on_linear_field():
    # x_t = (1-t) eps + t a, target a - eps: integrating the exact field from eps reaches a
    a, eps = torch.randn(4, 3), torch.randn(4, 3)
    x = eps.clone()
    n = 10
    ts = torch.linspace(0, 1, n + 1)
    for i in range(n):
        x = x + (ts[i + 1] - ts[i]) * (a - eps)
    assert torch.allclose(x, a, atol=1e-5)


def test_adamw_reference_step_matches_torch():
    p = torch.randn(50)
    g = torch.randn(50)
    q = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([q], lr=1e-2, weight_decay=0.1)
    m, v, w = torch.zeros(50), torch.zeros(50), p.clone()
    for step in range(1, 4):
        q.grad = g.clone()
        opt.step()
        ref.adamw_step(w, g, m, v, step, 1e-2, 0.9, 0.999, 1e-8, 0.1)
    assert torch.allclose(w, q.detach(), atol=1e-6)
