"""Property tests (hypothesis) of the CPU oracles and of the shard arithmetic, no GPU.

The oracles in ``wallx_b200.ops.ref`` are what every CUDA kernel is compared against, so they get
their own checks against independent restatements here: routing (the reference's permute /
unpermute semantics, modeling_qwen2_5_vl_act.py:138-157), position ids for random image layouts
and paddings (modeling_qwen2_5_vl_act.py:929-1149), ViT window order
(modeling_qwen2_5_vl.py:502-547), rotary forward / backward (modeling_qwen2_5_vl.py:731-773),
and the flat-buffer sharding and resharding at world sizes 1 / 2 / 4 / 8.
"""
import os

import pytest
import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from wallx_b200.ops import ref

_FAST = settings(max_examples=40, deadline=None, suppress_health_check=list(HealthCheck), derandomize=True, database=None)


# ----------------------------------------------------------------------------- routing
@_FAST
@given(st.lists(st.integers(0, 1), min_size=1, max_size=700), st.sampled_from([1, 16, 128]))
def test_route_plan_roundtrip_stable_aligned(types, align):
    t = torch.tensor(types)
    dest, seg = ref.route_plan(t, 2, align)
    n0, n1 = int((t == 0).sum()), int((t == 1).sum())
    assert int(seg[0, 1]) == n0 and int(seg[1, 1]) == n1  # real rows per expert
    assert int(seg[0, 0]) == 0 and int(seg[1, 0]) == int(seg[0, 2]) and int(seg[1, 0]) >= n0
    assert all(int(seg[e, 2]) % align == 0 and 0 <= int(seg[e, 2]) - int(seg[e, 1]) < align for e in range(2))
    assert dest.unique().numel() == len(types)  # injective
    for e, n in ((0, n0), (1, n1)):
        d = dest[t == e]
        assert torch.equal(d, int(seg[e, 0]) + torch.arange(n))  # token order kept inside an expert
    rows = int(seg[1, 0] + seg[1, 2])
    assert int(dest.max()) < rows
    x = torch.arange(len(types) * 3, dtype=torch.float32).view(-1, 3) + 1
    xp = ref.permute_rows(x, dest, rows)
    assert torch.equal(ref.unpermute_rows(xp, dest), x)
    assert xp.abs().sum() == x.abs().sum()  # pad rows are zero


# ----------------------------------------------------------------------------- ViT window order
_grid = st.tuples(st.integers(1, 2), st.integers(1, 12).map(lambda v: 2 * v), st.integers(1, 12).map(lambda v: 2 * v))


@_FAST
@given(st.lists(_grid, min_size=1, max_size=3))
def test_window_index_permutation_and_window_contents(grids):
    grids = [list(g) for g in grids]
    idx, cu = ref.window_index(grids, 112, 2, 14)
    n = sum(t * (h // 2) * (w // 2) for t, h, w in grids)
    assert sorted(idx.tolist()) == list(range(n))
    assert cu[0] == 0 and cu[-1] == 4 * n and all(b >= a for a, b in zip(cu[:-1], cu[1:]))
    # every window holds merged tokens of ONE frame of ONE image that lie in one 4 x 4 block
    owner = []
    for g, (t, h, w) in enumerate(grids):
        for ti in range(t):
            for hi in range(h // 2):
                for wi in range(w // 2):
                    owner.append((g, ti, hi // 4, wi // 4))
    for a, b in zip(cu[:-1], cu[1:]):
        assert a % 4 == 0 and b % 4 == 0
        toks = idx[a // 4:b // 4].tolist()
        assert len({owner[i] for i in toks}) <= 1
        assert len(toks) <= 16


# ----------------------------------------------------------------------------- position ids
IMG, VID, VS = 900, 901, 902


def _positions_direct(items, merge=2):
    """Independent restatement: ``items`` is a list of ("text", n) / ("image", (t, h, w))."""
    pos = [[], [], []]
    nxt = 0
    for kind, v in items:
        if kind == "text":
            for a in range(3):
                pos[a].extend(range(nxt, nxt + v))
            nxt += v
        else:
            t, h, w = v
            gh, gw = h // merge, w // merge
            for _ in range(t):
                for hi in range(gh):
                    for wi in range(gw):
                        pos[0].append(nxt)  # images: temporal index 0 for every frame
                        pos[1].append(nxt + hi)
                        pos[2].append(nxt + wi)
            nxt += max(gh, gw)
    return torch.tensor(pos), nxt


_image = st.tuples(st.just(1), st.integers(1, 5).map(lambda v: 2 * v), st.integers(1, 5).map(lambda v: 2 * v))


@_FAST
@given(st.lists(st.tuples(st.integers(0, 4), _image), min_size=1, max_size=3), st.integers(0, 5), st.integers(0, 4),
       st.booleans())
def test_rope_index_random_layouts(blocks, tail, pad, pad_left):
    toks, items, grids = [], [], []
    for n_text, g in blocks:
        toks += [5] * n_text + [VS] + [IMG] * (g[0] * (g[1] // 2) * (g[2] // 2))
        items += [("text", n_text + 1), ("image", g)]  # the vision-start token counts as text
        grids.append(list(g))
    toks += [7] * tail
    items.append(("text", tail))
    ids = [0] * pad + toks if pad_left else toks + [0] * pad
    am = [0] * pad + [1] * len(toks) if pad_left else [1] * len(toks) + [0] * pad
    pos, delta = ref.rope_index(torch.tensor([ids]), torch.tensor(grids), None, None, torch.tensor([am]), 2, IMG, VID, VS, 2.0)
    expect, nxt = _positions_direct(items)
    keep = torch.tensor(am) == 1
    assert torch.equal(pos[:, 0, keep], expect)
    assert (pos[:, 0, ~keep] == 1).all()
    assert int(delta) == int(expect.max()) + 1 - len(ids)


# ----------------------------------------------------------------------------- rotary
@_FAST
@given(st.integers(1, 9), st.integers(1, 3), st.sampled_from(["hf", "wallx_cuda"]), st.integers(0, 2 ** 31 - 1))
def test_rope_backward_is_rotation_by_minus_angle(T, H, layout, seed):
    g = torch.Generator().manual_seed(seed)
    D, sections = 16, [2, 3, 3]
    pos3 = torch.randint(0, 40, (3, T), generator=g)
    cos, sin = ref.mrope_cos_sin(pos3, ref.rope_inv_freq(D, 1e4), sections, layout)
    x = torch.randn(T, H, D, dtype=torch.float64, generator=g, requires_grad=True)
    dy = torch.randn(T, H, D, dtype=torch.float64, generator=g)
    y = ref.apply_rope(x, cos.double(), sin.double())
    (dx,) = torch.autograd.grad(y, x, dy)
    # in the Hugging Face layout both channels of a pair share the angle, so the transposed rotation (what the
    # kernels apply in backward) is the rotation by the negated angle
    if layout == "hf":
        assert torch.allclose(dx, ref.apply_rope(dy, cos.double(), -sin.double()), rtol=1e-5, atol=1e-5)  # the oracle computes in fp32
        assert torch.allclose(ref.apply_rope(y.detach(), cos.double(), -sin.double()), x.detach(), atol=1e-5)  # cos and sin are fp32 tables
    # in both layouts the map is linear in x
    y2 = ref.apply_rope(2.5 * x.detach(), cos.double(), sin.double())
    assert torch.allclose(y2, 2.5 * y.detach(), rtol=1e-5, atol=1e-5)  # the oracle computes in fp32


# ----------------------------------------------------------------------------- attention mask rules
@_FAST
@given(st.lists(st.integers(1, 9), min_size=1, max_size=4), st.integers(0, 4), st.booleans())
def test_attention_mask_rules(lens, n_bidir, causal):
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    bid = torch.zeros(T, dtype=torch.bool)
    for a, b in zip(cu[:-1], cu[1:]):
        bid[max(a, b - n_bidir):b] = True
    m = ref.attention_mask_varlen(cu, causal, bid, "cpu")
    assert m.shape == (T, T) and m.dtype == torch.bool
    seq_of = torch.repeat_interleave(torch.arange(len(lens)), torch.tensor(lens))
    for i in range(T):
        for j in range(T):
            same = bool(seq_of[i] == seq_of[j])
            allowed = same and (not causal or j <= i or (bool(bid[i]) and bool(bid[j])))
            assert bool(m[i, j]) == allowed, (i, j)


# ----------------------------------------------------------------------------- flat buffers: shard arithmetic
def _params(sizes, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [(f"p{i}", torch.nn.Parameter(torch.randn(*s, generator=g))) for i, s in enumerate(sizes)]


@_FAST
@given(st.lists(st.tuples(st.integers(1, 40), st.integers(1, 70)), min_size=1, max_size=6), st.sampled_from([1, 2, 4, 8]),
       st.data())
def test_flat_buffer_shards_partition_the_buffer(sizes, world, data):
    from wallx_b200.parallel.flat import FlatBuffer

    groups = [("decay", 1.0, 0.1) if len(s) == 2 and s[1] > 8 else ("no_decay", 1.0, 0.0) for s in sizes]
    touched = [data.draw(st.booleans()) for _ in sizes]
    bufs = [FlatBuffer(_params(sizes), world, r, groups, name="u") for r in range(world)]
    b0 = bufs[0]
    assert b0.padded % (FlatBuffer.ALIGN * world) == 0 and b0.padded >= b0.numel
    covered = torch.zeros(b0.padded, dtype=torch.int32)
    upd = torch.zeros(b0.padded, dtype=torch.int32)
    decay = torch.full((b0.padded,), -1.0)
    for r, b in enumerate(bufs):
        s0, s1 = b.shard_range
        assert s1 - s0 == b.shard_size == b0.padded // world and s0 == r * b.shard_size
        for lo, hi, seg in b.shard_segments():
            covered[s0 + lo:s0 + hi] += 1
            decay[s0 + lo:s0 + hi] = seg.weight_decay
        for lo, hi, seg in b.update_ranges(touched):
            upd[s0 + lo:s0 + hi] += 1
            assert 0 <= lo < hi <= b.shard_size
    assert (covered == 1).all()  # every element has exactly one owner and one hyper-parameter segment
    for i, (p, o) in enumerate(zip(b0.params, b0.offsets)):
        want = b0.segments[b0.seg_of_param[i]].weight_decay
        assert (decay[o:o + p.numel()] == want).all()
        if not all(touched):
            assert (upd[o:o + p.numel()] == (1 if touched[i] else 0)).all()
        # parameters are views of the flat storage
        assert p.data.data_ptr() == b0.param[o:].data_ptr()


def _tiny_engine(world, rank):
    from wallx_b200.parallel.engine import TrainEngine

    torch.manual_seed(7)
    m = torch.nn.Sequential(torch.nn.Linear(37, 53), torch.nn.Linear(53, 11))
    return TrainEngine(m, lr=1e-3, world=world, rank=rank, transport="dist")


@pytest.mark.parametrize("old_world,new_world", [(1, 2), (2, 4), (4, 8), (8, 1), (4, 2), (2, 1)])
def test_optimizer_state_reshards_between_world_sizes(tmp_path, old_world, new_world):
    """Shards written at one world size load at another with every element in place."""
    from wallx_b200.parallel.reshard import load_optimizer_shards

    g = torch.Generator().manual_seed(old_world * 10 + new_world)
    truth = None
    for r in range(old_world):
        eng = _tiny_engine(old_world, r)
        if truth is None:
            truth = [{k: torch.randn(b.numel, generator=g) for k in ("master", "exp_avg", "exp_avg_sq")} for b in eng.buffers]
        for b, t in zip(eng.buffers, truth):
            s0, s1 = b.shard_range
            for k, dst in (("master", b.master), ("exp_avg", b.exp_avg), ("exp_avg_sq", b.exp_avg_sq)):
                full = torch.cat([t[k], torch.zeros(b.padded - b.numel)])
                dst.copy_(full[s0:s1])
        eng.optimizer.step_count = 17
        torch.save(eng.optimizer_state(), os.path.join(tmp_path, f"optim_rank{r:05d}_of_{old_world:05d}.pt"))
    got = [{k: [] for k in ("master", "exp_avg", "exp_avg_sq")} for _ in truth]
    for r in range(new_world):
        eng = _tiny_engine(new_world, r)
        load_optimizer_shards(eng, str(tmp_path), old_world)
        assert eng.optimizer.step_count == 17
        for i, b in enumerate(eng.buffers):
            for k, src in (("master", b.master), ("exp_avg", b.exp_avg), ("exp_avg_sq", b.exp_avg_sq)):
                got[i][k].append(src.clone())
    for i, t in enumerate(truth):
        for k in t:
            full = torch.cat(got[i][k])
            assert torch.equal(full[: t[k].numel()], t[k]), (i, k)
            assert full[t[k].numel():].abs().sum() == 0  # padding stays zero


def test_missing_shard_is_reported(tmp_path):
    from wallx_b200.parallel.reshard import load_optimizer_shards

    eng = _tiny_engine(1, 0)
    with pytest.raises(FileNotFoundError):
        load_optimizer_shards(eng, str(tmp_path), 2)


# ----------------------------------------------------------------------------- data path
@_FAST
@given(st.integers(20, 2000), st.integers(20, 2000))
def test_smart_resize_bounds_and_alignment(h, w):
    from wallx_b200.data.synthetic import smart_resize

    if max(h, w) / min(h, w) > 200:
        return
    lo, hi = 4 * 28 * 28, 1280 * 28 * 28
    rh, rw = smart_resize(h, w, factor=28, min_pixels=lo, max_pixels=hi)
    assert rh % 28 == 0 and rw % 28 == 0 and rh >= 28 and rw >= 28
    assert lo <= rh * rw <= hi
    if lo <= round(h / 28) * 28 * round(w / 28) * 28 <= hi:  # in range: plain rounding, at most half a factor per side
        assert abs(rh - h) <= 14 and abs(rw - w) <= 14


@_FAST
@given(st.integers(1, 32), st.integers(1, 14), st.integers(0, 2 ** 31 - 1))
def test_dct_action_tokenizer_roundtrip_error_is_bounded(T, D, seed):
    import numpy as np

    from wallx_b200.data.fast_tokenizer import DctActionTokenizer

    rng = np.random.default_rng(seed)
    tok = DctActionTokenizer(2048, scale=10.0)
    a = rng.uniform(-1, 1, size=(2, T, D))
    ids = tok(a)
    assert len(ids) == 2 and all(0 < len(x) <= T * D and all(0 <= i < 2048 for i in x) for x in ids)
    back = tok.decode(ids, T, D)
    # an orthonormal transform with coefficients rounded to 1 / scale: per-element error <= sqrt(T) * 0.5 / scale
    assert np.abs(back - a).max() <= 0.5 / 10.0 * np.sqrt(T) + 1e-6
    assert np.sqrt(((back - a) ** 2).mean()) <= 0.5 / 10.0 + 1e-6  # Parseval: the RMS error is that of the rounding
    assert tok.decode([[5000]], T, D).any() == False  # noqa: E712  invalid ids decode to zeros


@_FAST
@given(st.lists(st.floats(-5, 5, allow_nan=False), min_size=3, max_size=3), st.lists(st.floats(0.125, 4), min_size=3, max_size=3),
       st.integers(0, 2 ** 31 - 1))
def test_normalizer_roundtrip_inside_the_range_and_clamp_outside(mins, deltas, seed):
    from wallx_b200.models.action_head import Normalizer

    stats = {"robot": {"arm": {"min": mins, "delta": deltas}}}
    nz = Normalizer(stats, {"arm": 3, "extra": 2})  # a key without statistics maps [0, 1] to [-1, 1]
    g = torch.Generator().manual_seed(seed)
    mn = torch.tensor(mins + [0.0, 0.0])
    dl = torch.tensor(deltas + [1.0, 1.0])
    x = mn + dl * torch.rand(1, 4, 5, generator=g)
    y = nz.normalize_data(x, ["robot"])
    assert y.min() >= -1 and y.max() <= 1
    assert torch.allclose(nz.unnormalize_data(y, ["robot"]), x, atol=1e-4)
    far = nz.normalize_data(x + 10 * dl, ["robot"])
    assert (far == 1).all()
    # masked unnormalize keeps the selected degrees of freedom only
    mask = torch.tensor([[1, 1, 1, 0, 0]]).expand(1, 5).unsqueeze(0)
    sel = nz.unnormalize_data(y[..., :3], ["robot"], dof_mask=mask)
    assert torch.allclose(sel, x[..., :3], atol=1e-4)
