"""Kernels of the cached decode / denoise step against plain PyTorch fp32 references: the few-row GEMM, the fused
rotary + cache write, and the small-query attention kernel (csrc/gemm_skinny.cuh, csrc/decode.cu)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _bf(x):
    return x.to(torch.bfloat16).cuda()


def _close(a, b, rtol, atol=None, what=""):
    a, b = a.float().cpu(), b.float().cpu()
    atol = atol if atol is not None else rtol * float(b.abs().max())
    err = float((a - b).abs().max())
    assert err <= atol + rtol * float(b.abs().max()), f"{what}: max abs err {err}"


@pytest.mark.parametrize("M", [1, 17, 32, 33, 64, 100, 128])
@pytest.mark.parametrize("N,K", [(32, 64), (96, 200), (2048, 2048), (2560, 512), (4096, 2048), (512, 8192)])
def test_few_row_gemm_matches_fp32_and_the_general_kernel(M, N, K):
    """force_bn 16: clusters of CTAs that split K (partial sums added in rank order); 17: the same kernel with one CTA
    per column tile, whose sum over K has the order of the general kernel and must equal it bit for bit."""
    from wallx_b200.ops import gemm as G

    g = torch.Generator().manual_seed(M * 7 + N + K)
    a = _bf(torch.randn(M, K, generator=g))
    w = _bf(torch.randn(N, K, generator=g) * 0.05)
    bias = _bf(torch.randn(N, generator=g))
    res = _bf(torch.randn(M, N, generator=g))
    ref = a.float() @ w.float().t() + bias.float() + res.float()
    split = G.gemm(a, w, bias=bias, residual=res, force_bn=16)
    again = G.gemm(a, w, bias=bias, residual=res, force_bn=16)
    single = G.gemm(a, w, bias=bias, residual=res, force_bn=17)
    wide = G.gemm(a, w, bias=bias, residual=res, force_bn=64)
    train = G.gemm(a, w, bias=bias, residual=res)
    with torch.no_grad(), G.inference_kernels():
        auto = G.gemm(a, w, bias=bias, residual=res)
    torch.cuda.synchronize()
    G.check_status()
    _close(split, ref, 1e-2, what="few-row gemm, K split over a cluster")
    _close(single, ref, 1e-2, what="few-row gemm, one CTA per column tile")
    assert torch.equal(single, wide), "few-row kernel (no split) and 64-wide tiles differ"
    assert torch.equal(split, again), "the sum over the cluster depends on timing"
    assert torch.equal(split, auto), "inference launches split K"
    assert torch.equal(single, train), "training launches do not"


@pytest.mark.parametrize("M,N,K", [(314, 2048, 11008), (200, 2560, 4096), (972, 1280, 4160), (1024, 2048, 8192),
                                   (314, 4096, 2048)])
def test_prefix_sized_gemm_on_k_splitting_clusters(M, N, K):
    """Launches made inside an ``inference_kernels`` region with autograd off may run a few hundred rows on 128 x 256
    tiles whose K range is split over a cluster; all other launches keep the general kernel. Both against fp32, and the
    split sum must not depend on timing."""
    from wallx_b200.ops import gemm as G

    g = torch.Generator().manual_seed(M + N + K)
    a = _bf(torch.randn(M, K, generator=g))
    w = _bf(torch.randn(N, K, generator=g) * 0.03)
    bias = _bf(torch.randn(N, generator=g))
    res = _bf(torch.randn(M, N, generator=g))
    ref = a.float() @ w.float().t() + bias.float() + res.float()
    train = G.gemm(a, w, bias=bias, residual=res)
    with torch.no_grad():
        plain = G.gemm(a, w, bias=bias, residual=res)
        with G.inference_kernels():
            infer = G.gemm(a, w, bias=bias, residual=res)
            again = G.gemm(a, w, bias=bias, residual=res)
    torch.cuda.synchronize()
    G.check_status()
    assert torch.equal(train, plain), "grad mode alone must not change the kernel"
    _close(train, ref, 1e-2, what="general kernel")
    _close(infer, ref, 1e-2, what="inference launch")
    assert torch.equal(infer, again)


def test_few_row_gemm_swiglu_fp32_out_and_device_side_sizes():
    from wallx_b200.ops import gemm as G, ref

    g = torch.Generator().manual_seed(3)
    M, K, I = 32, 512, 256
    a = _bf(torch.randn(M, K, generator=g))
    w = _bf(torch.randn(2 * I, K, generator=g) * 0.05)
    h = torch.empty(M, I, dtype=torch.bfloat16, device="cuda")
    G.launch([G.GemmSpec(a, w, h, flags=G.ACT_SWIGLU)], force_bn=16)
    want = ref.swiglu_interleaved((a.float() @ w.float().t()).to(torch.bfloat16).float())
    _close(h, want, 2e-2, what="few-row gate/up + SwiGLU")
    o32 = G.gemm(a, w, flags=G.OUT_FP32, force_bn=16)
    assert o32.dtype == torch.float32
    _close(o32, a.float() @ w.float().t(), 1e-2, what="fp32 output")
    # two problems in one launch, the second with no rows on the device: its CTAs leave, its output stays untouched
    out0 = torch.zeros(M, 2 * I, dtype=torch.bfloat16, device="cuda")
    out1 = torch.full((M, 2 * I), 7.0, dtype=torch.bfloat16, device="cuda")
    dyn0 = torch.tensor([0, 20, -1, -1], dtype=torch.int32, device="cuda")  # rows 0..19
    dyn1 = torch.tensor([0, 0, -1, -1], dtype=torch.int32, device="cuda")
    G.launch([G.GemmSpec(a, w, out0, dyn=dyn0), G.GemmSpec(a, w, out1, dyn=dyn1)], force_bn=16)
    torch.cuda.synchronize()
    G.check_status()
    full = a.float() @ w.float().t()
    _close(out0[:20], full[:20], 1e-2, what="rows given on the device")
    assert float(out0[20:].abs().max()) == 0.0
    assert bool((out1 == 7.0).all())


def test_few_row_kernel_is_refused_for_many_rows():
    from wallx_b200.ops import gemm as G

    a = _bf(torch.randn(129, 64))
    w = _bf(torch.randn(32, 64))
    with pytest.raises(RuntimeError):
        G.gemm(a, w, force_bn=16)


@pytest.mark.parametrize("hq,hkv,D", [(16, 2, 128), (4, 4, 64)])
def test_rotary_with_cache_write_matches_rotary_then_index_copy(hq, hkv, D):
    from wallx_b200.ops import functional as F_

    torch.manual_seed(2)
    T, rows = 37, 200
    qkv = _bf(torch.randn(T, (hq + 2 * hkv) * D))
    ang = torch.rand(T, D // 2) * 6.28
    cos = torch.cat([ang.cos(), ang.cos()], 1).float().cuda().contiguous()
    sin = torch.cat([ang.sin(), ang.sin()], 1).float().cuda().contiguous()
    cache_rows = torch.randperm(rows)[:T].cuda()
    cache = _bf(torch.randn(rows, 2 * hkv * D))
    want_cache = cache.clone()
    rot = F_.rope_qk(qkv, cos, sin, hq + hkv, D)
    want_cache.index_copy_(0, cache_rows, rot[:, hq * D:])
    with torch.no_grad():
        got = F_.rope_cache_(qkv.clone(), cos, sin, cache_rows, cache, hq, hkv, D)
    torch.cuda.synchronize()
    assert torch.equal(got[:, : hq * D], rot[:, : hq * D])
    assert torch.equal(cache, want_cache)


@pytest.mark.parametrize("causal,bid", [(True, False), (True, True), (False, False)])
@pytest.mark.parametrize("hq,hkv", [(16, 2), (8, 8), (6, 2)])
def test_small_query_attention_matches_fp32(causal, bid, hq, hkv):
    """Few new queries against a longer cached key range: the rule of the tensor-core kernel (bottom-right aligned
    causal limit, flagged queries see flagged keys), evaluated by the CPU oracle in fp32."""
    from wallx_b200.ops import functional as F_

    torch.manual_seed(5)
    D = 128
    cu_k, cu_q = [0, 300, 511, 520], [0, 32, 64, 65]
    Tq, Tk = cu_q[-1], cu_k[-1]
    q = torch.randn(Tq, hq * D)
    kv = torch.randn(Tk, 2 * hkv * D)  # one buffer, k columns then v columns, as the cache holds them
    bq = torch.ones(Tq, dtype=torch.bool) if bid else None
    bk = torch.zeros(Tk, dtype=torch.bool)
    bk[300 - 32:300] = True
    bk[511 - 32:511] = True
    mc = F_.AttnMeta(cu_q, "cuda", causal, bq.cuda() if bid else None, cu_k=cu_k, bidir_k=bk.cuda() if bid else None)
    mr = F_.AttnMeta(cu_q, "cpu", causal, bq, cu_k=cu_k, bidir_k=bk if bid else None)
    kvb = _bf(kv)
    qb = _bf(q)
    with torch.no_grad():
        o = F_.attention_decode(qb, kvb[:, : hkv * D], kvb[:, hkv * D:], mc, hq, hkv, D)
        o_tc = F_.attention(qb, kvb[:, : hkv * D], kvb[:, hkv * D:], mc, hq, hkv, D)
    kf = kvb.float().cpu()
    orf = F_.attention(qb.float().cpu(), kf[:, : hkv * D], kf[:, hkv * D:], mr, hq, hkv, D)
    _close(o, orf, 2e-2, what=f"small-query attention causal={causal} bidir={bid}")
    _close(o, o_tc, 2e-2, what="small-query kernel vs tensor-core kernel")


def test_denoise_step_uses_the_cached_step_kernels_and_matches_the_operator_path():
    """One velocity evaluation of the flow sampler with the fused rotary + cache write, the small-query attention and
    the single-expert FFN against the same evaluation through the general kernels."""
    from wallx_b200.config import tiny_config
    from wallx_b200.data.collator import add_pack_info
    from wallx_b200.data.synthetic import make_batch, make_processor
    from wallx_b200.models import Qwen2_5_VLMoEForAction
    from wallx_b200.models.inference import FlowSampler
    from wallx_b200.ops import functional as F_, gemm as G

    dev = torch.device("cuda", 0)
    cfg = tiny_config()
    proc = make_processor(cfg, 16)
    torch.manual_seed(0)
    model = Qwen2_5_VLMoEForAction(cfg, processor=proc).to(torch.bfloat16).to(dev)
    model.init_weights(seed=1)
    model.eval()
    g = torch.Generator().manual_seed(4)
    batch = make_batch(cfg, proc, 2, views=2, image_hw=(112, 112), prompt_len=16, horizon=16, mode="flow", generator=g)
    batch.pop("action_chunk", None)
    batch.pop("labels", None)
    batch = add_pack_info(dict(batch), cfg)
    batch = {k: (v.to(dev).to(torch.bfloat16) if isinstance(v, torch.Tensor) and v.is_floating_point()
                 else (v.to(dev) if isinstance(v, torch.Tensor) else v)) for k, v in batch.items()}
    t = torch.tensor(0.25, device=dev, dtype=torch.bfloat16)
    with torch.no_grad():
        s = FlowSampler(model, **batch)
        x = torch.randn(2, s.horizon, model.action_preprocessor.action_dim, device=dev, dtype=torch.bfloat16)
        assert s.ctx.plan is None or s.ctx.plan.single_expert == 1  # the suffix rows are all action tokens
        fast = s.velocity(t, x).float()
        # the same evaluation through the general kernels (the prefix cache is already filled)
        old_usable = F_.cached_step_kernels_usable
        F_.cached_step_kernels_usable = lambda qkv, d: False
        single = s.ctx.plan.single_expert if s.ctx.plan is not None else None
        try:
            if s.ctx.plan is not None:
                s.ctx.plan.single_expert = None
            slow = s.velocity(t, x).float()
        finally:
            F_.cached_step_kernels_usable = old_usable
            if s.ctx.plan is not None:
                s.ctx.plan.single_expert = single
    torch.cuda.synchronize()
    G.check_status()
    assert torch.isfinite(fast).all()
    err = float((fast - slow).abs().max())
    assert err <= 3e-2 * float(slow.abs().max()) + 1e-3, err
