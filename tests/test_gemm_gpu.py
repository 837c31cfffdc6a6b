"""tcgen05 GEMM core vs a plain fp32 PyTorch matmul (all four operand layouts, epilogues, groups)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(shape, seed, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).cuda()


def _ref(a, b, a_mn, b_mn):
    af = a.float().t() if a_mn else a.float()
    bf = b.float() if b_mn else b.float().t()
    return af @ bf


def _check(out, ref, K):
    tol = 2e-2 * (K ** 0.5) * 0.05 + 1e-2
    err = (out.float() - ref).abs().max().item()
    rel = err / (ref.abs().max().item() + 1e-6)
    assert rel < 1e-2 or err < tol, f"max abs err {err}, rel {rel}"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (200, 328, 136), (1000, 1280, 1176), (64, 40, 2048)])
@pytest.mark.parametrize("bn", [0, 32, 64, 128, 256, 512])  # 512 = CTA pairs, 256 x 256 tiles; 32 = K-major only
def test_layouts(a_mn, b_mn, M, N, K, bn):
    from wallx_b200.ops import gemm as G

    if bn == 32 and (a_mn or b_mn):
        pytest.skip("32-wide tiles exist for K-major operands only")
    if (a_mn and M % 8) or (b_mn and N % 8) or ((not a_mn or not b_mn) and K % 8):
        pytest.skip("pitch not 16-byte aligned for this layout")
    a = _mk((K, M) if a_mn else (M, K), 1)
    b = _mk((K, N) if b_mn else (N, K), 2)
    out = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, force_bn=bn)
    torch.cuda.synchronize()
    G.check_status()
    _check(out, _ref(a, b, a_mn, b_mn), K)


def test_epilogues():
    from wallx_b200.ops import gemm as G

    M, N, K = 300, 512, 320
    a, b = _mk((M, K), 3), _mk((N, K), 4, 0.1)
    bias = _mk((N,), 5)
    res = _mk((M, N), 6)
    ref = a.float() @ b.float().t()
    out = G.gemm(a, b, bias=bias)
    _check(out, ref + bias.float(), K)
    out = G.gemm(a, b, bias=bias, flags=G.ACT_GELU)
    _check(out, torch.nn.functional.gelu(ref + bias.float()), K)
    out = G.gemm(a, b, residual=res)
    _check(out, ref + res.float(), K)
    out = G.gemm(a, b, flags=G.OUT_FP32)
    assert out.dtype == torch.float32
    _check(out, ref, K)
    acc = torch.ones((M, N), device="cuda", dtype=torch.float32)
    G.gemm(a, b, out=acc, flags=G.OUT_FP32 | G.ACCUMULATE)
    _check(acc, ref + 1.0, K)
    accb = torch.ones((M, N), device="cuda", dtype=torch.bfloat16)
    G.gemm(a, b, out=accb, flags=G.ACCUMULATE)
    _check(accb, ref + 1.0, K)
    G.check_status()


def test_small_m_problems_and_forced_narrow_tiles():
    """Decode-sized problems (one row tile): bias, residual, SwiGLU. The few-row kernel without a K split (17) gives the
    bits of forced 32-wide tiles, and so does the default (training) path; inference launches split K over a cluster."""
    from wallx_b200.ops import gemm as G

    M, N, K = 32, 2560, 2048
    a, b = _mk((M, K), 30), _mk((N, K), 31, 0.05)
    bias, res = _mk((N,), 32), _mk((M, N), 33)
    ref = a.float() @ b.float().t()
    _check(G.gemm(a, b, bias=bias, residual=res), ref + bias.float() + res.float(), K)
    I = 1024
    wg, wu = _mk((I, K), 34, 0.05), _mk((I, K), 35, 0.05)
    w = torch.stack([wg.view(I // 16, 16, K), wu.view(I // 16, 16, K)], dim=1).reshape(2 * I, K).contiguous()
    h = torch.empty((M, I), device="cuda", dtype=torch.bfloat16)
    h32 = torch.empty_like(h)
    h17 = torch.empty_like(h)
    G.launch([G.GemmSpec(a, w, h, flags=G.ACT_SWIGLU)])
    G.launch([G.GemmSpec(a, w, h32, flags=G.ACT_SWIGLU)], force_bn=32)
    G.launch([G.GemmSpec(a, w, h17, flags=G.ACT_SWIGLU)], force_bn=17)
    g = (a.float() @ wg.float().t()).bfloat16().float()
    u = (a.float() @ wu.float().t()).bfloat16().float()
    _check(h, torch.nn.functional.silu(g) * u, K)
    _check(h32, torch.nn.functional.silu(g) * u, K)
    assert torch.equal(h17, h32) and torch.equal(h, h32)
    torch.cuda.synchronize()
    G.check_status()


def test_swiglu_interleaved():
    from wallx_b200.ops import gemm as G

    M, I, K = 260, 192, 256
    a = _mk((M, K), 7)
    wg, wu = _mk((I, K), 8, 0.1), _mk((I, K), 9, 0.1)
    w = torch.stack([wg.view(I // 16, 16, K), wu.view(I // 16, 16, K)], dim=1).reshape(2 * I, K).contiguous()
    raw = torch.empty((M, 2 * I), device="cuda", dtype=torch.bfloat16)
    h = torch.empty((M, I), device="cuda", dtype=torch.bfloat16)
    G.launch([G.GemmSpec(a, w, h, out2=raw, flags=G.ACT_SWIGLU)])
    g = (a.float() @ wg.float().t()).bfloat16().float()
    u = (a.float() @ wu.float().t()).bfloat16().float()
    _check(h, torch.nn.functional.silu(g) * u, K)
    _check(raw.view(M, I // 16, 2, 16)[:, :, 0].reshape(M, I), g, K)
    _check(raw.view(M, I // 16, 2, 16)[:, :, 1].reshape(M, I), u, K)
    G.check_status()


@pytest.mark.parametrize("bn", [0, 128, 256, 512])
def test_swiglu_backward_epilogue(bn):
    """dgrad of the down projection with the SwiGLU backward in its epilogue vs autograd in fp32."""
    from wallx_b200.ops import gemm as G

    M, I, H = 300, 192, 256
    dy = _mk((M, H), 20)
    w_dn = _mk((H, I), 21, 0.1)
    gu = _mk((M, 2 * I), 22)                      # raw [16 gate | 16 up] blocks
    dgu = torch.full((M, 2 * I), 9.0, device="cuda", dtype=torch.bfloat16)
    G.launch([G.GemmSpec(dy, w_dn, dgu, b_mn=True, out2=gu, flags=G.SWIGLU_BWD)], force_bn=bn)
    torch.cuda.synchronize()
    G.check_status()
    z = gu.float().view(M, I // 16, 2, 16)
    g = z[:, :, 0].reshape(M, I).clone().requires_grad_(True)
    u = z[:, :, 1].reshape(M, I).clone().requires_grad_(True)
    dh = dy.float() @ w_dn.float()
    (torch.nn.functional.silu(g) * u).backward(dh)
    ref = torch.stack([g.grad.view(M, I // 16, 16), u.grad.view(M, I // 16, 16)], dim=2).reshape(M, 2 * I)
    _check(dgu, ref, H)


def test_grouped_two_problems_with_row_map_and_dyn():
    from wallx_b200.ops import gemm as G

    K, N0, N1 = 256, 384, 128
    M0, M1 = 200, 72
    M0p = 256
    T = M0p + 128
    x = _mk((T, K), 10)
    w0, w1 = _mk((N0, K), 11, 0.1), _mk((N1, K), 12, 0.1)
    out = torch.zeros((T, N0), device="cuda", dtype=torch.bfloat16)
    dyn0 = torch.tensor([0, M0, 0, K], dtype=torch.int32, device="cuda")
    dyn1 = torch.tensor([M0p, M1, 0, K], dtype=torch.int32, device="cuda")
    perm = torch.randperm(T, device="cuda").to(torch.int32)
    G.launch([
        G.GemmSpec(x, w0, out, M=T, dyn=dyn0, row_map=perm),
        G.GemmSpec(x, w1, out, M=T, dyn=dyn1, row_map=perm),
    ])
    ref = torch.zeros((T, N0), device="cuda")
    ref[perm[:M0].long()] = x[:M0].float() @ w0.float().t()
    r1 = torch.zeros((M1, N0), device="cuda")
    r1[:, :N1] = x[M0p:M0p + M1].float() @ w1.float().t()
    ref[perm[M0p:M0p + M1].long()] = r1
    _check(out, ref, K)
    G.check_status()


def test_k_offset_segment_reduction():
    """wgrad over a token segment: reduction range [k0, k0+K) of MN-major operands."""
    from wallx_b200.ops import gemm as G

    T, N, H = 512, 256, 192
    dy, x = _mk((T, N), 13), _mk((T, H), 14)
    k0, K = 128, 256
    out = G.gemm(dy[: k0 + K], x[: k0 + K], a_mn=True, b_mn=True, flags=G.OUT_FP32) * 0  # shape only
    G.launch([G.GemmSpec(dy[: k0 + K], x[: k0 + K], out, a_mn=True, b_mn=True, K=K, k0=k0, flags=G.OUT_FP32)])
    ref = dy[k0:k0 + K].float().t() @ x[k0:k0 + K].float()
    _check(out, ref, K)
    G.check_status()


# --------------------------------------------------------------------------- CTA-pair kernel
def test_pair_kernel_epilogues_and_groups():
    """256 x 256 tiles over CTA pairs: every epilogue, two problems with device-side segments, the
    zero-fill of pad rows that must stop at the 128-row boundary of a segment, many tiles per pair."""
    from wallx_b200.ops import gemm as G

    M, N, K = 700, 640, 320
    a, b = _mk((M, K), 3), _mk((N, K), 4, 0.1)
    bias, res = _mk((N,), 5), _mk((M, N), 6)
    ref = a.float() @ b.float().t()
    _check(G.gemm(a, b, bias=bias, force_bn=512), ref + bias.float(), K)
    _check(G.gemm(a, b, bias=bias, flags=G.ACT_GELU, force_bn=512), torch.nn.functional.gelu(ref + bias.float()), K)
    _check(G.gemm(a, b, residual=res, force_bn=512), ref + res.float(), K)
    acc = torch.ones((M, N), device="cuda", dtype=torch.float32)
    G.gemm(a, b, out=acc, flags=G.OUT_FP32 | G.ACCUMULATE, force_bn=512)
    _check(acc, ref + 1.0, K)
    # two experts, segments at 128-aligned starts, zero padding only up to the next 128 boundary
    K2, I0, I1 = 256, 192, 64
    M0, M1 = 300, 100           # expert 0 rows [0, 300) padded to 384; expert 1 starts at 384
    T = 384 + 128
    x = _mk((T, K2), 10)
    w0, w1 = _mk((2 * I0, K2), 11, 0.1), _mk((2 * I1, K2), 12, 0.1)
    h = torch.full((T, I0), 7.0, device="cuda", dtype=torch.bfloat16)
    dyn0 = torch.tensor([0, M0, 0, K2], dtype=torch.int32, device="cuda")
    dyn1 = torch.tensor([384, M1, 0, K2], dtype=torch.int32, device="cuda")
    G.launch([G.GemmSpec(x, w0, h, M=T, dyn=dyn0, flags=G.ACT_SWIGLU | G.ZERO_PAD_ROWS),
              G.GemmSpec(x, w1, h, M=T, dyn=dyn1, flags=G.ACT_SWIGLU | G.ZERO_PAD_ROWS)], force_bn=512)

    def swiglu(xx, w):
        z = (xx.float() @ w.float().t()).bfloat16().float().view(xx.shape[0], -1, 2, 16)
        return (torch.nn.functional.silu(z[:, :, 0]) * z[:, :, 1]).reshape(xx.shape[0], -1)

    _check(h[:M0], swiglu(x[:M0], w0), K2)
    assert (h[M0:384] == 0).all()                       # pad rows of expert 0
    _check(h[384:384 + M1, :I1], swiglu(x[384:384 + M1], w1), K2)
    assert (h[384 + M1:512, :I1] == 0).all()            # pad rows of expert 1
    assert (h[384:, I1:] == 7.0).all()                  # columns expert 1 does not own are untouched
    # many tiles per pair + wgrad layout with fp32 accumulation
    dy, xx = _mk((4096, 1536), 13, 0.1), _mk((4096, 1024), 14)
    dw = torch.zeros((1536, 1024), device="cuda", dtype=torch.float32)
    G.launch([G.GemmSpec(dy, xx, dw, a_mn=True, b_mn=True, flags=G.OUT_FP32 | G.ACCUMULATE)], force_bn=512)
    _check(dw, dy.float().t() @ xx.float(), 4096)
    torch.cuda.synchronize()
    G.check_status()


# --------------------------------------------------------------------------- gathered-weight mode
# The shards of the "ranks" are separate tensors on one GPU: the puller CTAs only copy and publish
# flags, so the whole mechanism (bulk copies, flags, rotated tile order, bounded waits) runs in one
# kernel on one device.
def _ag_call(x, shards, transpose_w, flags=0, rank=0, n_pullers=0, epoch_flags=None, epoch=1, out=None):
    from wallx_b200.ops import _ext
    from wallx_b200.ops import gemm as G

    world = len(shards)
    rpr, cols = shards[0].shape
    rows = rpr * world
    staging = torch.full((rows, cols), float("nan"), dtype=torch.bfloat16, device=x.device)
    fl = epoch_flags if epoch_flags is not None else torch.zeros((rows + 255) // 256, dtype=torch.int32, device=x.device)
    N = cols if transpose_w else rows
    if out is None:
        out = torch.empty(x.shape[0], N // 2 if flags & G.ACT_SWIGLU else N, dtype=torch.bfloat16, device=x.device)
    spec = G.GemmSpec(x, staging, out, b_mn=transpose_w, flags=flags)
    _ext.get().gemm_ag([spec.as_tuple()], [[s.data_ptr() for s in shards]], [fl], rank, [rpr], n_pullers, [epoch])
    return out, staging, fl


@pytest.mark.parametrize("world,rows,cols,M,rank,n_pullers", [
    (1, 512, 256, 300, 0, 0),
    (2, 2560, 2048, 1000, 1, 0),     # fused QKV of the 2048-wide decoder
    (4, 1280, 1024, 4000, 2, 5),     # 320 rows per rank: shards straddle 256-row tiles
    (8, 2048, 11008, 700, 7, 3),     # down-projection shape: 22 KB rows, 16-byte-multiple chunks
    (2, 768, 136, 129, 0, 40),       # more pullers than chunks per tile
    (2, 2560, 2048, 8192, 1, 0),     # enough 256 x 256 tiles for the CTA-pair kernel (copy clusters + GEMM pairs)
    (8, 22016, 2048, 4096, 3, 8),    # gate/up shape on CTA pairs, 2752 rows per rank
])
def test_gemm_gathered_weight_forward(world, rows, cols, M, rank, n_pullers):
    from wallx_b200.ops import gemm as G

    torch.manual_seed(0)
    dev = torch.device("cuda")
    w = (torch.randn(rows, cols, device=dev) * 0.05).to(torch.bfloat16)
    shards = [w[r * (rows // world):(r + 1) * (rows // world)].clone() for r in range(world)]
    x = torch.randn(M, cols, device=dev).to(torch.bfloat16)
    y, staging, fl = _ag_call(x, shards, False, rank=rank, n_pullers=n_pullers)
    torch.cuda.synchronize()
    G.check_status()
    assert torch.equal(staging, w)
    assert int(fl.min()) == int(fl.max()) and int(fl.min()) > 0
    ref = x.float() @ w.float().t()
    torch.testing.assert_close(y.float(), ref, atol=2e-2 * ref.abs().max().item(), rtol=2e-2)
    # second call on the same flags (epoch 2) with changed shards must see the new weights
    shards2 = [s * 0.5 for s in shards]
    y2, staging2, _ = _ag_call(x, shards2, False, rank=rank, n_pullers=n_pullers, epoch_flags=fl, epoch=2)
    torch.cuda.synchronize()
    G.check_status()
    assert torch.equal(staging2, w * 0.5)
    torch.testing.assert_close(y2.float(), ref * 0.5, atol=2e-2 * ref.abs().max().item(), rtol=2e-2)


@pytest.mark.parametrize("world,rows,cols,M", [(2, 2560, 2048, 1000), (4, 1280, 1024, 515), (1, 256, 512, 128),
                                               (2, 2560, 2048, 8192), (8, 22016, 2048, 4096)])  # the last two: CTA pairs
def test_gemm_gathered_weight_dgrad(world, rows, cols, M):
    from wallx_b200.ops import gemm as G

    torch.manual_seed(1)
    dev = torch.device("cuda")
    w = (torch.randn(rows, cols, device=dev) * 0.05).to(torch.bfloat16)
    shards = [w[r * (rows // world):(r + 1) * (rows // world)].clone() for r in range(world)]
    dy = torch.randn(M, rows, device=dev).to(torch.bfloat16)
    dx, staging, _ = _ag_call(dy, shards, True)
    torch.cuda.synchronize()
    G.check_status()
    assert torch.equal(staging, w)
    ref = dy.float() @ w.float()
    torch.testing.assert_close(dx.float(), ref, atol=2e-2 * ref.abs().max().item(), rtol=2e-2)


def test_gemm_gathered_dual_gate_up():
    """Two experts' interleaved gate/up weights gathered and multiplied in one launch, SwiGLU epilogue."""
    from wallx_b200.ops import _ext
    from wallx_b200.ops import gemm as G

    torch.manual_seed(2)
    dev = torch.device("cuda")
    world, hidden = 2, 1024
    widths = (2816, 512)  # FFN widths of the two experts
    rows_tok = (900, 260)
    specs, peers, flags, rprs, outs, refs = [], [], [], [], [], []
    for e in range(2):
        wgu = (torch.randn(2 * widths[e], hidden, device=dev) * 0.05).to(torch.bfloat16)
        rpr = 2 * widths[e] // world
        shards = [wgu[r * rpr:(r + 1) * rpr].clone() for r in range(world)]
        x = torch.randn(rows_tok[e], hidden, device=dev).to(torch.bfloat16)
        staging = torch.empty_like(wgu)
        out = torch.empty(rows_tok[e], widths[e], dtype=torch.bfloat16, device=dev)
        specs.append(G.GemmSpec(x, staging, out, flags=G.ACT_SWIGLU))
        peers.append([s.data_ptr() for s in shards])
        flags.append(torch.zeros((2 * widths[e] + 255) // 256, dtype=torch.int32, device=dev))
        rprs.append(rpr)
        outs.append(out)
        refs.append((x, wgu, shards))
    _ext.get().gemm_ag([s.as_tuple() for s in specs], peers, flags, 1, rprs, 0, [1, 1])
    torch.cuda.synchronize()
    G.check_status()
    for e in range(2):
        x, wgu, _ = refs[e]
        z = (x.float() @ wgu.float().t()).to(torch.bfloat16).float().view(x.shape[0], -1, 2, 16)
        ref = torch.nn.functional.silu(z[:, :, 0]) * z[:, :, 1]
        ref = ref.reshape(x.shape[0], widths[e])
        torch.testing.assert_close(outs[e].float(), ref, atol=2e-2 * ref.abs().max().item(), rtol=3e-2)
