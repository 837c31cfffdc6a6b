"""Single-kernel workloads for roofline accounting and for profiler captures.

``python -m wallx_b200.bench.kernel_cases --case NAME [--iters 10]`` runs one named case (a few
launches of one hand-written kernel on inputs larger than L2 but at most a few GB), times it with
CUDA events and prints one JSON line with the achieved bytes/s or FLOP/s and its fraction of the
measured peak (``MEASURED_PEAKS.json`` at the repository root: STREAM-style copy bandwidth and
cuBLAS bf16 throughput). ``--case all`` runs every case; ``--list`` prints the names with the
kernel each exercises (the ``-k regex:`` to give a profiler). ``--profile`` runs exactly one warm-up
launch and two measured launches, so that a capture of the named kernel stays small.

The attention cases use the model's real shapes (LLM: 16 query / 2 KV heads of 128, 346-token
sequences, causal with a 32-token bidirectional action block; ViT: 16 heads of 80, 112-pixel
windows and full 324-patch images) with enough sequences that q/k/v exceed L2.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "of measured"
    except Exception:
        return 6650.0, 1590.0, "of fallback"


def _bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


# Each case returns (fn, kernel_regex, bytes, flops, note). bytes / flops are algorithmic (one
# read of every input, one write of every output).
def case_gemm(M, N, K, a_mn=False, b_mn=False, flags=0, extra=None, force_bn=0):
    def build():
        from wallx_b200.ops import gemm as G

        a = _bf(K, M) if a_mn else _bf(M, K)
        b = _bf(K, N) if b_mn else _bf(N, K, scale=0.05)
        width = N // 2 if flags & G.ACT_SWIGLU else N
        out = torch.empty(M, width, device="cuda", dtype=torch.float32 if flags & G.OUT_FP32 else torch.bfloat16)
        kw = {}
        nbytes = (M * K + N * K) * 2 + out.numel() * out.element_size()
        if extra == "swiglu_raw":
            kw["out2"] = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            nbytes += M * N * 2
        if extra == "swiglu_bwd":  # accumulator = dL/dh [M, N]; reads raw gate/up [M, 2N], writes dL/d(gate|up) [M, 2N]
            out = torch.empty(M, 2 * N, device="cuda", dtype=torch.bfloat16)
            kw["out2"] = _bf(M, 2 * N)
            nbytes = (M * K + N * K) * 2 + 2 * M * 2 * N * 2
        if extra == "residual":
            kw["residual"] = _bf(M, N)
            nbytes += M * N * 2
        spec = G.GemmSpec(a, b, out, a_mn=a_mn, b_mn=b_mn, flags=flags, **kw)
        name = "gemm_pair_kernel" if force_bn == 512 else "gemm_kernel"
        # library twin: the bare product through torch.matmul (cuBLAS), without this kernel's epilogue work
        aa = a.t() if a_mn else a
        bb = b if b_mn else b.t()
        lib_out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        lib = lambda: torch.matmul(aa, bb, out=lib_out)
        return ((lambda: G.launch([spec], force_bn)), name, nbytes, 2.0 * M * N * K,
                f"M={M} N={N} K={K} a_mn={a_mn} b_mn={b_mn}", lib, "torch.matmul (cuBLAS), bare product")
    return build


def case_gemm_dual():
    from wallx_b200.ops import functional as F_
    from wallx_b200.ops import gemm as G

    T, H, I0, I1 = 16384, 2048, 11008, 2048
    tt = (torch.rand(T, device="cuda") < 0.1).to(torch.int32)
    plan = F_.make_route_plan(tt, 2)
    n1 = int(tt.sum())
    xp = _bf(plan.rows, H)
    w0, w1 = _bf(2 * I0, H, scale=0.05), _bf(2 * I1, H, scale=0.05)
    h = torch.empty(plan.rows, I0, device="cuda", dtype=torch.bfloat16)
    specs = [G.GemmSpec(xp, w, h, M=plan.rows, dyn=plan.seg[e], flags=G.ACT_SWIGLU | G.ZERO_PAD_ROWS)
             for e, w in enumerate((w0, w1))]
    flops = 2.0 * H * 2 * ((T - n1) * I0 + n1 * I1)
    nbytes = (T * H + 2 * (I0 + I1) * H + (T - n1) * I0 + n1 * I1) * 2
    return (lambda: G.launch(specs)), "gemm_kernel", nbytes, flops, f"two experts, {T} tokens, 10% action, SwiGLU epilogue"


def case_gemm_gathered():
    """The fused weight gather with the ranks' shards as four local tensors (one kernel, one GPU)."""
    from wallx_b200.ops import _ext
    from wallx_b200.ops import gemm as G

    M, N, K, world = 8192, 22016, 2048, 4
    x = _bf(M, K)
    shards = [_bf(N // world, K, scale=0.05) for _ in range(world)]
    staging = torch.empty(N, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N // 2, device="cuda", dtype=torch.bfloat16)
    flags = torch.zeros((N + 255) // 256, dtype=torch.int32, device="cuda")
    spec = G.GemmSpec(x, staging, out, flags=G.ACT_SWIGLU)
    epoch = [0]

    def fn():
        epoch[0] += 1
        _ext.get().gemm_ag([spec.as_tuple()], [[s.data_ptr() for s in shards]], [flags], 1, [N // world], 0, [epoch[0]])

    nbytes = (M * K + 2 * N * K + N * K + M * N // 2) * 2  # shards read + staging written + staging read
    return fn, "gemm_kernel", nbytes, 2.0 * M * N * K, f"M={M} N={N} K={K}, 4 shards pulled by 12 copy CTAs inside the GEMM"


def _attn(cu, hq, hkv, D, causal, bidir_n, which):
    from wallx_b200.ops import functional as F_

    T = cu[-1]
    qkv = _bf(T, (hq + 2 * hkv) * D, scale=0.5).requires_grad_(which != "fwd")
    bid = None
    if bidir_n:
        bid = torch.zeros(T, dtype=torch.bool, device="cuda")
        for i in range(len(cu) - 1):
            bid[cu[i + 1] - bidir_n:cu[i + 1]] = True
    meta = F_.AttnMeta(cu, "cuda", causal, bid)
    meta.device_tables("cuda")
    fl = sum(4.0 * (cu[i + 1] - cu[i]) ** 2 * D * hq * (0.5 if causal else 1.0) for i in range(len(cu) - 1))
    # library twin: flash-attn 2 on the same tensors, the call the reference makes (flash_attn_varlen_func; plain
    # causal for the LLM, i.e. without the bidirectional action block, as its flash path runs it)
    lib_fwd = lib_bwd = None
    try:
        from flash_attn import flash_attn_varlen_func

        q3 = qkv.detach()[:, : hq * D].reshape(T, hq, D).contiguous().requires_grad_(which != "fwd")
        k3 = qkv.detach()[:, hq * D:(hq + hkv) * D].reshape(T, hkv, D).contiguous().requires_grad_(which != "fwd")
        v3 = qkv.detach()[:, (hq + hkv) * D:].reshape(T, hkv, D).contiguous().requires_grad_(which != "fwd")
        cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
        mx = max(cu[i + 1] - cu[i] for i in range(len(cu) - 1))

        def lib_fwd():
            with torch.no_grad():
                flash_attn_varlen_func(q3, k3, v3, cu_t, cu_t, mx, mx, causal=causal)

        if which != "fwd":
            o3 = flash_attn_varlen_func(q3, k3, v3, cu_t, cu_t, mx, mx, causal=causal)
            g3 = torch.randn_like(o3)

            def lib_bwd():
                q3.grad = k3.grad = v3.grad = None
                o3.backward(g3, retain_graph=True)
    except Exception:  # flash-attn is not importable here: the row simply has no library column
        lib_fwd = lib_bwd = None
    if which == "fwd":
        def fn():
            with torch.no_grad():
                F_.attention_packed(qkv, meta, hq, hkv, D)
        return (fn, "attn_fwd_kernel", T * (2 * hq + 2 * hkv) * D * 2, fl, f"T={T} hq={hq} hkv={hkv} d={D}", lib_fwd,
                "flash_attn_varlen_func forward")
    o = F_.attention_packed(qkv, meta, hq, hkv, D)
    g = torch.randn_like(o)

    def fn():
        qkv.grad = None
        o.backward(g, retain_graph=True)

    reg = "attn_dq_kernel" if which == "dq" else "attn_dkdv_kernel"
    return (fn, reg, T * (4 * hq + 4 * hkv) * D * 2, 2.5 * fl,
            f"backward (delta + dq + dk/dv kernels), T={T} hq={hq} hkv={hkv} d={D}", lib_bwd, "flash_attn_varlen_func backward")


def case_attn_llm(which):
    return lambda: _attn([346 * i for i in range(129)], 16, 2, 128, True, 32, which)


def case_attn_vit(kind, which):
    def build():
        if kind == "window":
            per, cu = [64, 64, 16, 64, 64, 16, 16, 16, 4], [0]
            for _ in range(192):
                for p in per:
                    cu.append(cu[-1] + p)
        else:
            cu = [324 * i for i in range(193)]
        return _attn(cu, 16, 16, 80, False, 0, which)
    return build


def case_rms_norm(which):
    def build():
        from wallx_b200.ops import _ext

        C = _ext.get()
        T, H = 65536, 2048
        x, w = _bf(T, H), _bf(H)
        if which == "fwd":
            return (lambda: C.rms_norm_fwd(x, w, 1e-6, None, 0)), "rms_norm_fwd_kernel", T * H * 4, 0, f"[{T}, {H}]"
        y, rstd = C.rms_norm_fwd(x, w, 1e-6, None, 0)
        dy = _bf(T, H)
        return (lambda: C.rms_norm_bwd(dy, x, w, rstd, None)), "rms_norm_bwd_kernel", T * H * 6, 0, f"[{T}, {H}]"
    return build


def case_swiglu_bwd():
    from wallx_b200.ops import _ext

    R, I = 16384, 11008
    dh, gu = _bf(R, I), _bf(R, 2 * I)
    return (lambda: _ext.get().swiglu_bwd(dh, gu)), "swiglu_bwd_kernel", R * I * 2 * 5, 0, f"dh [{R}, {I}]"


def case_rope():
    from wallx_b200.ops import _ext

    T, hq, hkv, D = 65536, 16, 2, 128
    qkv = _bf(T, (hq + 2 * hkv) * D)
    ang = torch.rand(T, D, device="cuda")
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    nbytes = T * (hq + hkv) * D * 2 * 2 + T * D * 8
    return (lambda: _ext.get().rope_qk(qkv, cos, sin, hq + hkv, D, False)), "rope_qk_kernel", nbytes, 0, f"qkv [{T}, {(hq + 2 * hkv) * D}]"


def case_permute(which):
    def build():
        from wallx_b200.ops import _ext
        from wallx_b200.ops import functional as F_

        C = _ext.get()
        T, H = 65536, 2048
        tt = (torch.rand(T, device="cuda") < 0.25).to(torch.int32)
        plan = F_.make_route_plan(tt, 2)
        x = _bf(T, H)
        if which == "permute":
            return (lambda: C.permute_rows(x, plan.dest, plan.rows)), "permute_rows_kernel", T * H * 4, 0, f"[{T}, {H}] 25% action"
        xp = C.permute_rows(x, plan.dest, plan.rows)
        return (lambda: C.gather_rows(xp, plan.dest)), "gather_rows_kernel", T * H * 4, 0, f"[{T}, {H}]"
    return build


def case_ce(which):
    def build():
        from wallx_b200.ops import _ext

        C = _ext.get()
        R, V = 4096, 151936 + 2048
        logits = _bf(R, V)
        labels = torch.randint(0, V, (R,), device="cuda")
        loss = torch.empty(R, device="cuda")
        lse = torch.empty(R, device="cuda")
        pred = torch.empty(R, device="cuda", dtype=torch.int64)
        if which == "fwd":
            return (lambda: C.ce_fwd(logits, labels, loss, lse, pred)), "ce_fwd_kernel", R * V * 2, 0, f"logits [{R}, {V}]"
        C.ce_fwd(logits, labels, loss, lse, pred)
        dl = torch.ones(R, device="cuda")
        return (lambda: C.ce_bwd(logits, labels, lse, dl)), "ce_bwd_kernel", R * V * 4, 0, f"logits [{R}, {V}] in place"
    return build


def case_adamw(fp32_grad):
    def build():
        from wallx_b200.ops import _ext

        C = _ext.get()
        n = 128 * 1024 * 1024
        p16 = _bf(n)
        p32 = p16.float()
        m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
        g = torch.randn(n, device="cuda") if fp32_grad else _bf(n)
        hyper = torch.tensor([1e-4, 0.9, 0.999, 1e-8, 0.1, 1.0, 1.0, 0.1, 0.001, 0, 0, 0], device="cuda")
        nbytes = n * (2 + 4 * 6 + (4 if fp32_grad else 2))
        if fp32_grad:
            return (lambda: C.adamw_step_f32g(p16, p32, m, v, g, hyper, None)), "adamw_f32g_kernel", nbytes, 0, f"{n} parameters"
        return (lambda: C.adamw_step(p16, p32, m, v, g, hyper, None)), "adamw_kernel", nbytes, 0, f"{n} parameters"
    return build


def case_column_sum():
    from wallx_b200.ops import _ext

    T, N = 65536, 3840
    x = _bf(T, N)
    return (lambda: _ext.get().column_sum(x)), "column_sum_kernel", T * N * 2, 0, f"[{T}, {N}]"


def case_reduce_scatter():
    """One-shot reduce-scatter + squared norm with four ranks' gradient arenas as local tensors."""
    from wallx_b200.ops import _ext

    world, shard = 4, 32 * 1024 * 1024
    arenas = [_bf(world * shard) for _ in range(world)]
    table = torch.tensor([[1 * shard, shard, 0]], dtype=torch.int64, device="cuda")  # rank 1's slice
    out = torch.empty(shard, device="cuda")
    ss = torch.zeros(1, device="cuda")
    fn = lambda: _ext.get().rs_reduce([a.data_ptr() for a in arenas], table, out, ss)
    return fn, "rs_reduce_kernel", shard * (2 * world + 4), 0, f"{world} ranks x {shard} bf16 -> fp32 shard"


def case_index(which):
    """The index-generation kernels at the benchmark batch (32 samples x 3 views of 18 x 18 patches, 346 tokens per
    sample): latency-bound single launches, reported in microseconds."""
    def build():
        from wallx_b200.config import wall_oss_config
        from wallx_b200.data.synthetic import make_batch, make_processor
        from wallx_b200.ops import _ext
        from wallx_b200.ops import functional as F_
        from wallx_b200.ops import index as IX

        C = _ext.get()
        B, views = 32, 3
        grid = torch.tensor([[1, 18, 18]] * (B * views), dtype=torch.int64, device="cuda")
        if which == "rope_index":
            cfg = wall_oss_config(action_expert_intermediate=2048, num_hidden_layers=1)
            proc = make_processor(cfg, 2048)
            b = make_batch(cfg, proc, B, views=views, image_hw=(256, 256), prompt_len=64, horizon=32, mode="flow",
                           generator=torch.Generator().manual_seed(0))
            ids, am, g = b["input_ids"].cuda(), b["attention_mask"].cuda(), b["image_grid_thw"].cuda()
            vc = cfg.vision_config
            fn = lambda: IX.get_rope_index(ids, g, None, None, am, vc.spatial_merge_size, cfg.image_token_id, cfg.video_token_id,
                                           cfg.vision_start_token_id, vc.tokens_per_second)
            return fn, "rope_index_kernel", ids.numel() * (8 + 24), 0, f"ids [{ids.shape[0]}, {ids.shape[1]}], {B * views} images"
        if which == "vit_rot_pos":
            inv = 1.0 / (10000.0 ** (torch.arange(0, 40, 2, dtype=torch.float, device="cuda") / 40))
            n = B * views * 324
            return (lambda: IX.rot_pos_emb(inv, grid, 2)), "vit_rot_pos_kernel", n * 40 * 4, 0, f"{B * views} grids of 18 x 18 -> [{n}, 40]"
        if which == "vit_window_index":
            n = B * views * 81
            return (lambda: IX.get_window_index(grid, 112, 2, 14)), "vit_window_index_kernel", n * 8, 0, f"{B * views} grids of 18 x 18, 112-pixel windows"
        T = B * 346
        tt = (torch.rand(T, device="cuda") < 0.09).to(torch.int32)
        return (lambda: F_.make_route_plan(tt, 2)), "route_plan_kernel", T * 12, 0, f"{T} tokens, 2 experts"
    return build


CASES = {
    "gemm_qkv": case_gemm(16384, 2560, 2048),
    "gemm_gate_up_swiglu": case_gemm(16384, 22016, 2048, flags=8, extra="swiglu_raw"),
    "gemm_down_residual": case_gemm(16384, 2048, 11008, extra="residual"),
    "gemm_dgrad": case_gemm(16384, 2048, 22016, b_mn=True),
    "gemm_wgrad_fp32_accumulate": case_gemm(22016, 2048, 16384, a_mn=True, b_mn=True, flags=3),
    "gemm_vit_qkv": case_gemm(62208, 3840, 1280),
    "gemm_qkv_pair": case_gemm(16384, 2560, 2048, force_bn=512),
    "gemm_gate_up_swiglu_pair": case_gemm(16384, 22016, 2048, flags=8, extra="swiglu_raw", force_bn=512),
    "gemm_down_residual_pair": case_gemm(16384, 2048, 11008, extra="residual", force_bn=512),
    "gemm_dgrad_pair": case_gemm(16384, 2048, 22016, b_mn=True, force_bn=512),
    "gemm_wgrad_fp32_accumulate_pair": case_gemm(22016, 2048, 16384, a_mn=True, b_mn=True, flags=3, force_bn=512),
    "gemm_vit_qkv_pair": case_gemm(62208, 3840, 1280, force_bn=512),
    "gemm_down_dgrad": case_gemm(16384, 11008, 2048, b_mn=True),
    "gemm_down_dgrad_swiglu_bwd": case_gemm(16384, 11008, 2048, b_mn=True, flags=32, extra="swiglu_bwd"),
    "gemm_dual_expert": case_gemm_dual,
    "gemm_gathered_weight": case_gemm_gathered,
    "attn_llm_fwd": case_attn_llm("fwd"),
    "attn_llm_dq": case_attn_llm("dq"),
    "attn_llm_dkdv": case_attn_llm("dkdv"),
    "attn_vit_window_fwd": case_attn_vit("window", "fwd"),
    "attn_vit_full_fwd": case_attn_vit("full", "fwd"),
    "attn_vit_full_dkdv": case_attn_vit("full", "dkdv"),
    "rms_norm_fwd": case_rms_norm("fwd"),
    "rms_norm_bwd": case_rms_norm("bwd"),
    "swiglu_bwd": case_swiglu_bwd,
    "rope_qk": case_rope,
    "permute_rows": case_permute("permute"),
    "gather_rows": case_permute("gather"),
    "ce_fwd": case_ce("fwd"),
    "ce_bwd": case_ce("bwd"),
    "adamw_bf16_grad": case_adamw(False),
    "adamw_fp32_grad": case_adamw(True),
    "column_sum": case_column_sum,
    "reduce_scatter_local": case_reduce_scatter,
    "rope_index": case_index("rope_index"),
    "vit_rot_pos": case_index("vit_rot_pos"),
    "vit_window_index": case_index("vit_window_index"),
    "route_plan": case_index("route_plan"),
}


def run_case(name, iters, profile, no_lib=False):
    from wallx_b200.ops import gemm as G

    torch.manual_seed(0)
    built = CASES[name]()
    fn, regex, nbytes, flops, note = built[:5]
    lib_fn, lib_name = (built[5], built[6]) if len(built) > 5 else (None, None)
    warm = 1 if profile else 3
    n = 2 if profile else iters

    def median_ms(f):
        for _ in range(warm):
            f()
        torch.cuda.synchronize()
        ts = []
        for _ in range(n):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            f()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        return ts[len(ts) // 2]

    ms = median_ms(fn)
    G.check_status()
    hbm, tf, tag = _peaks()
    rec = {"case": name, "kernel": regex, "ms": round(ms, 4), "note": note}
    if flops:
        rec["tflops"] = round(flops / ms / 1e9, 1)
        rec["frac_of_gemm_peak"] = round(flops / ms / 1e9 / tf, 3)
    rec["algorithmic_GBs"] = round(nbytes / ms / 1e6, 1)
    rec["frac_of_copy_bw"] = round(nbytes / ms / 1e6 / hbm, 3)
    rec["peaks"] = f"{hbm} GB/s copy, {tf} TFLOP/s cuBLAS bf16 burst, {tag}"
    if name.endswith("_dq") or name.endswith("_dkdv"):
        rec["timed"] = "whole attention backward (three kernels)"
    if lib_fn is not None and not profile and not no_lib:
        lib_ms = median_ms(lib_fn)
        rec["library"] = lib_name
        rec["library_ms"] = round(lib_ms, 4)
        rec["speedup_vs_library"] = round(lib_ms / ms, 3)
    return rec


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--no-lib", action="store_true", help="skip the library twin (cuBLAS / flash-attn 2) of each case")
    ap.add_argument("--out", default="")
    args = ap.parse_args(argv)
    if args.list:
        for k in CASES:
            print(k)
        return
    if not torch.cuda.is_available():
        print(json.dumps({"unavailable": "no CUDA device"}))
        return
    names = list(CASES) if args.case == "all" else args.case.split(",")
    lines = []
    for nm in names:
        rec = run_case(nm, args.iters, args.profile, args.no_lib)
        lines.append(json.dumps(rec))
        print(lines[-1], flush=True)
        torch.cuda.empty_cache()
    if args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        with open(args.out, "a") as f:
            f.write("\n".join(lines) + "\n")


if __name__ == "__main__":
    sys.exit(main())
