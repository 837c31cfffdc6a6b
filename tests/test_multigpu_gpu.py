"""Hand-written NVLink transport vs NCCL on 2 GPUs, and the bounded-wait failure path."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, tmp, transport):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    torch.distributed.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from wallx_b200.config import tiny_config
    from wallx_b200.data.collator import add_pack_info, to_device
    from wallx_b200.data.synthetic import make_batch, make_processor
    from wallx_b200.models import Qwen2_5_VLMoEForAction
    from wallx_b200.ops import gemm as G
    from wallx_b200.parallel.engine import TrainEngine

    cfg = tiny_config()
    proc = make_processor(cfg, 16)
    m = Qwen2_5_VLMoEForAction(cfg, processor=proc)
    m.init_weights(seed=0)
    m = m.to(torch.bfloat16).to(dev)
    symm = None
    overlap = transport == "symm_overlap"
    if overlap:
        transport = "symm"
    if transport == "symm":
        from wallx_b200.parallel.symm import SymmComm

        symm = SymmComm(torch.distributed.group.WORLD, dev)
    eng = TrainEngine(m, lr=1e-3, weight_decay=0.1, max_grad_norm=1.0, grad_accum=1, world=world, rank=rank,
                      transport=transport, symm=symm)
    eng.overlap_reduce = overlap
    g = torch.Generator().manual_seed(5)
    batches = []
    for _ in range(2 * world):
        b = add_pack_info(make_batch(cfg, proc, 2, views=1, image_hw=(112, 112), prompt_len=16, horizon=16, generator=g), cfg)
        b["flow_noise"] = torch.randn(b["action_chunk"].shape, generator=g)
        b["flow_time"] = torch.rand(2, generator=g)
        batches.append(b)
    norms = []
    for step in range(2):
        b = to_device(batches[step * world + rank], dev, torch.bfloat16)
        eng.backward(m(mode="train", **b).loss)
        eng.optimizer_step(1e-3)
        norms.append(eng.grad_norm().item())
    torch.cuda.synchronize()
    G.check_status()
    if symm is not None:
        symm.check()
    tag = "symm_overlap" if overlap else transport
    early = len(eng._early) if overlap else 0
    torch.save({"params": {n: p.detach().float().cpu() for n, p in m.named_parameters()}, "norms": norms,
                "early_units": early}, os.path.join(tmp, f"{tag}_{rank}.pt"))
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()


@pytest.mark.timeout(600)
def test_symm_transport_matches_nccl(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    for transport in ("dist", "symm", "symm_overlap"):
        mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), transport), nprocs=2, join=True)
    d0, d1 = torch.load(tmp_path / "dist_0.pt"), torch.load(tmp_path / "dist_1.pt")
    s0, s1 = torch.load(tmp_path / "symm_0.pt"), torch.load(tmp_path / "symm_1.pt")
    for k in s0["params"]:
        assert torch.equal(s0["params"][k], s1["params"][k]), k  # replicas identical
        assert torch.equal(d0["params"][k], d1["params"][k]), k
        # fp32 peer sum vs NCCL's bf16 reduction: equal up to one bf16 ulp of the stored parameter
        # (0.0039 at 1.0) plus a fraction of an lr-sized Adam step
        a, b = s0["params"][k], d0["params"][k]
        assert torch.allclose(a, b, atol=8e-3, rtol=8e-3), k
        assert ((a - b).abs() > 2.5e-3).float().mean() < 0.2, k
    assert abs(s0["norms"][0] - d0["norms"][0]) / d0["norms"][0] < 2e-2
    # reduce-scatter per unit during backward: the same kernels on the same data. Runs are not bit-identical
    # (fp32 atomics in the bias-gradient column sums and the squared norm land in another order), and Adam
    # turns last-bit differences of noise-level gradients (e.g. the key bias, whose true gradient is zero)
    # into sign flips of an lr-sized update, so the comparison is the same as for the NCCL transport.
    o0, o1 = torch.load(tmp_path / "symm_overlap_0.pt"), torch.load(tmp_path / "symm_overlap_1.pt")
    for k in s0["params"]:
        assert torch.equal(o0["params"][k], o1["params"][k]), k  # replicas identical
        a, b = o0["params"][k], s0["params"][k]
        assert torch.allclose(a, b, atol=8e-3, rtol=8e-3), k
        assert ((a - b).abs() > 2.5e-3).float().mean() < 0.2, k
    assert abs(o0["norms"][0] - s0["norms"][0]) / s0["norms"][0] < 1e-3
    assert o0["early_units"] >= 3 and o1["early_units"] >= 3


def test_barrier_wait_runs_out_and_reports_status():
    """A flag that nothing sets: the kernel gives up after its limit and the context stays usable."""
    from wallx_b200.ops import _ext

    C = _ext.get()
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    # "two ranks" whose flag arrays both live here; rank 1 never runs, so its signal never comes
    C.symm_barrier([flags.data_ptr(), flags[32:].data_ptr()], 0, 1, status)
    torch.cuda.synchronize()
    assert status[0].item() == 17
    assert flags[0].item() == 1 and flags[32].item() == 1  # our own signals were delivered
    x = torch.ones(8, device="cuda") * 2  # context still works
    assert x.sum().item() == 16


def _ag_worker(rank, world, port, tmp):
    import faulthandler

    faulthandler.enable()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    import torch.distributed as dist

    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from wallx_b200.ops import gemm as G
    from wallx_b200.parallel.ag_linear import AgLinear, GatherWorkspace

    torch.manual_seed(0)  # same full weight on every rank; each keeps its rows
    rows, cols, T = 2560, 2048, 1536
    full = (torch.randn(rows, cols, device=dev) * 0.03).to(torch.bfloat16)
    ws = GatherWorkspace(rows * cols, dev, slots=1)
    lin = AgLinear(cols, rows, dist.group.WORLD, dev, workspace=ws)
    lin.weight.load_full(full)
    torch.cuda.synchronize()
    dist.barrier()  # every shard is in place before any rank gathers
    torch.manual_seed(10 + rank)
    x = torch.randn(T, cols, device=dev).to(torch.bfloat16).requires_grad_(True)
    dy = torch.randn(T, rows, device=dev).to(torch.bfloat16)
    res = {}
    for it in range(2):
        x.grad = None
        y = lin(x)
        y.backward(dy)
        gshard = lin.reduce_scatter_grad()
    torch.cuda.synchronize()
    G.check_status()
    # reference: NCCL all-gather of the shards + fp32 matmuls
    parts = [torch.empty_like(lin.weight.shard) for _ in range(world)]
    dist.all_gather(parts, lin.weight.shard)
    w = torch.cat(parts).float()
    assert torch.equal(w.to(torch.bfloat16), full)
    y_ref = x.detach().float() @ w.t()
    dx_ref = dy.float() @ w
    dw = dy.float().t() @ x.detach().float()
    dist.all_reduce(dw, op=dist.ReduceOp.AVG)
    r0 = rank * (rows // world)
    res["y"] = (y.detach().float() - y_ref).abs().max().item() / y_ref.abs().max().item()
    res["dx"] = (x.grad.float() - dx_ref).abs().max().item() / dx_ref.abs().max().item()
    res["dw"] = (gshard - dw[r0:r0 + rows // world]).abs().max().item() / dw.abs().max().item()
    torch.save(res, os.path.join(tmp, f"ag_{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_gathered_weight_linear_two_gpus(tmp_path):
    """Weight shards pulled from the peer GPU inside the GEMM: forward, dgrad and sharded wgrad."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mp.spawn(_ag_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(tmp_path / f"ag_{r}.pt")
        assert res["y"] < 1e-2 and res["dx"] < 1e-2 and res["dw"] < 1e-2, res
