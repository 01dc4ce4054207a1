"""Two-GPU NCCL runs of the sharded forms (one process per GPU): the N-sharded linear with its
all-gather and the expert-parallel routed experts with all-to-all dispatch and combine, each against
the same computation on one GPU.  Skipped when the box has fewer than two GPUs."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _affine(g, dev, lead, n, k, bits):
    w = torch.randint(-2 ** 31, 2 ** 31 - 1, lead + (n, k * bits // 32), dtype=torch.int32, device=dev, generator=g)
    s = (torch.randn(lead + (n, k // 64), device=dev, generator=g) * 0.02).abs().to(torch.bfloat16)
    b = (torch.randn(lead + (n, k // 64), device=dev, generator=g) * 0.01).to(torch.bfloat16)
    return w, s, b


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from lisa_b200 import ops, parallel
    from lisa_b200.quant import QuantizedLinear, SwitchGlu

    ok = {}
    g = torch.Generator(device=dev)
    g.manual_seed(0)  # same tensors on every rank
    # ---- N-sharded 2-bit linear (config 3 geometry, shortened), M in {1, 8, 512}
    n, k, bits = 17408, 5120, 2
    w, s, b = _affine(g, dev, (), n, k, bits)
    lin = parallel.ShardedQuantizedLinear.from_full(w, s, b, world, rank, 64, bits)
    for m in (1, 8, 512):
        x = torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16)
        y = lin.forward(x)
        full = ops.quantized_matmul(x, w, s, b, True, 64, bits)
        # the shard's kernel plan (tile height, k segments) may differ from the full matrix's, so the
        # f32 summation order may too: a bf16 ulp, not equality
        ok[f"linear_m{m}"] = bool((y.float() - full.float()).abs().max() <= 1e-2 * full.float().abs().max())
    # ---- the same linear without NCCL: GEMV epilogue stores into every rank's buffer + peer barrier
    # (up to 8 rows), or the GEMM's epilogue does (more rows)
    fused = parallel.FusedShardedLinear(lin, max_rows=300)
    for m in (1, 8, 40, 300):
        x = torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16)
        full = ops.quantized_matmul(x, w, s, b, True, 64, bits)
        for rep in range(3):  # the buffers are reused: the barrier epochs must keep the ranks in step
            y = fused.forward(x)
            torch.cuda.synchronize()
            ok[f"fused_m{m}_{rep}"] = bool((y.float() - full.float()).abs().max() <= 1e-2 * full.float().abs().max())
            dist.barrier()  # nobody overwrites a buffer another rank is still comparing
    # ---- back-to-back calls of one instance without any host barrier between them: the instance alternates
    # between two output buffers, so the view of call i stays intact while call i+1 is stored
    xa = torch.randn((3, k), device=dev, generator=g).to(torch.bfloat16)
    xb = torch.randn((3, k), device=dev, generator=g).to(torch.bfloat16)
    fa, fb = (ops.quantized_matmul(t, w, s, b, True, 64, bits).float() for t in (xa, xb))
    good = True
    for rep in range(6):
        ya = fused.forward(xa)
        keep = ya.float()          # the consumer of call i, on the same stream, before call i+1
        yb = fused.forward(xb)
        good = good and bool((keep - fa).abs().max() <= 1e-2 * fa.abs().max())
        good = good and bool((yb.float() - fb).abs().max() <= 1e-2 * fb.abs().max())
    torch.cuda.synchronize()
    ok["fused_back_to_back"] = good
    dist.barrier()
    # ---- two sharded linears that read the same x: one launch, one barrier
    w2, s2, b2 = _affine(g, dev, (), 5120, k, bits)
    lin2 = parallel.ShardedQuantizedLinear.from_full(w2, s2, b2, world, rank, 64, bits)
    sib = parallel.FusedShardedSiblings([lin, lin2], max_rows=8)
    for m in (1, 3):
        x = torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16)
        fulls = [ops.quantized_matmul(x, w, s, b, True, 64, bits), ops.quantized_matmul(x, w2, s2, b2, True, 64, bits)]
        for rep in range(2):
            launches = ops.launch_count()
            ys = sib.forward(x)
            torch.cuda.synchronize()
            ok[f"siblings_m{m}_{rep}_launches"] = ops.launch_count() - launches == 2  # GEMV + barrier
            for j, (y, full) in enumerate(zip(ys, fulls)):
                ok[f"siblings_m{m}_{rep}_{j}"] = bool((y.float() - full.float()).abs().max() <= 1e-2 * full.float().abs().max())
            dist.barrier()
    # ---- GGUF K-quant matrices N-sharded: local matvec + NCCL all-gather of the f32 blocks, and the fused form
    for fmt, block in (("Q4K", 144), ("Q2K", 84)):
        rows_g, kg = 7168, 2048  # Q2_K rows must be whole 336-byte groups for the fused form: k a multiple of 1024
        nb = kg // 256
        gw = torch.randint(0, 256, (rows_g, nb, block), dtype=torch.uint8, device=dev, generator=g)
        dd = (torch.randn((rows_g, nb, 2), device=dev, generator=g) * 0.01).abs().to(torch.float16).view(torch.uint8)
        at = 0 if fmt == "Q4K" else 80
        gw[:, :, at:at + 4] = dd.reshape(rows_g, nb, 4)
        gw = gw.reshape(rows_g, nb * block).contiguous()
        glin = parallel.ShardedGgufLinear.from_full(fmt, gw, world, rank)
        gx = torch.randn((3, kg), device=dev, generator=g)
        full = ops.packed_matvec(fmt, gw, gx)
        ok[f"gguf_{fmt}_nccl"] = bool(torch.equal(glin.forward(gx), full))
        gf = parallel.FusedShardedGguf(glin, max_tokens=2)
        for rep in range(3):
            y1 = gf.forward(gx[:1].contiguous())
            torch.cuda.synchronize()
            ok[f"gguf_{fmt}_fused_{rep}"] = bool((y1 - full[:1]).abs().max() <= 1e-4 * full.abs().max())
            dist.barrier()
    ok["device_status"] = ops.device_status() == 0
    # ---- expert-parallel routed experts (config 4 geometry with 16 experts), tokens data-parallel
    experts, hidden, inter, top_k, tokens = 16, 2048, 768, 8, 64
    gate, up, down = (_affine(g, dev, (experts,), inter, hidden, 4), _affine(g, dev, (experts,), inter, hidden, 4),
                      _affine(g, dev, (experts,), hidden, inter, 4))
    x = torch.randn((tokens, hidden), device=dev, generator=g).to(torch.bfloat16)
    logits = torch.randn((tokens, experts), device=dev, generator=g)
    block = SwitchGlu(QuantizedLinear(*gate, 64, 4), QuantizedLinear(*up, 64, 4), QuantizedLinear(*down, 64, 4), top_k)
    ref = block.forward(x, logits)
    idx, wts = ops.moe_route(logits, top_k)
    e0, e1 = parallel.expert_range(experts, world, rank)
    mine = slice(rank * tokens // world, (rank + 1) * tokens // world)

    def local_experts(rows, local_ids):
        order = torch.sort(local_ids, stable=True).indices
        xs, ids = rows[order].contiguous(), local_ids[order].contiguous()
        sl = lambda t: tuple(a[e0:e1].contiguous() for a in t)
        r = rows.shape[0]
        gg = ops.gather_qmm(xs.reshape(r, 1, hidden), *sl(gate), None, ids, True, 64, 4, True).reshape(r, inter)
        uu = ops.gather_qmm(xs.reshape(r, 1, hidden), *sl(up), None, ids, True, 64, 4, True).reshape(r, inter)
        dd = ops.gather_qmm(ops.swiglu(gg, uu).reshape(r, 1, inter), *sl(down), None, ids, True, 64, 4, True).reshape(r, hidden)
        res = torch.empty_like(dd)
        res[order] = dd
        return res

    # the same exchange by the library's own kernels over peer memory (no collective on the data path)
    sl = lambda t: QuantizedLinear(*(a[e0:e1].contiguous() for a in t), 64, 4)
    ep = parallel.ExpertParallelMoe(SwitchGlu(sl(gate), sl(up), sl(down), top_k), experts, tokens, hidden)
    # three steps with the count matrix read on the device (small capacity: no host synchronisation), then three
    # with the host read that large capacities use; the buffers are reused throughout
    for rep in range(6):
        if rep == 3:
            ep.DEVICE_COUNT_ROWS = 0
        yp = ep.forward(x[mine].contiguous(), logits[mine].contiguous())
        torch.cuda.synchronize()
        dp = (yp.float() - ref[mine].float()).abs().max().item()
        ok[f"moe_peer_{rep}"] = dp <= 1e-2 * ref.float().abs().max().item()
    ok["device_status_ep"] = ops.device_status() == 0
    y = parallel.ep_moe_forward(x[mine].contiguous(), idx[mine].contiguous(), wts[mine].contiguous(), experts, local_experts)
    # the grouped GEMM tiles differ between the sharded and the single-GPU run (other rows per expert),
    # the per-row accumulation order does not: equality is expected, a bf16 ulp is tolerated
    diff = (y.float() - ref[mine].float()).abs().max().item()
    scale = ref.float().abs().max().item()
    ok["moe"] = diff <= 1e-2 * scale
    ok["moe_max_diff"] = diff
    out.put((rank, ok))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_nccl_sharded_linear_and_expert_parallel():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    [p.start() for p in procs]
    res = [q.get(timeout=300) for _ in procs]
    [p.join(timeout=60) for p in procs]
    for _, ok in res:
        assert all(v for k, v in ok.items() if k != "moe_max_diff"), res
