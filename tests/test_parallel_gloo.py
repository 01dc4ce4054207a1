"""World-size-2 gloo tests of the multi-GPU host logic (N-sharded linears + all-gather,
expert-parallel dispatch/combine) with the CPU oracle standing in for the CUDA operators."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lisa_b200 import parallel
from oracle import oracle as O
from tests import util


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _bits(t):  # bf16 tensor -> uint16 numpy
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def _bf16(a):  # uint16 numpy -> bf16 tensor
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


def _oracle_matmul(x, w, s, b, transpose, gs, bits):
    y = O.affine_matmul(_bits(x), w.numpy().view(np.uint32), _bits(s), _bits(b), gs, bits, threads=1)
    return _bf16(y)


def _worker_linear(rank, world, port, n, k, m, bits, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(0)  # same tensors on every rank
    w, s, b = util.affine_weights(rng, n, k, bits, 64)
    x = util.activations(rng, m, k)
    tw = torch.from_numpy(w.view(np.int32))
    lin = parallel.ShardedQuantizedLinear.from_full(tw, _bf16(s), _bf16(b), world, rank, 64, bits)
    y = lin.forward(_bf16(x), matmul=_oracle_matmul)
    full = O.affine_matmul(x, w, s, b, 64, bits, threads=1)
    ok = np.array_equal(_bits(y), full) and lin.n1 - lin.n0 > 0
    out.put((rank, bool(ok)))
    dist.destroy_process_group()


@pytest.mark.parametrize("n,m,bits", [(64, 1, 4), (72, 3, 2)])  # 72 rows: uneven 8-row blocks over 2 ranks
def test_n_sharded_linear_all_gather(n, m, bits):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker_linear, args=(r, world, port, n, 256, m, bits, q)) for r in range(world)]
    [p.start() for p in procs]
    res = [q.get(timeout=120) for _ in procs]
    [p.join(timeout=60) for p in procs]
    assert all(ok for _, ok in res), res


def _worker_gguf(rank, world, port, fmt, rows, k, tokens, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(2)
    w = util.gguf_weights(rng, fmt, rows, k)
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    lin = parallel.ShardedGgufLinear.from_full(fmt, torch.from_numpy(w), world, rank)

    def matvec(f, weights, xx):
        return torch.from_numpy(O.gguf_matvec(f, weights.numpy(), xx.numpy(), threads=1))

    y = lin.forward(torch.from_numpy(x), matvec=matvec)
    full = O.gguf_matvec(fmt, w, x, threads=1)
    out.put((rank, bool(np.array_equal(y.numpy(), full)) and (lin.r1 - lin.r0) % 8 == 0))
    dist.destroy_process_group()


@pytest.mark.parametrize("fmt,rows,tokens", [(O.Q4_K, 64, 1), (O.Q2_K, 72, 3)])  # 72 rows: uneven 8-row blocks
def test_n_sharded_gguf_matvec_all_gather_f32(fmt, rows, tokens):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker_gguf, args=(r, world, port, fmt, rows, 512, tokens, q)) for r in range(world)]
    [p.start() for p in procs]
    res = [q.get(timeout=120) for _ in procs]
    [p.join(timeout=60) for p in procs]
    assert all(ok for _, ok in res), res


def _worker_moe(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(1)
    experts, hidden, inter, top_k, tokens = 8, 128, 64, 2, 6
    gate = util.affine_weights(rng, inter, hidden, 4, 64, experts=experts)
    up = util.affine_weights(rng, inter, hidden, 4, 64, experts=experts)
    down = util.affine_weights(rng, hidden, inter, 4, 64, experts=experts)
    x = util.activations(rng, tokens, hidden)
    logits = rng.normal(size=(tokens, experts)).astype(np.float32)
    ref, aux = O.moe_forward(x, logits, gate, up, down, top_k, 64, 4)
    e0, e1 = parallel.expert_range(experts, world, rank)
    mine = slice(rank * tokens // world, (rank + 1) * tokens // world)  # tokens are data-parallel

    def local_experts(rows, local_ids):
        ids = local_ids.numpy().astype(np.int32)
        assert ids.min() >= 0 and ids.max() < e1 - e0  # only slots of owned experts arrive
        order = np.argsort(ids, kind="stable")
        xs = _bits(rows)[order]
        sl = [t[e0:e1] for t in gate], [t[e0:e1] for t in up], [t[e0:e1] for t in down]
        g = O.gather_qmm(xs, *sl[0], ids[order], 64, 4)
        u = O.gather_qmm(xs, *sl[1], ids[order], 64, 4)
        d = O.gather_qmm(O.swiglu_bf16(g, u), *sl[2], ids[order], 64, 4)
        res = np.empty_like(d)
        res[order] = d
        return _bf16(res)

    def combine(rows_sorted, weights, inverse, k):
        return _bf16(O.moe_combine(_bits(rows_sorted), weights.numpy(), inverse.numpy(), k))

    y = parallel.ep_moe_forward(_bf16(x[mine]), torch.from_numpy(aux["idx"][mine]), torch.from_numpy(aux["weights"][mine]),
                                experts, local_experts, combine=combine)
    out.put((rank, bool(np.array_equal(_bits(y), ref[mine]))))
    dist.destroy_process_group()


def test_expert_parallel_dispatch_and_combine():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker_moe, args=(r, world, port, q)) for r in range(world)]
    [p.start() for p in procs]
    res = [q.get(timeout=120) for _ in procs]
    [p.join(timeout=60) for p in procs]
    assert all(ok for _, ok in res), res


def test_shard_rows_and_expert_range_cover_everything():
    for n, w in [(17408, 8), (5120, 8), (5120, 3), (18432, 7), (64, 8)]:
        r = [parallel.shard_rows(n, w, k) for k in range(w)]
        assert r[0][0] == 0 and r[-1][1] == n
        assert all(r[i][1] == r[i + 1][0] for i in range(w - 1)) and all((b - a) % 8 == 0 for a, b in r)
    assert [parallel.expert_range(128, 8, r) for r in (0, 7)] == [(0, 16), (112, 128)]
    with pytest.raises(ValueError):
        parallel.expert_range(10, 4, 0)
