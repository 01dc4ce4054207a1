"""One-node multi-GPU forms of the path: N-sharded linears with an all-gather of the outputs, and
expert-parallel routed experts with all-to-all dispatch and combine.

The reference has no multi-device code (one Apple GPU); the only hook it offers is DS4's
contiguous expert-ownership rule ``first = rank * (E / world)``
(crates/lisa-mlx/src/shaders/deepseek41/iq.metal:976-982), which the expert-parallel split below
follows.  One process per GPU; ``torch.distributed`` (NCCL over NVLink on GPUs, gloo in the CPU
tests) is the plumbing.  The compute callables default to the CUDA operators of ``lisa_b200.ops``;
tests inject CPU stand-ins to exercise the sharding logic without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_rows(n: int, world: int, rank: int, multiple: int = 8) -> Tuple[int, int]:
    """Contiguous output-row range of `rank`: ranges are multiples of `multiple` rows (the GGUF
    kernels need rows % 8 == 0), the remainder goes to the last ranks one block at a time."""
    if n % multiple != 0:
        raise ValueError(f"N={n} is not a multiple of {multiple}")
    blocks = n // multiple
    base, extra = divmod(blocks, world)
    begin = rank * base + max(0, rank - (world - extra)) if extra else rank * base
    count = base + (1 if extra and rank >= world - extra else 0)
    return begin * multiple, (begin + count) * multiple


@dataclass
class ShardedQuantizedLinear:
    """Rank-local slice ``W[n0:n1, :]`` of a quantized linear (weights, scales, biases keep the
    reference layout); every rank holds the full activation and computes ``y[:, n0:n1]``."""
    weight: torch.Tensor
    scales: torch.Tensor
    biases: torch.Tensor
    n_total: int
    n0: int
    n1: int
    group_size: int = 64
    bits: int = 4

    @classmethod
    def from_full(cls, weight, scales, biases, world: int, rank: int, group_size: int = 64, bits: int = 4):
        n = weight.shape[0]
        n0, n1 = shard_rows(n, world, rank)
        return cls(weight[n0:n1].contiguous(), scales[n0:n1].contiguous(), biases[n0:n1].contiguous(), n, n0, n1,
                   group_size, bits)

    def forward(self, x: torch.Tensor, matmul: Optional[Callable] = None, group=None) -> torch.Tensor:
        """x [M, K] (same on every rank) -> y [M, N] on every rank: local slice, then all-gather."""
        if matmul is None:
            from . import ops
            matmul = ops.quantized_matmul
        local = matmul(x, self.weight, self.scales, self.biases, True, self.group_size, self.bits)
        return all_gather_columns(local, self.n_total, group=group)


def all_gather_columns(local: torch.Tensor, n_total: int, group=None) -> torch.Tensor:
    """Gathers column blocks [M, n_r] of all ranks into [M, N].  For M == 1 the gathered buffer is
    already the output; for M > 1 the [world, M, n_r] gather is laid out rank-major and permuted."""
    world = dist.get_world_size(group)
    m = local.shape[0]
    sizes = [shard_rows(n_total, world, r) for r in range(world)]
    widths = [b - a for a, b in sizes]
    if len(set(widths)) == 1:
        out = torch.empty((world * m, widths[0]), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out.view(world, m, widths[0]).permute(1, 0, 2).reshape(m, n_total)
    # uneven shards: pad every slice to the widest one, gather, drop the padding
    wmax = max(widths)
    padded = torch.zeros((m, wmax), dtype=local.dtype, device=local.device)
    padded[:, : local.shape[1]] = local
    out = torch.empty((world * m, wmax), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, padded, group=group)
    out = out.view(world, m, wmax)
    return torch.cat([out[r, :, : widths[r]] for r in range(world)], dim=1)


@dataclass
class ShardedGgufLinear:
    """Rank-local rows ``W[r0:r1]`` of a GGUF K-quant matrix (uint8 ``[rows, row_bytes]`` blocks, the layout of
    ``deepseek41::packed_matvec``); every rank holds the full f32 activation and computes ``y[:, r0:r1]``, the
    f32 column blocks are all-gathered.  Rows are independent, so the split is the dense linear's; ranges stay
    multiples of 8 rows (the kernels' limit, crates/lisa-mlx/src/models/deepseek41.rs:50-65)."""
    fmt: object
    weights: torch.Tensor
    rows_total: int
    r0: int
    r1: int

    @classmethod
    def from_full(cls, fmt, weights: torch.Tensor, world: int, rank: int):
        rows = weights.shape[0]
        r0, r1 = shard_rows(rows, world, rank)
        return cls(fmt, weights[r0:r1].contiguous(), rows, r0, r1)

    def forward(self, x: torch.Tensor, matvec: Optional[Callable] = None, group=None) -> torch.Tensor:
        """x f32 [tokens, K] (same on every rank) -> y f32 [tokens, rows_total] on every rank."""
        if matvec is None:
            from . import ops
            matvec = ops.packed_matvec
        local = matvec(self.fmt, self.weights, x)
        return all_gather_columns(local, self.rows_total, group=group)


def expert_range(experts: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous expert ownership, iq.metal:976-982: first = rank * (E / world)."""
    if experts % world != 0:
        raise ValueError(f"{experts} experts do not split over {world} ranks")
    per = experts // world
    return rank * per, (rank + 1) * per


def ep_dispatch_plan(idx: torch.Tensor, experts: int, world: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """For the local tokens' routing `idx` [T, top_k]: the destination rank of every slot, a stable
    order that groups slots by destination rank, and the number of slots per destination."""
    per = experts // world
    flat = idx.reshape(-1).to(torch.int64)
    dest = torch.div(flat, per, rounding_mode="floor")
    order = torch.sort(dest, stable=True).indices
    counts = torch.bincount(dest, minlength=world)
    return dest, order, counts


def ep_moe_forward(x: torch.Tensor, idx: torch.Tensor, weights: torch.Tensor, experts: int,
                   local_experts: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
                   combine: Optional[Callable] = None, group=None) -> torch.Tensor:
    """Expert-parallel routed experts for the tokens this rank owns.

    x [T, H] bf16 (rank-local tokens), idx int32 [T, top_k], weights f32 [T, top_k] from the
    replicated router.  `local_experts(rows [R, H], local_ids [R]) -> [R, H]` runs the rank's own
    experts (gate/up gather_qmm, SwiGLU, down gather_qmm) on rows sorted however it likes and
    returns them in the order given.  Exchange: slot counts (all-to-all of one int per peer), rows
    and expert ids to the owners (all-to-all), results back (all-to-all), then the weighted fold in
    original slot order on the token's rank (`combine(rows_sorted, weights, inverse, top_k)`,
    default the CUDA ``ops.moe_combine``)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    t, top_k = idx.shape
    hidden = x.shape[1]
    dest, order, send_counts = ep_dispatch_plan(idx, experts, world)
    token_of_slot = torch.div(order, top_k, rounding_mode="floor")
    send_rows = x[token_of_slot].contiguous()
    send_ids = idx.reshape(-1)[order].to(torch.int32).contiguous()
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    s_list, r_list = send_counts.tolist(), recv_counts.tolist()
    recv_rows = torch.empty((sum(r_list), hidden), dtype=x.dtype, device=x.device)
    recv_ids = torch.empty((sum(r_list),), dtype=torch.int32, device=x.device)
    dist.all_to_all_single(recv_rows, send_rows, r_list, s_list, group=group)
    dist.all_to_all_single(recv_ids, send_ids, r_list, s_list, group=group)
    e0, _ = expert_range(experts, world, rank)
    out_rows = local_experts(recv_rows, recv_ids - e0) if recv_rows.shape[0] else recv_rows
    back = torch.empty_like(send_rows)
    dist.all_to_all_single(back, out_rows.contiguous(), s_list, r_list, group=group)
    # `back` is in dispatch order; inverse[slot] = its row there.  Fold in original slot order.
    inverse = torch.empty_like(order)
    inverse[order] = torch.arange(order.numel(), device=order.device)
    if combine is None:
        from . import ops
        combine = ops.moe_combine
    return combine(back, weights.reshape(t, top_k), inverse.to(torch.int32), top_k)


# ---------------------------------------------------------------- fused GEMV + all-gather over peer memory
def _enable_peer_access(me: int, peer: int) -> None:
    """Makes memory of GPU `peer` addressable from kernels on GPU `me` (both directions are needed by the
    two ranks involved; each rank enables its own).  Raises when the pair has no peer path."""
    from cuda.bindings import runtime as rt

    (err, can) = rt.cudaDeviceCanAccessPeer(me, peer)
    if int(err) != 0 or not can:
        raise RuntimeError(f"GPU {me} cannot access GPU {peer} as a peer")
    torch.cuda.set_device(me)
    (err,) = rt.cudaDeviceEnablePeerAccess(peer, 0)
    if int(err) not in (0, int(rt.cudaError_t.cudaErrorPeerAccessAlreadyEnabled)):
        raise RuntimeError(f"cudaDeviceEnablePeerAccess({peer}) failed: {err}")
    rt.cudaGetLastError()  # clear the sticky "already enabled"


class _DevicePtr:
    """Wraps a raw device allocation for ``torch.as_tensor`` (CUDA array interface, zero copy)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"data": (ptr, False), "shape": tuple(shape), "typestr": typestr, "version": 3,
                                         "strides": None}


_TYPESTR = {torch.bfloat16: "<u2", torch.int64: "<i8", torch.float32: "<f4", torch.int32: "<i4"}  # bf16 as its bit pattern


class PeerBuffers:
    """A same-shaped device buffer on every rank of one node, with every rank holding pointers to all of
    them: its own ``cudaMalloc`` block and CUDA IPC mappings of the others', opened with this rank's GPU
    current and peer access enabled.  `ptrs()` is the pointer table
    `lisa_cuda_quantized_matmul_allgather` / `lisa_cuda_peer_barrier` take; `local` is a tensor view of
    this rank's block.  Every mapping is read once through ``cudaMemcpy`` before it is handed to a
    kernel, so that a pair without a working peer path fails here with an error code."""

    def __init__(self, shape, dtype, group=None):
        import ctypes as C

        from cuda.bindings import runtime as rt

        def ok(res, what):
            err = res[0]
            if int(err) != 0:
                raise RuntimeError(f"{what} failed: {err}")
            return res[1] if len(res) > 1 else None

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.cuda.current_device()
        torch.cuda.set_device(self.device)
        elem = torch.empty((), dtype=dtype).element_size()
        count = 1
        for d in shape:
            count *= int(d)
        self.nbytes = max(count * elem, 256)
        self._rt = rt
        self._ptr = int(ok(rt.cudaMalloc(self.nbytes), "cudaMalloc"))
        ok(rt.cudaMemset(self._ptr, 0, self.nbytes), "cudaMemset")
        ok(rt.cudaDeviceSynchronize(), "cudaDeviceSynchronize")
        handle = ok(rt.cudaIpcGetMemHandle(self._ptr), "cudaIpcGetMemHandle")
        gathered = [None] * self.world
        dist.all_gather_object(gathered, (bytes(handle.reserved), self.device), group=group)
        self._peer_ptrs = []
        scratch = ok(rt.cudaMalloc(256), "cudaMalloc")
        for r, (raw, dev_r) in enumerate(gathered):
            if r == self.rank:
                self._peer_ptrs.append(self._ptr)
                continue
            if dev_r != self.device:
                _enable_peer_access(self.device, dev_r)
            h = rt.cudaIpcMemHandle_t()
            h.reserved = raw
            ptr = int(ok(rt.cudaIpcOpenMemHandle(h, rt.cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle"))
            ok(rt.cudaMemcpy(scratch, ptr, min(self.nbytes, 256), rt.cudaMemcpyKind.cudaMemcpyDefault), "read of the peer mapping")
            self._peer_ptrs.append(ptr)
        ok(rt.cudaFree(scratch), "cudaFree")
        self.local = torch.as_tensor(_DevicePtr(self._ptr, shape, _TYPESTR[dtype]), device=torch.device("cuda", self.device))
        if dtype == torch.bfloat16:
            self.local = self.local.view(torch.bfloat16)
        self._table = (C.c_void_p * self.world)(*self._peer_ptrs)
        # the same pointers starting with the next rank and ending with this one: a kernel that stores into all
        # of them in table order then begins at a different peer on every rank instead of all at rank 0
        order = [(self.rank + 1 + i) % self.world for i in range(self.world)]
        self._table_rotated = (C.c_void_p * self.world)(*[self._peer_ptrs[r] for r in order])
        dist.barrier(group=group)

    def ptrs(self):
        return self._table

    def ptrs_rotated(self):
        """All ranks' pointers in the order rank+1, ..., rank (for stores whose order does not matter)."""
        return self._table_rotated

    def close(self):
        """Unmaps the peers' blocks and frees this rank's (after a barrier: nobody may still write to it)."""
        if self._ptr is None:
            return
        dist.barrier(group=self.group)
        for r, ptr in enumerate(self._peer_ptrs):
            if r != self.rank:
                self._rt.cudaIpcCloseMemHandle(ptr)
        dist.barrier(group=self.group)
        self.local = None
        self._rt.cudaFree(self._ptr)
        self._ptr = None


class FusedShardedLinear:
    """`ShardedQuantizedLinear` without a collective library: the epilogue of the GEMV (up to 8 rows) or of the
    tensor-core GEMM (more rows) stores this rank's column block into every rank's output buffer, and
    `lisa_cuda_peer_barrier` orders the ranks.

    Reuse rule.  The barrier of a call orders that call's stores (all ranks) before the reads that follow it on
    every rank; nothing orders one rank's reads of call i before another rank's stores of call i+1.  An instance
    therefore owns TWO output buffers and alternates between them: the stores of call i+2 into the buffer of
    call i come after the barrier of call i+1, which a rank only passes once every rank has enqueued -- behind
    its own consumer of call i, in stream order -- that barrier.  The returned view stays valid until the
    second-next `forward` of the same instance, provided its consumer runs on the same stream before the next
    `forward`.  A CUDA graph that captures `forward` fixes the buffer of every captured call: capture an even
    number of calls per instance, or a sequence in which other barriers separate two replays (a whole decoder
    stack does)."""

    def __init__(self, shard: ShardedQuantizedLinear, max_rows: int = 8, group=None):
        self.shard = shard
        self.outs = [PeerBuffers((max_rows, shard.n_total), torch.bfloat16, group) for _ in range(2)]
        self.flags = PeerBuffers((16,), torch.int64, group)
        self._turn = 0

    @property
    def out(self):
        return self.outs[0]

    def close(self):
        for o in self.outs:
            o.close()
        self.flags.close()

    def forward(self, x: torch.Tensor, stream=None) -> torch.Tensor:
        from . import _cabi

        sh = self.shard
        m, k = x.shape
        st = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        lib = _cabi.lib()
        out = self.outs[self._turn]
        self._turn ^= 1
        _cabi.check(lib.lisa_cuda_quantized_matmul_allgather(
            st, x.data_ptr(), m, k, sh.weight.data_ptr(), sh.scales.data_ptr(), sh.biases.data_ptr(), sh.n1 - sh.n0, 1,
            sh.group_size, sh.bits, _cabi.BF16, out.ptrs_rotated(), out.world, sh.n_total, sh.n0, _cabi.FLAG_PDL))
        # epoch 0: the barrier counts itself on the device, so the pair of launches replays from a CUDA graph
        _cabi.check(lib.lisa_cuda_peer_barrier(st, out.rank, out.world, self.flags.ptrs(), 0))
        return out.local[:m]


class FusedShardedGguf:
    """`ShardedGgufLinear` without a collective library, for the token counts the tensor-memory matvec takes (Q4_K:
    one or two, Q2_K: one): the kernel's epilogue stores this rank's f32 column block into every rank's output,
    `lisa_cuda_peer_barrier` orders the ranks.  Two output buffers taken in turn (the reuse rule of
    `FusedShardedLinear`).  `supported(tokens)` says whether the fused launch applies; otherwise use
    ``shard.forward`` (local matvec + collective all-gather)."""

    def __init__(self, shard: ShardedGgufLinear, max_tokens: int = 2, group=None):
        self.shard = shard
        self.outs = [PeerBuffers((max_tokens, shard.rows_total), torch.float32, group) for _ in range(2)]
        self.flags = PeerBuffers((16,), torch.int64, group)
        self._turn = 0
        self.max_tokens = max_tokens

    def close(self):
        for o in self.outs:
            o.close()
        self.flags.close()

    def forward(self, x: torch.Tensor, stream=None) -> torch.Tensor:
        from . import _cabi, ops

        sh = self.shard
        tokens = x.shape[0]
        st = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        out = self.outs[self._turn]
        self._turn ^= 1
        lib = _cabi.lib()
        code = ops._format_code(sh.fmt)
        _cabi.check(lib.lisa_cuda_gguf_packed_matvec_allgather(
            st, code, sh.weights.data_ptr(), sh.r1 - sh.r0, sh.weights.shape[1], x.data_ptr(), tokens, out.ptrs_rotated(),
            out.world, sh.rows_total, sh.r0))
        _cabi.check(lib.lisa_cuda_peer_barrier(st, out.rank, out.world, self.flags.ptrs(), 0))
        return out.local[:tokens]


class FusedShardedSiblings:
    """Several `ShardedQuantizedLinear`s that read the same x (gate|up, q|k|v): one launch whose epilogue stores
    every linear's column block into every rank's buffers, then ONE peer barrier.  Two sets of output buffers
    taken in turn, as in `FusedShardedLinear` (same reuse rule)."""

    def __init__(self, shards, max_rows: int = 8, group=None):
        import ctypes as C

        self.shards = list(shards)
        self.out_sets = [[PeerBuffers((max_rows, sh.n_total), torch.bfloat16, group) for sh in self.shards] for _ in range(2)]
        self.flags = PeerBuffers((16,), torch.int64, group)
        c, world = len(self.shards), self.out_sets[0][0].world
        self.world, self.rank = world, self.out_sets[0][0].rank
        self._w, self._s, self._b = (C.c_void_p * c)(), (C.c_void_p * c)(), (C.c_void_p * c)()
        self._n, self._nt, self._c0 = (C.c_int64 * c)(), (C.c_int64 * c)(), (C.c_int64 * c)()
        self._ys = [(C.c_void_p * (c * world))() for _ in range(2)]
        for i, sh in enumerate(self.shards):
            self._w[i], self._s[i], self._b[i] = sh.weight.data_ptr(), sh.scales.data_ptr(), sh.biases.data_ptr()
            self._n[i], self._nt[i], self._c0[i] = sh.n1 - sh.n0, sh.n_total, sh.n0
            for turn in range(2):
                ptrs = self.out_sets[turn][i].ptrs_rotated()
                for r in range(world):
                    self._ys[turn][i * world + r] = ptrs[r]
        self._turn = 0

    @property
    def outs(self):
        return self.out_sets[0]

    def close(self):
        for outs in self.out_sets:
            for o in outs:
                o.close()
        self.flags.close()

    def forward(self, x: torch.Tensor, stream=None):
        from . import _cabi

        sh = self.shards[0]
        m, k = x.shape
        st = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        lib = _cabi.lib()
        turn = self._turn
        self._turn ^= 1
        _cabi.check(lib.lisa_cuda_quantized_matmul_siblings_allgather(
            st, x.data_ptr(), m, k, len(self.shards), self._w, self._s, self._b, self._n, 1, sh.group_size, sh.bits, _cabi.BF16,
            self._ys[turn], self.world, self._nt, self._c0, _cabi.FLAG_PDL))
        _cabi.check(lib.lisa_cuda_peer_barrier(st, self.rank, self.world, self.flags.ptrs(), 0))
        return [o.local[:m] for o in self.out_sets[turn]]


class ExpertParallelMoe:
    """Routed experts, expert-parallel over the ranks of one node, with the exchange done by the library's own
    kernels over peer memory (`lisa_cuda_ep_counts / ep_dispatch / ep_return` + `lisa_cuda_peer_barrier`): no
    collective library on the data path.  Tokens are data-parallel; rank r owns experts
    ``[r * E / world, (r + 1) * E / world)`` (iq.metal:976-982).  `block` holds this rank's experts
    (`SwitchGlu` with E / world experts).  The only thing the host reads per call is the world x world count
    matrix, which sizes the owner's launches; when the receive capacity is small (`world * max_slots` up to
    DEVICE_COUNT_ROWS rows) not even that: the owner runs over its whole capacity, rows nobody sent carry an id
    outside its table, and the step has no host synchronisation (it can be captured in a CUDA graph)."""

    DEVICE_COUNT_ROWS = 16384

    def __init__(self, block, experts: int, max_tokens: int, hidden: int, group=None):
        self.block = block
        self.experts, self.top_k, self.hidden = experts, block.top_k, hidden
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.max_slots = max_tokens * block.top_k
        cap = self.world * self.max_slots           # every slot of every rank could land here
        self.matrix = PeerBuffers((self.world * self.world,), torch.int32, group)
        self.recv_x = PeerBuffers((cap, hidden), torch.bfloat16, group)
        self.recv_ids = PeerBuffers((cap,), torch.int32, group)
        self.back = PeerBuffers((self.max_slots, hidden), torch.bfloat16, group)
        self.flags = PeerBuffers((16,), torch.int64, group)
        self._host_matrix = torch.empty((self.world, self.world), dtype=torch.int32).pin_memory()

    def close(self):
        for b in (self.matrix, self.recv_x, self.recv_ids, self.back, self.flags):
            b.close()

    def _barrier(self, st):
        from . import _cabi
        _cabi.check(_cabi.lib().lisa_cuda_peer_barrier(st, self.rank, self.world, self.flags.ptrs(), 0))

    def forward(self, x: torch.Tensor, router_logits: torch.Tensor) -> torch.Tensor:
        """x bf16 [tokens, hidden] and router_logits f32 [tokens, E] of this rank's tokens -> [tokens, hidden]."""
        from . import _cabi, ops

        lib = _cabi.lib()
        st = torch.cuda.current_stream().cuda_stream
        blk, k = self.block, self.top_k
        tokens = x.shape[0]
        slots = tokens * k
        if slots > self.max_slots:
            raise _cabi.LisaError(_cabi.ERR_LIMIT, "ExpertParallelMoe: more tokens than the buffers were sized for")
        gs, bits = blk.gate.group_size, blk.gate.bits
        local_e = self.experts // self.world
        cap = self.world * self.max_slots
        on_device = cap <= self.DEVICE_COUNT_ROWS
        if on_device:
            self.recv_ids.local.fill_(local_e)       # rows nobody sends this step: an id outside the table
        idx, weights = ops.moe_route(router_logits, k)
        sorted_ids, token_rows, inverse = ops.moe_sort(idx, self.experts, k)   # by global expert: grouped by owner
        _cabi.check(lib.lisa_cuda_ep_counts(st, sorted_ids.data_ptr(), slots, self.experts, self.world, self.rank,
                                            self.matrix.ptrs()))
        self._barrier(st)
        if on_device:
            received = cap
        else:
            self._host_matrix.copy_(self.matrix.local.view(self.world, self.world), non_blocking=True)
            torch.cuda.current_stream().synchronize()      # the one host read: how many rows this rank receives
            received = int(self._host_matrix[:, self.rank].sum())
        _cabi.check(lib.lisa_cuda_ep_dispatch(st, x.data_ptr(), sorted_ids.data_ptr(), token_rows.data_ptr(), slots, self.hidden,
                                              self.experts, self.world, self.rank, self.matrix.local.data_ptr(),
                                              self.recv_x.ptrs(), self.recv_ids.ptrs(), _cabi.BF16))
        self._barrier(st)
        if received:
            ids = self.recv_ids.local[:received]
            s2, rows2, _ = ops.moe_sort(ids, local_e, 1)                     # top_k = 1: rows2 indexes recv_x
            xs = ops.gather_rows(self.recv_x.local[:received], rows2)
            g, u = ops.gather_qmm_siblings(xs, [(blk.gate.weight, blk.gate.scales, blk.gate.biases),
                                                (blk.up.weight, blk.up.scales, blk.up.biases)], s2, gs, bits)
            d = ops.gather_qmm(ops.swiglu(g, u), blk.down.weight, blk.down.scales, blk.down.biases, None, s2, True, gs, bits, True)
            _cabi.check(lib.lisa_cuda_ep_return(st, d.data_ptr(), rows2.data_ptr(), received, self.hidden, self.world, self.rank,
                                                self.matrix.local.data_ptr(), self.back.ptrs(), _cabi.BF16))
        self._barrier(st)
        return ops.moe_combine(self.back.local[:slots], weights, inverse, k)
