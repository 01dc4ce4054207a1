"""Host-side mirror of the reference's operator API for the quantized-weight matmul path.

Same names, argument meaning and error behaviour as ``lisa_mlx::ops`` and
``lisa_mlx::models::deepseek41`` (crates/lisa-mlx/src/ops/array_ops.rs:37-84,378-642;
crates/lisa-mlx/src/models/deepseek41.rs:93-283), over the C ABI of ``liblisa_cuda.so``.
torch is used only for device memory and streams: every call hands raw device pointers to
the library, which does all the work in hand-written sm_100a kernels.  The callee allocates
the output (as the reference does from its buffer pool) unless ``out=`` is given.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _cabi
from ._cabi import LisaError, check, lib

BlockFormat = {"Q2K": _cabi.GGUF_Q2_K, "Q4K": _cabi.GGUF_Q4_K, "Q5K": _cabi.GGUF_Q5_K}
_BLOCK_BYTES = {_cabi.GGUF_Q2_K: 84, _cabi.GGUF_Q4_K: 144, _cabi.GGUF_Q5_K: 176}


def _stream(stream=None) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _cabi.BF16
    if t.dtype == torch.float16:
        return _cabi.F16
    if t.dtype == torch.float32:
        return _cabi.F32
    raise LisaError(_cabi.ERR_UNSUPPORTED, f"unsupported compute dtype {t.dtype}")


def _need_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise LisaError(_cabi.ERR_BAD_ARG, "tensor is not on a CUDA device (no CPU fallback)")


def _words(w: torch.Tensor) -> torch.Tensor:
    if w.dtype not in (torch.uint32, torch.int32):
        raise LisaError(_cabi.ERR_BAD_ARG, f"packed weights must be uint32 words, got {w.dtype}")
    return w.contiguous()


def quantized_matmul(x: torch.Tensor, w: torch.Tensor, scales: torch.Tensor,
                     biases: Optional[torch.Tensor], transpose: bool = True, group_size: int = 64,
                     bits: int = 4, *, stream=None, out: Optional[torch.Tensor] = None,
                     flags: int = 0) -> torch.Tensor:
    """``ops::quantized_matmul`` (array_ops.rs:378-493): y = x . dequant(w)^T over the last
    axis of x; x is flattened to [M, K]; output shape x.shape[:-1] + [N]."""
    _need_cuda(x, w, scales, biases)
    k = x.shape[-1]
    m = x.numel() // k
    n = w.shape[0]
    x2 = x.reshape(m, k).contiguous()
    w = _words(w)
    sc = scales.contiguous()
    bi = biases.contiguous() if biases is not None else None
    if w.shape[-1] * 32 // bits != k or sc.shape[-1] * group_size != k:
        raise LisaError(_cabi.ERR_BAD_ARG, "quantized_matmul: shapes of x, w and scales disagree")
    y = out if out is not None else torch.empty((m, n), dtype=x2.dtype, device=x2.device)
    rc = lib().lisa_cuda_quantized_matmul_ex(
        _stream(stream), x2.data_ptr(), m, k, w.data_ptr(), sc.data_ptr(),
        bi.data_ptr() if bi is not None else None, n, int(bool(transpose)), group_size, bits,
        _dtype_code(x2), y.data_ptr(), flags)
    check(rc)
    return y.reshape(*x.shape[:-1], n)


def quantized_matmul_siblings(x: torch.Tensor, linears, transpose: bool = True, group_size: int = 64,
                               bits: int = 4, *, stream=None, flags: int = 0):
    """One to three quantized linears applied to the same x (q|k|v, gate|up); `linears` is a sequence of
    (w, scales, biases).  Returns the list of outputs, each x.shape[:-1] + [N_i]: what as many
    ``quantized_matmul`` calls return, from one launch when the rows are few."""
    import ctypes as C

    k = x.shape[-1]
    m = x.numel() // k
    x2 = x.reshape(m, k).contiguous()
    count = len(linears)
    keep, ys = [], []
    wp, sp, bp, yp = (C.c_void_p * count)(), (C.c_void_p * count)(), (C.c_void_p * count)(), (C.c_void_p * count)()
    ns = (C.c_int64 * count)()
    for i, (w, sc, bi) in enumerate(linears):
        _need_cuda(x, w, sc, bi)
        w = _words(w)
        sc, bi = sc.contiguous(), bi.contiguous()
        if w.shape[-1] * 32 // bits != k or sc.shape[-1] * group_size != k:
            raise LisaError(_cabi.ERR_BAD_ARG, "quantized_matmul_siblings: shapes of x, w and scales disagree")
        y = torch.empty((m, w.shape[0]), dtype=x2.dtype, device=x2.device)
        keep.append((w, sc, bi))
        ys.append(y)
        wp[i], sp[i], bp[i], yp[i], ns[i] = w.data_ptr(), sc.data_ptr(), bi.data_ptr(), y.data_ptr(), w.shape[0]
    rc = lib().lisa_cuda_quantized_matmul_siblings(_stream(stream), x2.data_ptr(), m, k, count, wp, sp, bp, ns,
                                                   int(bool(transpose)), group_size, bits, _dtype_code(x2), yp, flags)
    check(rc)
    return [y.reshape(*x.shape[:-1], y.shape[-1]) for y in ys]


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor, eps: float, *, stream=None):
    """(sum, normed): sum = bf16(x + residual), normed = rms_norm(sum) * norm_weight with the reference's
    rounding points (crates/lisa-mlx/src/jit/matmul.rs:304-316)."""
    _need_cuda(x, residual, norm_weight)
    k = x.shape[-1]
    m = x.numel() // k
    x2, r2 = x.reshape(m, k).contiguous(), residual.reshape(m, k).contiguous()
    total, normed = torch.empty_like(x2), torch.empty_like(x2)
    check(lib().lisa_cuda_add_rmsnorm(_stream(stream), x2.data_ptr(), r2.data_ptr(), norm_weight.contiguous().data_ptr(),
                                      float(eps), m, k, _dtype_code(x2), total.data_ptr(), normed.data_ptr()))
    return total.reshape(x.shape), normed.reshape(x.shape)


def quantized_matmul_addnorm(x: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor, eps: float, linears,
                             group_size: int = 64, bits: int = 4, *, write_norm: bool = True, stream=None, flags: int = 0):
    """Residual add + RMSNorm + one to three quantized linears on the normed rows (affine_qmv_fast_addnorm,
    crates/lisa-mlx/src/jit/matmul.rs:304-470): returns (outputs, sum, normed or None).  Decode rows run as one
    launch; other shapes need `write_norm` (the normed rows are then the matmul's input buffer)."""
    import ctypes as C

    _need_cuda(x, residual, norm_weight)
    k = x.shape[-1]
    m = x.numel() // k
    x2, r2 = x.reshape(m, k).contiguous(), residual.reshape(m, k).contiguous()
    count = len(linears)
    keep, ys = [], []
    wp, sp, bp, yp = (C.c_void_p * count)(), (C.c_void_p * count)(), (C.c_void_p * count)(), (C.c_void_p * count)()
    ns = (C.c_int64 * count)()
    for i, (w, sc, bi) in enumerate(linears):
        _need_cuda(w, sc, bi)
        w = _words(w)
        sc, bi = sc.contiguous(), bi.contiguous()
        if w.shape[-1] * 32 // bits != k or sc.shape[-1] * group_size != k:
            raise LisaError(_cabi.ERR_BAD_ARG, "quantized_matmul_addnorm: shapes of x, w and scales disagree")
        y = torch.empty((m, w.shape[0]), dtype=x2.dtype, device=x2.device)
        keep.append((w, sc, bi))
        ys.append(y)
        wp[i], sp[i], bp[i], yp[i], ns[i] = w.data_ptr(), sc.data_ptr(), bi.data_ptr(), y.data_ptr(), w.shape[0]
    total = torch.empty_like(x2)
    normed = torch.empty_like(x2) if write_norm else None
    rc = lib().lisa_cuda_quantized_matmul_addnorm(_stream(stream), x2.data_ptr(), r2.data_ptr(), norm_weight.contiguous().data_ptr(),
                                                  float(eps), m, k, count, wp, sp, bp, ns, 1, group_size, bits, _dtype_code(x2), yp,
                                                  total.data_ptr(), None if normed is None else normed.data_ptr(), flags)
    check(rc)
    outs = [y.reshape(*x.shape[:-1], y.shape[-1]) for y in ys]
    return outs, total.reshape(x.shape), None if normed is None else normed.reshape(x.shape)


def quantized_matmul_swiglu(gate: torch.Tensor, up: torch.Tensor, w, scales, biases, group_size: int = 64, bits: int = 4, *,
                            write_act: bool = False, stream=None, flags: int = 0):
    """swiglu(gate, up) . dequant(w)^T: the down projection of an MLP reading the gate and up outputs.  Returns
    (y, act or None); decode rows run as one launch, other shapes need `write_act`."""
    _need_cuda(gate, up, w, scales, biases)
    k = gate.shape[-1]
    m = gate.numel() // k
    g2, u2 = gate.reshape(m, k).contiguous(), up.reshape(m, k).contiguous()
    w = _words(w)
    y = torch.empty((m, w.shape[0]), dtype=g2.dtype, device=g2.device)
    act = torch.empty_like(g2) if write_act else None
    check(lib().lisa_cuda_quantized_matmul_swiglu(_stream(stream), g2.data_ptr(), u2.data_ptr(), m, k, w.data_ptr(),
                                                  scales.contiguous().data_ptr(), biases.contiguous().data_ptr(), w.shape[0], 1,
                                                  group_size, bits, _dtype_code(g2), y.data_ptr(),
                                                  None if act is None else act.data_ptr(), flags))
    return y.reshape(*gate.shape[:-1], w.shape[0]), None if act is None else act.reshape(gate.shape)


def quantized_matmul_serial_rows(x, w, scales, biases, transpose: bool = True, group_size: int = 64,
                                 bits: int = 4, *, stream=None) -> torch.Tensor:
    """``ops::quantized_matmul_serial_rows`` (array_ops.rs:500-555)."""
    _need_cuda(x, w, scales, biases)
    k = x.shape[-1]
    rows = x.numel() // k
    n = w.shape[0]
    x2 = x.reshape(rows, k).contiguous()
    w = _words(w)
    y = torch.empty((rows, n), dtype=x2.dtype, device=x2.device)
    rc = lib().lisa_cuda_quantized_matmul_serial_rows(
        _stream(stream), x2.data_ptr(), rows, k, w.data_ptr(), scales.contiguous().data_ptr(),
        biases.contiguous().data_ptr() if biases is not None else None, n, int(bool(transpose)),
        group_size, bits, _dtype_code(x2), y.data_ptr())
    check(rc)
    return y.reshape(*x.shape[:-1], n)


def dequantize(w: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, group_size: int = 64,
               bits: int = 4, *, stream=None) -> torch.Tensor:
    """``ops::dequantize`` (array_ops.rs:37-84): output dtype = scales dtype, shape [..., K]."""
    _need_cuda(w, scales, biases)
    w = _words(w)
    kq = w.shape[-1]
    k = kq * 32 // bits
    rows = w.numel() // kq
    out = torch.empty(w.shape[:-1] + (k,), dtype=scales.dtype, device=w.device)
    rc = lib().lisa_cuda_dequantize(_stream(stream), w.data_ptr(), scales.contiguous().data_ptr(),
                                    biases.contiguous().data_ptr(), rows, k, group_size, bits,
                                    _dtype_code(scales), out.data_ptr())
    check(rc)
    return out


def dequantize_rows(w: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, ids: torch.Tensor, group_size: int = 64,
                    bits: int = 4, *, stream=None) -> torch.Tensor:
    """Rows ``ids`` of a quantized table, dequantized: what ``QuantizedEmbedding::forward`` computes with
    take_axis + ``ops::dequantize`` (crates/lisa-engine/src/core/quant.rs:449-455).  ids of any integer dtype,
    any shape; returns ids.shape + [K]; an id outside the table gives zeros."""
    _need_cuda(w, scales, biases, ids)
    w = _words(w)
    vocab, kq = w.shape[0], w.shape[-1]
    k = kq * 32 // bits
    flat = ids.reshape(-1).to(torch.int32).contiguous()
    out = torch.empty((flat.numel(), k), dtype=scales.dtype, device=w.device)
    check(lib().lisa_cuda_dequantize_rows(_stream(stream), w.data_ptr(), scales.contiguous().data_ptr(),
                                          biases.contiguous().data_ptr(), flat.data_ptr(), flat.numel(), vocab, k,
                                          group_size, bits, _dtype_code(scales), out.data_ptr()))
    return out.reshape(*ids.shape, k)


def quantize(w: torch.Tensor, group_size: Optional[int] = None, bits: Optional[int] = None, *, stream=None):
    """``ops::quantize`` (array_ops.rs:218-290): returns (wq uint32 [..., K*bits/32], scales, biases [..., K/group])
    in w's dtype; defaults group 64, 4 bits."""
    _need_cuda(w)
    gs = 64 if group_size is None else int(group_size)
    b = 4 if bits is None else int(bits)
    k = w.shape[-1]
    rows = w.numel() // k
    if b not in (2, 4, 8) or gs < 1 or k % gs != 0 or gs % (32 // b) != 0:
        raise LisaError(_cabi.ERR_BAD_ARG, f"quantize: group size {gs} incompatible with K={k}, bits={b}")
    w2 = w.reshape(rows, k).contiguous()
    wq = torch.empty((rows, k * b // 32), dtype=torch.int32, device=w.device)
    sc = torch.empty((rows, k // gs), dtype=w.dtype, device=w.device)
    bi = torch.empty_like(sc)
    check(lib().lisa_cuda_quantize(_stream(stream), w2.data_ptr(), rows, k, gs, b, _dtype_code(w2), wq.data_ptr(),
                                   sc.data_ptr(), bi.data_ptr()))
    lead = w.shape[:-1]
    return wq.reshape(*lead, k * b // 32), sc.reshape(*lead, k // gs), bi.reshape(*lead, k // gs)


def gather_qmm(x: torch.Tensor, w: torch.Tensor, scales: torch.Tensor, biases: Optional[torch.Tensor],
               lhs_indices: Optional[torch.Tensor], rhs_indices: Optional[torch.Tensor],
               transpose: bool = True, group_size: int = 64, bits: int = 4,
               sorted_indices: bool = True, *, stream=None,
               workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``ops::gather_qmm`` (array_ops.rs:561-642): x [rows, 1, K] or [rows, K]; w [E, N, K*bits/32];
    rhs_indices [rows] sorted; returns [rows, 1, N] / [rows, N]."""
    _need_cuda(x, w, scales, biases, rhs_indices)
    k = x.shape[-1]
    rows = x.numel() // k
    experts, n = w.shape[0], w.shape[-2]
    x2 = x.reshape(rows, k).contiguous()
    w = _words(w)
    y = torch.empty((rows, n), dtype=x2.dtype, device=x2.device)
    need = lib().lisa_cuda_gather_qmm_workspace_bytes(rows, experts)
    if workspace is None and need:
        workspace = torch.empty(need, dtype=torch.uint8, device=x2.device)
    ids = rhs_indices.to(torch.int32).contiguous() if rhs_indices is not None else None
    rc = lib().lisa_cuda_gather_qmm(
        _stream(stream), x2.data_ptr(), rows, k, w.data_ptr(), scales.contiguous().data_ptr(),
        biases.contiguous().data_ptr() if biases is not None else None,
        lhs_indices.data_ptr() if lhs_indices is not None else None,
        ids.data_ptr() if ids is not None else None, experts, n, int(bool(transpose)), group_size,
        bits, int(bool(sorted_indices)), _dtype_code(x2), y.data_ptr(),
        workspace.data_ptr() if workspace is not None else None,
        workspace.numel() if workspace is not None else 0)
    check(rc)
    return y.reshape(*x.shape[:-1], n)


def gather_qmm_siblings(x: torch.Tensor, linears, rhs_indices: torch.Tensor, group_size: int = 64, bits: int = 4, *, stream=None,
                        workspace: Optional[torch.Tensor] = None):
    """``gather_qmm`` for one to three linears that share x, the sorted ids and their shape (gate | up of a routed
    block; the grouped gate|up launch of crates/lisa-mlx/src/models/qwen4/prefill_indirect.rs:127-170): `linears`
    is a sequence of (w [E, N, K*bits/32], scales, biases); returns the list of outputs [rows, N]."""
    import ctypes as C

    _need_cuda(x, rhs_indices)
    k = x.shape[-1]
    rows = x.numel() // k
    x2 = x.reshape(rows, k).contiguous()
    count = len(linears)
    experts, n = linears[0][0].shape[0], linears[0][0].shape[-2]
    keep, ys = [], []
    wp, sp, bp, yp = (C.c_void_p * count)(), (C.c_void_p * count)(), (C.c_void_p * count)(), (C.c_void_p * count)()
    for i, (w, sc, bi) in enumerate(linears):
        _need_cuda(w, sc, bi)
        w = _words(w)
        if w.shape[0] != experts or w.shape[-2] != n:
            raise LisaError(_cabi.ERR_BAD_ARG, "gather_qmm_siblings: the linears must have one shape")
        sc, bi = sc.contiguous(), bi.contiguous()
        y = torch.empty((rows, n), dtype=x2.dtype, device=x2.device)
        keep.append((w, sc, bi))
        ys.append(y)
        wp[i], sp[i], bp[i], yp[i] = w.data_ptr(), sc.data_ptr(), bi.data_ptr(), y.data_ptr()
    need = lib().lisa_cuda_gather_qmm_workspace_bytes(rows, experts)
    if workspace is None and need:
        workspace = torch.empty(need, dtype=torch.uint8, device=x2.device)
    ids = rhs_indices.to(torch.int32).contiguous()
    check(lib().lisa_cuda_gather_qmm_siblings(_stream(stream), x2.data_ptr(), rows, k, count, wp, sp, bp, ids.data_ptr(), experts, n,
                                              1, group_size, bits, 1, _dtype_code(x2), yp,
                                              workspace.data_ptr() if workspace is not None else None,
                                              workspace.numel() if workspace is not None else 0))
    return [y.reshape(*x.shape[:-1], n) for y in ys]


def _format_code(fmt) -> int:
    return BlockFormat[fmt] if isinstance(fmt, str) else int(fmt)


def packed_matvec(fmt, weights: torch.Tensor, input: torch.Tensor, *, stream=None) -> torch.Tensor:
    """``deepseek41::packed_matvec`` (deepseek41.rs:93-110): weights uint8 [rows, row_bytes],
    input f32 [tokens, K] -> f32 [tokens, rows]."""
    _need_cuda(weights, input)
    code = _format_code(fmt)
    if weights.dim() != 2 or weights.dtype != torch.uint8 or not weights.is_contiguous():
        raise LisaError(_cabi.ERR_BAD_ARG, "unsupported GGUF quantized matvec layout")
    if input.dim() != 2 or input.dtype != torch.float32:
        raise LisaError(_cabi.ERR_BAD_ARG, "invalid GGUF matvec input rows")
    rows, row_bytes = weights.shape
    block = _BLOCK_BYTES.get(code, 0)
    if block and row_bytes % block == 0 and input.shape[1] != row_bytes // block * 256:
        raise LisaError(_cabi.ERR_BAD_ARG, "GGUF matvec input width does not match the packed rows")
    tokens = input.shape[0]
    y = torch.empty((tokens, rows), dtype=torch.float32, device=input.device)
    rc = lib().lisa_cuda_gguf_packed_matvec(_stream(stream), code, weights.data_ptr(), rows, row_bytes,
                                            input.contiguous().data_ptr(), tokens, y.data_ptr())
    check(rc)
    return y


def packed_matmul(fmt, weights: torch.Tensor, input: torch.Tensor, *, workspace: Optional[torch.Tensor] = None,
                  stream=None) -> torch.Tensor:
    """``packed_matvec`` for many tokens with a workspace: products of 32 tokens or more run on the
    tensor cores (operands as hi + lo bf16 planes, f32 accumulate and output, ~1e-4 of the matvec);
    everything else is the exact matvec."""
    _need_cuda(weights, input)
    code = _format_code(fmt)
    if weights.dim() != 2 or weights.dtype != torch.uint8 or not weights.is_contiguous():
        raise LisaError(_cabi.ERR_BAD_ARG, "unsupported GGUF quantized matvec layout")
    if input.dim() != 2 or input.dtype != torch.float32:
        raise LisaError(_cabi.ERR_BAD_ARG, "invalid GGUF matvec input rows")
    rows, row_bytes = weights.shape
    tokens = input.shape[0]
    need = lib().lisa_cuda_gguf_packed_matmul_workspace_bytes(tokens, row_bytes, code)
    if workspace is None and need:
        workspace = torch.empty(need, dtype=torch.uint8, device=input.device)
    y = torch.empty((tokens, rows), dtype=torch.float32, device=input.device)
    rc = lib().lisa_cuda_gguf_packed_matmul(_stream(stream), code, weights.data_ptr(), rows, row_bytes,
                                            input.contiguous().data_ptr(), tokens, y.data_ptr(),
                                            workspace.data_ptr() if workspace is not None else None,
                                            workspace.numel() if workspace is not None else 0)
    check(rc)
    return y


def expert_matvec(fmt, weights: torch.Tensor, input: torch.Tensor, ids: torch.Tensor, *,
                  stream=None) -> torch.Tensor:
    """``deepseek41::expert_matvec`` (deepseek41.rs:204-283): weights uint8 [E, rows, row_bytes],
    input f32 [tokens, 1 or top_k, K], ids int32 [tokens, top_k] -> f32 [tokens, top_k, rows]."""
    _need_cuda(weights, input, ids)
    code = _format_code(fmt)
    if weights.dim() != 3 or weights.dtype != torch.uint8 or not weights.is_contiguous():
        raise LisaError(_cabi.ERR_BAD_ARG, "unsupported GGUF quantized matvec layout")
    if ids.dim() != 2 or ids.dtype != torch.int32 or input.dim() != 3 or input.dtype != torch.float32:
        raise LisaError(_cabi.ERR_BAD_ARG, "invalid GGUF expert matvec geometry")
    experts, rows, row_bytes = weights.shape
    tokens, top_k = ids.shape
    slots = input.shape[1]
    if input.shape[0] != tokens:
        raise LisaError(_cabi.ERR_BAD_ARG, "invalid GGUF expert matvec geometry")
    y = torch.empty((tokens, top_k, rows), dtype=torch.float32, device=input.device)
    rc = lib().lisa_cuda_gguf_expert_matvec(_stream(stream), code, weights.data_ptr(), experts, rows,
                                            row_bytes, input.contiguous().data_ptr(), tokens, slots,
                                            ids.contiguous().data_ptr(), top_k, y.data_ptr())
    check(rc)
    return y


# ---------------------------------------------------------------- MoE routing
def moe_route(logits: torch.Tensor, top_k: int, *, stream=None) -> Tuple[torch.Tensor, torch.Tensor]:
    _need_cuda(logits)
    logits = logits.contiguous().to(torch.float32)
    tokens, experts = logits.shape
    idx = torch.empty((tokens, top_k), dtype=torch.int32, device=logits.device)
    wts = torch.empty((tokens, top_k), dtype=torch.float32, device=logits.device)
    check(lib().lisa_cuda_moe_route(_stream(stream), logits.data_ptr(), tokens, experts, top_k,
                                    idx.data_ptr(), wts.data_ptr()))
    return idx, wts


def moe_sort(idx: torch.Tensor, experts: int, top_k: int, *, stream=None):
    _need_cuda(idx)
    flat = idx.reshape(-1).contiguous()
    slots = flat.numel()
    dev = flat.device
    sorted_ids = torch.empty(slots, dtype=torch.int32, device=dev)
    token_rows = torch.empty(slots, dtype=torch.int32, device=dev)
    inverse = torch.empty(slots, dtype=torch.int32, device=dev)
    need = lib().lisa_cuda_moe_sort_workspace_bytes(slots, experts)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
    check(lib().lisa_cuda_moe_sort(_stream(stream), flat.data_ptr(), slots, experts, top_k,
                                   sorted_ids.data_ptr(), token_rows.data_ptr(), inverse.data_ptr(),
                                   ws.data_ptr(), ws.numel()))
    return sorted_ids, token_rows, inverse


def moe_sort_static(idx: torch.Tensor, experts: int, top_k: int, out=None, *, stream=None):
    """``moe_sort`` through the entry point that allocates nothing: the count table is a device
    array built into the library.  Pass ``out=(sorted_ids, token_rows, inverse)`` to reuse the
    caller's buffers, as a caller that cannot allocate would; limit ceil(slots/256)*experts <= 65536."""
    _need_cuda(idx)
    flat = idx.reshape(-1).contiguous()
    slots = flat.numel()
    if out is None:
        out = tuple(torch.empty(slots, dtype=torch.int32, device=flat.device) for _ in range(3))
    sorted_ids, token_rows, inverse = out
    check(lib().lisa_cuda_moe_sort_static(_stream(stream), flat.data_ptr(), slots, experts, top_k,
                                          sorted_ids.data_ptr(), token_rows.data_ptr(), inverse.data_ptr()))
    return sorted_ids, token_rows, inverse


def gather_rows(x: torch.Tensor, token_rows: torch.Tensor, *, stream=None) -> torch.Tensor:
    _need_cuda(x, token_rows)
    x = x.contiguous()
    rows, width = token_rows.numel(), x.shape[-1]
    out = torch.empty((rows, width), dtype=x.dtype, device=x.device)
    check(lib().lisa_cuda_gather_rows(_stream(stream), x.data_ptr(), token_rows.data_ptr(), rows, width,
                                      _dtype_code(x), out.data_ptr()))
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor, *, stream=None) -> torch.Tensor:
    _need_cuda(gate, up)
    gate, up = gate.contiguous(), up.contiguous()
    act = torch.empty_like(gate)
    check(lib().lisa_cuda_swiglu(_stream(stream), gate.data_ptr(), up.data_ptr(), gate.numel(),
                                 _dtype_code(gate), act.data_ptr()))
    return act


def moe_combine(down_sorted: torch.Tensor, weights: torch.Tensor, inverse: torch.Tensor, top_k: int, *,
                stream=None) -> torch.Tensor:
    _need_cuda(down_sorted, weights, inverse)
    down_sorted = down_sorted.contiguous()
    hidden = down_sorted.shape[-1]
    tokens = inverse.numel() // top_k
    out = torch.empty((tokens, hidden), dtype=down_sorted.dtype, device=down_sorted.device)
    check(lib().lisa_cuda_moe_combine(_stream(stream), down_sorted.data_ptr(),
                                      weights.contiguous().data_ptr(), inverse.contiguous().data_ptr(),
                                      tokens, top_k, hidden, _dtype_code(down_sorted), out.data_ptr()))
    return out


def moe_gate_up_act(x: torch.Tensor, idx: torch.Tensor, gate, up, group_size: int, bits: int, *, xrow=None,
                    stream=None) -> torch.Tensor:
    """moe_decode::gate_up_act (crates/lisa-mlx/src/models/qwen4/moe_decode.rs:136-184) without the shared
    expert: x [tokens, hidden], idx int32 [tokens, top_k], gate / up = (weight [E, inter, hidden*bits/32],
    scales, biases) -> act [tokens * top_k, inter]."""
    _need_cuda(x, idx, *gate, *up)
    x = x.contiguous()
    idx = idx.contiguous()
    top_k = idx.shape[-1]
    slots = idx.numel()
    experts, inter = gate[0].shape[0], gate[0].shape[1]
    hidden = x.shape[-1]
    act = torch.empty((slots, inter), dtype=x.dtype, device=x.device)
    check(lib().lisa_cuda_moe_gate_up_act(_stream(stream), x.data_ptr(), idx.data_ptr(),
                                          None if xrow is None else xrow.contiguous().data_ptr(), slots, top_k, experts,
                                          hidden, inter, gate[0].data_ptr(), gate[1].data_ptr(), gate[2].data_ptr(),
                                          up[0].data_ptr(), up[1].data_ptr(), up[2].data_ptr(), group_size, bits,
                                          _dtype_code(x), act.data_ptr()))
    return act


def moe_down_combine(act: torch.Tensor, idx: torch.Tensor, weights: torch.Tensor, down, group_size: int, bits: int, *,
                     stream=None) -> torch.Tensor:
    """moe_decode::down_combine (moe_decode.rs:214-298) without the shared expert and its gate: act
    [tokens * top_k, inter], idx / weights [tokens, top_k], down = (weight [E, hidden, inter*bits/32], scales,
    biases) -> [tokens, hidden]."""
    _need_cuda(act, idx, weights, *down)
    act = act.contiguous()
    idx = idx.contiguous()
    tokens, top_k = idx.shape
    experts, hidden = down[0].shape[0], down[0].shape[1]
    inter = act.shape[-1]
    out = torch.empty((tokens, hidden), dtype=act.dtype, device=act.device)
    check(lib().lisa_cuda_moe_down_combine(_stream(stream), act.data_ptr(), idx.data_ptr(),
                                           weights.contiguous().data_ptr(), tokens, top_k, experts, inter, hidden,
                                           down[0].data_ptr(), down[1].data_ptr(), down[2].data_ptr(), group_size, bits,
                                           _dtype_code(act), out.data_ptr()))
    return out


def launch_count() -> int:
    return int(lib().lisa_cuda_launch_count())


def device_status() -> int:
    return int(lib().lisa_cuda_device_status())


def clear_device_status() -> None:
    """Resets the sticky status word after the caller has handled a reported failure."""
    check(lib().lisa_cuda_clear_device_status())
