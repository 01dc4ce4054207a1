"""Engine-side holders of quantized weights, mirroring ``lisa-engine``'s callers of the path.

``QuantizedLinear`` / ``QuantizedEmbedding`` / ``detect_group_size`` follow
crates/lisa-engine/src/core/quant.rs:273-321,408-492;
``SwitchGlu.forward`` is the generic routed-expert block of
crates/lisa-engine/src/models/qwen4/moe.rs:352-481 without the Qwen4-specific shared expert.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import ops


def detect_group_size(weight_cols: int, scales_cols: int, bits: int) -> Optional[int]:
    """Group size implied by the packed shapes, or None when they are inconsistent
    (quant.rs:273-287)."""
    if weight_cols <= 0 or scales_cols <= 0 or bits <= 0 or 32 % bits != 0:
        return None
    k = weight_cols * (32 // bits)
    if k % scales_cols != 0:
        return None
    group = k // scales_cols
    return group if 1 <= group <= 4096 else None


@dataclass
class QuantizedLinear:
    """weight uint32 [N, K*bits/32]; scales, biases bf16 [N, K/group_size] (quant.rs:292-299)."""
    weight: torch.Tensor
    scales: torch.Tensor
    biases: torch.Tensor
    group_size: int = 64
    bits: int = 4

    def dims_out(self) -> int:
        return self.weight.shape[0]

    def forward(self, x: torch.Tensor, *, flags: int = 0) -> torch.Tensor:
        """[..., K] -> [..., N]; the input is flattened to 2-D first (quant.rs:306-321)."""
        k = x.shape[-1]
        flat = x.reshape(-1, k)
        out = ops.quantized_matmul(flat, self.weight, self.scales, self.biases, True, self.group_size,
                                   self.bits, flags=flags)
        return out.reshape(*x.shape[:-1], self.dims_out())

    def forward_serial_rows(self, x: torch.Tensor) -> torch.Tensor:
        return ops.quantized_matmul_serial_rows(x, self.weight, self.scales, self.biases, True,
                                                self.group_size, self.bits)

    def set_quant(self, group_size: int, bits: int) -> None:
        """Overrides the geometry: the group size is re-derived from the packed shapes for `bits`,
        `group_size` is the fallback (quant.rs:400-406)."""
        self.bits = bits
        self.group_size = detect_group_size(self.weight.shape[-1], self.scales.shape[-1], bits) or group_size

    @classmethod
    def load(cls, shard, prefix: str, key: str = "", device="cuda", bits: int = 4, group_size: int = 64):
        """``{prefix}.{key}.weight/.scales/.biases`` of a safetensors shard (`lisa_b200.files.Shard`), copied to
        `device`; the group size comes from the shapes (quant.rs:408-432)."""
        w, s, b, gs, bits = shard.quantized_triplet(prefix, key, bits=bits, group_size_hint=group_size)
        return cls(_to_device_words(w, device), _to_device_bf16(s, device), _to_device_bf16(b, device), gs, bits)


def _to_device_words(a, device):
    import numpy as np
    return torch.from_numpy(np.array(a, copy=True).view(np.int32)).to(device)


def _to_device_bf16(a, device):
    import numpy as np
    return torch.from_numpy(np.array(a, copy=True).view(np.int16)).to(device).view(torch.bfloat16)


@dataclass
class QuantizedEmbedding:
    """An affine-quantized embedding table; lookups dequantize only the gathered rows (quant.rs:436-492).
    weight uint32 [V, K*bits/32]; scales, biases bf16 [V, K/group_size]."""
    weight: torch.Tensor
    scales: torch.Tensor
    biases: torch.Tensor
    group_size: int = 64
    bits: int = 4

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        """Token ids (any integer dtype, any shape) -> [..., K] rows."""
        return ops.dequantize_rows(self.weight, self.scales, self.biases, ids, self.group_size, self.bits)

    def as_linear(self, x: torch.Tensor) -> torch.Tensor:
        """The tied output head: [..., K] -> [..., V]."""
        return ops.quantized_matmul(x, self.weight, self.scales, self.biases, True, self.group_size, self.bits)

    def set_quant(self, group_size: int, bits: int) -> None:
        self.bits = bits
        self.group_size = detect_group_size(self.weight.shape[-1], self.scales.shape[-1], bits) or group_size

    @classmethod
    def load(cls, shard, prefix: str, device="cuda", bits: int = 4, group_size: int = 64):
        w, s, b, gs, bits = shard.quantized_triplet(prefix, "", bits=bits, group_size_hint=group_size)
        return cls(_to_device_words(w, device), _to_device_bf16(s, device), _to_device_bf16(b, device), gs, bits)


@dataclass
class SwitchGlu:
    """Routed experts: gate/up [E, inter, hidden*bits/32], down [E, hidden, inter*bits/32]."""
    gate: QuantizedLinear
    up: QuantizedLinear
    down: QuantizedLinear
    top_k: int
    # below this many (token, expert) slots the per-slot path is used; from it on the sorted one, which reads every
    # expert once (measured cross-over on the 128-expert top-8 block: three tokens 0.066 against 0.079 ms, four
    # tokens 0.082 against 0.088)
    DECODE_SLOTS = 32

    def forward(self, x: torch.Tensor, router_logits: torch.Tensor) -> torch.Tensor:
        """x [tokens, hidden] bf16, router_logits f32 [tokens, E] -> [tokens, hidden]:
        route, stable sort by expert, gate/up gather_qmm, SwiGLU, down gather_qmm, weighted
        un-sort (moe.rs:352-481)."""
        experts = self.gate.weight.shape[0]
        gs, bits = self.gate.group_size, self.gate.bits
        idx, weights = ops.moe_route(router_logits, self.top_k)
        if x.shape[0] * self.top_k < self.DECODE_SLOTS:
            # a handful of tokens (forward_decode, moe.rs:116-350): three launches, every slot streams its own expert
            g, u, d = ((l.weight, l.scales, l.biases) for l in (self.gate, self.up, self.down))
            act = ops.moe_gate_up_act(x, idx, g, u, gs, bits)
            return ops.moe_down_combine(act, idx, weights, d, gs, bits)
        sorted_ids, token_rows, inverse = ops.moe_sort(idx, experts, self.top_k)
        x_sorted = ops.gather_rows(x, token_rows)
        # gate and up read the same rows: one tile table, one grouped launch (prefill_indirect.rs:127-170)
        g, u = ops.gather_qmm_siblings(x_sorted, [(self.gate.weight, self.gate.scales, self.gate.biases),
                                                  (self.up.weight, self.up.scales, self.up.biases)], sorted_ids, gs, bits)
        act = ops.swiglu(g, u)
        d = ops.gather_qmm(act, self.down.weight, self.down.scales, self.down.biases, None, sorted_ids,
                           True, gs, bits, True)
        return ops.moe_combine(d, weights, inverse, self.top_k)
