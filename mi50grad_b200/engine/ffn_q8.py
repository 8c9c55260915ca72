"""The FFN of one layer on the INT8-activation path.

The reference's engine takes `quant_format` in {'w4a16', 'w8a8', 'w4a8'} and, for the last two, runs
gate / up / down through its INT8 GEMV kernels with a dynamic activation quantisation in front of
each (reference: src/inference/engine.py:463-482, 1767-1771; tests/test_engine_w8a8_w4a8.py).  Here
the whole-model step is w4a16 (INT4 weights with fp16 activations already stream the fewest bytes on
this part), and the INT8 formats are offered per layer through this class: the same three products
on the int8 tensor-core kernels, for any number of rows.
"""
from __future__ import annotations

import torch

from ..utils import quant as Q


class FfnQ8:
    """gate/up/down of one layer converted from GPTQ-Int4 to W8A8 or W4A8 and kept on the device.

    forward(x fp16 [T, H]) -> fp32 [T, H] = down(silu(gate(x)) * up(x)), activations quantised to
    int8 per row before each product."""

    def __init__(self, gate: Q.Int4Linear, up: Q.Int4Linear, down: Q.Int4Linear, quant_format: str = "w8a8",
                 device="cuda"):
        if quant_format not in ("w8a8", "w4a8"):
            raise ValueError("quant_format must be w8a8 or w4a8")
        self.quant_format = quant_format
        self.group = gate.group_size
        conv = Q.int4_to_w8a8 if quant_format == "w8a8" else Q.int4_to_w4a8
        dev = torch.device(device)
        self.w = {}
        for name, lin in (("gate", gate), ("up", up), ("down", down)):
            w, s = conv(lin)
            self.w[name] = (w.contiguous().to(dev), s.contiguous().to(dev))

    def _linear(self, name: str, xq: torch.Tensor, sx: torch.Tensor, out_dtype) -> torch.Tensor:
        from ..ops import kernels as K
        w, s = self.w[name]
        if self.quant_format == "w8a8":
            return K.linear_w8a8(w, s, xq, sx, out_dtype=out_dtype)
        return K.linear_w4a8(w, s, xq, sx, group=self.group, out_dtype=out_dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from ..ops import kernels as K
        x = x.half().contiguous()
        xq, sx = K.act_quant_int8(x)
        gate = self._linear("gate", xq, sx, torch.float16)
        up = self._linear("up", xq, sx, torch.float16)
        act = K.silu_mul(gate, up)
        aq, sa = K.act_quant_int8(act)
        return self._linear("down", aq, sa, torch.float32)

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() + s.numel() * s.element_size() for w, s in self.w.values())


def reference_ffn(gate: Q.Int4Linear, up: Q.Int4Linear, down: Q.Int4Linear, x: torch.Tensor) -> torch.Tensor:
    """fp32 FFN with the dequantised INT4 weights (what the w4a16 path computes)."""
    xf = x.float()
    h = torch.nn.functional.silu(xf @ gate.dense().t()) * (xf @ up.dense().t())
    return h @ down.dense().t()
