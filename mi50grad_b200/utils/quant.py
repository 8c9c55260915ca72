"""INT4 weight-only quantisation formats: pack, unpack, dequantise, convert.

Three checkpoint layouts are understood (all 4-bit, unsigned nibbles):

* GPTQ  : qweight[K/8, N] int32 (nibble b of word r holds k = 8r+b),
          scales[ceil(K/g), N] fp16, qzeros[ceil(K/g), N/8] int32 packed along N
          (nibble b of word c holds column 8c+b); w = (q - zero) * scale
          (reference: src/model/weight_loader.py:95-119, 145-171).
* "AWQ" as the reference defines it: the GPTQ tensors without qzeros and
          w = q * scale (reference: src/model/awq_loader.py:88-121).
* compressed-tensors: weight_packed[N, K/8] int32 (nibble b of word c holds
          k = 8c+b), weight_scale[N, K/g], symmetric with an implicit zero of 8
          (reference: src/model/compressed_tensors_loader.py:98-186).

Everything is converted to one engine form, `Int4Linear`: K-packed qweight,
fp16 scales and fp16 zeros of shape [groups, N], plus `group_offset`, the number
of k-elements by which row 0 of this (possibly row-sharded) matrix sits inside
its first quantisation group.  `group_offset` is what lets a row-parallel shard
start in the middle of a group (FFN width 704 split over 2 ranks is 2.75 groups
of 128 each), a case the reference's sharder silently assumes away
(reference: src/model/weight_loader.py:374-385).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

NIBBLES = 8


def pack_int4_rows(q: torch.Tensor) -> torch.Tensor:
    """[K, N] values 0..15 -> [K/8, N] int32, nibble b of row r holds k = 8r+b."""
    K, N = q.shape
    if K % NIBBLES:
        raise ValueError("K must be a multiple of 8")
    q = q.to(torch.int64).reshape(K // NIBBLES, NIBBLES, N)
    shifts = (torch.arange(NIBBLES, dtype=torch.int64, device=q.device) * 4).view(1, NIBBLES, 1)
    word = (q << shifts).sum(dim=1)
    return _to_i32(word)


def unpack_int4_rows(qweight: torch.Tensor) -> torch.Tensor:
    """[K/8, N] int32 -> [K, N] uint8."""
    R, N = qweight.shape
    w = qweight.to(torch.int64) & 0xFFFFFFFF
    shifts = (torch.arange(NIBBLES, dtype=torch.int64, device=qweight.device) * 4).view(1, NIBBLES, 1)
    q = (w.unsqueeze(1) >> shifts) & 0xF
    return q.reshape(R * NIBBLES, N).to(torch.uint8)


def pack_int4_cols(q: torch.Tensor) -> torch.Tensor:
    """[R, C] values 0..15 -> [R, C/8] int32, nibble b of word c holds column 8c+b."""
    return pack_int4_rows(q.t().contiguous()).t().contiguous()


def unpack_int4_cols(packed: torch.Tensor) -> torch.Tensor:
    """[R, C/8] int32 -> [R, C] uint8."""
    return unpack_int4_rows(packed.t().contiguous()).t().contiguous()


def _to_i32(word: torch.Tensor) -> torch.Tensor:
    word = word & 0xFFFFFFFF
    word = torch.where(word >= 2**31, word - 2**32, word)
    return word.to(torch.int32)


def unpack_gptq_qzeros(qzeros: torch.Tensor, sym: bool = True) -> torch.Tensor:
    """GPTQ packed zeros -> fp16 [groups, N].  Symmetric checkpoints store the
    zero itself (8); legacy asymmetric ones store zero-1."""
    z = unpack_int4_cols(qzeros).to(torch.float16)
    return z if sym else z + 1


def pack_gptq_qzeros(zeros: torch.Tensor, sym: bool = True) -> torch.Tensor:
    z = zeros.to(torch.int64)
    if not sym:
        z = z - 1
    return pack_int4_cols(z)


@dataclass
class DenseLinear:
    """y = W x with W[N, K] (HuggingFace out_features x in_features)."""
    weight: torch.Tensor

    @property
    def out_features(self) -> int:
        return self.weight.shape[0]

    @property
    def in_features(self) -> int:
        return self.weight.shape[1]

    def dense(self, dtype=torch.float32) -> torch.Tensor:
        return self.weight.to(dtype)

    def to(self, device) -> "DenseLinear":
        return DenseLinear(self.weight.to(device))


@dataclass
class Int4Linear:
    """Engine form of a 4-bit weight-only linear layer computing y = Wᵀx with
    the quantised matrix stored input-major: qweight[K/8, N]."""
    qweight: torch.Tensor              # int32 [K/8, N]
    scales: torch.Tensor               # fp16  [G, N]
    zeros: Optional[torch.Tensor]      # fp16  [G, N]; None means zero = 0 (AWQ form)
    group_size: int = 128
    group_offset: int = 0              # k-elements of the first group that precede row 0

    @property
    def in_features(self) -> int:
        return self.qweight.shape[0] * NIBBLES

    @property
    def out_features(self) -> int:
        return self.qweight.shape[1]

    @property
    def num_groups(self) -> int:
        return self.scales.shape[0]

    def expected_groups(self) -> int:
        return -(-(self.in_features + self.group_offset) // self.group_size)

    def validate(self):
        if self.scales.shape != (self.expected_groups(), self.out_features):
            raise ValueError(
                f"scales {tuple(self.scales.shape)} do not cover K={self.in_features} "
                f"(offset {self.group_offset}, g={self.group_size}), N={self.out_features}")
        if self.zeros is not None and self.zeros.shape != self.scales.shape:
            raise ValueError("zeros must match scales")

    def group_index(self) -> torch.Tensor:
        k = torch.arange(self.in_features, device=self.qweight.device)
        return (k + self.group_offset) // self.group_size

    def dense(self, dtype=torch.float32) -> torch.Tensor:
        """Dequantised W[N, K]."""
        q = unpack_int4_rows(self.qweight).to(torch.float32)          # [K, N]
        gi = self.group_index()
        s = self.scales.to(torch.float32)[gi]
        if self.zeros is not None:
            q = q - self.zeros.to(torch.float32)[gi]
        return (q * s).t().contiguous().to(dtype)

    def to(self, device) -> "Int4Linear":
        return Int4Linear(self.qweight.to(device), self.scales.to(device),
                          None if self.zeros is None else self.zeros.to(device),
                          self.group_size, self.group_offset)


def quantize_int4(weight: torch.Tensor, group_size: int = 128, sym: bool = True,
                  awq: bool = False) -> Int4Linear:
    """Round-to-nearest 4-bit quantisation of W[N, K] (test helper; checkpoints
    come pre-quantised)."""
    N, K = weight.shape
    w = weight.to(torch.float32).t().contiguous()                     # [K, N]
    G = -(-K // group_size)
    pad = G * group_size - K
    wp = torch.cat([w, w.new_zeros(pad, N)]) if pad else w
    wg = wp.reshape(G, group_size, N)
    if awq:
        # zero-less form: q*scale with q in 0..15 can only hold non-negative weights
        mx = wg.amax(dim=1).clamp_min(1e-8)
        scale = mx / 15.0
        q = torch.round(wg / scale.unsqueeze(1)).clamp(0, 15)
        zeros = None
    elif sym:
        mx = wg.abs().amax(dim=1).clamp_min(1e-8)
        scale = mx / 7.0
        q = (torch.round(wg / scale.unsqueeze(1)) + 8).clamp(0, 15)
        zeros = torch.full((G, N), 8.0, dtype=torch.float16)
    else:
        lo, hi = wg.amin(dim=1), wg.amax(dim=1)
        scale = ((hi - lo) / 15.0).clamp_min(1e-8)
        zp = torch.round(-lo / scale).clamp(0, 15)
        q = (torch.round(wg / scale.unsqueeze(1)) + zp.unsqueeze(1)).clamp(0, 15)
        zeros = zp.to(torch.float16)
    q = q.reshape(G * group_size, N)[:K]
    return Int4Linear(pack_int4_rows(q.to(torch.uint8)), scale.to(torch.float16), zeros,
                      group_size, 0)


def random_int4_linear(K: int, N: int, group_size: int = 128,
                       generator: Optional[torch.Generator] = None,
                       device="cpu", zeros: Optional[float] = 8.0,
                       scale_lo: float = 0.002, scale_hi: float = 0.02) -> Int4Linear:
    """Random-init weights of the benchmark's form: nibbles uniform 0..15,
    zero 8, fp16 scales U(scale_lo, scale_hi)."""
    G = -(-K // group_size)
    qweight = torch.randint(-2**31, 2**31 - 1, (K // NIBBLES, N), dtype=torch.int64,
                            generator=generator, device=device).to(torch.int32)
    scales = (torch.rand((G, N), generator=generator, device=device)
              * (scale_hi - scale_lo) + scale_lo).to(torch.float16)
    z = None if zeros is None else torch.full((G, N), zeros, dtype=torch.float16, device=device)
    return Int4Linear(qweight, scales, z, group_size, 0)


# -- compressed-tensors (N-major) -------------------------------------------

def ct_to_engine(weight_packed: torch.Tensor, weight_scale: torch.Tensor,
                 group_size: int = 32) -> Int4Linear:
    """compressed-tensors pack-quantized [N, K/8] + scale [N, K/g] -> engine form.
    The stored nibble is unsigned with an implicit zero of 8."""
    q = unpack_int4_cols(weight_packed)                # [N, K]
    qweight = pack_int4_rows(q.t().contiguous())       # [K/8, N]
    scales = weight_scale.to(torch.float16).t().contiguous()
    zeros = torch.full_like(scales, 8.0)
    return Int4Linear(qweight, scales, zeros, group_size, 0)


def ct_dequantize(weight_packed: torch.Tensor, weight_scale: torch.Tensor,
                  group_size: int = 32) -> torch.Tensor:
    return ct_to_engine(weight_packed, weight_scale, group_size).dense()


def engine_to_ct(lin: Int4Linear) -> Tuple[torch.Tensor, torch.Tensor]:
    q = unpack_int4_rows(lin.qweight).t().contiguous()
    return pack_int4_cols(q), lin.scales.t().contiguous()


# -- true AutoAWQ GEMM layout (recognised and converted explicitly) ---------

AUTOAWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)


def is_autoawq_layout(qweight_shape, scales_shape) -> bool:
    """AutoAWQ packs along N: qweight[K, N/8] with scales[K/g, N]."""
    return (len(qweight_shape) == 2 and len(scales_shape) == 2
            and qweight_shape[1] * NIBBLES == scales_shape[1]
            and qweight_shape[0] > scales_shape[0] * NIBBLES // 2)


def autoawq_to_engine(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor,
                      group_size: int = 128) -> Int4Linear:
    def unpack_awq(p):
        R, C = p.shape
        w = p.to(torch.int64) & 0xFFFFFFFF
        out = torch.empty(R, C * NIBBLES, dtype=torch.uint8)
        for slot, col in enumerate(AUTOAWQ_ORDER):
            out[:, col::NIBBLES] = ((w >> (4 * slot)) & 0xF).to(torch.uint8)
        return out
    q = unpack_awq(qweight)                       # [K, N]
    z = unpack_awq(qzeros).to(torch.float16)      # [G, N]
    return Int4Linear(pack_int4_rows(q), scales.to(torch.float16), z, group_size, 0)


# -- INT8 / W4A8 conversions (reference: src/model/weight_loader.py:122-249) -

def int4_to_w8a8(lin: Int4Linear) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dequantise then re-quantise per output channel to signed int8.
    Returns (W_int8[N, K], scale_w[N] fp32)."""
    w = lin.dense()
    mx = w.abs().amax(dim=1) + 1e-12
    scale = (mx / 127.0).to(torch.float32)
    return torch.round(w / scale[:, None]).clamp(-128, 127).to(torch.int8), scale


def int4_to_w4a8(lin: Int4Linear) -> Tuple[torch.Tensor, torch.Tensor]:
    """N-major signed-nibble repack: returns (W_packed[N, K/8] int32 with the
    zero already subtracted and clamped to [-8, 7], scales[G, N] fp16)."""
    q = unpack_int4_rows(lin.qweight).to(torch.int64)
    z = 0 if lin.zeros is None else lin.zeros.to(torch.int64)[lin.group_index()]
    s = (q - z).clamp(-8, 7) & 0xF
    return pack_int4_cols(s.t().contiguous()), lin.scales.clone()


def int4_to_w4a8_per_channel(lin: Int4Linear) -> Tuple[torch.Tensor, torch.Tensor]:
    """The same nibbles with ONE scale per output channel, the mean of its group scales
    (reference: src/kernels/repack_w4a8.py:119-138, a test aid: it gives up the per-group accuracy).
    Returns (W_packed[N, K/8] int32, scale[N] fp32)."""
    packed, scales = int4_to_w4a8(lin)
    return packed, scales.to(torch.float32).mean(dim=0)


def dense_to_w4a8(w: torch.Tensor, group_size: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantise a real matrix W[N, K] straight to the W4A8 layout: symmetric, scale = max|w| / 7 per
    (group, channel) (reference: src/kernels/repack_w4a8.py:177-208).  Returns (packed, scales[G, N] fp16)."""
    N, K = w.shape
    assert K % group_size == 0 and K % 8 == 0
    wg = w.to(torch.float32).reshape(N, K // group_size, group_size)
    scale = (wg.abs().amax(dim=2) / 7.0).clamp_min(1e-8).to(torch.float16)           # [N, G]
    q = torch.round(wg / scale.to(torch.float32)[:, :, None]).clamp(-8, 7).to(torch.int64).reshape(N, K)
    return pack_int4_cols(q & 0xF), scale.t().contiguous()


def w4a8_roundtrip_error(w: torch.Tensor, group_size: int = 128) -> float:
    """max |W - dequant(quant(W))| / max|W| (reference: src/kernels/repack_w4a8.py:211-227)."""
    packed, scales = dense_to_w4a8(w, group_size)
    back = dequantize_w4a8(packed, scales, group_size)
    return float((back - w.to(torch.float32)).abs().max() / w.abs().max().clamp_min(1e-12))


def dequantize_w4a8(w_packed: torch.Tensor, scales: torch.Tensor,
                    group_size: int = 128) -> torch.Tensor:
    q = unpack_int4_cols(w_packed).to(torch.int64)       # [N, K]
    q = torch.where(q >= 8, q - 16, q).to(torch.float32)
    K = q.shape[1]
    gi = torch.arange(K) // group_size
    return q * scales.to(torch.float32).t()[:, gi]


def quantize_activation_int8(x: torch.Tensor, per_row: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dynamic symmetric int8 (reference: src/kernels/activation_quant.hip): one scale for the
    tensor, or with `per_row` one per row of a 2-D input (what the device kernel computes)."""
    xf = x.to(torch.float32)
    amax = (xf.abs().amax(dim=-1, keepdim=True) if per_row else xf.abs().amax()).clamp_min(1e-12)
    scale = amax / 127.0
    q = torch.round(xf / scale).clamp(-128, 127).to(torch.int8)
    return q, (scale.squeeze(-1) if per_row else scale)
