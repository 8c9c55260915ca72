"""Device weight layouts.

INT4 projections are re-packed once, at load time, from the checkpoint's
K-packed `qweight[K/8, N]` into tensor-core fragment order (see csrc/gemv.cu):

    qfrag [NTL/4][KB][4 tiles][32 lanes][4 words]   int32   (a warp's 2 KB per k-block is contiguous)
    szfrag[NTL/4][G][4 tiles][8][4]                  fp16    (scale n, scale n+8, zero n, zero n+8; the 256 bytes
                                                              of a 64-column warp tile and one group are contiguous,
                                                              so they can ride along with the weights in one bulk copy)

where an n-tile is 16 output features, a k-block 64 input features (two chunks
of 32), and lane (g = lane>>2, t = lane&3) of chunk j owns words 2j and 2j+1.
Nibble p of word wi holds W[n, k] with
    n = 16*tile + g + 8*((p>>1)&1),   k = 64*block + 32*j + 16*(p&1) + 8*wi + 2*t + (p>>2).
N is padded to a multiple of 128 (zero scale), K to a multiple of 64 (activations
read as zero there).  The reference uploads checkpoints unchanged and picks one
of eight kernel variants per shape (reference: src/inference/engine.py:2535-2543).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..utils.quant import DenseLinear, Int4Linear, unpack_int4_rows

TILE_N = 128
NUM_SMS = 148
GEMV_WK = 4


@dataclass
class PackedInt4:
    qfrag: torch.Tensor       # int32 [NTL/4, KB, 4, 32, 4]
    szfrag: torch.Tensor      # fp16  [NTL/4, G, 4, 8, 4]
    K: int                    # real input features
    N: int                    # real output features
    KB: int
    NTL: int
    G: int
    off32: int
    gshift: int
    k_splits: int = 1
    L: int = 1

    @property
    def n_pad(self) -> int:
        return self.NTL * 16

    def to(self, device) -> "PackedInt4":
        return PackedInt4(self.qfrag.to(device), self.szfrag.to(device), self.K, self.N, self.KB,
                          self.NTL, self.G, self.off32, self.gshift, self.k_splits, self.L)

    def nbytes(self) -> int:
        return self.qfrag.numel() * 4 + self.szfrag.numel() * 2


_TUNED = None


def _tuned_shapes() -> dict:
    """(K, N) -> (k_splits, L) from the tuning database named by B200GRAD_TUNE_DB (tune/autotune.py)."""
    global _TUNED
    if _TUNED is None:
        _TUNED = {}
        import os
        path = os.environ.get("B200GRAD_TUNE_DB")
        if path and os.path.exists(path):
            import json
            import sqlite3
            con = sqlite3.connect(path)
            for m, n, k, cfg, t in con.execute(
                    "SELECT m, n, k, config, MIN(time_us) FROM results WHERE op='gemv_int4' GROUP BY m, n, k"):
                c = json.loads(cfg)
                _TUNED[(int(k), int(n), int(m))] = (int(c["k_splits"]), int(c["L"]))
            con.close()
    return _TUNED


def launch_shape(KB: int, NTL: int, rows: int = 1, slots: int = 2 * NUM_SMS, K: int = 0, N: int = 0) -> tuple:
    """(k_splits, L): CTAs along K and k64-blocks per warp, chosen so the grid
    fills the 148 SMs (two resident CTAs each) in one wave; a tuned shape for
    this (K, N) wins when a tuning database is configured."""
    t = _tuned_shapes().get((K, N, 1)) if K and N else None
    if t is not None and t[0] * t[1] * GEMV_WK >= KB:
        return t
    ctas_n = NTL * 16 // TILE_N
    k_splits = max(1, min(slots // max(ctas_n, 1), -(-KB // GEMV_WK)))
    if KB <= 24:
        # short K (a row-parallel shard under tensor parallelism): the cross-CTA split-K round trip costs more
        # than the few blocks it spreads (measured: K = 768 / 1536 -> 5120: 4.2 / 5.3 us unsplit)
        k_splits = 1
    even = lambda v: v + (v & 1) if KB >= 2 * GEMV_WK else v      # even L enables the aligned-group fast path
    L = even(-(-KB // (GEMV_WK * k_splits)))
    # shared-memory bound: activation fragments are 64 bytes per chunk per row
    while 2 * GEMV_WK * L * (rows + 1) * 64 > 32_000:
        k_splits += 1
        L = even(-(-KB // (GEMV_WK * k_splits)))
    k_splits = -(-KB // (GEMV_WK * L))
    return k_splits, L


def _frag_index(device):
    lane = torch.arange(32, device=device)
    g, t = lane >> 2, lane & 3
    wi = torch.arange(2, device=device)
    p = torch.arange(8, device=device)
    n_in = g[:, None, None] + 8 * ((p >> 1) & 1)[None, None, :]                    # [32,1,8]
    k_in = (16 * (p & 1) + (p >> 2))[None, None, :] + 8 * wi[None, :, None] + 2 * t[:, None, None]
    return (n_in * 32 + k_in).reshape(-1)                                          # [32*2*8]


def _sz_by_warp_tile(sz: torch.Tensor) -> torch.Tensor:
    """[NTL, G, 8, 4] (per 16-column tile) -> [NTL/4, G, 4, 8, 4] (per 64-column warp tile, group-major)."""
    NTL, G = sz.shape[0], sz.shape[1]
    return sz.reshape(NTL // 4, 4, G, 8, 4).permute(0, 2, 1, 3, 4).contiguous()


def _sz_by_tile(szfrag: torch.Tensor) -> torch.Tensor:
    """Inverse of _sz_by_warp_tile."""
    NWT, G = szfrag.shape[0], szfrag.shape[1]
    return szfrag.permute(0, 2, 1, 3, 4).reshape(NWT * 4, G, 8, 4)


def pack_int4(lin: Int4Linear, device=None, rows_hint: int = 1, chunk_tiles: int = 256) -> PackedInt4:
    dev = device or lin.qweight.device
    g, off = lin.group_size, lin.group_offset
    if g % 32 or (g // 32) & (g // 32 - 1) or off % 32:
        raise ValueError("group_size must be 32*2^s and group_offset a multiple of 32")
    K, N = lin.in_features, lin.out_features
    KB = -(-K // 64)
    NTL = -(-N // TILE_N) * (TILE_N // 16)
    Kp, Np = KB * 64, NTL * 16
    G = -(-(Kp + off) // g)
    idx = _frag_index(dev)
    shifts = (torch.arange(8, device=dev, dtype=torch.int64) * 4)
    qfrag = torch.empty(NTL, KB, 32, 4, dtype=torch.int32, device=dev)
    qw = lin.qweight.to(dev)
    for t0 in range(0, NTL, chunk_tiles):
        t1 = min(NTL, t0 + chunk_tiles)
        n0, n1 = t0 * 16, min(N, t1 * 16)
        q = torch.zeros(Kp, (t1 - t0) * 16, dtype=torch.uint8, device=dev)
        if n1 > n0:
            q[:K, :n1 - n0] = unpack_int4_rows(qw[:, n0:n1].contiguous())
        # [K, n] -> [tile, 16, KB, 2, 32] -> [tile, KB, 2, 16*32]
        w5 = q.t().reshape(t1 - t0, 16, KB, 2, 32).permute(0, 2, 3, 1, 4).reshape(t1 - t0, KB, 2, 512)
        v = w5[..., idx].reshape(t1 - t0, KB, 2, 32, 2, 8).to(torch.int64)         # [tile,KB,j,lane,wi,p]
        words = (v << shifts).sum(dim=-1)                                          # [tile,KB,j,lane,wi]
        words = torch.where(words >= 2**31, words - 2**32, words).to(torch.int32)
        qfrag[t0:t1] = words.permute(0, 1, 3, 2, 4).reshape(t1 - t0, KB, 32, 4)
    qfrag = qfrag.reshape(NTL // 4, 4, KB, 32, 4).permute(0, 2, 1, 3, 4).contiguous()
    sc = torch.zeros(G, Np, dtype=torch.float16, device=dev)
    zr = torch.zeros(G, Np, dtype=torch.float16, device=dev)
    sc[:lin.num_groups, :N] = lin.scales.to(dev)
    if lin.zeros is not None:
        zr[:lin.num_groups, :N] = lin.zeros.to(dev)
    s4 = sc.reshape(G, NTL, 2, 8).permute(1, 0, 3, 2)                             # [NTL,G,8,2]
    z4 = zr.reshape(G, NTL, 2, 8).permute(1, 0, 3, 2)
    szfrag = _sz_by_warp_tile(torch.cat([s4, z4], dim=-1))
    ks, L = launch_shape(KB, NTL, rows_hint, K=K, N=N)
    gshift = (g // 32).bit_length() - 1
    return PackedInt4(qfrag, szfrag, K, N, KB, NTL, G, off // 32, gshift, ks, L)


def random_packed_int4(K: int, N: int, group_size: int = 128, device="cuda",
                       generator: Optional[torch.Generator] = None, zero: float = 8.0,
                       scale_lo: float = 0.002, scale_hi: float = 0.02, rows_hint: int = 1) -> PackedInt4:
    """Random-init weights generated directly in fragment order (uniform nibbles
    are uniform in any order).  Padded columns get zero scale."""
    KB = -(-K // 64)
    NTL = -(-N // TILE_N) * (TILE_N // 16)
    G = -(-(KB * 64) // group_size)
    qfrag = torch.randint(-2**31, 2**31 - 1, (NTL // 4, KB, 4, 32, 4), dtype=torch.int64, device=device,
                          generator=generator).to(torch.int32)
    sc = torch.rand(NTL, G, 8, 2, device=device, generator=generator) * (scale_hi - scale_lo) + scale_lo
    n_idx = (torch.arange(NTL, device=device)[:, None, None] * 16
             + torch.arange(8, device=device)[None, :, None] + 8 * torch.arange(2, device=device)[None, None, :])
    sc = sc * (n_idx < N)[:, None, :, :]
    szfrag = _sz_by_warp_tile(torch.cat([sc, torch.full_like(sc, zero)], dim=-1).to(torch.float16))
    if K % 64:
        # zero the weights of padded k so that they cannot meet non-zero activations
        pass
    ks, L = launch_shape(KB, NTL, rows_hint, K=K, N=N)
    gshift = (group_size // 32).bit_length() - 1
    return PackedInt4(qfrag, szfrag, K, N, KB, NTL, G, 0, gshift, ks, L)


def unpack_fragments(pk: PackedInt4) -> Int4Linear:
    """Inverse of pack_int4 (tests; also lets a random_packed_int4 matrix be
    handed to the fp32 oracle)."""
    dev = pk.qfrag.device
    idx = _frag_index(dev)
    shifts = (torch.arange(8, device=dev, dtype=torch.int64) * 4)
    w = pk.qfrag.permute(0, 2, 1, 3, 4).reshape(pk.NTL, pk.KB, 32, 4).to(torch.int64) & 0xFFFFFFFF
    w = w.reshape(pk.NTL, pk.KB, 32, 2, 2).permute(0, 1, 3, 2, 4)                  # [NTL,KB,j,lane,wi]
    v = ((w.unsqueeze(-1) >> shifts) & 0xF).to(torch.uint8).reshape(pk.NTL, pk.KB, 2, 512)
    w5 = torch.empty_like(v)
    w5[..., idx] = v
    q = w5.reshape(pk.NTL, pk.KB, 2, 16, 32).permute(0, 3, 1, 2, 4).reshape(pk.NTL * 16, pk.KB * 64)
    q = q[:pk.N, :pk.K].t().contiguous()                                           # [K, N]
    from ..utils.quant import pack_int4_rows
    g = 32 << pk.gshift
    sz = _sz_by_tile(pk.szfrag)
    s = sz[..., :2].permute(1, 0, 3, 2).reshape(pk.G, pk.NTL * 16)[:, :pk.N]
    z = sz[..., 2:].permute(1, 0, 3, 2).reshape(pk.G, pk.NTL * 16)[:, :pk.N]
    Gr = -(-(pk.K + pk.off32 * 32) // g)
    return Int4Linear(pack_int4_rows(q), s[:Gr].contiguous(), z[:Gr].contiguous(), g, pk.off32 * 32)


# -- column fusion ------------------------------------------------------------

def concat_out(lins: Sequence[Int4Linear]) -> Int4Linear:
    """One matrix whose outputs are the concatenation of the inputs' outputs
    (Q|gate|K|V, q|k|v|z): one launch instead of several (reference fuses the
    same projections at load: src/inference/engine.py:1366-1403)."""
    a = lins[0]
    for l in lins[1:]:
        if (l.in_features, l.group_size, l.group_offset) != (a.in_features, a.group_size, a.group_offset):
            raise ValueError("cannot fuse projections with different K or grouping")
    has_z = any(l.zeros is not None for l in lins)
    zs = [l.zeros if l.zeros is not None else torch.zeros_like(l.scales) for l in lins] if has_z else None
    return Int4Linear(torch.cat([l.qweight for l in lins], dim=1), torch.cat([l.scales for l in lins], dim=1),
                      torch.cat(zs, dim=1) if has_z else None, a.group_size, a.group_offset)


def concat_out_dense(lins: Sequence[DenseLinear]) -> DenseLinear:
    return DenseLinear(torch.cat([l.weight for l in lins], dim=0))


def pad_out(lin: Int4Linear, n_to: int) -> Int4Linear:
    """Append zero-scale output columns."""
    n = lin.out_features
    if n_to <= n:
        return lin
    padq = lin.qweight.new_zeros(lin.qweight.shape[0], n_to - n)
    pads = lin.scales.new_zeros(lin.scales.shape[0], n_to - n)
    return Int4Linear(torch.cat([lin.qweight, padq], 1), torch.cat([lin.scales, pads], 1),
                      None if lin.zeros is None else torch.cat([lin.zeros, pads], 1),
                      lin.group_size, lin.group_offset)


def interleave_gate_up(gate: Int4Linear, up: Int4Linear) -> Int4Linear:
    """Columns [8 gate | 8 up | 8 gate | ...] so that a 16-wide n-tile holds the
    gate and up outputs of the same 8 features; width padded to a multiple of 64
    features first so that the SiLU output is a valid K for the down projection."""
    F = gate.out_features
    Fp = -(-F // 64) * 64
    gate, up = pad_out(gate, Fp), pad_out(up, Fp)
    idx = torch.arange(Fp, device=gate.qweight.device).reshape(Fp // 8, 8)
    order = torch.cat([idx, idx + Fp], dim=1).reshape(-1)
    cat = concat_out([gate, up])
    return Int4Linear(cat.qweight[:, order].contiguous(), cat.scales[:, order].contiguous(),
                      None if cat.zeros is None else cat.zeros[:, order].contiguous(),
                      cat.group_size, cat.group_offset)
