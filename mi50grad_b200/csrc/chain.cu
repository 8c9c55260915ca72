// Persistent projection chain for the decode step (1..8 token rows), sm_100a.
//
// One launch runs up to four dependent INT4 projections back to back, e.g.
//   out_proj (+residual) -> gate/up (+SiLU) -> down (+residual) -> next layer's in-projection,
// which the stand-alone GEMV path issues as four kernels.  The reference issues
// every projection as its own launch from a C loop (reference:
// src/runtime/c_dispatch.c:975-1213) and only sketched a persistent kernel
// (reference: src/kernels/persistent_decode.hip:271-468).
//
// Why one kernel: a decode step streams weights once and is bound by HBM, but a
// short launch never reaches HBM speed: it ramps up, drains its pipeline at the
// end, and its successor cannot read a byte it depends on until then.  Here
//  * one CTA per SM stays resident; each of its warps owns a contiguous slice
//    of every projection's weights and pulls it through a private shared-memory
//    ring with bulk asynchronous copies (cp.async.bulk + mbarrier, one
//    instruction per 4 KB).  Weights depend on nothing, so the ring keeps
//    filling across the boundaries between projections: while the grid waits
//    for the last tile of projection i, ~20 MB of projection i+1 is already
//    on chip and HBM never idles;
//  * the weights of a projection are one linear sequence of 2 KB units
//    (64 output columns x 64 k); warp w of the grid takes units [w U, (w+1) U),
//    so every SM streams the same number of bytes whatever the matrix shape;
//  * a warp's slice of one 64-column tile is a split-K "piece": pieces go to an
//    L2-resident scratch, the warp that delivers the last piece of a tile sums
//    them in a fixed order (deterministic) and runs the epilogue for the tile;
//  * dependencies are counters in global memory: a projection's consumers wait
//    until all of its tiles are complete.  Every wait is time-bounded and
//    reports through CommCtx::status;
//  * under tensor parallelism the warp that completes a tile of a row-parallel
//    projection stores it into every peer's staging area (plain peer stores
//    over NVLink), raises that tile's flag on the peer, waits for the peers'
//    copies of the same tile and adds them up in rank order.  All tiles are
//    exchanged concurrently by the warps that finish them; there is no
//    grid-wide collection point and no serial tail.
#include <cstdlib>
#include <cstring>
#include "chain.cuh"

// ---------------------------------------------------------------------------
// small PTX helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ch_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ch_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void ch_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool ch_mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait for a weight copy to land.
__device__ __forceinline__ bool ch_mbar_wait(uint32_t bar, uint32_t parity, long long budget_ns) {
    if (ch_mbar_try_wait(bar, parity)) return true;
    const long long t0 = globaltimer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (ch_mbar_try_wait(bar, parity)) return true;
        if (globaltimer_ns() - t0 > budget_ns) return false;
    }
}
__device__ __forceinline__ void ch_bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t ch_ld_acquire_gpu(const int* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void ch_mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t ch_nib_lo(uint32_t w) {      // halves: 1024 + q
    uint32_t r;
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(r) : "r"(w));
    return r;
}
__device__ __forceinline__ uint32_t ch_nib_hi(uint32_t w) {      // halves: 1024 + 16 q
    uint32_t r;
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(r) : "r"(w));
    return r;
}

// ---------------------------------------------------------------------------
// Work split.  A projection's weights are NWT * KB units of 2 KB; units are
// handed out in granules of `gsz` units (2 = one k128 quantisation group when KB
// is even) in two levels: granules are spread evenly over the CTAs (so every SM
// streams the same number of bytes, +-1 granule), and a CTA's share evenly over
// its warps.  Slice s = cta * CH_WARPS + warp; slices are contiguous and
// ascending in s, some may be empty.
// ---------------------------------------------------------------------------
struct ChSlice { int g0, g1; };

__device__ __forceinline__ ChSlice ch_slice(const ChainOp& op, int s) {
    const int cta = s / CH_WARPS, warp = s % CH_WARPS;
    const int n_c = op.cBase + (cta < op.cRem ? 1 : 0);
    const int start = cta * op.cBase + (cta < op.cRem ? cta : op.cRem);
    const int wB = n_c / CH_WARPS, wR = n_c % CH_WARPS;
    ChSlice r;
    r.g0 = start + warp * wB + (warp < wR ? warp : wR);
    r.g1 = r.g0 + wB + (warp < wR ? 1 : 0);
    return r;
}
// The slice that holds granule g.
__device__ __forceinline__ int ch_slice_of(const ChainOp& op, int g) {
    const int lim = op.cRem * (op.cBase + 1);
    const int cta = g < lim ? g / (op.cBase + 1) : op.cRem + (g - lim) / op.cBase;
    const int n_c = op.cBase + (cta < op.cRem ? 1 : 0);
    const int start = cta * op.cBase + (cta < op.cRem ? cta : op.cRem);
    const int wB = n_c / CH_WARPS, wR = n_c % CH_WARPS;
    const int off = g - start, lim2 = wR * (wB + 1);
    const int warp = off < lim2 ? off / (wB + 1) : wR + (off - lim2) / wB;
    return cta * CH_WARPS + warp;
}

// Position of a warp inside its slice of one projection.
struct ChCursor {
    int o;        // projection
    int wt;       // 64-column warp tile
    int kb;       // k64-block inside the tile
    int left;     // units left in this warp's slice of projection o
};

__device__ __forceinline__ bool ch_cursor_set(ChCursor& c, const ChainOp& op, int gw) {
    const ChSlice sl = ch_slice(op, gw);
    if (sl.g1 <= sl.g0) { c.left = 0; return false; }
    const int u0 = sl.g0 * op.gsz;
    c.wt = u0 / op.KB;
    c.kb = u0 - c.wt * op.KB;
    c.left = (sl.g1 - sl.g0) * op.gsz;
    return true;
}
__device__ __forceinline__ void ch_cursor_enter(ChCursor& c, const ChainParams& p, int gw) {
    // skip projections in which this warp has no units
    while (c.o < p.n_ops) {
        if (ch_cursor_set(c, p.op[c.o], gw)) return;
        ++c.o;
    }
    c.left = 0;
}
__device__ __forceinline__ int ch_cursor_blocks(const ChCursor& c, int KB) {
    int n = KB - c.kb;
    n = n < c.left ? n : c.left;
    return n < 2 ? n : 2;
}
__device__ __forceinline__ void ch_fence_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
// {value, tag} pairs: written with one 8-byte store, polled with loads that go to L2 every time.
__device__ __forceinline__ float2 ch_ld_pair(const float2* p) {
    float2 v;
    asm volatile("ld.volatile.global.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ch_ld_pair2(const float2* p) {     // two adjacent pairs (16-byte aligned)
    float4 v;
    asm volatile("ld.volatile.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint2 ch_ld_upair(const uint2* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void ch_st_pair(float2* p, float v, uint32_t tag) {
    asm volatile("st.volatile.global.v2.f32 [%0], {%1,%2};" :: "l"(p), "f"(v), "f"(__uint_as_float(tag)) : "memory");
}
// Poll one pair until its tag matches (bounded).  Returns false on expiry.
__device__ __forceinline__ bool ch_wait_pair(const float2* p, uint32_t tag, long long budget_ns, float& out) {
    float2 v = ch_ld_pair(p);
    if (__float_as_uint(v.y) != tag) {
        const long long t0 = globaltimer_ns();
        for (;;) {
#pragma unroll 1
            for (int i = 0; i < 32 && __float_as_uint(v.y) != tag; ++i) v = ch_ld_pair(p);
            if (__float_as_uint(v.y) == tag || globaltimer_ns() - t0 > budget_ns) break;
        }
    }
    out = v.x;
    return __float_as_uint(v.y) == tag;
}

// ---------------------------------------------------------------------------
// Activation staging.  Item (chunk cl, quarter tt) is the B fragment of four lanes: fp16 pairs at
// k = 32 cl + 2 tt + {0, 8, 16, 24}; the pairs at +16 and +24 are pre-scaled by 1/16 (they meet the
// high nibbles).  LAZY: x = h * rsqrt(sum(ss)/H + eps) * w formed here.  IT items per thread are
// loaded (or polled, when the input is a tagged hand-off) before any is used.
// ---------------------------------------------------------------------------
template <bool FAST, bool LAZY, int IT>
__device__ __forceinline__ bool ch_stage(const ChainParams& p, const ChainOp& op, int M, int Mpad, uint4* xf, float2* cs,
                                         uint32_t itag, long long wait_ns, int c0, int ncl) {
    // chunks c0 .. c0 + ncl - 1 (modulo the projection's chunk count) are staged at positions 0 .. ncl - 1
    const int tid = threadIdx.x, lane = tid & 31;
    const int items = ncl * 4, nCh = 2 * op.KB;
    auto k_of = [&](int item) -> int {
        int cl = c0 + (item >> 2);
        cl = cl >= nCh ? cl - nCh : cl;
        return cl * 32 + 2 * (item & 3);
    };
    bool ok = true;
    for (int m = 0; m < M; ++m) {
        const __half* xr = LAZY ? nullptr : op.x + (size_t)m * op.ldx;
        const float* hr = LAZY ? op.ln.h + (size_t)m * op.ln.H : nullptr;
        float inv = 0.f;
        for (int base0 = 0; base0 < items; base0 += CH_THREADS * IT) {
            float2 hv[LAZY ? IT : 1][4];
            uint32_t xv16[LAZY ? 1 : IT][4];
            const bool tagged = LAZY ? op.th_in != nullptr : op.tact_in != nullptr;
            unsigned long long need = 0;
#pragma unroll
            for (int it = 0; it < IT; ++it) {
                const int item = base0 + it * CH_THREADS + tid;
                const int k0 = k_of(item);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int k = k0 + 8 * q;
                    const bool in = item < items && k < op.K;
                    if (LAZY) hv[it][q] = make_float2(0.f, 0.f); else xv16[it][q] = 0u;
                    if (!in) continue;
                    if (tagged) need |= 1ull << (it * 4 + q);
                    else if (LAZY) hv[it][q] = __ldcg((const float2*)(hr + k));
                    else xv16[it][q] = __ldcg((const uint32_t*)(xr + k));
                }
            }
            // tagged input: poll until every pair carries this launch's tag of the producing projection
            long long t0 = 0;
            while (need) {
#pragma unroll
                for (int it = 0; it < IT; ++it) {
                    const int item = base0 + it * CH_THREADS + tid;
                    const int k0 = k_of(item);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        if (need & (1ull << (it * 4 + q))) {
                            const int k = k0 + 8 * q;
                            if (LAZY) {
                                const float4 v = ch_ld_pair2(op.th_in + (size_t)m * p.tag_h_cols + k);
                                if (__float_as_uint(v.y) == itag && __float_as_uint(v.w) == itag) {
                                    hv[it][q] = make_float2(v.x, v.z);
                                    need &= ~(1ull << (it * 4 + q));
                                }
                            } else {
                                const uint2 v = ch_ld_upair(op.tact_in + (size_t)m * p.tag_act_cols + k / 2);
                                if (v.y == itag) { xv16[it][q] = v.x; need &= ~(1ull << (it * 4 + q)); }
                            }
                        }
                    }
                }
                if (need) {
                    if (t0 == 0) t0 = globaltimer_ns();
                    else if (globaltimer_ns() - t0 > wait_ns) { ok = false; break; }
                }
            }
            if (LAZY && base0 == 0) {
                // every warp forms 1/rms of the row itself: no block-wide hand-off in front of the loads
                float s = 0.f;
                for (int i0 = 0; i0 < op.ln.np; i0 += 128) {
                    float v[4];
                    float2 pv[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int i = i0 + u * 32 + lane;
                        v[u] = 0.f;
                        pv[u] = make_float2(0.f, __uint_as_float(itag));
                        if (i < op.ln.np) {
                            if (op.tss_in) pv[u] = ch_ld_pair(op.tss_in + (size_t)m * p.tag_ss_cols + i);
                            else v[u] = __ldcg(op.ln.ss + (size_t)m * op.ln.np + i);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int i = i0 + u * 32 + lane;
                        if (op.tss_in && i < op.ln.np) {
                            if (__float_as_uint(pv[u].y) == itag) v[u] = pv[u].x;
                            else if (!ch_wait_pair(op.tss_in + (size_t)m * p.tag_ss_cols + i, itag, wait_ns, v[u])) ok = false;
                        }
                        s += v[u];
                    }
                }
                s = warp_sum(s);
                inv = rsqrtf(s / (float)op.ln.H + op.ln.eps);
            }
#pragma unroll
            for (int it = 0; it < IT; ++it) {
                const int item = base0 + it * CH_THREADS + tid;
                const bool valid = item < items;
                const int tt = item & 3, cl = item >> 2;      // cl: position in the staged window
                const int k0 = k_of(item);
                __half2 v[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    if (LAZY) {
                        const int k = k0 + 8 * q;
                        float2 wv = make_float2(0.f, 0.f);
                        if (valid && k < op.K) wv = __half22float2(*(const __half2*)(op.ln.w + k));
                        v[q] = __floats2half2_rn(hv[it][q].x * inv * wv.x, hv[it][q].y * inv * wv.y);
                    } else {
                        v[q] = *(__half2*)&xv16[it][q];
                    }
                }
                const __half2 sixteenth = __float2half2_rn(0.0625f);
                v[2] = __hmul2(v[2], sixteenth);
                v[3] = __hmul2(v[3], sixteenth);
                float2 fa0 = __half22float2(v[0]), fa1 = __half22float2(v[1]);
                float2 fb0 = __half22float2(v[2]), fb1 = __half22float2(v[3]);
                float sa = fa0.x + fa0.y + fa1.x + fa1.y;
                float sb = fb0.x + fb0.y + fb1.x + fb1.y;
                sa += __shfl_xor_sync(0xffffffffu, sa, 1);
                sb += __shfl_xor_sync(0xffffffffu, sb, 1);
                sa += __shfl_xor_sync(0xffffffffu, sa, 2);
                sb += __shfl_xor_sync(0xffffffffu, sb, 2);
                if (FAST) {
                    // a group is four consecutive chunks = sixteen consecutive lanes
                    sa += __shfl_xor_sync(0xffffffffu, sa, 4);
                    sb += __shfl_xor_sync(0xffffffffu, sb, 4);
                    sa += __shfl_xor_sync(0xffffffffu, sa, 8);
                    sb += __shfl_xor_sync(0xffffffffu, sb, 8);
                }
                if (valid) {
                    uint4 w4;
                    w4.x = *(uint32_t*)&v[0]; w4.y = *(uint32_t*)&v[1]; w4.z = *(uint32_t*)&v[2]; w4.w = *(uint32_t*)&v[3];
                    xf[((size_t)cl * M + m) * 4 + tt] = w4;
                    if (FAST) {
                        if ((item & 15) == 0) cs[(size_t)(cl >> 2) * Mpad + m] = make_float2(1024.f * (sa + sb), sa + 16.f * sb);
                    } else if (tt == 0) {
                        cs[(size_t)cl * Mpad + m] = make_float2(1024.f * (sa + sb), sa + 16.f * sb);
                    }
                }
            }
        }
    }
    return ok;
}

// Poll N pairs at once: all loads are issued before any tag is checked.
template <int N>
__device__ __forceinline__ bool ch_wait_pairs(const float2* const (&ptr)[N], const bool (&want)[N], uint32_t tag,
                                              long long budget_ns, float (&out)[N]) {
    float2 v[N];
    unsigned need = 0;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        v[i] = make_float2(0.f, 0.f);
        if (want[i]) v[i] = ch_ld_pair(ptr[i]);
    }
#pragma unroll
    for (int i = 0; i < N; ++i) {
        if (want[i] && __float_as_uint(v[i].y) != tag) need |= 1u << i;
        out[i] = v[i].x;
    }
    if (!need) return true;
    const long long t0 = globaltimer_ns();
    for (;;) {
#pragma unroll
        for (int i = 0; i < N; ++i) {
            if (need & (1u << i)) {
                const float2 w = ch_ld_pair(ptr[i]);
                if (__float_as_uint(w.y) == tag) { out[i] = w.x; need &= ~(1u << i); }
            }
        }
        if (!need) return true;
        if (globaltimer_ns() - t0 > budget_ns) return false;
    }
}

// ---------------------------------------------------------------------------
// Epilogue of one finished 64-column tile.  Lane l holds, for every token row m,
// columns ca = 16 (l>>3) + (l&7) and cb = ca + 8 of the tile in ya[m], yb[m]
// (a gate/up pair when the projection is the interleaved gate|up matrix).
// Returns false if a peer's tile did not arrive in time.
// ---------------------------------------------------------------------------
template <int MT>
__device__ __forceinline__ bool ch_epilogue(const ChainParams& p, const ChainOp& op, int o, int wt, int lane,
                                            float (&ya)[MT], float (&yb)[MT], uint32_t epoch, uint32_t gen4,
                                            long long wait_ns) {
    const GemvEpi& e = op.epi;
    const int M = MT == 1 ? 1 : p.rows;
    const int n0 = wt * 64;
    const int ca = n0 + 16 * (lane >> 3) + (lane & 7), cb = ca + 8;
    const uint32_t otag = gen4 + (uint32_t)o + 1u;                     // tag of this op's outputs in this launch
    bool ok = true;
    if (e.mode == EPI_STORE_F16) {
        __half* out = (__half*)e.out;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < M) {
                if (ca < e.n_valid) out[(size_t)m * e.ldo + ca] = __float2half(ya[m]);
                if (cb < e.n_valid) out[(size_t)m * e.ldo + cb] = __float2half(yb[m]);
            }
        }
    } else if (e.mode == EPI_STORE_F32) {
        float* out = (float*)e.out;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < M) {
                if (ca < e.n_valid) out[(size_t)m * e.ldo + ca] = ya[m];
                if (cb < e.n_valid) out[(size_t)m * e.ldo + cb] = yb[m];
            }
        }
    } else if (e.mode == EPI_SILU_PAIR) {
        __half* out = (__half*)e.out;
        const int o = n0 / 2 + 8 * (lane >> 3) + (lane & 7);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < M) {
                const __half v = __float2half(silu_f(ya[m]) * yb[m]);
                if (o < e.n_valid) out[(size_t)m * e.ldo + o] = v;
                if (op.tact_out) {
                    // the consumer reads fp16 pairs: even lanes store {pair, tag} for themselves and their neighbour
                    const unsigned short mine = __half_as_ushort(v);
                    const unsigned short next = (unsigned short)__shfl_down_sync(0xffffffffu, (unsigned)mine, 1);
                    if (!(lane & 1) && o < e.n_valid) {
                        uint2 pr;
                        pr.x = (uint32_t)mine | ((uint32_t)next << 16); pr.y = otag;
                        asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};"
                                     :: "l"(op.tact_out + (size_t)m * p.tag_act_cols + o / 2), "r"(pr.x), "r"(pr.y) : "memory");
                    }
                }
            }
        }
    } else {   // EPI_FINISH
        const CommCtx& c = p.comm;
        const bool va = ca < e.n_valid, vb = cb < e.n_valid;
        const bool local = (e.fin_flags & FIN_NO_COMM) || c.tp <= 1;
        // the residual stream does not depend on this projection: fetch it before anything is waited for
        float hra[MT], hrb[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            hra[m] = hrb[m] = 0.f;
            if (m < M) {
                if (op.th_res) {
                    const uint32_t rtag = gen4 + (uint32_t)op.res_op + 1u;
                    const float2* const ptr[2] = {op.th_res + (size_t)m * p.tag_h_cols + ca, op.th_res + (size_t)m * p.tag_h_cols + cb};
                    const bool want[2] = {va, vb};
                    float got[2];
                    ok = ch_wait_pairs<2>(ptr, want, rtag, wait_ns, got) && ok;
                    hra[m] = got[0]; hrb[m] = got[1];
                } else {
                    if (va) hra[m] = __ldcg(e.h + (size_t)m * e.n_valid + ca);
                    if (vb) hrb[m] = __ldcg(e.h + (size_t)m * e.n_valid + cb);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < M) {
                const size_t off = (size_t)m * e.n_valid;
                if (e.fin_flags & FIN_ADD_EXTRA) {
                    if (va) ya[m] += __ldcg(e.extra + off + ca);
                    if (vb) yb[m] += __ldcg(e.extra + off + cb);
                }
                if (e.fin_flags & FIN_SAVE_EXTRA) {
                    if (va) e.extra[off + ca] = ya[m];
                    if (vb) e.extra[off + cb] = yb[m];
                }
            }
        }
        if (e.fin_flags & FIN_SAVE_EXTRA) __threadfence();   // `extra` is read by a later op of this launch: before any tag
        if (!local) {
            // ---- exchange this tile: every value goes to every peer as a {value, epoch} pair in one 8-byte
            // store over NVLink; the peers' copies are polled in place and added in rank order (every rank
            // forms the same sum).  No flag, no fence: the data is its own arrival signal.
            const size_t par = (size_t)(epoch & 1) * c.tp * B2_MAX_ROWS * c.tile_h;
            const size_t mine = par + (size_t)c.rank * B2_MAX_ROWS * c.tile_h;
            if (!(e.fin_flags & FIN_TEST_WITHHOLD_SIGNAL)) {
#pragma unroll
                for (int pr = 0; pr < B2_MAX_TP; ++pr) {
                    if (pr < c.tp && pr != c.rank) {
                        float2* dst = c.tpart[pr] + mine;
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            if (m < M) {
                                if (va) ch_st_pair(dst + (size_t)m * c.tile_h + ca, ya[m], epoch);
                                if (vb) ch_st_pair(dst + (size_t)m * c.tile_h + cb, yb[m], epoch);
                            }
                        }
                    }
                }
            }
            const float2* src = c.tpart[c.rank] + par;
            int late = -1;
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                if (m < M) {
                    // the peers' copies of this row are polled together, then added in rank order
                    const float2* ptr[2 * B2_MAX_TP];
                    bool want[2 * B2_MAX_TP];
                    float got[2 * B2_MAX_TP];
#pragma unroll
                    for (int pr = 0; pr < B2_MAX_TP; ++pr) {
                        const float2* q = src + ((size_t)(pr < c.tp ? pr : 0) * B2_MAX_ROWS + m) * c.tile_h;
                        ptr[2 * pr] = q + ca; ptr[2 * pr + 1] = q + cb;
                        want[2 * pr] = pr < c.tp && pr != c.rank && va;
                        want[2 * pr + 1] = pr < c.tp && pr != c.rank && vb;
                    }
                    if (late < 0 && !ch_wait_pairs<2 * B2_MAX_TP>(ptr, want, epoch, wait_ns, got)) late = c.rank == 0 ? 1 : 0;
                    float sa = 0.f, sb = 0.f;
#pragma unroll
                    for (int pr = 0; pr < B2_MAX_TP; ++pr) {
                        if (pr < c.tp) {
                            sa += pr == c.rank ? ya[m] : got[2 * pr];
                            sb += pr == c.rank ? yb[m] : got[2 * pr + 1];
                        }
                    }
                    if (late < 0) { ya[m] = sa; yb[m] = sb; }
                }
            }
            if (late >= 0) { report_timeout(c, B2_KID_CHAIN_TILE, late, epoch); ok = false; }
            ok = __all_sync(0xffffffffu, ok);
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < M) {
                const size_t off = (size_t)m * e.n_valid;
                float ha = 0.f, hb = 0.f;
                if (va) { ha = hra[m] + ya[m]; e.hout[off + ca] = ha; }
                if (vb) { hb = hrb[m] + yb[m]; e.hout[off + cb] = hb; }
                if (op.th_out) {
                    if (va) ch_st_pair(op.th_out + (size_t)m * p.tag_h_cols + ca, ha, otag);
                    if (vb) ch_st_pair(op.th_out + (size_t)m * p.tag_h_cols + cb, hb, otag);
                }
                const float tot = warp_sum(ha * ha + hb * hb);
                if (lane == 0) {
                    e.ss_part[(size_t)m * e.ss_np + wt] = tot;
                    if (op.tss_out) ch_st_pair(op.tss_out + (size_t)m * p.tag_ss_cols + wt, tot, otag);
                }
            }
        }
    }
    return ok;
}

// ---------------------------------------------------------------------------
// The kernel.  MT: compile-time bound of the token rows (1, or B2_MAX_ROWS).
// FAST: every projection has groups of 128 k aligned to its k64-block pairs, so
// a ring stage is exactly one quantisation group and the loop carries no group
// bookkeeping.
// ---------------------------------------------------------------------------
#define CH_HDR_BYTES (CH_WARPS * CH_MAX_STAGES * 8 + 128)   // mbarriers, then per-segment arrival counts and the abort flag
#define CH_STAGE_IT 4          // activation items per thread whose loads are in flight together
#define CH_W_BYTES 4096        // weights of a stage: two k64-blocks of a warp tile
#define CH_SZ_BYTES 256        // scale/zero pairs of one quantisation group of a warp tile

template <int MT, bool FAST>
__global__ void __launch_bounds__(CH_THREADS, MT == 1 ? 2 : 1) chain_kernel(const __grid_constant__ ChainParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int M = MT == 1 ? 1 : p.rows, Mpad = (M + 1) & ~1;
    const int NST = p.stages;
    const int cta = blockIdx.x;
    const int gw = cta * CH_WARPS + warp;
    const long long wait_ns = p.comm.wait_ns > 0 ? p.comm.wait_ns : 2000000000ll;
    const int la = 16 * (lane >> 3) + (lane & 7);                      // this lane's columns in an epilogue: la, la + 8
    const int g_eff = g < M ? g : 0;                                   // token row this lane feeds to the MMA (rows >= M: ignored)

    // ---- shared memory carve-up (offsets match b2_chain's size computation)
    const int maxCh = p.xf_chunks;                                     // widest staged window of any projection (32-k chunks)
    uint64_t* bars = (uint64_t*)smem;                                  // [CH_WARPS][CH_MAX_STAGES]
    int* seg_cnt = (int*)(smem + CH_HDR_BYTES - 128);                  // [CH_WARPS] arrivals per shared tile segment
    int* s_abort = (int*)(smem + CH_HDR_BYTES - 64);
    float* part = (float*)(smem + CH_HDR_BYTES);                       // [2 * CH_WARPS][M][64] partial tiles of the warps
    unsigned char* ptr = smem + CH_HDR_BYTES + (size_t)2 * CH_WARPS * M * 256;
    uint4* xf = (uint4*)ptr;                                           // [maxCh][M][4]
    ptr += (size_t)maxCh * M * 4 * 16;
    float2* cs = (float2*)ptr;                                         // [maxCh (FAST: groups)][Mpad] (+ slack)
    ptr += ((size_t)maxCh * Mpad + 8) * 8;
    ptr = (unsigned char*)(((uintptr_t)ptr + 127) & ~(uintptr_t)127);
    unsigned char* ring = ptr + (size_t)warp * NST * CH_STAGE_BYTES;   // stage: [4096 weights][<= 4 x 256 scale/zero]
    const uint32_t bar0 = ch_smem_u32(bars + warp * CH_MAX_STAGES);
    const uint32_t ring0 = ch_smem_u32(ring);

    if (tid == 0) *s_abort = 0;
    if (tid < CH_WARPS) seg_cnt[tid] = 0;
    if (lane == 0) {
        for (int s = 0; s < NST; ++s) ch_mbar_init(bar0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    // ---- weight ring: the issue cursor runs NST stages ahead of the consume cursor, across projections.
    // A stage carries two k64-blocks of weights and the scale/zero pairs of every group they touch.
    ChCursor ic;
    ic.o = 0; ic.wt = ic.kb = ic.left = 0;
    ch_cursor_enter(ic, p, gw);
    int issued = 0, consumed = 0;
    int islot = 0, cslot = 0;                // issued % NST, consumed % NST
    uint32_t cphase = 0;                     // (consumed / NST) & 1
    auto issue_one = [&]() {
        if (ic.o >= p.n_ops) return;
        const ChainOp& op = p.op[ic.o];
        const int n = FAST ? 2 : ch_cursor_blocks(ic, op.KB);
        if (lane == 0) {
            int g_lo, ng;
            if (FAST) { g_lo = ic.kb >> 1; ng = 1; }
            else {
                g_lo = (2 * ic.kb + op.off32) >> op.gshift;
                ng = ((2 * (ic.kb + n) - 1 + op.off32) >> op.gshift) - g_lo + 1;
            }
            const uint32_t wbytes = (uint32_t)n * 2048u, sbytes = (uint32_t)ng * CH_SZ_BYTES;
            const uint32_t dst = ring0 + islot * CH_STAGE_BYTES, bar = bar0 + 8 * islot;
            ch_mbar_expect_tx(bar, wbytes + sbytes);
            ch_bulk_g2s(dst, op.qfrag + ((size_t)ic.wt * op.KB + ic.kb) * 128, wbytes, bar);
            ch_bulk_g2s(dst + CH_W_BYTES, op.szfrag + ((size_t)ic.wt * op.G + g_lo) * 32, sbytes, bar);
        }
        ++issued;
        islot = islot + 1 == NST ? 0 : islot + 1;
        ic.kb += n; ic.left -= n;
        if (ic.kb == op.KB) { ic.kb = 0; ++ic.wt; }
        if (ic.left == 0) { ++ic.o; ch_cursor_enter(ic, p, gw); }
    };
    for (int s = 0; s < NST; ++s) issue_one();
    pdl_launch_dependents();

    uint32_t epoch0 = 0, gen4 = 0;
    int n_exchanged = 0;          // exchanges of projections before the current one
    bool failed = false;

    for (int o = 0; o < p.n_ops; ++o) {
        const ChainOp& op = p.op[o];
        // ---- the first projection reads what earlier kernels wrote; the others poll the tagged values
        // their producer leaves behind, so there is no grid-wide wait between projections
        if (o == 0) {
            pdl_wait();
            if (p.comm.tp > 1) epoch0 = *(volatile uint32_t*)p.comm.epoch;
            gen4 = ((volatile unsigned int*)p.counters)[1] << 2;
        }
        long long* pr = p.prof ? p.prof + ((size_t)gw * CH_MAX_OPS + o) * 8 : nullptr;
        long long cyc_wait = 0, cyc_fin = 0, n_stage = 0, cyc_issue = 0;
        if (pr && lane == 0) pr[0] = globaltimer_ns();
        const bool exchanges = op.epi.mode == EPI_FINISH && p.comm.tp > 1 && !(op.epi.fin_flags & FIN_NO_COMM);
        const uint32_t epoch = epoch0 + 1u + (uint32_t)n_exchanged;

        // ---- stage the activations in MMA B-fragment order, with the bias sums per 32-k chunk (FAST: per
        // group of four chunks); all loads of a pass are in flight together
        const int nCh = 2 * op.KB;
        // a CTA without a share of this projection reads none of its input; one whose share is shorter than
        // a tile's K stages only the window of k it will meet (it may wrap around the end of K)
        const bool has_share = op.cBase + (cta < op.cRem ? 1 : 0) > 0;
        int win0 = 0, win_n = nCh;
        {
            const int nc = op.cBase + (cta < op.cRem ? 1 : 0);
            const int u0 = (cta * op.cBase + (cta < op.cRem ? cta : op.cRem)) * op.gsz, un = nc * op.gsz;
            if (un < op.KB) { win0 = 2 * (u0 % op.KB); win_n = 2 * un; }
        }
        if (has_share) {
            const uint32_t itag = gen4 + (uint32_t)op.in_op + 1u;
            bool staged;
            if (op.ln.h) staged = ch_stage<FAST, true, 3>(p, op, M, Mpad, xf, cs, itag, wait_ns, win0, win_n);
            else staged = ch_stage<FAST, false, 5>(p, op, M, Mpad, xf, cs, itag, wait_ns, win0, win_n);
            if (!staged) *s_abort = 1;
        }
        if (Mpad != M)
            for (int cl = tid; cl < (FAST ? win_n / 4 : win_n); cl += CH_THREADS) cs[(size_t)cl * Mpad + M] = make_float2(0.f, 0.f);
        __syncthreads();
        if (pr && lane == 0) pr[1] = globaltimer_ns();

        // ---- this CTA's and this warp's share of the projection (units)
        const int n_c = op.cBase + (cta < op.cRem ? 1 : 0);
        const int c_start = cta * op.cBase + (cta < op.cRem ? cta : op.cRem);            // granules
        const int cu0 = c_start * op.gsz, cu1 = (c_start + n_c) * op.gsz;
        const int wB = n_c / CH_WARPS, wR = n_c % CH_WARPS;
        auto warp_of = [&](int gran) -> int {                       // warp of this CTA that holds granule `gran`
            const int off = gran - c_start, lim2 = wR * (wB + 1);
            return off < lim2 ? off / (wB + 1) : wR + (off - lim2) / wB;
        };
        auto warp_start = [&](int w) -> int {                       // first unit of warp w's slice
            return (c_start + w * wB + (w < wR ? w : wR)) * op.gsz;
        };
        ChCursor cc;
        cc.o = o; cc.left = 0; cc.wt = cc.kb = 0;
        ch_cursor_set(cc, op, gw);
        float accl[4][4], acch[4][4], tot[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int r = 0; r < 4; ++r) accl[i][r] = acch[i][r] = tot[i][r] = 0.f;
        float c1r0 = 0.f, c1r1 = 0.f, c2r0 = 0.f, c2r1 = 0.f;
        int cur = -1;
        uint2 szc[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) szc[i] = make_uint2(0u, 0u);
        const uint4* xfl = xf + (size_t)g_eff * 4 + t;               // this lane's B-fragment words: xfl[cl * M * 4]

        while (cc.left > 0 && !failed) {
            const int n = FAST ? 2 : ch_cursor_blocks(cc, op.KB);
            const long long c0 = pr ? clock64() : 0;
            const bool landed = ch_mbar_wait(bar0 + 8 * cslot, cphase, wait_ns);
            if (pr) { cyc_wait += clock64() - c0; ++n_stage; }
            if (!landed) {
                if (lane == 0 && p.comm.status &&
                    atomicCAS(p.comm.status, B2_STATUS_OK, B2_STATUS_WAIT_TIMEOUT) == B2_STATUS_OK) {
                    p.comm.status[1] = B2_KID_CHAIN_COPY; p.comm.status[2] = o; p.comm.status[3] = (int)blockIdx.x;
                }
                failed = true;
                *s_abort = 1;
                break;
            }
            const uint4* rp = (const uint4*)(ring + (size_t)cslot * CH_STAGE_BYTES) + lane;
            const uint2* szs = (const uint2*)(ring + (size_t)cslot * CH_STAGE_BYTES + CH_W_BYTES) + g;
            auto flush = [&]() {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float2 s = __half22float2(*(__half2*)&szc[i].x), z = __half22float2(*(__half2*)&szc[i].y);
                    tot[i][0] += s.x * (accl[i][0] + acch[i][0] - c1r0 - z.x * c2r0);
                    tot[i][1] += s.x * (accl[i][1] + acch[i][1] - c1r1 - z.x * c2r1);
                    tot[i][2] += s.y * (accl[i][2] + acch[i][2] - c1r0 - z.y * c2r0);
                    tot[i][3] += s.y * (accl[i][3] + acch[i][3] - c1r1 - z.y * c2r1);
#pragma unroll
                    for (int r = 0; r < 4; ++r) accl[i][r] = acch[i][r] = 0.f;
                }
                c1r0 = c1r1 = c2r0 = c2r1 = 0.f;
            };
            auto mma_chunk = [&](const uint4 (&w)[4], int j, const uint4 xv) {
                // eight independent accumulators per chunk: the tensor pipe's latency overlaps
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t w0 = j ? w[i].z : w[i].x, w1 = j ? w[i].w : w[i].y;
                    ch_mma16816(accl[i], ch_nib_lo(w0), ch_nib_lo(w0 >> 8), ch_nib_lo(w1), ch_nib_lo(w1 >> 8), xv.x, xv.y);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t w0 = j ? w[i].z : w[i].x, w1 = j ? w[i].w : w[i].y;
                    ch_mma16816(acch[i], ch_nib_hi(w0), ch_nib_hi(w0 >> 8), ch_nib_hi(w1), ch_nib_hi(w1 >> 8), xv.z, xv.w);
                }
            };
            if (FAST) {
                // the stage is one group: its scale/zero pairs and bias sums are read once
#pragma unroll
                for (int i = 0; i < 4; ++i) szc[i] = szs[i * 8];
                int rel = 2 * cc.kb - win0;                    // position of the stage's first chunk in the staged window
                rel = rel < 0 ? rel + nCh : rel;
                const float4 cv = *(const float4*)(cs + (size_t)(rel >> 2) * Mpad + 2 * t);
                if (2 * t < Mpad) { c1r0 = cv.x; c2r0 = cv.y; c1r1 = cv.z; c2r1 = cv.w; }
                const uint4* xp = xfl + (size_t)rel * M * 4;
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    uint4 w[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) w[i] = rp[(b * 4 + i) * 32];
#pragma unroll
                    for (int j = 0; j < 2; ++j) mma_chunk(w, j, xp[(size_t)(2 * b + j) * M * 4]);
                }
                flush();
            } else {
                const int g_lo = (2 * cc.kb + op.off32) >> op.gshift;
                for (int b = 0; b < n; ++b) {
                    uint4 w[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) w[i] = rp[(b * 4 + i) * 32];
                    const int cl0 = 2 * (cc.kb + b);
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int cl = cl0 + j;
                        const int grp = (cl + op.off32) >> op.gshift;
                        if (grp != cur) {
                            if (cur >= 0) flush();
                            cur = grp;
                            // scale/zero pairs of a group are taken from the stage in which the group starts
#pragma unroll
                            for (int i = 0; i < 4; ++i) szc[i] = szs[((grp - g_lo) * 4 + i) * 8];
                        }
                        int rel = cl - win0;
                        rel = rel < 0 ? rel + nCh : rel;
                        const float4 cv = *(const float4*)(cs + (size_t)rel * Mpad + 2 * t);
                        if (2 * t < Mpad) { c1r0 += cv.x; c2r0 += cv.y; c1r1 += cv.z; c2r1 += cv.w; }
                        mma_chunk(w, j, xfl[(size_t)rel * M * 4]);
                    }
                }
            }
            // the slot is free once every lane's registers hold its words: refill it
            __syncwarp();
            ++consumed;
            if (++cslot == NST) { cslot = 0; cphase ^= 1u; }
            {
                const long long i0 = pr ? clock64() : 0;
                issue_one();
                if (pr) cyc_issue += clock64() - i0;
            }
            const int wt = cc.wt;
            cc.kb += n; cc.left -= n;
            const bool tile_end = cc.kb == op.KB;
            if (tile_end) { cc.kb = 0; ++cc.wt; }
            if (!tile_end && cc.left > 0) continue;

            // ---- end of this warp's share of tile `wt`
            const long long f0 = pr ? clock64() : 0;
            if (!FAST && cur >= 0) flush();
            cur = -1;
            // level 1: the warps of this CTA that share the tile add up through shared memory; the last
            // of them to arrive carries the CTA's sum on
            const int tb = wt * op.KB, te = tb + op.KB;
            const int sb = tb > cu0 ? tb : cu0, se = te < cu1 ? te : cu1;       // this CTA's units of the tile
            const int wf = warp_of(sb / op.gsz), wl = warp_of((se - 1) / op.gsz);
            const int nw = wl - wf + 1;
            float ya[MT], yb[MT];
            bool carry = true;
            {
                // slot 0: the head of a warp's slice (a tile it shares with the warp before it); slot 1: the
                // tail of its slice, and every tile it holds alone on the way there
                float* mine = part + (size_t)(2 * warp + ((nw > 1 && warp_start(warp) >= tb) ? 0 : 1)) * M * 64;
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const int row = 2 * t + (r & 1), col = 16 * i + g + 8 * (r >> 1);
                        if (row < M) mine[row * 64 + col] = tot[i][r];
                        tot[i][r] = 0.f;
                    }
                if (nw > 1) {
                    __threadfence_block();
                    __syncwarp();
                    int old = 0;
                    if (lane == 0) {
                        old = atomicAdd(&seg_cnt[wf], 1);
                        if (old == nw - 1) seg_cnt[wf] = 0;
                    }
                    old = __shfl_sync(0xffffffffu, old, 0);
                    carry = old == nw - 1;
                    __threadfence_block();
                } else {
                    __syncwarp();
                }
                if (carry) {
#pragma unroll
                    for (int m = 0; m < MT; ++m) ya[m] = yb[m] = 0.f;
                    for (int w2 = wf; w2 <= wl; ++w2) {
                        const volatile float* src = part + (size_t)(2 * w2 + ((nw > 1 && (w2 > wf || warp_start(w2) >= tb)) ? 0 : 1)) * M * 64;
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            if (m < M) {
                                ya[m] += src[m * 64 + la];
                                yb[m] += src[m * 64 + la + 8];
                            }
                        }
                    }
                    __syncwarp();
                }
            }
            // level 2: CTAs that share the tile.  The first of them (which reaches the tile at the end of its
            // share, when the others are done with it) collects the others' sums from the scratch
            if (carry) {
                const int cfirst = ch_slice_of(op, tb / op.gsz) / CH_WARPS, clast = ch_slice_of(op, (te - 1) / op.gsz) / CH_WARPS;
                const int npc = clast - cfirst + 1;
                const uint32_t otag = gen4 + (uint32_t)o + 1u;
                bool epi = true;
                if (npc > 1 && cta != cfirst) {
                    float2* piece = p.scratch + (((size_t)wt * op.pmax + (cta - cfirst)) * M) * 64;
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        if (m < M) { ch_st_pair(piece + m * 64 + la, ya[m], otag); ch_st_pair(piece + m * 64 + la + 8, yb[m], otag); }
                    }
                    epi = false;
                } else if (npc > 1) {
                    const float2* base = p.scratch + ((size_t)wt * op.pmax * M) * 64;
                    bool ok = true;
                    for (int q = 1; q < npc && ok; ++q) {
                        const float2* ptr[2 * MT];
                        bool want[2 * MT];
                        float got[2 * MT];
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            ptr[2 * m] = base + ((size_t)q * M + (m < M ? m : 0)) * 64 + la;
                            ptr[2 * m + 1] = ptr[2 * m] + 8;
                            want[2 * m] = want[2 * m + 1] = m < M;
                        }
                        ok = ch_wait_pairs<2 * MT>(ptr, want, otag, wait_ns, got);
#pragma unroll
                        for (int m = 0; m < MT; ++m)
                            if (m < M) { ya[m] += got[2 * m]; yb[m] += got[2 * m + 1]; }
                    }
                    if (!__all_sync(0xffffffffu, ok)) {
                        if (lane == 0 && p.comm.status && atomicCAS(p.comm.status, B2_STATUS_OK, B2_STATUS_WAIT_TIMEOUT) == B2_STATUS_OK) {
                            p.comm.status[1] = B2_KID_CHAIN_DEP; p.comm.status[2] = o; p.comm.status[3] = (int)blockIdx.x;
                        }
                        *s_abort = 1;
                    }
                }
                if (epi) ch_epilogue<MT>(p, op, o, wt, lane, ya, yb, epoch, gen4, wait_ns);
            }
            if (pr) cyc_fin += clock64() - f0;
        }
        if (pr && lane == 0) { pr[2] = globaltimer_ns(); pr[4] = cyc_wait; pr[5] = cyc_fin; pr[6] = n_stage; pr[7] = cyc_issue; }
        if (exchanges) ++n_exchanged;
        __syncthreads();                      // every warp is done with the staged activations
        if (pr && lane == 0) pr[3] = globaltimer_ns();
        if (*s_abort) { failed = true; break; }
    }

    // ---- leave nothing in flight: wait (bounded) for copies that were issued but not consumed
    while (consumed < issued) {
        if (!ch_mbar_wait(bar0 + 8 * cslot, cphase, wait_ns)) break;
        ++consumed;
        if (++cslot == NST) { cslot = 0; cphase ^= 1u; }
    }
    __syncthreads();
    // ---- the last CTA to leave starts the next launch generation and advances the exchange epoch
    if (tid == 0) {
        __threadfence();
        const unsigned old = atomicAdd(p.counters, 1u);
        if (old == gridDim.x - 1) {
            p.counters[0] = 0;
            p.counters[1] = (gen4 >> 2) + 1u;
            if (p.comm.tp > 1 && n_exchanged > 0) *p.comm.epoch = epoch0 + (uint32_t)n_exchanged;
            __threadfence();
        }
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
static int ch_grid() {
    static int sms[B2_MAX_DEVICES] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= B2_MAX_DEVICES) return 0;
    if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    return sms[dev];
}

// Work split of one projection over `grid` CTAs (see ch_slice).
static void ch_split(ChainOp& op, int grid) {
    op.gsz = (op.KB % 2 == 0) ? 2 : 1;
    const long long TG = (long long)op.NWT * op.KB / op.gsz;
    op.cBase = (int)(TG / grid);
    op.cRem = (int)(TG % grid);
    // pieces of a tile in the scratch: one per CTA that shares it (a non-empty CTA holds at least cBase granules)
    const int KBg = op.KB / op.gsz;
    int pm = KBg / (op.cBase > 0 ? op.cBase : 1) + 2;
    op.pmax = pm < KBg + 1 ? pm : KBg + 1;
}

// Cross-CTA scratch a projection needs ({value, tag} pairs), for the device this is called on.
B2_API long long b2_chain_scratch_floats(int KB, int NWT, int rows) {
    const int sms = ch_grid();
    if (sms <= 0) return 0;
    long long need = 0;
    for (int per = 1; per <= 2; ++per) {          // either grid size may be used, depending on the rows of a launch
        ChainOp op;
        memset(&op, 0, sizeof(op));
        op.KB = KB; op.NWT = NWT;
        ch_split(op, sms * per);
        const long long n = (long long)NWT * op.pmax * rows * 64 * 2;
        need = n > need ? n : need;
    }
    return need;
}
// CTAs per SM of a launch: the one-row kernels fit two (128 registers, half the shared memory each), which
// doubles the warps that hide the loop's latencies; more rows need the registers of one CTA per SM.
static int ch_ctas_per_sm(int rows) { return rows == 1 ? 2 : 1; }
static size_t ch_smem_limit(int rows) { return ch_ctas_per_sm(rows) == 2 ? (size_t)113 * 1024 : (size_t)227 * 1024; }

// Widest window of 32-k chunks any CTA stages (see the kernel: a share shorter than K stages only its k).
static int ch_xf_chunks(const ChainParams* p, int grid) {
    int mx = 0;
    for (int o = 0; o < p->n_ops; ++o) {
        ChainOp t = p->op[o];
        ch_split(t, grid);
        const int un = (t.cBase + (t.cRem > 0 ? 1 : 0)) * t.gsz;
        const int ch = 2 * (un < t.KB ? un : t.KB);
        mx = ch > mx ? ch : mx;
    }
    return mx;
}

static size_t ch_fixed_smem(const ChainParams* p, int grid) {
    const size_t maxCh = (size_t)ch_xf_chunks(p, grid), M = p->rows, Mpad = (M + 1) & ~(size_t)1;
    size_t s = CH_HDR_BYTES + 2 * CH_WARPS * M * 256;
    s += maxCh * M * 4 * 16;
    s += (maxCh * Mpad + 8) * 8;
    return s + 128;                               // alignment slack before the rings
}

static int ch_stages(const ChainParams* p, int grid) {
    const size_t fixed = ch_fixed_smem(p, grid), limit = ch_smem_limit(p->rows);
    if (fixed >= limit) return 0;
    size_t st = (limit - fixed) / ((size_t)CH_WARPS * CH_STAGE_BYTES);
    // B200GRAD_CHAIN_STAGES caps the ring depth (tuning)
    static const int cap = [] { const char* e = getenv("B200GRAD_CHAIN_STAGES"); int v = e ? atoi(e) : 0; return v >= CH_MIN_STAGES && v <= CH_MAX_STAGES ? v : CH_MAX_STAGES; }();
    return (int)(st > (size_t)cap ? (size_t)cap : st);
}

// Wire the hand-off between consecutive projections (each one must read what its predecessor writes)
// and check the shapes.  Returns false if the projections cannot run as one launch.
static bool ch_wire(ChainParams* q) {
    if (q->n_ops < 1 || q->n_ops > CH_MAX_OPS || q->rows < 1 || q->rows > B2_MAX_ROWS) return false;
    if (!q->scratch || !q->counters) return false;
    for (int o = 0; o < q->n_ops; ++o) {
        ChainOp& op = q->op[o];
        if (!op.qfrag || !op.szfrag || op.KB < 1 || op.NWT < 1) return false;
        if (!op.x && !op.ln.h) return false;
        op.th_out = nullptr; op.tss_out = nullptr; op.tact_out = nullptr;
        op.th_in = nullptr; op.tss_in = nullptr; op.tact_in = nullptr; op.th_res = nullptr;
        op.in_op = op.res_op = 0;
        if (op.epi.mode == EPI_FINISH) {
            if (op.epi.ss_np < op.NWT) return false;
            const bool comm = q->comm.tp > 1 && !(op.epi.fin_flags & FIN_NO_COMM);
            if (comm && (q->comm.tile_h < op.epi.n_valid || !q->comm.tpart[0])) return false;
        }
    }
    for (int o = 1; o < q->n_ops; ++o) {
        ChainOp& op = q->op[o];
        ChainOp& prev = q->op[o - 1];
        if (op.ln.h && prev.epi.mode == EPI_FINISH && op.ln.h == prev.epi.hout && op.ln.ss == prev.epi.ss_part) {
            if (!q->tag_h || !q->tag_ss || prev.epi.n_valid > q->tag_h_cols || prev.NWT > q->tag_ss_cols ||
                op.ln.np != prev.NWT || op.ln.H != prev.epi.n_valid || (q->tag_h_cols & 1))
                return false;
            prev.th_out = q->tag_h; prev.tss_out = q->tag_ss;
            op.th_in = q->tag_h; op.tss_in = q->tag_ss; op.in_op = o - 1;
        } else if (op.x && prev.epi.mode == EPI_SILU_PAIR && (const void*)op.x == (const void*)prev.epi.out &&
                   op.ldx == prev.epi.ldo) {
            if (!q->tag_act || (prev.epi.n_valid + 1) / 2 > q->tag_act_cols || op.K > prev.epi.n_valid) return false;
            prev.tact_out = q->tag_act;
            op.tact_in = q->tag_act; op.in_op = o - 1;
        } else {
            return false;
        }
    }
    // a FINISH projection whose residual stream is written earlier in the same launch reads the tagged copy
    for (int o = 1; o < q->n_ops; ++o) {
        ChainOp& op = q->op[o];
        if (op.epi.mode != EPI_FINISH) continue;
        for (int j = o - 1; j >= 0; --j) {
            const ChainOp& w = q->op[j];
            if (w.epi.mode == EPI_FINISH && w.epi.hout == op.epi.h) {
                if (!w.th_out) return false;              // written here but not tagged: cannot be ordered
                // nothing between j and o may overwrite the tagged copy
                for (int k = j + 1; k < o; ++k) if (q->op[k].th_out) return false;
                op.th_res = q->tag_h; op.res_op = j;
                break;
            }
        }
    }
    return true;
}

// 1 if the chain can run as one launch (shapes, shared memory for `rows`), else 0: the caller then
// issues the projections as separate GEMV launches.
B2_API int b2_chain_feasible(const ChainParams* p) {
    ChainParams q = *p;
    const int grid = ch_grid() * ch_ctas_per_sm(p->rows);
    return ch_wire(&q) && grid > 0 && ch_stages(p, grid) >= CH_MIN_STAGES ? 1 : 0;
}

B2_API int b2_chain(const ChainParams* p, cudaStream_t stream) {
    const int per_sm_want = ch_ctas_per_sm(p->rows);
    const int grid = ch_grid() * per_sm_want;
    if (grid <= 0) return cudaErrorInvalidDevice;
    ChainParams q = *p;
    if (!ch_wire(&q)) return cudaErrorInvalidValue;
    q.stages = ch_stages(p, grid);
    q.xf_chunks = ch_xf_chunks(p, grid);
    if (q.stages < CH_MIN_STAGES) return cudaErrorInvalidValue;
    for (int o = 0; o < q.n_ops; ++o) ch_split(q.op[o], grid);
    const size_t smem = ch_fixed_smem(p, grid) + (size_t)CH_WARPS * q.stages * CH_STAGE_BYTES;
    // groups of 128 k aligned to block pairs in every projection: the loop without group bookkeeping
    bool fast = true;
    for (int o = 0; o < q.n_ops; ++o) fast = fast && q.op[o].gshift == 2 && q.op[o].off32 == 0 && q.op[o].KB % 2 == 0;
    const int variant = (q.rows == 1 ? 0 : 2) + (fast ? 1 : 0);
    const void* kern = variant == 0 ? (const void*)chain_kernel<1, false> : variant == 1 ? (const void*)chain_kernel<1, true>
                     : variant == 2 ? (const void*)chain_kernel<B2_MAX_ROWS, false> : (const void*)chain_kernel<B2_MAX_ROWS, true>;
    static SmemOptIn optin[4];
    {
        cudaError_t e = optin[variant].ensure(kern, ch_smem_limit(q.rows));
        if (e != cudaSuccess) return e;
    }
    // the grid's CTAs wait on one another: all of them must be resident at once (one per SM)
    static int resident[4][B2_MAX_DEVICES] = {{0}};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= B2_MAX_DEVICES) return cudaErrorInvalidDevice;
    if (!resident[variant][dev]) {
        int per_sm = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, CH_THREADS, smem);
        if (e != cudaSuccess) return e;
        if (per_sm < per_sm_want) return cudaErrorLaunchOutOfResources;
        resident[variant][dev] = per_sm;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(CH_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    void* args[1] = {(void*)&q};
    return cudaLaunchKernelExC(&cfg, kern, args);
}

B2_API int b2_sizeof_chain_params() { return (int)sizeof(ChainParams); }
B2_API int b2_sizeof_chain_op() { return (int)sizeof(ChainOp); }
