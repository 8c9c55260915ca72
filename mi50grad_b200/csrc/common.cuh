// Shared device helpers for the sm_100a kernels of this package.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define B2_MAX_TP 8
#define B2_MAX_ROWS 8          // token rows one decode-path launch can carry

#define B2_API extern "C" __attribute__((visibility("default")))

// Error/status codes written to CommCtx::status by kernels whose bounded waits expire.
#define B2_STATUS_OK 0
#define B2_STATUS_WAIT_TIMEOUT 1

// ---------------------------------------------------------------------------
// Symmetric-memory communicator as the kernels see it.  Every rank allocates
// the same buffers; part[r] / sig[r] are this process's mappings of rank r's
// copies.  mc_part is the NVSwitch multicast mapping of the partial buffer
// (null when multimem is not used).
// ---------------------------------------------------------------------------
struct CommCtx {
    int tp;                       // ranks
    int rank;                     // this rank
    int part_stride;              // floats per parity half of the partial buffer
    int pad0;
    float* part[B2_MAX_TP];       // [2][part_stride] fp32 partial sums, per rank
    uint32_t* sig[B2_MAX_TP];     // [B2_MAX_TP] arrival words, per rank: sig[dst][src]
    float* mc_part;               // multicast address of part (or null)
    uint32_t* epoch;              // local: number of collective calls completed
    int* status;                  // local: [0]=code [1]=kernel id [2]=peer [3]=epoch
    long long wait_ns;            // bound of every spin-wait
    long long* trace;             // optional [8] globaltimer stamps of the last exchange (null: off)
    // Tile-granular exchange of the persistent chain kernel: every 64-column output tile is pushed
    // to the peers by the warp that completes it and announced with its own flag word.
    float2* tpart[B2_MAX_TP];     // [2][tp][B2_MAX_ROWS][tile_h] {partial, epoch} pairs by (parity, source rank), per rank:
                                  // every value travels with its arrival tag in one 8-byte store
    uint32_t* tsig[B2_MAX_TP];    // reserved
    int tile_h;                   // row length the tile area was sized for (0: no tile area)
    int tile_flags;               // reserved
};

// Device-resident description of one token row of a decode/verify step.  A
// captured CUDA graph reads these instead of host-patched kernel arguments.
struct RowMeta {
    int seq;                      // sequence slot (KV cache / DeltaNet state index)
    int pos;                      // RoPE position
    int slot;                     // KV cache slot this row's K/V is written to
    int ctx;                      // cache slots [0, ctx) are visible to this row
    unsigned long long mask;      // bit j: slot ctx+j is visible (self and draft ancestors)
};

struct SeqState {
    int len;                      // committed tokens in the cache
    int token;                    // last sampled token (input of the next step)
    int pad[2];
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum; `red` needs 32 floats of shared memory.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (l == 0) red[w] = v;
    __syncthreads();
    float t = (l < nw) ? red[l] : 0.f;
    t = warp_sum(t);
    return t;
}

__device__ __forceinline__ uint4 ldg_nc_v4(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ uint2 ldg_nc_v2(const void* p) {
    uint2 r;
    asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
    return r;
}
// Loads that must observe another GPU's (or another CTA's) fresh writes.
// Data loads that follow an acquire of the producer's flag: weak loads that bypass L1 (peer and
// local memory alike are then read at the home L2), not volatile, so that many are in flight.
__device__ __forceinline__ float4 ld_relaxed_sys_v4(const float* p) { return __ldcg((const float4*)p); }
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    uint32_t s = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(s), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async8(void* smem_dst, const void* gmem_src) {
    uint32_t s = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" :: "r"(s), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }
// L2 loads (bypass L1) of data another CTA of this kernel wrote before a fence
// + counter handshake.  Not volatile, so independent loads pipeline.
__device__ __forceinline__ float4 ld_cg_v4(const float* p) { return __ldcg((const float4*)p); }
__device__ __forceinline__ float ld_cg_f32(const float* p) { return __ldcg(p); }
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 multimem_ld_reduce_v4(const float* mc) {
    float4 r;
    asm("multimem.ld_reduce.weak.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
        : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "l"(mc));
    return r;
}
__device__ __forceinline__ void multimem_st_v4(float* mc, float4 v) {
    asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1,%2,%3,%4};"
                 :: "l"(mc), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ long long globaltimer_ns() {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Spin until *p has reached `target` (wrap-safe) or `budget_ns` has passed.
// Never unbounded: on expiry the caller records a status and carries on.
__device__ __forceinline__ uint32_t ld_relaxed_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ bool wait_reached(const uint32_t* p, uint32_t target, long long budget_ns) {
    // spin on relaxed loads, then one acquire fence orders the data reads that follow
    bool ok = (int)(ld_relaxed_sys_u32(p) - target) >= 0;
    if (!ok) {
        long long t0 = globaltimer_ns();
        for (;;) {
#pragma unroll 1
            for (int i = 0; i < 256 && !ok; ++i) ok = (int)(ld_relaxed_sys_u32(p) - target) >= 0;
            if (ok || globaltimer_ns() - t0 > budget_ns) break;
        }
    }
    asm volatile("fence.acquire.sys;" ::: "memory");
    return ok;
}

__device__ __forceinline__ void report_timeout(const CommCtx& c, int kernel_id, int peer, uint32_t epoch) {
    if (atomicCAS(c.status, B2_STATUS_OK, B2_STATUS_WAIT_TIMEOUT) == B2_STATUS_OK) {
        c.status[1] = kernel_id;
        c.status[2] = peer;
        c.status[3] = (int)epoch;
    }
}

// Programmatic dependent launch.  A kernel that calls pdl_launch_dependents() lets the
// next kernel in the stream start (if that one was launched with the programmatic
// stream-serialisation attribute); the dependent must call pdl_wait() before it touches
// anything its predecessors produce.  pdl_wait() returns once every predecessor grid has
// completed and its memory is visible.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch `kern` so that it may become resident while its predecessor in the stream is still running
// (programmatic dependent launch).  The kernel must call pdl_wait() before it reads anything that a
// predecessor of the same step writes.
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }

// The opt-in to more than 48 KB of dynamic shared memory is an attribute of (kernel, device), not of
// the process: remember it per device, under a lock, so that a process that drives several GPUs or
// launches from several threads opts in on each device exactly once.
#include <mutex>
#define B2_MAX_DEVICES 64
struct SmemOptIn {
    size_t have[B2_MAX_DEVICES] = {0};
    std::mutex mu;
    template <typename F>
    cudaError_t ensure(F kernel, size_t bytes) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (dev < 0 || dev >= B2_MAX_DEVICES) return cudaErrorInvalidDevice;
        std::lock_guard<std::mutex> lock(mu);
        if (bytes > have[dev]) {
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
            if (e != cudaSuccess) return e;
            have[dev] = bytes;
        }
        return cudaSuccess;
    }
};

#define B2_KID_GEMV_FIN 1
#define B2_KID_ALLREDUCE 2
#define B2_KID_ARGMAX 3
#define B2_KID_BARRIER 4
#define B2_KID_TEST 5
#define B2_KID_GEMM_RS 6
#define B2_KID_GEMV_SPLITK 12     // GEMV: a split-K partner's tagged partial sums did not arrive
#define B2_KID_SEQPAR 11         // reduce-scatter + norm + all-gather: a peer never arrived
#define B2_KID_SAMPLE 10         // distributed sampler: a peer's candidate list did not arrive
#define B2_KID_CHAIN_DEP 7      // chain kernel: an op's producers did not finish
#define B2_KID_CHAIN_TILE 8     // chain kernel: a peer's tile did not arrive
#define B2_KID_CHAIN_COPY 9     // chain kernel: a weight copy did not land
