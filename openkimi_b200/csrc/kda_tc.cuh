// sm_100a building blocks for the tensor-core stages: mbarriers with bounded waits, 1-D bulk
// TMA copies, TMEM allocation / load / store, tcgen05.mma issue, and the shared-memory /
// instruction descriptors of the canonical (un-swizzled) core-matrix layout.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace kda {
namespace tc {

// ---------------------------------------------------------------------------------------
// Core-matrix ("CM") layout.  A [R x Cc] tile of 16-bit elements is stored as 8x8-element
// core matrices of 128 contiguous bytes (8 rows of 16 bytes), core matrices ordered
// [R/8][Cc/8].  The same bytes serve two tcgen05 operand views:
//   * K-major view, rows = M/N index, cols = K index:   SBO = (Cc/8)*128 (next 8 rows),
//     LBO = 128 (next 8 k);  one K=16 instruction step advances the start by 256 bytes.
//   * MN-major view, cols = M/N index, rows = K index:  SBO = 128 (next 8 along M/N),
//     LBO = (Cc/8)*128 (next 8 k); one K=16 step advances the start by 2 * LBO.
// ---------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ int cm_idx(int r, int c, int cols) {
    return (((r >> 3) * (cols >> 3) + (c >> 3)) << 6) + ((r & 7) << 3) + (c & 7);
}

// ---------------------------------------------------------------------------------------
// Row-major [rows][128] tiles (the kept prologue: G in FP32, q^ and k^ in BF16) are stored with
// their 16-byte chunks XOR-swizzled by the row: chunk c of row r sits at chunk position
// c ^ (r & 7).  A warp that reads eight ROWS at the same channels (the operand stage of the
// forward) then touches eight different 16-byte bank groups instead of one, while every access
// that walks the channels of one row (thread = channel, or a half warp per row) stays
// conflict-free, because the swizzle permutes chunks inside an aligned group of eight.
// ---------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ int swz_f32(int r, int d) { return r * 128 + ((((d >> 2) ^ (r & 7)) << 2) | (d & 3)); }
__host__ __device__ __forceinline__ int swz_bf16(int r, int d) { return r * 128 + ((((d >> 3) ^ (r & 7)) << 3) | (d & 7)); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// 64-bit shared-memory matrix descriptor, no swizzle, descriptor version 1 (sm_100)
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

// instruction descriptor for kind::f16 with BF16 operands and FP32 accumulation
__host__ __device__ constexpr uint32_t make_idesc(int M, int N, bool a_mn_major, bool b_mn_major, bool neg_a = false,
                                                 bool neg_b = false) {
    return (1u << 4)            // D format F32
           | (1u << 7)          // A format BF16
           | (1u << 10)         // B format BF16
           | ((neg_a ? 1u : 0u) << 13) | ((neg_b ? 1u : 0u) << 14)
           | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16)
           | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// ---------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2^22 polls (each try_wait already blocks for a
// hardware-defined interval), records the failure and returns false.
constexpr uint32_t WAIT_LIMIT = 1u << 22;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code,
                                          uint32_t limit = WAIT_LIMIT) {
    for (uint32_t it = 0; it < limit; ++it)
        if (mbar_try_wait(bar, parity)) return true;
    if (status) atomicOr(status, code);
    return false;
}
// The same wait inside kda_fwd / kda_bwd kernels (P = KdaParams): the thread whose wait gave up also leaves the
// status word in the caller's pinned host word (status_host, device-mapped), so that the host can notice by
// reading its own memory, without a copy, a synchronisation or one more launch.
template <class P>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const P& p, int code) {
    for (uint32_t it = 0; it < WAIT_LIMIT; ++it)
        if (mbar_try_wait(bar, parity)) return true;
    int v = code;
    if (p.status) v |= atomicOr(p.status, code);
    if (p.status_host) *reinterpret_cast<volatile int32_t*>(p.status_host) = v;
    return false;
}
// account for `bytes` of a transaction that will never arrive (used when a wait is abandoned, so that
// the barrier still completes once the copies that ARE in flight have landed)
__device__ __forceinline__ void mbar_complete_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.complete_tx.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

// ---------------------------------------------------------------------------------------
// TMA: 1-D bulk copy global -> shared, completion on an mbarrier (bytes % 16 == 0, both
// addresses 16-byte aligned)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_1d(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// shared -> global bulk store (bulk async-group completion)
__device__ __forceinline__ void tma_store_1d(void* dst_gmem, const void* src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem), "r"(smem_u32(src_smem)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// hint: bring a record into L2 ahead of the bulk copy that will read it
__device__ __forceinline__ void l2_prefetch_bulk(const void* gmem, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gmem), "r"(bytes) : "memory");
}

// generic-proxy writes to shared memory -> visible to the async proxy (TMA, tcgen05)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------------------------------
// TMEM
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {  // one full warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // one full warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 bit, 16 consecutive columns: thread t of the warp gets lane (base lane + t)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
                 "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

// ---------------------------------------------------------------------------------------
// tcgen05.mma (one thread issues).  D[tmem] (+)= A * B, A from shared memory or from TMEM.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// arrive on an mbarrier once every tcgen05 operation issued so far by this thread is done
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

}  // namespace tc
}  // namespace kda

// ---------------------------------------------------------------------------------------
// Optional phase timing (compiled in only with -DKDA_PHASE_TIMING; development aid).  Thread 0
// of every CTA adds the nanoseconds since its previous mark to slot n of a per-file counter
// array; KDA_PHASE_EXPORT(name) defines the C entry point that reads and clears it.
// ---------------------------------------------------------------------------------------
#ifdef KDA_PHASE_TIMING
static __device__ unsigned long long g_phase_ns[32];
__device__ __forceinline__ unsigned long long kda_phase_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define KDA_PHASE_BEGIN() unsigned long long _ph_t = kda_phase_now()
#define KDA_PHASE(n)                                               \
    do {                                                           \
        if (threadIdx.x == 0) {                                    \
            unsigned long long _now = kda_phase_now();             \
            atomicAdd(&g_phase_ns[n], _now - _ph_t);               \
            _ph_t = _now;                                          \
        }                                                          \
    } while (0)
#define KDA_PHASE_EXPORT(name)                                                            \
    extern "C" int name(unsigned long long* out) {                                        \
        unsigned long long z[32] = {0};                                                   \
        if (cudaMemcpyFromSymbol(out, g_phase_ns, sizeof(z)) != cudaSuccess) return 1;    \
        return cudaMemcpyToSymbol(g_phase_ns, z, sizeof(z)) == cudaSuccess ? 0 : 1;       \
    }
#else
#define KDA_PHASE_BEGIN() do {} while (0)
#define KDA_PHASE(n) do {} while (0)
#define KDA_PHASE_EXPORT(name)
#endif

// ---------------------------------------------------------------------------------------
// small vector helpers
// ---------------------------------------------------------------------------------------
namespace kda {
namespace tc {
__device__ __forceinline__ void bf16x8_to_f32(const uint4& u, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __bfloat1622float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ uint4 f32_to_bf16x8(const float (&f)[8]) {
    return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}
// Span guard of one [16 rows x 32 channels] tile of the cumulative log2 gate, evaluated by the
// warp whose lanes hold the 32 channels (experiments/kda_sm90/patch_fla_guarded_intra.py:35-63;
// oracle: experiments/kda_sm90/guarded_diagonal_oracle.py:131-141): every channel monotone
// non-increasing and finite, and the largest per-channel (max - min) <= limit.  A negative
// limit rejects every tile.  Returns the decision (uniform over the warp) and this lane's
// midpoint (max + min) / 2.
__device__ __forceinline__ bool guard_tile(const float (&G)[16], float limit, float& mid) {
    float gmax = -INFINITY, gmin = INFINITY, prev = INFINITY;
    bool good = true;
#pragma unroll
    for (int r = 0; r < 16; ++r) {
        good = good && (G[r] <= prev) && isfinite(G[r]);
        prev = G[r];
        gmax = fmaxf(gmax, G[r]);
        gmin = fminf(gmin, G[r]);
    }
    mid = 0.5f * (gmax + gmin);
    float span = gmax - gmin;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) span = fmaxf(span, __shfl_xor_sync(0xffffffffu, span, o));
    return __all_sync(0xffffffffu, good) && isfinite(span) && span <= limit;
}

// 2^x by the hardware approximation alone (results below 2^-126 flush to zero); exp2f wraps the
// same instruction in a rescaling for denormal results that no decay factor here needs
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 16-byte asynchronous copy global -> shared (L2 only); !valid writes zeros and reads nothing
__device__ __forceinline__ void cp_async16_z(void* dst_smem, const void* src, bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(src), "r"(valid ? 16 : 0)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// sum over the 16 lanes of a half warp
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
}  // namespace tc
}  // namespace kda
