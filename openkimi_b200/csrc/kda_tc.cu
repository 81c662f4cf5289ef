// Tensor-core (tcgen05 / TMEM) stages of the KDA op for BF16 operands.
#include "kda_common.cuh"
#include "kda_tc.cuh"
#include "kda_tmap.cuh"

namespace kda {

using namespace tc;

// ---------------------------------------------------------------------------------------
// Self-test of the MMA building block: D[128 x N] = A[128 x K] * B[K x N] with one CTA,
// operands converted to BF16 and laid out by the kernel in the core-matrix layout.  The
// host chooses the operand views and passes the descriptor strides, so the layout rules
// of kda_tc.cuh are checked against a plain matrix product.
//   a_mode 0: shared, K-major (stored CM rows=m, cols=k)   1: shared, MN-major (CM rows=k, cols=m)
//          2: tensor memory (lane = m, two BF16 per 32-bit column)
//   b_mode 0: shared, K-major (stored CM rows=n, cols=k)   1: shared, MN-major (CM rows=k, cols=n)
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128, 1)
mma_selftest_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ D, int N, int K,
                    int a_mode, int b_mode, int lbo_a, int sbo_a, int step_a, int lbo_b, int sbo_b, int step_b,
                    int neg_a, int m_rows, int* status) {
    extern __shared__ __align__(128) unsigned char dyn[];
    __nv_bfloat16* sA = reinterpret_cast<__nv_bfloat16*>(dyn);
    __nv_bfloat16* sB = sA + 128 * 128;
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_base_s;
    const int tid = threadIdx.x, warp = tid >> 5;
    if (warp == 0) {
        tmem_alloc(&tmem_base_s, 256);
        tmem_relinquish();
    }
    if (tid == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    for (int idx = tid; idx < 128 * K; idx += 128) {
        int m = idx / K, k = idx % K;
        __nv_bfloat16 v = __float2bfloat16_rn(A[idx]);
        if (a_mode == 0) sA[cm_idx(m, k, K)] = v;
        else if (a_mode == 1) sA[cm_idx(k, m, 128)] = v;
    }
    for (int idx = tid; idx < K * N; idx += 128) {
        int k = idx / N, n = idx % N;
        __nv_bfloat16 v = __float2bfloat16_rn(B[idx]);
        if (b_mode == 0) sB[cm_idx(n, k, K)] = v;
        else sB[cm_idx(k, n, N)] = v;
    }
    fence_async_smem();
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
    if (m_rows != 128) {  // clear the accumulator so that untouched lanes read as zero
        uint32_t z[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) z[j] = 0u;
        for (int c0 = 0; c0 < N; c0 += 16) tmem_st16(tmem + lane_off + c0, z);
        tmem_wait_st();
    }
    if (a_mode == 2) {
        for (int c0 = 0; c0 < K / 2; c0 += 16) {
            uint32_t r[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] = pack_bf16(A[tid * K + 2 * (c0 + j)], A[tid * K + 2 * (c0 + j) + 1]);
            tmem_st16(tmem + lane_off + 128 + c0, r);
        }
        tmem_wait_st();
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
        tc_fence_after();
        const uint32_t idesc = make_idesc(m_rows, N, a_mode == 1, b_mode == 1, neg_a != 0);
        for (int s = 0; s < K / 16; ++s) {
            uint64_t bd = make_desc(smem_u32(sB) + s * step_b, lbo_b, sbo_b);
            if (a_mode == 2) mma_ts(tmem, tmem + 128 + s * 8, bd, idesc, s > 0);
            else mma_ss(tmem, make_desc(smem_u32(sA) + s * step_a, lbo_a, sbo_a), bd, idesc, s > 0);
        }
        mma_commit(&bar);
    }
    const bool ok = mbar_wait(&bar, 0, status, 1);
    tc_fence_after();
    if (ok) {
        for (int c0 = 0; c0 < N; c0 += 16) {
            uint32_t r[16];
            tmem_ld16(tmem + lane_off + c0, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) D[tid * N + c0 + j] = __uint_as_float(r[j]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

// ---------------------------------------------------------------------------------------
// Self-test of the bounded wait: one CTA allocates tensor memory, arms an mbarrier for
// 2 * bytes, issues ONE bulk copy of `bytes`, and polls at most `poll_limit` times.  The
// wait must run out: the kernel records `code` in the status word, accounts for the bytes that
// were never sent so that the barrier completes as soon as the copy that IS in flight has
// landed, waits for that (bounded), frees its tensor memory and returns.  Nothing hangs.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128, 1) wait_selftest_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                               uint32_t poll_limit, int code, int* status) {
    __shared__ __align__(128) float buf[64];
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_base_s;
    const int tid = threadIdx.x, warp = tid >> 5;
    constexpr uint32_t BYTES = 64 * sizeof(float);
    if (warp == 0) {
        tmem_alloc(&tmem_base_s, 32);
        tmem_relinquish();
    }
    if (tid == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (tid == 0) {
        mbar_expect_tx(&bar, 2 * BYTES);  // twice what the copy below delivers
        tma_load_1d(buf, src, BYTES, &bar);
    }
    bool ok = mbar_wait(&bar, 0, status, code, poll_limit);
    ok = __syncthreads_and(ok);
    if (!ok) {
        if (tid == 0) mbar_complete_tx(&bar, BYTES);
        const bool landed = mbar_wait(&bar, 0, status, code << 8);  // the copy in flight, default limit
        if (__syncthreads_and(landed) && tid < 64) dst[tid] = buf[tid];
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base_s, 32);
}

// ---------------------------------------------------------------------------------------
// fwd_state on tensor cores.  One CTA per (sequence, head); thread t owns value column
// e = t, which is TMEM lane t.  The state is kept TRANSPOSED in tensor memory for the whole
// sequence: Sacc[e][d] (FP32, 128 columns).  Per chunk:
//   A  read Sacc -> BF16 copy Sbf (MMA operand, also the chunk-entry checkpoint), decay Sacc
//   1  WSacc = Sbf * W^T        (V'^T = U^T - WSacc)        Oacc  = Sbf * Qt^T
//   B  V'^T -> BF16 Vbf (MMA operand) and the V' record
//   2  Oacc += Vbf * Aqk^T      Sacc += Vbf * Kh
//   C  o = Oacc
// The per-chunk records arrive by linear bulk TMA copies into a two-stage ring.
// ---------------------------------------------------------------------------------------
namespace fs {
constexpr int D = 128, NTHR = 256;
constexpr uint32_t WT = 0, QT = 16384, KH = 32768, UT = 49152, AQ = 65536, GAM = 73728, STAGE = 74240;
constexpr uint32_t OUT = 2 * STAGE, TOTAL = OUT + 16384;  // output tile bf16 [64][128] behind the two stages
constexpr uint32_t SACC = 0, SBF = 128, WSACC = 192, OACC = 256, VBF = 320, TMEM_COLS = 512;
}  // namespace fs

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __bfloat1622float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

__global__ void __launch_bounds__(fs::NTHR, 1) kda_fwd_state_tc(const KdaParams p, const __grid_constant__ RowMaps maps) {
    using namespace fs;
    extern __shared__ __align__(128) unsigned char dyn[];
    __shared__ uint64_t full[2];
    __shared__ uint64_t mmabar;
    __shared__ uint32_t tmem_s;
    // thread (half, e) = (tid / 128, tid % 128): TMEM lane e (value column e), and half of the accumulator
    // columns in every conversion phase (two warps share a lane quadrant)
    const int tid = threadIdx.x, warp = tid >> 5, e = tid & 127, half = tid >> 7;
    const int h = blockIdx.x, n = blockIdx.y;
    int c0, nc;
    seq_chunks(p, n, c0, nc);
    long long tok_first, tok_end;
    seq_tokens(p, n, tok_first, tok_end);
    const WsLayout L = ws_layout(p.NT, p.H, p.dk, p.dv, p.dtype);
    char* ws = (char*)p.workspace;
    if (warp == 0) {
        tmem_alloc(&tmem_s, TMEM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        mbar_init(&mmabar, 2);  // two issuing threads per MMA group (one accumulator each): a single thread spends
                                // ~50 ns on every MMA it issues, which is on the critical path of the chunk loop
        mbar_fence_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_s + ((uint32_t)((warp & 3) * 32) << 16);  // this warp's lane quadrant
    const uint32_t tmem0 = tmem_s;
    const size_t sbase = ((size_t)n * p.H + h) * D * D;
    const bool save = !(p.flags & KDA_FLAG_NO_SAVE);  // forward-only calls write no checkpoint and no V' record

    for (int d0 = 64 * half; d0 < 64 * half + 64; d0 += 16) {
        uint32_t r[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(p.h0 ? p.h0[sbase + state_idx(p, d0 + j, e)] : 0.f);
        tmem_st16(tmem + SACC + d0, r);
    }
    tmem_wait_st();

    // the six records of a chunk: one copy each from lane 0 of six warps (a thread spends ~30 ns on every bulk
    // copy it issues, and the chunk step waits for the slowest thread)
    auto issue_loads = [&](int lc, int stage) {
        if ((tid & 31) != 0 || warp >= 6) return;
        const size_t rec = (size_t)(c0 + lc) * p.H + h;
        unsigned char* b = dyn + stage * STAGE;
        if (warp == 0) {
            mbar_expect_tx(&full[stage], STAGE);
            tma_load_1d(b + WT, (const __nv_bfloat16*)(ws + L.W) + rec * C * D, 16384, &full[stage]);
        } else if (warp == 1) {
            tma_load_1d(b + UT, (const __nv_bfloat16*)(ws + L.U) + rec * C * D, 16384, &full[stage]);
        } else if (warp == 2) {
            tma_load_1d(b + QT, (const __nv_bfloat16*)(ws + L.Qt) + rec * C * D, 16384, &full[stage]);
        } else if (warp == 3) {
            tma_load_1d(b + KH, (const __nv_bfloat16*)(ws + L.Kh) + rec * C * D, 16384, &full[stage]);
        } else if (warp == 4) {
            tma_load_1d(b + AQ, (const __nv_bfloat16*)(ws + L.Aqk) + rec * C * C, 8192, &full[stage]);
        } else {
            tma_load_1d(b + GAM, (const float*)(ws + L.gamC) + rec * D, 512, &full[stage]);
        }
    };
    if (nc > 0) issue_loads(0, 0);

    uint32_t mma_phase = 0;
    bool ok = true;
    KDA_PHASE_BEGIN();
    __nv_bfloat16* o = (__nv_bfloat16*)p.o;
    for (int lc = 0; lc < nc; ++lc) {
        const int stage = lc & 1;
        unsigned char* b = dyn + stage * STAGE;
        const ChunkInfo ci = chunk_of_seq(n, lc, tok_first, tok_end);
        const size_t rec = (size_t)(c0 + lc) * p.H + h;
        // the next chunk's records are requested first thing (the other stage was last read by the previous
        // chunk's MMAs, which completed before that chunk's iteration ended): a whole chunk step ahead of their use
        if (lc + 1 < nc) issue_loads(lc + 1, stage ^ 1);
        tma_store_wait_read();  // the previous chunk's output rows have left the staging tile
        ok = mbar_wait(&full[stage], (lc >> 1) & 1, p, 2);
        if (!__syncthreads_and(ok)) { ok = false; break; }
        KDA_PHASE(0);

        // ---- A: BF16 copy of the entering state, checkpoint, decay
        {
            const float* gam = reinterpret_cast<const float*>(b + GAM);
            __nv_bfloat16* gS0 = (__nv_bfloat16*)(ws + L.S0) + rec * D * D;
            for (int d0 = 64 * half; d0 < 64 * half + 64; d0 += 16) {
                uint32_t r[16], pk[8];
                tmem_ld16(tmem + SACC + d0, r);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 8; ++j) pk[j] = pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                tmem_st8(tmem + SBF + d0 / 2, pk);
                if (save) {
                    *reinterpret_cast<uint4*>(gS0 + cm_idx(e, d0, D)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    *reinterpret_cast<uint4*>(gS0 + cm_idx(e, d0 + 8, D)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * gam[d0 + j]);
                tmem_st16(tmem + SACC + d0, r);
            }
            tmem_wait_st();
        }
        KDA_PHASE(1);
        tc_fence_before();
        __syncthreads();
        if ((tid & 31) == 0 && warp < 2) {
            tc_fence_after();
            const uint32_t sb = smem_u32(b);
            constexpr uint32_t id_mn = make_idesc(128, 64, false, true);
            constexpr uint32_t id_k = make_idesc(128, 64, false, false);
            if (warp == 0) {
#pragma unroll
                for (int s = 0; s < 8; ++s)  // WSacc = Sbf (K = d) * W^T record, MN-major B
                    mma_ts(tmem0 + WSACC, tmem0 + SBF + s * 8, make_desc(sb + WT + s * 2048, 1024, 128), id_mn, s > 0);
            } else {
#pragma unroll
                for (int s = 0; s < 8; ++s)  // Oacc = Sbf * Qt^T, K-major B (rows = i)
                    mma_ts(tmem0 + OACC, tmem0 + SBF + s * 8, make_desc(sb + QT + s * 256, 128, 2048), id_k, s > 0);
            }
            mma_commit(&mmabar);
        }
        ok = mbar_wait(&mmabar, mma_phase, p, 4);
        mma_phase ^= 1;
        tc_fence_after();
        if (!__syncthreads_and(ok)) { ok = false; break; }
        KDA_PHASE(2);

        // ---- B: V'^T = U^T - (W S)^T
        {
            const __nv_bfloat16* sU = reinterpret_cast<const __nv_bfloat16*>(b + UT);
            __nv_bfloat16* gV = (__nv_bfloat16*)(ws + L.U) + rec * C * D;
            for (int i0 = 32 * half; i0 < 32 * half + 32; i0 += 16) {
                uint32_t r[16], pk[8];
                float u[16];
                tmem_ld16(tmem + WSACC + i0, r);
                tmem_wait_ld();
                {
                    float t8[8];
                    unpack8(*reinterpret_cast<const uint4*>(sU + cm_idx(e, i0, C)), t8);
#pragma unroll
                    for (int j = 0; j < 8; ++j) u[j] = t8[j];
                    unpack8(*reinterpret_cast<const uint4*>(sU + cm_idx(e, i0 + 8, C)), t8);
#pragma unroll
                    for (int j = 0; j < 8; ++j) u[8 + j] = t8[j];
                }
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    pk[j] = pack_bf16(u[2 * j] - __uint_as_float(r[2 * j]), u[2 * j + 1] - __uint_as_float(r[2 * j + 1]));
                tmem_st8(tmem + VBF + i0 / 2, pk);
                if (save) {
                    *reinterpret_cast<uint4*>(gV + cm_idx(e, i0, C)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    *reinterpret_cast<uint4*>(gV + cm_idx(e, i0 + 8, C)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                }
            }
            tmem_wait_st();
        }
        KDA_PHASE(3);
        tc_fence_before();
        __syncthreads();
        if ((tid & 31) == 0 && warp < 2) {
            tc_fence_after();
            const uint32_t sb = smem_u32(b);
            constexpr uint32_t id_k = make_idesc(128, 64, false, false);
            constexpr uint32_t id_s = make_idesc(128, 128, false, true);
            if (warp == 0) {
#pragma unroll
                for (int s = 0; s < 4; ++s)  // Oacc += Vbf (K = j) * Aqk^T, K-major B (rows = i)
                    mma_ts(tmem0 + OACC, tmem0 + VBF + s * 8, make_desc(sb + AQ + s * 256, 128, 1024), id_k, true);
            } else {
#pragma unroll
                for (int s = 0; s < 4; ++s)  // Sacc += Vbf (K = i) * Kh, MN-major B
                    mma_ts(tmem0 + SACC, tmem0 + VBF + s * 8, make_desc(sb + KH + s * 4096, 2048, 128), id_s, true);
            }
            mma_commit(&mmabar);
        }
        ok = mbar_wait(&mmabar, mma_phase, p, 4);
        mma_phase ^= 1;
        tc_fence_after();
        if (!__syncthreads_and(ok)) { ok = false; break; }
        KDA_PHASE(4);

        // ---- C: output rows.  The accumulator holds O^T (lane = channel), so the tile is transposed through
        //      shared memory and goes out with one bulk-tensor store (row by row for a partial chunk)
        {
            __nv_bfloat16* sO = reinterpret_cast<__nv_bfloat16*>(dyn + OUT);
#pragma unroll
            for (int i0 = 32 * half; i0 < 32 * half + 32; i0 += 16) {
                uint32_t r[16];
                tmem_ld16(tmem + OACC + i0, r);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 16; ++j) sO[(i0 + j) * D + e] = __float2bfloat16_rn(__uint_as_float(r[j]));
            }
            fence_async_smem();
            __syncthreads();
            if (maps.ok && ci.len == C) {  // the whole tile with one bulk-tensor store
                if (tid == 0) {
                    tma_store_tile(&maps.m[0], h * D, (int)ci.tok0, sO);
                    tma_store_commit();
                }
            } else if (tid < ci.len) {
                tma_store_1d(o + ((size_t)(ci.tok0 + tid) * p.H + h) * D, sO + tid * D, D * 2);
                tma_store_commit();
            }
        }
        KDA_PHASE(5);
    }
    if (ok && p.ht) {
        for (int d0 = 64 * half; d0 < 64 * half + 64; d0 += 16) {
            uint32_t r[16];
            tmem_ld16(tmem + SACC + d0, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) p.ht[sbase + state_idx(p, d0 + j, e)] = __uint_as_float(r[j]);
        }
    }
    tma_store_wait_all();
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem0, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------
// bwd_state on tensor cores: same organisation, reverse chunk order, dS^T resident in TMEM.
//   A  dSacc -> BF16 dSbf (operand + checkpoint of the dS entering the chunk), decay dSacc
//   1  dVacc = dO^T * Aqk + dSbf * Kh^T          dSacc += dO^T * Qt
//   B  dV'^T -> BF16 dVbf and the dV' record
//   2  dSacc -= dVbf * W
// ---------------------------------------------------------------------------------------
namespace bs {
constexpr int D = 128, NTHR = 256;
constexpr uint32_t WT = 0, QT = 16384, KH = 32768, DO = 49152, AQ = 65536, GAM = 73728, STAGE = 74240;
constexpr uint32_t TMA_BYTES = 16384 * 3 + 8192 + 512;
constexpr uint32_t SACC = 0, SBF = 128, VACC = 192, VBF = 256, TMEM_COLS = 512;
}  // namespace bs

__global__ void __launch_bounds__(bs::NTHR, 1) kda_bwd_state_tc(const KdaParams p) {
    using namespace bs;
    extern __shared__ __align__(128) unsigned char dyn[];
    __shared__ uint64_t full[3];  // three stages: the records of a chunk are requested two chunk steps ahead of their use
    __shared__ uint64_t mmabar, mmabar2;
    __shared__ uint32_t tmem_s;
    // thread (half, e) = (tid / 128, tid % 128): TMEM lane e, and half of the columns of every conversion phase
    const int tid = threadIdx.x, warp = tid >> 5, e = tid & 127, half = tid >> 7;
    const int h = blockIdx.x, n = blockIdx.y;
    int c0, nc;
    seq_chunks(p, n, c0, nc);
    long long tok_first, tok_end;
    seq_tokens(p, n, tok_first, tok_end);
    const WsLayout L = ws_layout(p.NT, p.H, p.dk, p.dv, p.dtype);
    const char* ws = (const char*)p.workspace;
    char* sc = (char*)p.bwd_scratch;
    const __nv_bfloat16* dO = (const __nv_bfloat16*)p.grad_o;
    if (warp == 0) {
        tmem_alloc(&tmem_s, TMEM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        mbar_init(&full[2], 1);
        mbar_init(&mmabar, 2);   // first group: one issuing thread per accumulator
        mbar_init(&mmabar2, 1);  // second group: a single product
        mbar_fence_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_s + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t tmem0 = tmem_s;
    const size_t sbase = ((size_t)n * p.H + h) * D * D;

    for (int d0 = 64 * half; d0 < 64 * half + 64; d0 += 16) {
        uint32_t r[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(p.grad_ht ? p.grad_ht[sbase + state_idx(p, d0 + j, e)] : 0.f);
        tmem_st16(tmem + SACC + d0, r);
    }
    tmem_wait_st();

    // step k = 0..nc-1 processes chunk lc = nc-1-k
    auto issue_loads = [&](int k, int stage) {
        const int lc = nc - 1 - k;
        const size_t rec = (size_t)(c0 + lc) * p.H + h;
        unsigned char* b = dyn + stage * STAGE;
        if ((tid & 31) == 0) {  // one bulk copy each from lane 0 of five warps
            if (warp == 0) {
                mbar_expect_tx(&full[stage], TMA_BYTES);
                tma_load_1d(b + WT, (const __nv_bfloat16*)(ws + L.W) + rec * C * D, 16384, &full[stage]);
            } else if (warp == 1) {
                tma_load_1d(b + QT, (const __nv_bfloat16*)(ws + L.Qt) + rec * C * D, 16384, &full[stage]);
            } else if (warp == 2) {
                tma_load_1d(b + KH, (const __nv_bfloat16*)(ws + L.Kh) + rec * C * D, 16384, &full[stage]);
            } else if (warp == 3) {
                tma_load_1d(b + AQ, (const __nv_bfloat16*)(ws + L.Aqk) + rec * C * C, 8192, &full[stage]);
            } else if (warp == 4) {
                tma_load_1d(b + GAM, (const float*)(ws + L.gamC) + rec * D, 512, &full[stage]);
            }
        }
        // dO tile -> core-matrix layout cm(i, e; 128), 16-byte chunks, zero rows past the end
        const ChunkInfo ci = chunk_of_seq(n, lc, tok_first, tok_end);
        __nv_bfloat16* sdo = reinterpret_cast<__nv_bfloat16*>(b + DO);
        for (int q = tid; q < C * (D / 8); q += NTHR) {
            const int i = q >> 4, e8 = (q & 15) * 8;
            const bool valid = i < ci.len;
            const size_t row = (size_t)(ci.tok0 + (valid ? i : 0)) * p.H + h;
            cp_async16_z(sdo + cm_idx(i, e8, D), dO + row * D + e8, valid);
        }
        cp_async_commit();
    };
    if (nc > 0) issue_loads(0, 0);
    if (nc > 1) issue_loads(1, 1);

    bool ok = true;
    int stage = 0;
    uint32_t ring_phase = 0;  // parity of full[stage]: flips every time the ring wraps
    for (int k = 0; k < nc; ++k) {
        const int lc = nc - 1 - k;
        unsigned char* b = dyn + stage * STAGE;
        const size_t rec = (size_t)(c0 + lc) * p.H + h;
        if (k + 2 < nc) {  // (the stage behind this one was last read by the previous step's MMAs, which have completed)
            issue_loads(k + 2, stage == 0 ? 2 : stage - 1);
            cp_async_wait<2>();
        } else if (k + 1 < nc) {
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        fence_async_smem();
        ok = mbar_wait(&full[stage], ring_phase, p, 2);
        if (!__syncthreads_and(ok)) { ok = false; break; }

        {
            const float* gam = reinterpret_cast<const float*>(b + GAM);
            __nv_bfloat16* gdS = (__nv_bfloat16*)(sc + L.dS) + rec * D * D;
            for (int d0 = 64 * half; d0 < 64 * half + 64; d0 += 16) {
                uint32_t r[16], pk[8];
                tmem_ld16(tmem + SACC + d0, r);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 8; ++j) pk[j] = pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                tmem_st8(tmem + SBF + d0 / 2, pk);
                *reinterpret_cast<uint4*>(gdS + cm_idx(e, d0, D)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                *reinterpret_cast<uint4*>(gdS + cm_idx(e, d0 + 8, D)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * gam[d0 + j]);
                tmem_st16(tmem + SACC + d0, r);
            }
            tmem_wait_st();
        }
        tc_fence_before();
        __syncthreads();
        if ((tid & 31) == 0 && warp < 2) {
            tc_fence_after();
            const uint32_t sb = smem_u32(b);
            constexpr uint32_t id_v1 = make_idesc(128, 64, true, true);    // dO^T (MN-major A) * Aqk (MN-major B)
            constexpr uint32_t id_v2 = make_idesc(128, 64, false, false);  // dSbf (TMEM) * Kh^T (K-major B)
            constexpr uint32_t id_s1 = make_idesc(128, 128, true, true);   // dO^T * Qt (MN-major B)
            if (warp == 0) {
#pragma unroll
                for (int s = 0; s < 4; ++s)
                    mma_ss(tmem0 + VACC, make_desc(sb + DO + s * 4096, 2048, 128), make_desc(sb + AQ + s * 2048, 1024, 128), id_v1,
                           s > 0);
#pragma unroll
                for (int s = 0; s < 8; ++s)
                    mma_ts(tmem0 + VACC, tmem0 + SBF + s * 8, make_desc(sb + KH + s * 256, 128, 2048), id_v2, true);
            } else {
#pragma unroll
                for (int s = 0; s < 4; ++s)
                    mma_ss(tmem0 + SACC, make_desc(sb + DO + s * 4096, 2048, 128), make_desc(sb + QT + s * 4096, 2048, 128), id_s1,
                           true);
            }
            mma_commit(&mmabar);
        }
        ok = mbar_wait(&mmabar, k & 1, p, 4);
        tc_fence_after();
        if (!__syncthreads_and(ok)) { ok = false; break; }

        {
            __nv_bfloat16* gdV = (__nv_bfloat16*)(sc + L.dVn) + rec * C * D;
            for (int i0 = 32 * half; i0 < 32 * half + 32; i0 += 16) {
                uint32_t r[16], pk[8];
                tmem_ld16(tmem + VACC + i0, r);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 8; ++j) pk[j] = pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                tmem_st8(tmem + VBF + i0 / 2, pk);
                *reinterpret_cast<uint4*>(gdV + cm_idx(e, i0, C)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                *reinterpret_cast<uint4*>(gdV + cm_idx(e, i0 + 8, C)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            }
            tmem_wait_st();
        }
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            const uint32_t sb = smem_u32(b);
            constexpr uint32_t id_w = make_idesc(128, 128, false, false, true);  // -dVbf (TMEM) * W (K-major B, rows = d)
#pragma unroll
            for (int s = 0; s < 4; ++s)
                mma_ts(tmem0 + SACC, tmem0 + VBF + s * 8, make_desc(sb + WT + s * 256, 128, 1024), id_w, true);
            mma_commit(&mmabar2);
        }
        ok = mbar_wait(&mmabar2, k & 1, p, 4);
        tc_fence_after();
        if (!__syncthreads_and(ok)) { ok = false; break; }
        if (++stage == 3) {
            stage = 0;
            ring_phase ^= 1;
        }
    }
    if (ok && p.grad_h0) {
        for (int d0 = 64 * half; d0 < 64 * half + 64; d0 += 16) {
            uint32_t r[16];
            tmem_ld16(tmem + SACC + d0, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) p.grad_h0[sbase + state_idx(p, d0 + j, e)] = __uint_as_float(r[j]);
        }
    }
    cp_async_wait<0>();
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem0, TMEM_COLS);
}

cudaError_t simt_stage(const KdaParams& p, int stage, cudaStream_t s);
cudaError_t launch_fwd_intra_tc(const KdaParams& p, cudaStream_t s);
cudaError_t launch_bwd_intra(const KdaParams& p, cudaStream_t s);
cudaError_t launch_bwd_wy_tc(const KdaParams& p, cudaStream_t s);
void prof_mark(cudaStream_t s);

enum { ST_FWD_INTRA = 0, ST_FWD_STATE = 1, ST_BWD_STATE = 2, ST_BWD_CHUNK = 3, ST_PARAM_REDUCE = 4 };

bool tc_supported(const KdaParams& p) { return p.dtype == KDA_DTYPE_BF16 && p.dk == 128 && p.dv == 128; }

static bool stage_simt(const KdaParams& p, int stage) { return (p.flags >> (5 + stage)) & 1; }

cudaError_t tc_fwd(const KdaParams& p, cudaStream_t s) {
    cudaError_t e;
    if ((e = stage_simt(p, ST_FWD_INTRA) ? simt_stage(p, ST_FWD_INTRA, s) : launch_fwd_intra_tc(p, s)) != cudaSuccess) return e;
    prof_mark(s);
    if (stage_simt(p, ST_FWD_STATE)) {
        if ((e = simt_stage(p, ST_FWD_STATE, s)) != cudaSuccess) return e;
    } else {
        constexpr int smem = fs::TOTAL;
        if ((e = cudaFuncSetAttribute(kda_fwd_state_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) != cudaSuccess)
            return e;
        RowMaps maps = {};
        maps.ok = !(p.flags & KDA_FLAG_ROW_COPIES) && make_row_map(&maps.m[0], p.o, (long long)p.B * p.T, p.H, C);
        kda_fwd_state_tc<<<dim3(p.H, p.N), fs::NTHR, smem, s>>>(p, maps);
    }
    prof_mark(s);
    return cudaGetLastError();
}

cudaError_t tc_bwd(const KdaParams& p, cudaStream_t s) {
    cudaError_t e;
    if (stage_simt(p, ST_BWD_STATE)) {
        if ((e = simt_stage(p, ST_BWD_STATE, s)) != cudaSuccess) return e;
    } else {
        constexpr int smem = 3 * bs::STAGE;
        if ((e = cudaFuncSetAttribute(kda_bwd_state_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) != cudaSuccess)
            return e;
        kda_bwd_state_tc<<<dim3(p.H, p.N), bs::NTHR, smem, s>>>(p);
    }
    prof_mark(s);
    if (stage_simt(p, ST_BWD_CHUNK)) {  // fused FP32-math kernel
        if ((e = simt_stage(p, ST_BWD_CHUNK, s)) != cudaSuccess) return e;
        prof_mark(s);
    } else {  // chunk-level adjoints, then the guarded intra kernel
        if ((e = stage_simt(p, 4) ? simt_stage(p, 5, s) : launch_bwd_wy_tc(p, s)) != cudaSuccess) return e;
        prof_mark(s);
        if ((e = launch_bwd_intra(p, s)) != cudaSuccess) return e;
        prof_mark(s);
    }
    if (p.flags & KDA_FLAG_GATE) {
        if ((e = simt_stage(p, ST_PARAM_REDUCE, s)) != cudaSuccess) return e;
    }
    prof_mark(s);
    return cudaGetLastError();
}

}  // namespace kda

extern "C" int kda_selftest_mma(const float* A, const float* B, float* D, int N, int K, int a_mode, int b_mode, int lbo_a,
                                int sbo_a, int step_a, int lbo_b, int sbo_b, int step_b, int neg_a, int m_rows,
                                int* status, void* stream) {
    if (!A || !B || !D || !status) return KDA_ERR_NULL;
    if (N < 16 || N > 128 || N % 16 || K < 16 || K > 128 || K % 16 || (m_rows != 64 && m_rows != 128)) return KDA_ERR_SHAPE;
    // the strides must keep every operand read inside the tile the kernel wrote
    if (lbo_a < 16 || sbo_a < 16 || lbo_b < 16 || sbo_b < 16 || lbo_a > 4096 || sbo_a > 4096 || lbo_b > 4096 || sbo_b > 4096)
        return KDA_ERR_SHAPE;
    size_t smem = 2 * 128 * 128 * sizeof(__nv_bfloat16);
    cudaError_t e = cudaFuncSetAttribute(kda::mma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return KDA_ERR_LAUNCH;
    kda::mma_selftest_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(A, B, D, N, K, a_mode, b_mode, lbo_a, sbo_a, step_a,
                                                                     lbo_b, sbo_b, step_b, neg_a, m_rows, status);
    return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

extern "C" int kda_selftest_wait(const float* src, float* dst, int poll_limit, int code, int* status, void* stream) {
    if (!src || !dst || !status) return KDA_ERR_NULL;
    if (poll_limit < 1 || poll_limit > 4096 || code < 1 || code > 255) return KDA_ERR_SHAPE;
    if (((uintptr_t)src & 15) != 0) return KDA_ERR_ALIGN;
    kda::wait_selftest_kernel<<<1, 128, 0, (cudaStream_t)stream>>>(src, dst, (uint32_t)poll_limit, code, status);
    return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

KDA_PHASE_EXPORT(kda_debug_phases_state)
