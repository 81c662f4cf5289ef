// bwd_wy on tensor cores (BF16 path, d = 128): the chunk-level adjoints of the WY / state
// products; one CTA per SM walks the (chunk, head) units (UnitWalk); every [64 x d] result is
// computed TRANSPOSED so that the accumulator rows (TMEM lanes) are the 128 channels:
//
//   S1   dAqk = dO V'^T (M = 64)        dWn^T = S0 dV'^T        dQt^T = S0 dO^T
//        dKh^T = dS V'^T                dVb^T = dV'^T T
//   S2   dKb^T = -dWn^T T               Z^T   = -dWn^T T + S0 dVb^T
//   S3   dMn   = Z W^T + dVb V'^T (M = 64);   dM = -strict_lower(dMn)
//
// (dWn = dV' S0^T = -dW.  With M = I + diag(beta) L, T = M^-1, W = T (beta K~), U = T (beta V) =
// V' + W S0, the gradient of M is -(T^T dW)(beta K~)^T T^T - (T^T dV')(beta V)^T T^T
// = -(dKb W^T + dVb U^T) = -((dKb + dVb S0^T) W^T + dVb V'^T); only its strictly lower part is
// used, for which masking the intermediate T-gradient is irrelevant.)
//
// Outputs: dv, the beta gradient collected so far, dGamma_C * Gamma_C, and the hand-over
// records of bwd_intra (dAqk, dM as three-way BF16 splits in operand layout; dQt, dKh, dKb in BF16,
// channel-major: handover_idx).
#include "kda_common.cuh"
#include "kda_conv_bwd.cuh"
#include "kda_tc.cuh"
#include "kda_tmap.cuh"

namespace kda {

using namespace tc;

// sixteen consecutive entries (row i, columns j0 .. j0 + 15) of a [64 x 64] FP32 matrix -> the three
// BF16 tiles cm(i, j; 64) whose sum it is (tile p at base + p * 4096 elements)
__device__ __forceinline__ void store_split_row(__nv_bfloat16* base, int i, int j0, const float (&f)[16]) {
    uint32_t p0[8], p1[8], p2[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) split3_bf16(f[2 * j], f[2 * j + 1], p0[j], p1[j], p2[j]);
    __nv_bfloat16* a = base + cm_idx(i, j0, C);
    __nv_bfloat16* b = base + cm_idx(i, j0 + 8, C);
    *reinterpret_cast<uint4*>(a) = make_uint4(p0[0], p0[1], p0[2], p0[3]);
    *reinterpret_cast<uint4*>(b) = make_uint4(p0[4], p0[5], p0[6], p0[7]);
    *reinterpret_cast<uint4*>(a + C * C) = make_uint4(p1[0], p1[1], p1[2], p1[3]);
    *reinterpret_cast<uint4*>(b + C * C) = make_uint4(p1[4], p1[5], p1[6], p1[7]);
    *reinterpret_cast<uint4*>(a + 2 * C * C) = make_uint4(p2[0], p2[1], p2[2], p2[3]);
    *reinterpret_cast<uint4*>(b + 2 * C * C) = make_uint4(p2[4], p2[5], p2[6], p2[7]);
}

// sixteen consecutive rows (i0 .. i0 + 15) of channel ch of a hand-over array: two 16-byte stores from the
// accumulator registers into the array's staging tile (layout: handover_idx; the tile then leaves as one bulk copy)
__device__ __forceinline__ void store_handover16(__nv_bfloat16* rec_base, int ch, int i0, const uint32_t (&r)[16]) {
    uint32_t pk[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) pk[j] = pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
    *reinterpret_cast<uint4*>(rec_base + handover_idx(i0, ch)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    *reinterpret_cast<uint4*>(rec_base + handover_idx(i0 + 8, ch)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
}

// ---------------------------------------------------------------------------------------
// The loads are taken off the critical path.  The operands that only the first and last MMA
// groups touch exist twice (V'^T, dV'^T, dO: set it % 2), so the NEXT unit's copies of them are
// requested as soon as the current unit's first MMA group is issued; S0 and T follow when the
// second group has read them; dS, W and the v rows are requested at the start of their unit
// and are first needed one MMA group (dS), a conversion stage (v) or nearly the whole unit (W)
// later.  The beta row sums are reduced in registers (a transposing butterfly over the 32
// channels of a warp) instead of through a 32 KB FP32 staging tile, which is what makes room for
// the second operand set.
// CONVB: the backward of the short convolution of v runs here too (KdaParams.grad_conv_*): dv of
// the convolved rows stays in shared memory and grad_v receives the gradient of the v
// projection.  The projection rows it needs (-3 .. 63) are fetched once dS is dead, into the half
// of its tile that stays free until the second conversion stage.
// ---------------------------------------------------------------------------------------
namespace bp {
constexpr int D = 128, NTHR = 512;
constexpr uint32_t VT = 0;                   // V'^T  cm(e, i; 64), two sets
constexpr uint32_t DVT = VT + 2 * 16384;     // dV'^T cm(e, i; 64), two sets;  later Z^T  cm(d, i; 64)
constexpr uint32_t DOT = DVT + 2 * 16384;    // dO    cm(i, e; 128), two sets; later dVb^T cm(e, i; 64)
constexpr uint32_t S0T = DOT + 2 * 16384;    // S0^T  cm(e, d; 128)
constexpr uint32_t DST = S0T + 32768;        // dS^T  cm(e, d; 128); later staging of dQt / dKb
constexpr uint32_t TT = DST + 32768;         // T     cm(i, j; 64)
constexpr uint32_t WT = TT + 8192;           // W^T   cm(d, j; 64)
constexpr uint32_t SV = WT + 16384;          // v bf16 [64][128] row-major; later dv
constexpr uint32_t SKH = SV + 16384;         // bf16 staging of dKh (dQt and dKb are staged in the two halves of DST once dS is dead)
constexpr uint32_t SBETA = SKH + 16384;      // f32: beta [64], row sums [64], partial dGamma_C [4][128], partial row sums [4][64]
constexpr uint32_t TOTAL = SBETA + 256 + 256 + 2048 + 1024;
constexpr uint32_t XVM = DST + 16384;        // fused conv backward only: pre-convolution v rows 0 .. 63, bf16 [64][128] (dS is dead by then)
constexpr uint32_t XVH = TOTAL;              //                          rows -3 .. -1, bf16 [3][128]
constexpr uint32_t XTAPS = XVH + 3 * 256;     //                          f32 [128][4] padded filter taps of v
constexpr uint32_t TOTAL_CONVB = XTAPS + 128 * 16;
constexpr uint32_t DAQK = 0, DWN = 64, DQT = 128, DKH = 192, DVB = 256, DKB = 320, DMN = 384, WBF = 448, TMEM_COLS = 512;
}  // namespace bp

// Sums of 16 values per lane over the 32 lanes of a warp: afterwards the lane holds the sum of value
// number r = 8 b4 + 4 b3 + 2 b2 + b1 (b_k = bit k of the lane index); lanes 2m and 2m + 1 hold the same sum.
__device__ __forceinline__ float warp_sum16(const float (&v)[16], int lane, int& r) {
    const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4, b1 = lane & 2;
    float a8[8], a4[4], a2[2];
#pragma unroll
    for (int t = 0; t < 8; ++t) a8[t] = (b4 ? v[t + 8] : v[t]) + __shfl_xor_sync(0xffffffffu, b4 ? v[t] : v[t + 8], 16);
#pragma unroll
    for (int t = 0; t < 4; ++t) a4[t] = (b3 ? a8[t + 4] : a8[t]) + __shfl_xor_sync(0xffffffffu, b3 ? a8[t] : a8[t + 4], 8);
#pragma unroll
    for (int t = 0; t < 2; ++t) a2[t] = (b2 ? a4[t + 2] : a4[t]) + __shfl_xor_sync(0xffffffffu, b2 ? a4[t] : a4[t + 2], 4);
    float a1 = (b1 ? a2[1] : a2[0]) + __shfl_xor_sync(0xffffffffu, b1 ? a2[0] : a2[1], 2);
    a1 += __shfl_xor_sync(0xffffffffu, a1, 1);
    r = (b4 ? 8 : 0) + (b3 ? 4 : 0) + (b2 ? 2 : 0) + (b1 ? 1 : 0);
    return a1;
}

template <bool CONVB>
__global__ void __launch_bounds__(bp::NTHR, 1) kda_bwd_wy_tc_pf(const KdaParams p, const __grid_constant__ RowMaps maps) {
    using namespace bp;
    extern __shared__ __align__(128) unsigned char dyn[];
    __shared__ uint64_t fullA[2], fullS, fullD, fullW, mma1, mma2, mma3;
    __shared__ uint32_t tmem_s;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const WsLayout L = ws_layout(p.NT, p.H, p.dk, p.dv, p.dtype);
    const char* ws = (const char*)p.workspace;
    char* sc = (char*)p.bwd_scratch;
    float* sbeta = reinterpret_cast<float*>(dyn + SBETA);
    float* srow = sbeta + 64;
    float* spart = srow + 64;   // [4][128]
    float* srp = spart + 512;   // [4][64]
    const __nv_bfloat16* dO = (const __nv_bfloat16*)p.grad_o;
    const __nv_bfloat16* v = (const __nv_bfloat16*)p.v;

    if (warp == 0) {
        tmem_alloc(&tmem_s, TMEM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        mbar_init(&fullA[0], 1);
        mbar_init(&fullA[1], 1);
        mbar_init(&fullS, 1);
        mbar_init(&fullD, 1);
        mbar_init(&fullW, 1);
        mbar_init(&mma1, 5);  // one issuing thread per accumulator
        mbar_init(&mma2, 2);
        mbar_init(&mma3, 2);
        mbar_fence_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem0 = tmem_s;
    const uint32_t tmem = tmem0 + ((uint32_t)((warp & 3) * 32) << 16);  // this warp's lane quadrant
    const int ch = tid & 127, qtr = tid >> 7;                             // channel (TMEM lane) and column quarter (16 columns)
    const uint32_t sb = smem_u32(dyn);

    const int n_units = p.NT * p.H;
    auto request_set = [&](size_t r, int set) {  // V'^T and dV'^T of unit record r (one thread)
        mbar_expect_tx(&fullA[set], 2 * 16384);
        tma_load_1d(dyn + VT + set * 16384, (const __nv_bfloat16*)(ws + L.U) + r * C * D, 16384, &fullA[set]);
        tma_load_1d(dyn + DVT + set * 16384, (const __nv_bfloat16*)(sc + L.dVn) + r * C * D, 16384, &fullA[set]);
    };
    auto request_state = [&](size_t r) {  // S0 and T (one thread)
        mbar_expect_tx(&fullS, 32768 + 8192);
        tma_load_1d(dyn + S0T, (const __nv_bfloat16*)(ws + L.S0) + r * D * D, 32768, &fullS);
        tma_load_1d(dyn + TT, (const __nv_bfloat16*)(ws + L.Tm) + r * C * C, 8192, &fullS);
    };
    auto request_dS = [&](size_t r) {  // (one thread)
        mbar_expect_tx(&fullD, 32768);
        tma_load_1d(dyn + DST, (const __nv_bfloat16*)(sc + L.dS) + r * D * D, 32768, &fullD);
    };
    auto request_dO = [&](const ChunkInfo& cn, int hu, int set) {  // dO rows of a unit into core-matrix layout (all threads; one cp.async group)
        __nv_bfloat16* sdo = reinterpret_cast<__nv_bfloat16*>(dyn + DOT + set * 16384);
        for (int qq = tid; qq < C * (D / 8); qq += NTHR) {
            const int i = qq >> 4, e8 = (qq & 15) * 8;
            const bool valid = i < cn.len;
            cp_async16_z(sdo + cm_idx(i, e8, D), dO + ((size_t)(cn.tok0 + (valid ? i : 0)) * p.H + hu) * D + e8, valid);
        }
    };

    uint32_t it = 0;
    float beta_nx = 0.f;
    bool ok = true, ahead = false, early = false;  // copies for the next unit are in flight
    UnitWalk uw;
    uw.init(blockIdx.x, gridDim.x, p.H);
    ChunkInfo ci = chunk_info(p, uw.c);
    for (; uw.unit < n_units; uw.next(), ++it) {
    const int set = it & 1;
    const uint32_t par = it & 1;
    const int c = uw.c, h = uw.head();
    const size_t rec = (size_t)c * p.H + h;
    UnitWalk un = uw;  // the next unit of this CTA
    un.next();
    const bool more = un.unit < n_units;
    ChunkInfo ci_nx = ci;
    ahead = early = false;
    // with the short convolution fused into the forward, p.v is the pre-convolution projection and
    // the convolved rows come from the forward's record
    const __nv_bfloat16* vrec = p.conv_q ? (const __nv_bfloat16*)(ws + L.Vc) + rec * C * D : nullptr;
    auto tok = [&](int i) { return ((size_t)(ci.tok0 + i) * p.H + h); };
    const float gam_c = tid < D ? ((const float*)(ws + L.gamC))[rec * D + tid] : 0.f;
    const uint32_t oVT = VT + set * 16384, oDVT = DVT + set * 16384, oDOT = DOT + set * 16384;

    KDA_PHASE_BEGIN();
    if (tid == 0) {
        if (it == 0) {
            request_set(rec, 0);
            request_state(rec);
        }
        request_dS(rec);
        mbar_expect_tx(&fullW, 16384);
        tma_load_1d(dyn + WT, (const __nv_bfloat16*)(ws + L.W) + rec * C * D, 16384, &fullW);
    }
    if (it == 0) {
        request_dO(ci, h, 0);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    {
        __nv_bfloat16* sv = reinterpret_cast<__nv_bfloat16*>(dyn + SV);
        for (int qq = tid; qq < C * (D / 8); qq += NTHR) {
            const int i = qq >> 4, e8 = (qq & 15) * 8;
            const bool valid = i < ci.len;
            cp_async16_z(sv + i * D + e8, vrec ? vrec + (valid ? i : 0) * D + e8 : v + tok(valid ? i : 0) * D + e8, valid);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (tid < C) sbeta[tid] = it == 0 ? ((const float*)(ws + L.aux))[rec * 3 * C + 2 * C + tid] : beta_nx;  // beta kept by the forward
        asm volatile("cp.async.wait_group 1;" ::: "memory");  // dO of this unit (requested one unit ago) has landed
        fence_async_smem();
    }
    ok = mbar_wait(&fullA[set], (it >> 1) & 1, p, 16);
    ok = mbar_wait(&fullS, par, p, 16) && ok;
    tc_fence_before();
    ok = __syncthreads_and(ok);
    KDA_PHASE(0);

    // ---- S1: lane 0 of warps 0..4 issues the product of one accumulator each (dKh waits for dS)
    if (lane == 0 && warp < 5 && ok) {
        tc_fence_after();
        constexpr uint32_t id_aqk = make_idesc(64, 64, false, true);
        constexpr uint32_t id_mm = make_idesc(128, 64, true, true);
        constexpr uint32_t id_mk = make_idesc(128, 64, true, false);
        constexpr uint32_t id_km = make_idesc(128, 64, false, true);
        if (warp == 0) {
#pragma unroll
            for (int s = 0; s < 8; ++s)  // dAqk = dO (K-major) * V' (MN-major view of V'^T)
                mma_ss(tmem0 + DAQK, make_desc(sb + oDOT + s * 256, 128, 2048), make_desc(sb + oVT + s * 2048, 1024, 128), id_aqk, s > 0);
        } else if (warp == 1) {
#pragma unroll
            for (int s = 0; s < 8; ++s)  // dWn^T = S0 (MN-major view of S0^T) * dV'^T (MN-major)
                mma_ss(tmem0 + DWN, make_desc(sb + S0T + s * 4096, 2048, 128), make_desc(sb + oDVT + s * 2048, 1024, 128), id_mm, s > 0);
        } else if (warp == 2) {
#pragma unroll
            for (int s = 0; s < 8; ++s)  // dQt^T = S0 * dO^T (K-major, rows = i)
                mma_ss(tmem0 + DQT, make_desc(sb + S0T + s * 4096, 2048, 128), make_desc(sb + oDOT + s * 256, 128, 2048), id_mk, s > 0);
        } else if (warp == 3) {
            if (mbar_wait(&fullD, par, p, 16)) {
#pragma unroll
                for (int s = 0; s < 8; ++s)  // dKh^T = dS * V'^T
                    mma_ss(tmem0 + DKH, make_desc(sb + DST + s * 4096, 2048, 128), make_desc(sb + oVT + s * 2048, 1024, 128), id_mm, s > 0);
            }
        } else {
#pragma unroll
            for (int s = 0; s < 4; ++s)  // dVb^T = dV'^T (K-major, rows = e) * T (MN-major, rows = j)
                mma_ss(tmem0 + DVB, make_desc(sb + oDVT + s * 256, 128, 1024), make_desc(sb + TT + s * 2048, 1024, 128), id_km, s > 0);
        }
        mma_commit(&mma1);
    }
    // the next unit's V'^T, dV'^T and dO go to the other operand set (its last readers were the previous unit's MMAs)
    if (more && ok) {
        ci_nx = chunk_info(p, un.c);
        if (tid == 5 * 32) request_set(un.rec(), set ^ 1);
        request_dO(ci_nx, un.head(), set ^ 1);
        if (tid < C) beta_nx = ((const float*)(ws + L.aux))[un.rec() * 3 * C + 2 * C + tid];  // (in a register until then)
        ahead = true;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");  // (an empty group when there is no next unit: the waits below count groups)
    ok = mbar_wait(&fullD, par, p, 16) && ok;
    {   // while the first MMA group runs:
        // dGamma_C[d] = sum_e dS[d][e] S0[d][e].  Both records are cm(e, d; 128): a warp reads, for one
        // octet of e, 8 rows x 4 channel groups = four contiguous 128-byte core matrices per load.
        const __nv_bfloat16* s0 = reinterpret_cast<const __nv_bfloat16*>(dyn + S0T);
        const __nv_bfloat16* ds = reinterpret_cast<const __nv_bfloat16*>(dyn + DST);
        const int e7 = lane & 7, d8 = 8 * (4 * (warp & 3) + (lane >> 3)), eh = warp >> 2;
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll 2
        for (int eo = 0; eo < 4; ++eo) {
            const int e = 8 * (4 * eh + eo) + e7;
            float a[8], b[8];
            bf16x8_to_f32(*reinterpret_cast<const uint4*>(ds + cm_idx(e, d8, D)), a);
            bf16x8_to_f32(*reinterpret_cast<const uint4*>(s0 + cm_idx(e, d8, D)), b);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = fmaf(a[j], b[j], acc[j]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 1);
            acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 2);
            acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 4);
        }
        if (e7 == 0) {
#pragma unroll
            for (int j = 0; j < 8; ++j) spart[128 * eh + d8 + j] = acc[j];
        }
    }
    ok = ok && mbar_wait(&mma1, par, p, 32);
    tc_fence_after();
    asm volatile("cp.async.wait_group 1;" ::: "memory");  // my share of the v rows has landed (the next unit's dO may still be on its way)
    ok = __syncthreads_and(ok);  // every warp is done reading dS: its tile becomes the staging area of dQt
    if constexpr (CONVB) {  // ... and, in its second half, receives rows 0 .. 63 of the v projection (zero where a row does not exist)
        if (ok) {
            __nv_bfloat16* sxv = reinterpret_cast<__nv_bfloat16*>(dyn + XVM);
            __nv_bfloat16* sxh = reinterpret_cast<__nv_bfloat16*>(dyn + XVH);
            for (int qq = tid; qq < C * (D / 8); qq += NTHR) {
                const int r = qq >> 4, e8 = (qq & 15) * 8;
                const bool valid = r < ci.len;
                cp_async16_z(sxv + r * D + e8, v + tok(valid ? r : 0) * D + e8, valid);
            }
            if (tid < 3 * (D / 8)) {  // rows -3 .. -1: they exist unless the chunk starts its sequence
                const int r = tid >> 4, e8 = (tid & 15) * 8;
                const bool valid = ci.lc > 0;
                cp_async16_z(sxh + r * D + e8, v + ((size_t)(ci.tok0 + (valid ? r - 3 : 0)) * p.H + h) * D + e8, valid);
            }
            if (tid >= 64 && tid < 64 + D) stage_taps(reinterpret_cast<float4*>(dyn + XTAPS) + tid - 64, p.conv_v, h, tid - 64, p.conv_ksize);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    KDA_PHASE(2);

    // ---- conversions after S1
    if (ok) {
        __nv_bfloat16* sdvb = reinterpret_cast<__nv_bfloat16*>(dyn + oDOT);
        __nv_bfloat16* sv = reinterpret_cast<__nv_bfloat16*>(dyn + SV);
        {
            const int i0 = 16 * qtr;
            uint32_t r[16], pk[8];
            tmem_ld16(tmem + DWN + i0, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 8; ++j) pk[j] = pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
            tmem_st8(tmem + WBF + i0 / 2, pk);
            tmem_ld16(tmem + DQT + i0, r);
            tmem_wait_ld();
            store_handover16(reinterpret_cast<__nv_bfloat16*>(dyn + DST), ch, i0, r);
            tmem_ld16(tmem + DKH + i0, r);
            tmem_wait_ld();
            store_handover16(reinterpret_cast<__nv_bfloat16*>(dyn + SKH), ch, i0, r);
            tmem_ld16(tmem + DVB + i0, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 8; ++j) pk[j] = pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
            *reinterpret_cast<uint4*>(sdvb + cm_idx(ch, i0, C)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            *reinterpret_cast<uint4*>(sdvb + cm_idx(ch, i0 + 8, C)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            float xv[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int i = i0 + j;
                const float x = __uint_as_float(r[j]);
                const float vv = __bfloat162float(sv[i * D + ch]);  // zero on padding rows
                sv[i * D + ch] = __float2bfloat16_rn(sbeta[i] * x);  // dv takes the place of v
                xv[j] = x * vv;
            }
            // beta row sums: over the 32 channels of the warp in registers, over the four channel groups below
            int rr;
            const float part = warp_sum16(xv, lane, rr);
            if (!(lane & 1)) srp[(warp & 3) * C + i0 + rr] = part;
        }
        // dAqk: rows of the M = 64 accumulator sit in lanes 0..15 of every warp's quadrant.  It leaves as
        // three BF16 tiles cm(i, j; 64) (24-bit split, strictly lower triangle) plus its diagonal
        {
            __nv_bfloat16* gAM = (__nv_bfloat16*)(sc + L.dAM) + rec * 6 * C * C;
            float* gAd = (float*)(sc + L.dAd) + rec * C;
            const int i = 16 * (warp & 3) + (lane & 15);
            const int j0 = 16 * qtr;
            uint32_t r[16];
            tmem_ld16(tmem + DAQK + j0, r);
            tmem_wait_ld();
            if (lane < 16) {
                float f[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    f[j] = (j0 + j < i) ? __uint_as_float(r[j]) : 0.f;
                    if (j0 + j == i) gAd[i] = __uint_as_float(r[j]);
                }
                store_split_row(gAM, i, j0, f);
            }
        }
        tmem_wait_st();
        fence_async_smem();
    }
    tc_fence_before();
    __syncthreads();
    if (!ok) {
    } else if (tid == 0) {
        tma_store_1d((__nv_bfloat16*)(sc + L.dQt) + rec * C * D, dyn + DST, C * D * 2);
        tma_store_1d((__nv_bfloat16*)(sc + L.dKh) + rec * C * D, dyn + SKH, C * D * 2);
        tma_store_commit();
    } else if (CONVB) {  // (dv stays on chip for the convolution backward below)
    } else if (maps.ok && ci.len == C) {  // dv: the whole tile with one bulk-tensor store
        if (tid == 64) {
            tma_store_tile(&maps.m[0], h * D, (int)ci.tok0, dyn + SV);
            tma_store_commit();
        }
    } else if (tid >= 64 && tid - 64 < ci.len) {
        const int i = tid - 64;
        tma_store_1d((__nv_bfloat16*)p.grad_v + tok(i) * D, dyn + SV + i * D * 2, D * 2);
        tma_store_commit();
    }
    KDA_PHASE(3);

    // ---- S2: two issuing threads (the products into dWn form one chain)
    if (lane == 0 && warp < 2 && ok) {
        tc_fence_after();
        constexpr uint32_t id_neg = make_idesc(128, 64, false, true, true);  // -WBF (TMEM) * T (MN-major)
        constexpr uint32_t id_mm = make_idesc(128, 64, true, true);
        if (warp == 0) {
#pragma unroll
            for (int s = 0; s < 4; ++s) mma_ts(tmem0 + DKB, tmem0 + WBF + s * 8, make_desc(sb + TT + s * 2048, 1024, 128), id_neg, s > 0);
        } else {
#pragma unroll
            for (int s = 0; s < 4; ++s) mma_ts(tmem0 + DWN, tmem0 + WBF + s * 8, make_desc(sb + TT + s * 2048, 1024, 128), id_neg, s > 0);
#pragma unroll
            for (int s = 0; s < 8; ++s)  // Z^T += S0 * dVb^T (MN-major B from cm(e, i; 64))
                mma_ss(tmem0 + DWN, make_desc(sb + S0T + s * 4096, 2048, 128), make_desc(sb + oDOT + s * 2048, 1024, 128), id_mm, true);
        }
        mma_commit(&mma2);
    }
    if constexpr (CONVB) {
        // meanwhile: backward of the short convolution of v.  dv (BF16, as the unfused path would store it) is
        // in shared memory; thread (channel, 16-row block) walks its rows, the four blocks' filter-gradient
        // shares meet in the (now dead) dV'^T tile, and dx goes out in place of dv.
        if (ok) {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();  // the projection rows have landed
            __nv_bfloat16* sv = reinterpret_cast<__nv_bfloat16*>(dyn + SV);
            float* sdw = reinterpret_cast<float*>(dyn + oDVT);  // [4][128][4]
            int c0s, ncs;
            seq_chunks(p, ci.seq, c0s, ncs);
            const bool has_next = ci.lc + 1 < ncs;
            float w4[4], dw[4] = {0.f, 0.f, 0.f, 0.f}, out[16];
            {
                const float4 t4 = reinterpret_cast<const float4*>(dyn + XTAPS)[ch];
                w4[0] = t4.x; w4[1] = t4.y; w4[2] = t4.z; w4[3] = t4.w;
            }
            float* cvh = (float*)(sc + L.cv_head) + ((rec * 3 + 2) * 3) * D;
            float* cvt = (float*)(sc + L.cv_tail) + ((rec * 3 + 2) * 3) * D;
            conv_bwd_block(reinterpret_cast<const __nv_bfloat16*>(dyn + XVH), reinterpret_cast<const __nv_bfloat16*>(dyn + XVM), sv, w4, ch,
                           qtr, cvh, cvt, dw, out);
            *reinterpret_cast<float4*>(sdw + (qtr * D + ch) * 4) = make_float4(dw[0], dw[1], dw[2], dw[3]);
            __syncthreads();  // every read of dv is done, the filter-gradient shares are visible
#pragma unroll
            for (int r = 0; r < 16; ++r) sv[(16 * qtr + r) * D + ch] = __float2bfloat16_rn(out[r]);
            if (qtr == 0) {
                float4 t = *reinterpret_cast<const float4*>(sdw + ch * 4);
#pragma unroll
                for (int b = 1; b < 4; ++b) {
                    const float4 u = *reinterpret_cast<const float4*>(sdw + (b * D + ch) * 4);
                    t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
                }
                *reinterpret_cast<float4*>((float*)(sc + L.cv_part) + ((rec * 3 + 2) * D + ch) * 4) = t;
            }
            fence_async_smem();
            __syncthreads();
            const int lim = has_next ? 61 : ci.len;  // rows 61..63 of a chunk with a successor wait for the fix-up
            if (tid >= 64 && tid - 64 < lim) {
                const int i = tid - 64;
                tma_store_1d((__nv_bfloat16*)p.grad_v + tok(i) * D, dyn + SV + i * D * 2, D * 2);
                tma_store_commit();
            }
        }
    }
    if (tid < C) srow[tid] = (srp[tid] + srp[C + tid]) + (srp[2 * C + tid] + srp[3 * C + tid]);
    KDA_PHASE(4);
    ok = ok && mbar_wait(&mma2, par, p, 32);
    tc_fence_after();
    ok = __syncthreads_and(ok);
    if (tid == 0 && more && ok) {  // S0 and T are dead: their tiles take the next unit's
        request_state(un.rec());
        early = true;
    }
    KDA_PHASE(5);
    if (ok && tid < C) ((float*)(sc + L.dbp))[rec * C + tid] = srow[tid];
    if (ok && tid < D) ((float*)(sc + L.gC))[rec * D + tid] = ((spart[tid] + spart[128 + tid]) + (spart[256 + tid] + spart[384 + tid])) * gam_c;

    // ---- conversions after S2
    if (ok) {
        __nv_bfloat16* sz = reinterpret_cast<__nv_bfloat16*>(dyn + oDVT);
        const int i0 = 16 * qtr;
        uint32_t r[16];
        tmem_ld16(tmem + DKB + i0, r);
        tmem_wait_ld();
        store_handover16(reinterpret_cast<__nv_bfloat16*>(dyn + DST + 16384), ch, i0, r);  // second half: dQt may still be leaving the first
        tmem_ld16(tmem + DWN + i0, r);
        tmem_wait_ld();
        *reinterpret_cast<uint4*>(sz + cm_idx(ch, i0, C)) =
            make_uint4(pack_bf16(__uint_as_float(r[0]), __uint_as_float(r[1])), pack_bf16(__uint_as_float(r[2]), __uint_as_float(r[3])),
                       pack_bf16(__uint_as_float(r[4]), __uint_as_float(r[5])), pack_bf16(__uint_as_float(r[6]), __uint_as_float(r[7])));
        *reinterpret_cast<uint4*>(sz + cm_idx(ch, i0 + 8, C)) =
            make_uint4(pack_bf16(__uint_as_float(r[8]), __uint_as_float(r[9])), pack_bf16(__uint_as_float(r[10]), __uint_as_float(r[11])),
                       pack_bf16(__uint_as_float(r[12]), __uint_as_float(r[13])), pack_bf16(__uint_as_float(r[14]), __uint_as_float(r[15])));
        fence_async_smem();
    }
    ok = ok && mbar_wait(&fullW, par, p, 16);  // W, for the last MMA group
    tc_fence_before();
    ok = __syncthreads_and(ok);
    if (tid == 0 && ok) {
        tma_store_1d((__nv_bfloat16*)(sc + L.dKb) + rec * C * D, dyn + DST + 16384, C * D * 2);
        tma_store_commit();
    }
    KDA_PHASE(6);

    // ---- S3: the two products of dMn go to two accumulators (the second one where dAqk was), one issuing thread each
    if (lane == 0 && warp < 2 && ok) {
        tc_fence_after();
        constexpr uint32_t id = make_idesc(64, 64, true, true);
        if (warp == 0) {
#pragma unroll
            for (int s = 0; s < 8; ++s)  // Z (MN-major view of Z^T) * W^T (MN-major view of the W^T record)
                mma_ss(tmem0 + DMN, make_desc(sb + oDVT + s * 2048, 1024, 128), make_desc(sb + WT + s * 2048, 1024, 128), id, s > 0);
        } else {
#pragma unroll
            for (int s = 0; s < 8; ++s)  // dVb * V'^T
                mma_ss(tmem0 + DAQK, make_desc(sb + oDOT + s * 2048, 1024, 128), make_desc(sb + oVT + s * 2048, 1024, 128), id, s > 0);
        }
        mma_commit(&mma3);
    }
    ok = ok && mbar_wait(&mma3, par, p, 32);
    tc_fence_after();
    KDA_PHASE(7);
    if (ok) {
        __nv_bfloat16* gMM = (__nv_bfloat16*)(sc + L.dAM) + rec * 6 * C * C + 3 * C * C;
        const int i = 16 * (warp & 3) + (lane & 15);
        const int j0 = 16 * qtr;
        uint32_t r[16], r2[16];
        tmem_ld16(tmem + DMN + j0, r);
        tmem_ld16(tmem + DAQK + j0, r2);
        tmem_wait_ld();
        if (lane < 16) {
            float f[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) f[j] = (j0 + j < i) ? -(__uint_as_float(r[j]) + __uint_as_float(r2[j])) : 0.f;
            store_split_row(gMM, i, j0, f);
        }
    }
    tma_store_wait_all();
    fence_async_smem();  // (the tiles this unit wrote are about to receive the next units' copies)
    tc_fence_before();
    ok = __syncthreads_and(ok);
    KDA_PHASE(8);
    if (!ok) break;  // a wait gave up (recorded in the status word): no further unit is started
    ci = ci_nx;
    }
    if (!ok) {  // the copies in flight for the next unit land before the CTA leaves
        if (ahead) mbar_wait(&fullA[(it + 1) & 1], ((it + 1) >> 1) & 1, p, 16);
        if (early) mbar_wait(&fullS, (it + 1) & 1, p, 16);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem0, TMEM_COLS);
}

cudaError_t launch_bwd_wy_tc(const KdaParams& p, cudaStream_t s) {
    const bool convb = p.grad_conv_q != nullptr;
    const int units = p.NT * p.H, sms = sm_count();
    RowMaps maps = {};
    maps.ok = !(p.flags & KDA_FLAG_ROW_COPIES) && make_row_map(&maps.m[0], p.grad_v, (long long)p.B * p.T, p.H, C);
    auto kern = convb ? kda_bwd_wy_tc_pf<true> : kda_bwd_wy_tc_pf<false>;
    const int smem = convb ? (int)bp::TOTAL_CONVB : (int)bp::TOTAL;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    kern<<<units < sms ? units : sms, bp::NTHR, smem, s>>>(p, maps);
    return cudaGetLastError();
}

}  // namespace kda

KDA_PHASE_EXPORT(kda_debug_phases_bwd_wy)
