// bwd_intra (BF16 path, d = 128): the guarded-diagonal intra-chunk backward, the reverse
// cumulative sum of the gate gradient and the chain rule through gate / L2 norm / sigmoid.
// One CTA per (chunk, head), one thread per channel d, so that everything that runs along
// the token axis of one channel -- the pairwise decays, the cumulative sums -- is
// thread-local, and one warp covers exactly the [16 rows x 32 channels] tile on which the
// reference evaluates its span guard (experiments/kda_sm90/patch_fla_guarded_intra.py:35-63).
//
// With D_ij = 2^(G_i - G_j) per channel (i >= j inside the chunk), dA = dAqk (lower
// triangle), dM the gradient of I + diag(beta) L (strictly lower):
//   row side   a1_i = sum_{j<i} dA_ij k_j D_ij          a2_i = sum_{j<i} dM_ij k_j D_ij
//   col side   c1_j = sum_{i>j} (scale dA_ij q_i + beta_i dM_ij k_i) D_ij
// The chunk is cut into four 16-row blocks.  Off-diagonal block pairs always factorise
// D_ij = 2^(G_i - r) 2^(r - G_j) with r = G at the first row of the later block (both factors
// <= 1).  A diagonal block uses the midpoint factorisation 2^(G_i - m) 2^(m - G_j),
// m = (max + min) / 2 per channel, only if its tile passes the guard (per-channel monotone
// non-increasing, finite, max-over-channels span <= the runtime limit); otherwise every pair
// gets its own exp2.  A negative limit therefore gives the exact evaluation everywhere.
#include "kda_common.cuh"
#include "kda_tc.cuh"

namespace kda {

using namespace tc;

namespace bi {
constexpr int D = 128, NTHR = 256, B = 16, HB = 8;
constexpr uint32_t SQ = 0;                   // q^ bf16 [64][128]
constexpr uint32_t SK = SQ + 16384;          // k^ bf16 [64][128]
constexpr uint32_t SG = SK + 16384;          // G f32 [64][128]
constexpr uint32_t SDA = SG + 32768;         // dAqk f32 [64][64]
constexpr uint32_t SDM = SDA + 16384;        // dM   f32 [64][64]
constexpr uint32_t STG = SDM + 16384;        // staging f32 [3][16][128]: dq, dk, dbeta terms of one block
constexpr uint32_t PF = STG + 24576;         // bf16 [3][64][128]: dQt, dKh, dKb of the whole chunk
constexpr uint32_t SBETA = PF + 49152;       // f32 [64] 1/|q|, [64] 1/|k|, [64] beta, [64] dbeta
constexpr uint32_t SX = SBETA + 1024;        // f32 [2][2][128] block totals of dG, f32 [2][128] scratch
constexpr uint32_t SRED = SX + 3072;         // f32 [8]
constexpr uint32_t TOTAL = SRED + 64 + 256;
}  // namespace bi

// 256 threads: thread (gp, d) = (tid / 128, tid % 128) owns channel d and, inside every 16-row
// block, the 8 tokens 8 gp .. 8 gp + 7: their row sums a1, a2, their column sums c1 and their
// final assembly all stay in its registers.
// u[0..7] += dA[0..7] * qf + dM[0..7] * kf as packed two-wide FP32 FMAs (one issue slot per two
// products); dA and dM point at eight consecutive floats in shared memory, 16-byte aligned
__device__ __forceinline__ void col_accumulate(float2 (&u)[4], const float* dA, const float* dM, float qf, float kf) {
    const float4 a0 = *reinterpret_cast<const float4*>(dA), a4 = *reinterpret_cast<const float4*>(dA + 4);
    const float4 m0 = *reinterpret_cast<const float4*>(dM), m4 = *reinterpret_cast<const float4*>(dM + 4);
    const float2 q2 = make_float2(qf, qf), k2 = make_float2(kf, kf);
    u[0] = __ffma2_rn(make_float2(a0.x, a0.y), q2, __ffma2_rn(make_float2(m0.x, m0.y), k2, u[0]));
    u[1] = __ffma2_rn(make_float2(a0.z, a0.w), q2, __ffma2_rn(make_float2(m0.z, m0.w), k2, u[1]));
    u[2] = __ffma2_rn(make_float2(a4.x, a4.y), q2, __ffma2_rn(make_float2(m4.x, m4.y), k2, u[2]));
    u[3] = __ffma2_rn(make_float2(a4.z, a4.w), q2, __ffma2_rn(make_float2(m4.z, m4.w), k2, u[3]));
}

__global__ void __launch_bounds__(bi::NTHR, 1) kda_bwd_intra(const KdaParams p) {
    using namespace bi;
    extern __shared__ __align__(128) unsigned char dyn[];
    __shared__ uint64_t barA, barB;
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(dyn + SQ);
    __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(dyn + SK);
    float* sG = reinterpret_cast<float*>(dyn + SG);
    float* sdA = reinterpret_cast<float*>(dyn + SDA);
    float* sdM = reinterpret_cast<float*>(dyn + SDM);
    float* stg = reinterpret_cast<float*>(dyn + STG);
    const __nv_bfloat16* spf = reinterpret_cast<const __nv_bfloat16*>(dyn + PF);
    float* srq = reinterpret_cast<float*>(dyn + SBETA);  // aux record order: 1/|q|, 1/|k|, beta
    float* srk = srq + 64;
    float* sbeta = srq + 128;
    float* sdb = srq + 192;
    float* stotal = reinterpret_cast<float*>(dyn + SX);  // [parity][gp][d]
    float* sscr = stotal + 512;                          // [gp][d]
    float* sred = reinterpret_cast<float*>(dyn + SRED);
    float* sdiag = sred + 8;  // f32 [64]: diagonal of dAqk (cleared in sdA so that the pair loops need no mask)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, d = tid & 127, gp = tid >> 7;
    const int c = blockIdx.x / p.H, h = blockIdx.x % p.H;
    const ChunkInfo ci = chunk_info(p, c);
    const WsLayout L = ws_layout(p.NT, p.H, p.dk, p.dv, p.dtype);
    char* sc = (char*)p.bwd_scratch;
    const size_t rec = (size_t)c * p.H + h;
    const __nv_bfloat16* gdQt = (const __nv_bfloat16*)(sc + L.dQt) + rec * C * D;
    const __nv_bfloat16* gdKh = (const __nv_bfloat16*)(sc + L.dKh) + rec * C * D;
    const __nv_bfloat16* gdKb = (const __nv_bfloat16*)(sc + L.dKb) + rec * C * D;
    const bool l2 = p.flags & KDA_FLAG_QK_L2NORM, gate = p.flags & KDA_FLAG_GATE, sig = p.flags & KDA_FLAG_BETA_SIGMOID;
    const float scale = p.scale;
    const float expA = gate ? expf(p.A_log[h]) : 1.f;
    const float negA = -expA, rcpA = 1.f / expA;
    auto tok = [&](int i) { return ((size_t)(ci.tok0 + i) * p.H + h); };
    KDA_PHASE_BEGIN();
    // ---- everything the kernel reads arrives by bulk TMA: on barA what the pair sums need (G, the
    //      normalised q and k, the row norms and beta kept by the forward; dAqk and dM from bwd_wy),
    //      on barB the three [64][128] hand-over arrays that only the assembly needs
    if (tid == 0) {
        mbar_init(&barA, 1);
        mbar_init(&barB, 1);
        mbar_fence_init();
        const char* ws = (const char*)p.workspace;
        mbar_expect_tx(&barA, C * D * 4 + 2 * C * D * 2 + 2 * C * C * 4 + 3 * C * 4);
        tma_load_1d(sG, (const float*)(ws + L.Gc) + rec * C * D, C * D * 4, &barA);
        tma_load_1d(sQ, (const __nv_bfloat16*)(ws + L.Qn) + rec * C * D, C * D * 2, &barA);
        tma_load_1d(sK, (const __nv_bfloat16*)(ws + L.Kn) + rec * C * D, C * D * 2, &barA);
        tma_load_1d(sdA, (const float*)(sc + L.dAqk) + rec * C * C, C * C * 4, &barA);
        tma_load_1d(sdM, (const float*)(sc + L.dM) + rec * C * C, C * C * 4, &barA);
        tma_load_1d(srq, (const float*)(ws + L.aux) + rec * 3 * C, 3 * C * 4, &barA);  // 1/|q|, 1/|k|, beta
        mbar_expect_tx(&barB, 3 * C * D * 2);
        tma_load_1d(dyn + PF, gdQt, C * D * 2, &barB);
        tma_load_1d(dyn + PF + C * D * 2, gdKh, C * D * 2, &barB);
        tma_load_1d(dyn + PF + 2 * C * D * 2, gdKb, C * D * 2, &barB);
    }
    const int c8 = (tid & 15) * 8;
    if (tid < C) sdb[tid] = ((const float*)(sc + L.dbp))[rec * C + tid];
    __syncthreads();  // barrier initialisation is visible
    if (!mbar_wait(&barA, 0, p.status, 64)) return;  // uniform: every thread polls the same barrier
    KDA_PHASE(0);
    const float gl = sG[(C - 1) * D + d];
    KDA_PHASE(1);
    KDA_PHASE(2);

    if (tid < C) {
        sdiag[tid] = sdA[tid * C + tid];
        sdA[tid * C + tid] = 0.f;
    }
    __syncthreads();
    float carry = ((const float*)(sc + L.gC))[rec * D + d];
    float dA_acc = 0.f, dbias_acc = 0.f;
    __nv_bfloat16* dq_out = (__nv_bfloat16*)p.grad_q;
    __nv_bfloat16* dk_out = (__nv_bfloat16*)p.grad_k;
    __nv_bfloat16* dg_out = (__nv_bfloat16*)p.grad_g;
    const int h0 = HB * gp;  // first of my 8 tokens inside a block
    KDA_PHASE(3);

    for (int I = 3; I >= 0; --I) {
        float Gb[B], a1[HB], a2[HB], c1[HB], Gm[HB];
#pragma unroll
        for (int r = 0; r < B; ++r) Gb[r] = sG[(B * I + r) * D + d];
#pragma unroll
        for (int i = 0; i < HB; ++i) {
            a1[i] = 0.f;
            a2[i] = 0.f;
            c1[i] = 0.f;
            Gm[i] = gp ? Gb[HB + i] : Gb[i];
        }
        // guard of this block's diagonal tile (one tile = 16 rows x this warp's 32 channels)
        float mid;
        const bool guarded = guard_tile(Gb, p.guard_span, mid);
        // ---- row sums of my 8 tokens over the earlier blocks: k_j 2^(r - G_j), r = G at this block's first row
        for (int J = 0; J < I; ++J) {
            float kd[B];
#pragma unroll
            for (int j = 0; j < B; ++j) {
                const int jj = B * J + j;
                kd[j] = __bfloat162float(sK[jj * D + d]) * ex2_approx(Gb[0] - sG[jj * D + d]);
            }
#pragma unroll
            for (int i = 0; i < HB; ++i) {
                const int ii = B * I + h0 + i;
                float2 u1 = make_float2(0.f, 0.f), u2 = u1;  // even / odd j in the two halves
#pragma unroll
                for (int j4 = 0; j4 < B; j4 += 4) {
                    const float4 a = *reinterpret_cast<const float4*>(sdA + ii * C + B * J + j4);
                    const float4 m = *reinterpret_cast<const float4*>(sdM + ii * C + B * J + j4);
                    const float2 k01 = make_float2(kd[j4], kd[j4 + 1]), k23 = make_float2(kd[j4 + 2], kd[j4 + 3]);
                    u1 = __ffma2_rn(make_float2(a.x, a.y), k01, __ffma2_rn(make_float2(a.z, a.w), k23, u1));
                    u2 = __ffma2_rn(make_float2(m.x, m.y), k01, __ffma2_rn(make_float2(m.z, m.w), k23, u2));
                }
                const float Pi = ex2_approx(Gm[i] - Gb[0]);
                a1[i] = fmaf(Pi, u1.x + u1.y, a1[i]);
                a2[i] = fmaf(Pi, u2.x + u2.y, a2[i]);
            }
        }
        // ---- column sums of my 8 tokens over the later blocks: reference r' = G at their first row
        for (int Ip = I + 1; Ip < 4; ++Ip) {
            const float r2 = sG[(B * Ip) * D + d];
            float2 u[HB / 2];
#pragma unroll
            for (int j = 0; j < HB / 2; ++j) u[j] = make_float2(0.f, 0.f);
#pragma unroll
            for (int i = 0; i < B; ++i) {
                const int ii = B * Ip + i;
                const float Pi = ex2_approx(sG[ii * D + d] - r2);
                const float qp = scale * __bfloat162float(sQ[ii * D + d]) * Pi;
                const float kp = sbeta[ii] * __bfloat162float(sK[ii * D + d]) * Pi;
                col_accumulate(u, sdA + ii * C + B * I + h0, sdM + ii * C + B * I + h0, qp, kp);
            }
#pragma unroll
            for (int j = 0; j < HB; ++j) c1[j] = fmaf(ex2_approx(r2 - Gm[j]), j & 1 ? u[j >> 1].y : u[j >> 1].x, c1[j]);
        }
        // ---- diagonal block: pairs (i, j) with j < i, at least one of them mine
        {
            float kj[B], qs[B], kb[B];
#pragma unroll
            for (int r = 0; r < B; ++r) {
                const int rr = B * I + r;
                const float kk = __bfloat162float(sK[rr * D + d]);
                kj[r] = kk;
                qs[r] = scale * __bfloat162float(sQ[rr * D + d]);
                kb[r] = sbeta[rr] * kk;
            }
            if (guarded) {  // midpoint factorisation 2^(G_i - m) 2^(m - G_j), m = (max + min) / 2 per channel
#pragma unroll
                for (int r = 0; r < B; ++r) {
                    const float P = ex2_approx(Gb[r] - mid), N = ex2_approx(mid - Gb[r]);
                    kj[r] *= N;   // key side of the row sums
                    qs[r] *= P;   // row side of the column sums
                    kb[r] *= P;
                }
#pragma unroll
                for (int i = 0; i < HB; ++i) {  // dA, dM vanish for j >= i (the diagonal of dA was moved to sdiag)
                    const int ii = B * I + h0 + i;
                    float2 u1 = make_float2(0.f, 0.f), u2 = u1;
#pragma unroll
                    for (int j4 = 0; j4 < B; j4 += 4) {
                        const float4 a = *reinterpret_cast<const float4*>(sdA + ii * C + B * I + j4);
                        const float4 m = *reinterpret_cast<const float4*>(sdM + ii * C + B * I + j4);
                        const float2 k01 = make_float2(kj[j4], kj[j4 + 1]), k23 = make_float2(kj[j4 + 2], kj[j4 + 3]);
                        u1 = __ffma2_rn(make_float2(a.x, a.y), k01, __ffma2_rn(make_float2(a.z, a.w), k23, u1));
                        u2 = __ffma2_rn(make_float2(m.x, m.y), k01, __ffma2_rn(make_float2(m.z, m.w), k23, u2));
                    }
                    const float Pi = ex2_approx(Gm[i] - mid);
                    a1[i] = fmaf(Pi, u1.x + u1.y, a1[i]);
                    a2[i] = fmaf(Pi, u2.x + u2.y, a2[i]);
                }
                {  // column side: dA, dM vanish for i <= j
                    float2 u[HB / 2];
#pragma unroll
                    for (int j = 0; j < HB / 2; ++j) u[j] = make_float2(0.f, 0.f);
#pragma unroll
                    for (int i = 1; i < B; ++i) {
                        const int ii = B * I + i;
                        col_accumulate(u, sdA + ii * C + B * I + h0, sdM + ii * C + B * I + h0, qs[i], kb[i]);
                    }
#pragma unroll
                    for (int j = 0; j < HB; ++j) c1[j] = fmaf(ex2_approx(mid - Gm[j]), j & 1 ? u[j >> 1].y : u[j >> 1].x, c1[j]);
                }
            } else {  // one exp2 per pair
#pragma unroll
                for (int i = 0; i < HB; ++i) {
                    const int li = h0 + i, ii = B * I + li;
#pragma unroll
                    for (int j = 0; j < B - 1; ++j) {
                        const bool on = j < li;
                        const float kp = on ? kj[j] * ex2_approx(Gm[i] - Gb[j]) : 0.f;
                        a1[i] = fmaf(sdA[ii * C + B * I + j], kp, a1[i]);
                        a2[i] = fmaf(sdM[ii * C + B * I + j], kp, a2[i]);
                    }
                }
#pragma unroll
                for (int j = 0; j < HB; ++j) {
                    const int lj = h0 + j, jj = B * I + lj;
#pragma unroll
                    for (int i = 1; i < B; ++i) {
                        const bool on = i > lj;
                        const float e = on ? ex2_approx(Gb[i] - Gm[j]) : 0.f;
                        const float t = sdA[(B * I + i) * C + jj] * qs[i] + sdM[(B * I + i) * C + jj] * kb[i];
                        c1[j] = fmaf(t, e, c1[j]);
                    }
                }
            }
        }
        KDA_PHASE(4 + 4 * (3 - I));
        if (I == 3) {
            if (!mbar_wait(&barB, 0, p.status, 64)) return;
            // term of the last row: dGamma_C Gamma_C + sum_i dKh_i Kh_i (each group sums its 32 rows);
            // it joins the carry after the barrier that follows the assembly
            float s = 0.f;
#pragma unroll 8
            for (int r = 0; r < 32; ++r) {
                const int i = 32 * gp + r;
                s = fmaf(__bfloat162float(spf[(C + i) * D + d]), __bfloat162float(sK[i * D + d]) * ex2_approx(gl - sG[i * D + d]), s);
            }
            sscr[128 * gp + d] = s;
        }
        KDA_PHASE(5 + 4 * (3 - I));

        // ---- assembly of my 8 tokens, last first; run[i] = dG summed over the tokens >= i of my half
        float runl[HB];
        {
            float acc = 0.f;
#pragma unroll
            for (int i = HB - 1; i >= 0; --i) {
                const int li = h0 + i, ii = B * I + li;
                const float qi = __bfloat162float(sQ[ii * D + d]), ki = __bfloat162float(sK[ii * D + d]);
                const float bi_ = sbeta[ii];
                const float gam = ex2_approx(Gm[i]), eta = ex2_approx(gl - Gm[i]);
                const float dQt = __bfloat162float(spf[ii * D + d]), dKh = __bfloat162float(spf[(C + ii) * D + d]),
                            dKb = __bfloat162float(spf[(2 * C + ii) * D + d]);
                const float diag = scale * sdiag[ii];
                const float dq_in = scale * a1[i], dk_row = bi_ * a2[i], dKt = bi_ * dKb;
                stg[(0 * B + li) * D + d] = dq_in + diag * ki + scale * dQt * gam;
                stg[(1 * B + li) * D + d] = dk_row + c1[i] + diag * qi + dKt * gam + dKh * eta;
                stg[(2 * B + li) * D + d] = ki * a2[i] + dKb * (ki * gam);
                acc += qi * dq_in + ki * dk_row - ki * c1[i] + dQt * (scale * qi * gam) + dKt * (ki * gam) - dKh * (ki * eta);
                runl[i] = acc;
            }
            stotal[((I & 1) * 2 + gp) * D + d] = acc;
        }
        // gate chain for one half: base = everything after my half's last token
        auto finish = [&](float base) {
#pragma unroll
            for (int i = HB - 1; i >= 0; --i) {
                const int ii = B * I + h0 + i;
                if (ii < ci.len) {
                    const float run = base + runl[i];
                    const size_t off = tok(ii) * D + d;
                    if (gate) {
                        // per-token log decay g = (G_i - G_{i-1}) ln 2; sigmoid(x + b) = 1 - exp(-softplus) = -expm1(g / e^A)
                        const float gprev = ii > 0 ? (i > 0 ? Gm[i - 1] : sG[(ii - 1) * D + d]) : 0.f;
                        const float gnat = (Gm[i] - gprev) * 0.6931471805599453f;
                        dA_acc = fmaf(run, gnat, dA_acc);
                        const float dx = run * negA * (1.f - ex2_approx(gnat * rcpA * LOG2E));
                        dbias_acc += dx;
                        dg_out[off] = __float2bfloat16_rn(dx);
                    } else {
                        dg_out[off] = __float2bfloat16_rn(run);
                    }
                }
            }
        };
        __syncthreads();
        KDA_PHASE(6 + 4 * (3 - I));
        if (I == 3) carry += sscr[d] + sscr[128 + d];
        const float upper = stotal[((I & 1) * 2 + 1) * D + d];
        finish(gp == 0 ? carry + upper : carry);
        carry += upper + stotal[((I & 1) * 2 + 0) * D + d];
        // ---- row-wise (one half warp per token): L2-norm chain, beta gradient, 16-byte stores
        {
            const int i = tid >> 4, ii = B * I + i;
            float dq8[8], dk8[8], q8[8], k8[8], db = 0.f, dotq = 0.f, dotk = 0.f;
            bf16x8_to_f32(*reinterpret_cast<const uint4*>(sQ + ii * D + c8), q8);
            bf16x8_to_f32(*reinterpret_cast<const uint4*>(sK + ii * D + c8), k8);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                dq8[j] = stg[(0 * B + i) * D + c8 + j];
                dk8[j] = stg[(1 * B + i) * D + c8 + j];
                db += stg[(2 * B + i) * D + c8 + j];
                dotq = fmaf(q8[j], dq8[j], dotq);
                dotk = fmaf(k8[j], dk8[j], dotk);
            }
            db = half_warp_sum(db);
            if (l2) {
                dotq = half_warp_sum(dotq);
                dotk = half_warp_sum(dotk);
                const float rq = srq[ii], rk = srk[ii];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    dq8[j] = (dq8[j] - q8[j] * dotq) * rq;
                    dk8[j] = (dk8[j] - k8[j] * dotk) * rk;
                }
            }
            if (ii < ci.len) {
                const size_t row = tok(ii);
                *reinterpret_cast<uint4*>(dq_out + row * D + c8) = f32_to_bf16x8(dq8);
                *reinterpret_cast<uint4*>(dk_out + row * D + c8) = f32_to_bf16x8(dk8);
                if ((tid & 15) == 0) {
                    float b = sbeta[ii], v = sdb[ii] + db;
                    if (sig) v *= b * (1.f - b);
                    ((__nv_bfloat16*)p.grad_beta)[row] = __float2bfloat16_rn(v);
                }
            }
        }
        __syncthreads();  // the staging buffer may be overwritten
        KDA_PHASE(7 + 4 * (3 - I));
    }
    if (gate) {
        sscr[128 * gp + d] = dbias_acc;
        dA_acc = warp_sum(dA_acc);
        if (lane == 0) sred[warp] = dA_acc;
        __syncthreads();
        if (gp == 0) ((float*)(sc + L.dbias_part))[rec * D + d] = sscr[d] + sscr[128 + d];
        if (tid == 0) {
            float t = 0.f;
            for (int w = 0; w < 8; ++w) t += sred[w];
            ((float*)(sc + L.dA_part))[rec] = t;
        }
    }
}

cudaError_t launch_bwd_intra(const KdaParams& p, cudaStream_t s) {
    cudaError_t e = cudaFuncSetAttribute(kda_bwd_intra, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bi::TOTAL);
    if (e != cudaSuccess) return e;
    kda_bwd_intra<<<p.NT * p.H, bi::NTHR, bi::TOTAL, s>>>(p);
    return cudaGetLastError();
}


// ---------------------------------------------------------------------------------------
// Stand-alone form of the guarded diagonal tile with the reference's own interface
// (experiments/kda_sm90/guarded_diagonal_oracle.py:57-180): gate, q, k [N,16,32], beta [N,16],
// dAqk, dAkk [N,16,16] -> dq, dk, dkt [N,16,32], hits [N].  One warp per tile, one lane per
// channel; same guard (guard_tile) and the same two evaluation rules as kda_bwd_intra.
//   dq[i]  = sum_{j<=i} dAqk[i][j] k[j] 2^(g_i-g_j)       dk[i] = sum_{j<=i} dAkk[i][j] k[j] 2^(g_i-g_j)
//   dkt[i] = sum_{j>=i} (dAqk[i][j] q[j] + dAkk[i][j] beta[j] k[j]) 2^(g_j-g_i)
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(32) kda_diag_tile_kernel(const float* __restrict__ gate, const float* __restrict__ q,
                                                           const float* __restrict__ k, const float* __restrict__ beta,
                                                           const float* __restrict__ dAqk, const float* __restrict__ dAkk,
                                                           float* __restrict__ dq, float* __restrict__ dk,
                                                           float* __restrict__ dkt, int* __restrict__ hits, float limit) {
    const int n = blockIdx.x, ch = threadIdx.x;
    float G[16], Q[16], K[16], Bt[16];
#pragma unroll
    for (int r = 0; r < 16; ++r) {
        G[r] = gate[(n * 16 + r) * 32 + ch];
        Q[r] = q[(n * 16 + r) * 32 + ch];
        K[r] = k[(n * 16 + r) * 32 + ch];
        Bt[r] = beta[n * 16 + r];
    }
    float mid;
    const bool pass = guard_tile(G, limit, mid);
    if (ch == 0) hits[n] = pass ? 1 : 0;
    const float* A = dAqk + n * 256;
    const float* M = dAkk + n * 256;
    float P[16], N[16];
    if (pass) {
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            P[r] = ex2_approx(G[r] - mid);
            N[r] = ex2_approx(mid - G[r]);
        }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float sq = 0.f, sk = 0.f, st = 0.f;
        if (pass) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if (j <= i) {
                    sq = fmaf(A[i * 16 + j], K[j] * N[j], sq);
                    sk = fmaf(M[i * 16 + j], K[j] * N[j], sk);
                }
                if (j >= i) st = fmaf(A[i * 16 + j], Q[j] * P[j], fmaf(M[i * 16 + j], Bt[j] * K[j] * P[j], st));
            }
            sq *= P[i];
            sk *= P[i];
            st *= N[i];
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if (j <= i) {
                    const float kp = K[j] * ex2_approx(G[i] - G[j]);
                    sq = fmaf(A[i * 16 + j], kp, sq);
                    sk = fmaf(M[i * 16 + j], kp, sk);
                }
                if (j >= i) st = fmaf(A[i * 16 + j] * Q[j] + M[i * 16 + j] * (Bt[j] * K[j]), ex2_approx(G[j] - G[i]), st);
            }
        }
        dq[(n * 16 + i) * 32 + ch] = sq;
        dk[(n * 16 + i) * 32 + ch] = sk;
        dkt[(n * 16 + i) * 32 + ch] = st;
    }
}

}  // namespace kda

extern "C" int kda_guarded_diagonal_tiles(const float* gate, const float* q, const float* k, const float* beta,
                                          const float* dAqk, const float* dAkk, float* dq, float* dk, float* dkt, int* hits,
                                          int n_tiles, float max_log2_span, void* stream) {
    if (!gate || !q || !k || !beta || !dAqk || !dAkk || !dq || !dk || !dkt || !hits) return KDA_ERR_NULL;
    if (n_tiles <= 0) return KDA_ERR_SHAPE;
    if (!(max_log2_span < 0.f) && !(isfinite(max_log2_span) && max_log2_span < 252.f)) return KDA_ERR_GUARD;
    kda::kda_diag_tile_kernel<<<n_tiles, 32, 0, (cudaStream_t)stream>>>(gate, q, k, beta, dAqk, dAkk, dq, dk, dkt, hits,
                                                                       max_log2_span);
    return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

KDA_PHASE_EXPORT(kda_debug_phases_bwd_intra)
