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
constexpr int D = 128, NTHR = 128, B = 16;
constexpr uint32_t SQ = 0;                   // q^ bf16 [64][128]
constexpr uint32_t SK = SQ + 16384;          // k^ bf16 [64][128]
constexpr uint32_t SG = SK + 16384;          // G f32 [64][128]
constexpr uint32_t SDA = SG + 32768;         // dAqk f32 [64][64]
constexpr uint32_t SDM = SDA + 16384;        // dM   f32 [64][64]
constexpr uint32_t SC1 = SDM + 16384;        // c1 f32 [64][128]
constexpr uint32_t STG = SC1 + 32768;        // staging f32 [3][16][128]: dq, dk, dbeta terms
constexpr uint32_t SBETA = STG + 24576;      // f32 [64] beta, [64] 1/|q|, [64] 1/|k|, [64] dbeta
constexpr uint32_t SRED = SBETA + 1024;      // f32 [8]
constexpr uint32_t TOTAL = SRED + 64;
}  // namespace bi

__global__ void __launch_bounds__(bi::NTHR, 1) kda_bwd_intra(const KdaParams p) {
    using namespace bi;
    extern __shared__ __align__(128) unsigned char dyn[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(dyn + SQ);
    __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(dyn + SK);
    float* sG = reinterpret_cast<float*>(dyn + SG);
    float* sdA = reinterpret_cast<float*>(dyn + SDA);
    float* sdM = reinterpret_cast<float*>(dyn + SDM);
    float* sC1 = reinterpret_cast<float*>(dyn + SC1);
    float* stg = reinterpret_cast<float*>(dyn + STG);
    float* sbeta = reinterpret_cast<float*>(dyn + SBETA);
    float* srq = sbeta + 64;
    float* srk = sbeta + 128;
    float* sdb = sbeta + 192;
    float* sred = reinterpret_cast<float*>(dyn + SRED);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, d = tid;
    const int c = blockIdx.x / p.H, h = blockIdx.x % p.H;
    const ChunkInfo ci = chunk_info(p, c);
    const WsLayout L = ws_layout(p.NT, p.H, p.dk, p.dv, p.dtype);
    char* sc = (char*)p.bwd_scratch;
    const size_t rec = (size_t)c * p.H + h;
    const __nv_bfloat16* q = (const __nv_bfloat16*)p.q;
    const __nv_bfloat16* k = (const __nv_bfloat16*)p.k;
    const __nv_bfloat16* g = (const __nv_bfloat16*)p.g;
    const __nv_bfloat16* beta = (const __nv_bfloat16*)p.beta;
    const float* gdQt = (const float*)(sc + L.dQt) + rec * C * D;
    const float* gdKh = (const float*)(sc + L.dKh) + rec * C * D;
    const float* gdKb = (const float*)(sc + L.dKb) + rec * C * D;
    const bool l2 = p.flags & KDA_FLAG_QK_L2NORM, gate = p.flags & KDA_FLAG_GATE, sig = p.flags & KDA_FLAG_BETA_SIGMOID;
    const float scale = p.scale;
    const float negA = gate ? -expf(p.A_log[h]) : 0.f;
    const float bias = (gate && p.dt_bias) ? p.dt_bias[h * D + d] : 0.f;
    auto tok = [&](int i) { return ((size_t)(ci.tok0 + i) * p.H + h); };

    // ---- 0a: q, k row-wise (half warp per row): L2 norm, BF16 copies; beta
    {
        const int hw = tid >> 4, c8 = (tid & 15) * 8;
        for (int m = 0; m < 8; ++m) {
            const int i = hw + 8 * m;
            const bool valid = i < ci.len;
            const size_t row = tok(valid ? i : 0);
            float qf[8], kf[8];
            const uint4 z = make_uint4(0, 0, 0, 0);
            bf16x8_to_f32(valid ? *reinterpret_cast<const uint4*>(q + row * D + c8) : z, qf);
            bf16x8_to_f32(valid ? *reinterpret_cast<const uint4*>(k + row * D + c8) : z, kf);
            float rq = 1.f, rk = 1.f;
            if (l2) {
                float ssq = 0.f, ssk = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    ssq += qf[j] * qf[j];
                    ssk += kf[j] * kf[j];
                }
                ssq = half_warp_sum(ssq);
                ssk = half_warp_sum(ssk);
                rq = 1.f / fmaxf(sqrtf(ssq), 1e-6f);
                rk = 1.f / fmaxf(sqrtf(ssk), 1e-6f);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    qf[j] *= rq;
                    kf[j] *= rk;
                }
            }
            *reinterpret_cast<uint4*>(sQ + i * D + c8) = f32_to_bf16x8(qf);
            *reinterpret_cast<uint4*>(sK + i * D + c8) = f32_to_bf16x8(kf);
            if ((tid & 15) == 0) {
                float b = 0.f;
                if (valid) {
                    b = __bfloat162float(beta[row]);
                    if (sig) b = sigmoid_f(b);
                }
                sbeta[i] = b;
                srq[i] = rq;
                srk[i] = rk;
            }
        }
    }
    // ---- 0b: gate channel-wise -> cumulative log2 decay G
    {
        float run = 0.f;
#pragma unroll 8
        for (int i = 0; i < C; ++i) {
            float gl = 0.f;
            if (i < ci.len) {
                const float x = __bfloat162float(g[tok(i) * D + d]);
                gl = gate ? negA * softplus_f(x + bias) : x;
            }
            run += gl * LOG2E;
            sG[i * D + d] = run;
        }
    }
    // ---- 0c: dAqk, dM (FP32 row-major) and the beta gradient collected by bwd_wy
    {
        const float4* gdA = reinterpret_cast<const float4*>((const float*)(sc + L.dAqk) + rec * C * C);
        const float4* gdM = reinterpret_cast<const float4*>((const float*)(sc + L.dM) + rec * C * C);
        for (int qq = tid; qq < C * C / 4; qq += NTHR) {
            reinterpret_cast<float4*>(sdA)[qq] = gdA[qq];
            reinterpret_cast<float4*>(sdM)[qq] = gdM[qq];
        }
        if (tid < C) sdb[tid] = ((const float*)(sc + L.dbp))[rec * C + tid];
    }
    __syncthreads();

    // ---- guard of the four diagonal tiles (one tile = 16 rows x this warp's 32 channels)
    unsigned guard_mask = 0;
    {
        const float thr = p.guard_span;
#pragma unroll
        for (int I = 0; I < 4; ++I) {
            float gmax = -INFINITY, gmin = INFINITY, prev = INFINITY;
            bool good = true;
#pragma unroll
            for (int r = 0; r < B; ++r) {
                const float x = sG[(B * I + r) * D + d];
                good = good && (x <= prev) && isfinite(x);
                prev = x;
                gmax = fmaxf(gmax, x);
                gmin = fminf(gmin, x);
            }
            float span = gmax - gmin;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) span = fmaxf(span, __shfl_xor_sync(0xffffffffu, span, o));
            const bool pass = __all_sync(0xffffffffu, good) && isfinite(span) && span <= thr;
            if (pass) guard_mask |= 1u << I;
        }
    }

    // decays of one diagonal block: e[i][j] for j < i, i.e. e_idx(i, j) = i (i - 1) / 2 + j
    // (kept implicit: the two passes below recompute them the same way)
    auto diag_factors = [&](int I, const float (&Gb)[B], float (&P)[B], float (&N)[B]) {
        float gmax = Gb[0], gmin = Gb[0];
#pragma unroll
        for (int r = 1; r < B; ++r) {
            gmax = fmaxf(gmax, Gb[r]);
            gmin = fminf(gmin, Gb[r]);
        }
        const float m = 0.5f * (gmax + gmin);
#pragma unroll
        for (int r = 0; r < B; ++r) {
            P[r] = exp2f(Gb[r] - m);
            N[r] = exp2f(m - Gb[r]);
        }
        (void)I;
    };

    // ---- pass C: column sums c1_j, block by block
    for (int J = 0; J < 4; ++J) {
        float c1[B], Gj[B];
#pragma unroll
        for (int j = 0; j < B; ++j) {
            c1[j] = 0.f;
            Gj[j] = sG[(B * J + j) * D + d];
        }
        {  // diagonal block: pairs i > j
            float qs[B], kb[B];
#pragma unroll
            for (int i = 0; i < B; ++i) {
                qs[i] = scale * __bfloat162float(sQ[(B * J + i) * D + d]);
                kb[i] = sbeta[B * J + i] * __bfloat162float(sK[(B * J + i) * D + d]);
            }
            if ((guard_mask >> J) & 1) {
                float P[B], N[B];
                diag_factors(J, Gj, P, N);
#pragma unroll
                for (int i = 1; i < B; ++i)
#pragma unroll
                    for (int j = 0; j < i; ++j) {
                        const float t = sdA[(B * J + i) * C + B * J + j] * qs[i] + sdM[(B * J + i) * C + B * J + j] * kb[i];
                        c1[j] = fmaf(t, P[i] * N[j], c1[j]);
                    }
            } else {
#pragma unroll
                for (int i = 1; i < B; ++i)
#pragma unroll
                    for (int j = 0; j < i; ++j) {
                        const float t = sdA[(B * J + i) * C + B * J + j] * qs[i] + sdM[(B * J + i) * C + B * J + j] * kb[i];
                        c1[j] = fmaf(t, exp2f(Gj[i] - Gj[j]), c1[j]);
                    }
            }
        }
        for (int I = J + 1; I < 4; ++I) {  // later blocks, reference r = G at their first row
            const float r = sG[(B * I) * D + d];
            float N[B];
#pragma unroll
            for (int j = 0; j < B; ++j) N[j] = exp2f(r - Gj[j]);
#pragma unroll
            for (int i = 0; i < B; ++i) {
                const int ii = B * I + i;
                const float Pi = exp2f(sG[ii * D + d] - r);
                const float qs = scale * __bfloat162float(sQ[ii * D + d]) * Pi;
                const float kb = sbeta[ii] * __bfloat162float(sK[ii * D + d]) * Pi;
#pragma unroll
                for (int j = 0; j < B; ++j) {
                    const float t = sdA[ii * C + B * J + j] * qs + sdM[ii * C + B * J + j] * kb;
                    c1[j] = fmaf(t, N[j], c1[j]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < B; ++j) sC1[(B * J + j) * D + d] = c1[j];
    }

    // ---- term of the last row: sum_i dKh_i Kh_i + dGamma_C Gamma_C
    const float gl = sG[(C - 1) * D + d];
    float run = ((const float*)(sc + L.gC))[rec * D + d];
    {
        float s = 0.f;
#pragma unroll 8
        for (int i = 0; i < C; ++i)
            s = fmaf(gdKh[i * D + d], __bfloat162float(sK[i * D + d]) * exp2f(gl - sG[i * D + d]), s);
        run += s;
    }

    // ---- pass R: row sums a1_i, a2_i per block (last block first) and the final assembly
    float dA_acc = 0.f, dbias_acc = 0.f;
    __nv_bfloat16* dq_out = (__nv_bfloat16*)p.grad_q;
    __nv_bfloat16* dk_out = (__nv_bfloat16*)p.grad_k;
    __nv_bfloat16* dg_out = (__nv_bfloat16*)p.grad_g;
    for (int I = 3; I >= 0; --I) {
        float a1[B], a2[B], Gi[B];
#pragma unroll
        for (int i = 0; i < B; ++i) {
            a1[i] = 0.f;
            a2[i] = 0.f;
            Gi[i] = sG[(B * I + i) * D + d];
        }
        {  // earlier blocks
            float P[B];
#pragma unroll
            for (int i = 0; i < B; ++i) P[i] = exp2f(Gi[i] - Gi[0]);
            for (int J = 0; J < I; ++J) {
#pragma unroll
                for (int j = 0; j < B; ++j) {
                    const int jj = B * J + j;
                    const float kd = __bfloat162float(sK[jj * D + d]) * exp2f(Gi[0] - sG[jj * D + d]);
#pragma unroll
                    for (int i = 0; i < B; ++i) {
                        const float kp = kd * P[i];
                        a1[i] = fmaf(sdA[(B * I + i) * C + jj], kp, a1[i]);
                        a2[i] = fmaf(sdM[(B * I + i) * C + jj], kp, a2[i]);
                    }
                }
            }
        }
        {  // diagonal block: pairs j < i
            float kj[B];
#pragma unroll
            for (int j = 0; j < B; ++j) kj[j] = __bfloat162float(sK[(B * I + j) * D + d]);
            if ((guard_mask >> I) & 1) {
                float P[B], N[B];
                diag_factors(I, Gi, P, N);
#pragma unroll
                for (int i = 1; i < B; ++i)
#pragma unroll
                    for (int j = 0; j < i; ++j) {
                        const float kp = kj[j] * (P[i] * N[j]);
                        a1[i] = fmaf(sdA[(B * I + i) * C + B * I + j], kp, a1[i]);
                        a2[i] = fmaf(sdM[(B * I + i) * C + B * I + j], kp, a2[i]);
                    }
            } else {
#pragma unroll
                for (int i = 1; i < B; ++i)
#pragma unroll
                    for (int j = 0; j < i; ++j) {
                        const float kp = kj[j] * exp2f(Gi[i] - Gi[j]);
                        a1[i] = fmaf(sdA[(B * I + i) * C + B * I + j], kp, a1[i]);
                        a2[i] = fmaf(sdM[(B * I + i) * C + B * I + j], kp, a2[i]);
                    }
            }
        }
        // assembly of the 16 tokens of this block, last token first (running suffix sum of dG)
#pragma unroll
        for (int i = B - 1; i >= 0; --i) {
            const int ii = B * I + i;
            const float qi = __bfloat162float(sQ[ii * D + d]), ki = __bfloat162float(sK[ii * D + d]);
            const float bi_ = sbeta[ii];
            const float gam = exp2f(Gi[i]), eta = exp2f(gl - Gi[i]);
            const float dQt = gdQt[ii * D + d], dKh = gdKh[ii * D + d], dKb = gdKb[ii * D + d];
            const float c1 = sC1[ii * D + d];
            const float diag = scale * sdA[ii * C + ii];
            const float dq_in = scale * a1[i], dk_row = bi_ * a2[i], dKt = bi_ * dKb;
            const float dqv = dq_in + diag * ki + scale * dQt * gam;
            const float dkv = dk_row + c1 + diag * qi + dKt * gam + dKh * eta;
            const float dG = qi * dq_in + ki * dk_row - ki * c1 + dQt * (scale * qi * gam) + dKt * (ki * gam) - dKh * (ki * eta);
            stg[(0 * B + i) * D + d] = dqv;
            stg[(1 * B + i) * D + d] = dkv;
            stg[(2 * B + i) * D + d] = ki * a2[i] + dKb * (ki * gam);
            run += dG;
            if (ii < ci.len) {
                const size_t off = tok(ii) * D + d;
                if (gate) {
                    const float z = __bfloat162float(g[off]) + bias;
                    dA_acc = fmaf(run, negA * softplus_f(z), dA_acc);
                    const float dx = run * negA * sigmoid_f(z);
                    dbias_acc += dx;
                    dg_out[off] = __float2bfloat16_rn(dx);
                } else {
                    dg_out[off] = __float2bfloat16_rn(run);
                }
            }
        }
        __syncthreads();
        {  // row-wise: L2-norm chain, beta gradient, 16-byte stores
            const int hw = tid >> 4, c8 = (tid & 15) * 8;
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                const int i = hw + 8 * m, ii = B * I + i;
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
        }
        __syncthreads();
    }
    if (gate) {
        ((float*)(sc + L.dbias_part))[rec * D + d] = dbias_acc;
        dA_acc = warp_sum(dA_acc);
        if (lane == 0) sred[warp] = dA_acc;
        __syncthreads();
        if (tid == 0) ((float*)(sc + L.dA_part))[rec] = sred[0] + sred[1] + sred[2] + sred[3];
    }
}

cudaError_t launch_bwd_intra(const KdaParams& p, cudaStream_t s) {
    cudaError_t e = cudaFuncSetAttribute(kda_bwd_intra, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bi::TOTAL);
    if (e != cudaSuccess) return e;
    kda_bwd_intra<<<p.NT * p.H, bi::NTHR, bi::TOTAL, s>>>(p);
    return cudaGetLastError();
}

}  // namespace kda
