// Recurrent (single-token) KDA step for decoding: one iteration of the reference recurrence
// (k3mini/model.py:121-128) per (sequence, head), FP32 state in and out.
//
//   S~ = diag(alpha) S          pred = k^T S~          S' = S~ + k (beta (v - pred))^T          o = scale S'^T q
//
// The step is pure HBM traffic (the dk x dv FP32 state is read once and written once, 2 x 64 KB per
// (sequence, head) at d = 128).  One CTA per (sequence, head): the state arrives in shared memory by
// one linear bulk TMA copy, is updated in place there and leaves by one bulk store; several CTAs
// per SM overlap each other's copies.  Thread (e, half) owns value column e and half of the key
// channels.  Both state layouts use conflict-free shared-memory accesses: [dk][dv] is read row by
// row (the lanes hold consecutive e), [dv][dk] along diagonals (lane e visits channel (j + e) mod dk
// in step j).
#include "kda_common.cuh"
#include "kda_tc.cuh"

namespace kda {

using namespace tc;

template <typename T, int D>
__global__ void __launch_bounds__(2 * D) kda_recurrent_step_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                                    const T* __restrict__ v, const T* __restrict__ g,
                                                                    const T* __restrict__ beta, const float* __restrict__ A_log,
                                                                    const float* __restrict__ dt_bias,
                                                                    const float* __restrict__ state_in, float* __restrict__ state_out,
                                                                    T* __restrict__ o, int H, int flags, float scale, int* status) {
    extern __shared__ __align__(128) unsigned char dyn[];
    float* S = reinterpret_cast<float*>(dyn);  // [D][D] in the caller's layout
    float* ska = S + D * D;                    // k_d alpha_d
    float* sal = ska + D;                      // alpha_d
    float* skk = sal + D;                      // k_d
    float* sqq = skk + D;                      // scale q_d
    float* spart = sqq + D;                    // [2][D]
    float* sred = spart + 2 * D;               // [2][2 * D / 32]
    __shared__ uint64_t bar;
    const int tid = threadIdx.x, e = tid & (D - 1), half = tid / D, warp = tid >> 5, lane = tid & 31;
    const int nh = blockIdx.x, h = nh % H;
    const bool l2 = flags & KDA_FLAG_QK_L2NORM, gate = flags & KDA_FLAG_GATE, sig = flags & KDA_FLAG_BETA_SIGMOID;
    const bool vfirst = flags & KDA_FLAG_STATE_V_FIRST;
    const size_t sbase = (size_t)nh * D * D;
    if (tid == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
        mbar_expect_tx(&bar, D * D * 4);
        tma_load_1d(S, state_in + sbase, D * D * 4, &bar);
    }
    // ---- prologue of the token while the state is on its way (k3mini/model.py:217-223)
    float qv = 0.f, kv = 0.f;
    if (half == 0) {
        qv = ldf(q + (size_t)nh * D + e);
        kv = ldf(k + (size_t)nh * D + e);
    }
    if (l2) {
        float sq2 = warp_sum(qv * qv), sk2 = warp_sum(kv * kv);
        if (lane == 0) {
            sred[warp] = sq2;
            sred[2 * D / 32 + warp] = sk2;
        }
    }
    __syncthreads();  // (also: the barrier initialisation is visible)
    if (half == 0) {
        if (l2) {
            float sq2 = 0.f, sk2 = 0.f;
#pragma unroll
            for (int w = 0; w < D / 32; ++w) {
                sq2 += sred[w];
                sk2 += sred[2 * D / 32 + w];
            }
            qv *= 1.f / fmaxf(sqrtf(sq2), 1e-6f);
            kv *= 1.f / fmaxf(sqrtf(sk2), 1e-6f);
            if (sizeof(T) == 2) {  // BF16 activations: the reference rounds the normalised rows back (model.py:218-219)
                qv = __bfloat162float(__float2bfloat16_rn(qv));
                kv = __bfloat162float(__float2bfloat16_rn(kv));
            }
        }
        float gl = ldf(g + (size_t)nh * D + e);
        if (gate) gl = -expf(A_log[h]) * softplus_f(gl + (dt_bias ? dt_bias[h * D + e] : 0.f));
        const float al = expf(gl);
        ska[e] = kv * al;
        sal[e] = al;
        skk[e] = kv;
        sqq[e] = scale * qv;
    }
    float b = ldf(beta + nh);
    if (sig) b = sigmoid_f(b);
    const float ve = ldf(v + (size_t)nh * D + e);
    const bool ok = mbar_wait(&bar, 0, status, 128);
    if (!__syncthreads_and(ok)) return;  // (no tensor memory, no store in flight: nothing to clean up)
    auto at = [&](int j) {  // step j of this thread: key channel and shared-memory index of S[d][e]
        const int d = vfirst ? (j + e) & (D - 1) : j;
        return make_int2(d, vfirst ? e * D + d : d * D + e);
    };
    const int j0 = half * (D / 2);
    {
        float pa = 0.f, pb = 0.f;
#pragma unroll 8
        for (int j = j0; j < j0 + D / 2; j += 2) {
            const int2 a = at(j), c = at(j + 1);
            pa = fmaf(ska[a.x], S[a.y], pa);
            pb = fmaf(ska[c.x], S[c.y], pb);
        }
        spart[half * D + e] = pa + pb;
    }
    __syncthreads();
    const float err = b * (ve - (spart[e] + spart[D + e]));
    {
        float oa = 0.f, ob = 0.f;
#pragma unroll 8
        for (int j = j0; j < j0 + D / 2; j += 2) {
            const int2 a = at(j), c = at(j + 1);
            const float s0 = fmaf(sal[a.x], S[a.y], skk[a.x] * err), s1 = fmaf(sal[c.x], S[c.y], skk[c.x] * err);
            S[a.y] = s0;
            S[c.y] = s1;
            oa = fmaf(sqq[a.x], s0, oa);
            ob = fmaf(sqq[c.x], s1, ob);
        }
        __syncthreads();  // every read of the partial predictions is done
        spart[half * D + e] = oa + ob;
    }
    fence_async_smem();
    __syncthreads();
    if (half == 0) stf(o + (size_t)nh * D + e, spart[e] + spart[D + e]);
    if (tid == 0) {
        tma_store_1d(state_out + sbase, S, D * D * 4);
        tma_store_commit();
        tma_store_wait_all();
    }
}

template <typename T, int D>
static cudaError_t launch_step(const void* q, const void* k, const void* v, const void* g, const void* beta, const float* A_log,
                               const float* dt_bias, const float* state_in, float* state_out, void* o, int N, int H, int flags,
                               float scale, int* status, cudaStream_t s) {
    constexpr size_t smem = (size_t)(D * D + 6 * D + 4 * (2 * D / 32)) * 4;
    auto kern = kda_recurrent_step_kernel<T, D>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    kern<<<N * H, 2 * D, smem, s>>>((const T*)q, (const T*)k, (const T*)v, (const T*)g, (const T*)beta, A_log, dt_bias, state_in,
                                    state_out, (T*)o, H, flags, scale, status);
    return cudaGetLastError();
}

}  // namespace kda

extern "C" int kda_recurrent_step(const void* q, const void* k, const void* v, const void* g, const void* beta,
                                  const float* A_log, const float* dt_bias, const float* state_in, float* state_out, void* o,
                                  int32_t N, int32_t H, int32_t dk, int32_t dv, int32_t dtype, int32_t flags, float scale,
                                  int32_t* status, void* stream) {
    using namespace kda;
    if (!q || !k || !v || !g || !beta || !state_in || !state_out || !o) return KDA_ERR_NULL;
    if ((flags & KDA_FLAG_GATE) && !A_log) return KDA_ERR_NULL;
    if (N <= 0 || H <= 0 || dk != dv || (dk != 64 && dk != 128)) return KDA_ERR_SHAPE;
    if (dtype != KDA_DTYPE_F32 && dtype != KDA_DTYPE_BF16) return KDA_ERR_DTYPE;
    if (((uintptr_t)state_in & 15) || ((uintptr_t)state_out & 15)) return KDA_ERR_ALIGN;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == KDA_DTYPE_F32)
        e = dk == 64 ? launch_step<float, 64>(q, k, v, g, beta, A_log, dt_bias, state_in, state_out, o, N, H, flags, scale, status, s)
                     : launch_step<float, 128>(q, k, v, g, beta, A_log, dt_bias, state_in, state_out, o, N, H, flags, scale, status, s);
    else
        e = dk == 64 ? launch_step<__nv_bfloat16, 64>(q, k, v, g, beta, A_log, dt_bias, state_in, state_out, o, N, H, flags, scale,
                                                      status, s)
                     : launch_step<__nv_bfloat16, 128>(q, k, v, g, beta, A_log, dt_bias, state_in, state_out, o, N, H, flags,
                                                       scale, status, s);
    return e == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}
