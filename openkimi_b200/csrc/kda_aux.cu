// HBM-bound companions of the KDA op inside the KimiDeltaAttention sublayer:
// causal depthwise short convolution + SiLU (k3mini/model.py:76-88) and the headwise
// RMSNorm * sigmoid(gate) output stage (k3mini/model.py:91-98).  Both are single passes
// with 16-byte vector accesses; parameter gradients are reduced in a fixed order.
#include <mutex>

#include "kda_common.cuh"
#include "kda_conv_bwd.cuh"

namespace kda {

// Scratch of kda_short_conv_bwd_static: the per-token-group partial sums of the filter
// gradient, [CONV_STATIC_PARTIALS][C * ksize] floats, resident in every GPU that loads the
// library (2 MiB) from load until exit.  In host code this name is only a handle for
// cudaGetSymbolAddress -- it is not a device address and must never be handed to a kernel.
constexpr int CONV_STATIC_PARTIALS = 64;
constexpr int CONV_STATIC_MAX_WEIGHTS = 8192;  // C * ksize, e.g. 2048 channels with 4 taps
static __device__ __align__(256) float g_conv_static_partial[CONV_STATIC_PARTIALS * CONV_STATIC_MAX_WEIGHTS];

template <typename T> struct Vec;
template <> struct Vec<float> {
    static constexpr int N = 4;
    using raw = float4;
    __device__ static void load(const float* p, float (&v)[4]) {
        float4 r = *reinterpret_cast<const float4*>(p);
        v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
    }
    __device__ static void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) {
        uint4 r = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
    __device__ static void store(__nv_bfloat16* p, const float (&v)[8]) {
        uint4 r;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = r;
    }
};

constexpr int CONV_TT = 16;  // tokens per thread tile
constexpr int CONV_KMAX = 4;

// index of the document that contains flattened token t (fixed length: t / T)
__device__ __forceinline__ int doc_of(const int64_t* cu, int N, long long t, int T) {
    if (!cu) return (int)(t / T);
    int lo = 0, hi = N;  // cu[lo] <= t < cu[hi]
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (cu[mid] <= t) lo = mid; else hi = mid;
    }
    return lo;
}


// the filter padded to four taps: tap j multiplies x[t - 3 + j]
template <int V>
__device__ __forceinline__ void load_taps(const float* __restrict__ w, int c0, int K, float (&wt)[CONV_KMAX][V]) {
#pragma unroll
    for (int j = 0; j < CONV_KMAX; ++j)
#pragma unroll
        for (int i = 0; i < V; ++i) wt[j][i] = (j >= CONV_KMAX - K) ? w[(c0 + i) * K + j - (CONV_KMAX - K)] : 0.f;
}

// y[t, c] = silu(sum_j w[c][j] * x[t - (K-1) + j, c]); taps before the document start are 0.
// One thread walks CONV_TT consecutive tokens of one 16-byte channel group with a sliding
// window held in registers, so every x element is loaded once per thread.
template <typename T>
__global__ void __launch_bounds__(128) short_conv_fwd_kernel(const T* __restrict__ x, const float* __restrict__ w,
                                                             T* __restrict__ y, long long total, int Tlen, int Cch, int K,
                                                             const int64_t* cu, int N) {
    constexpr int V = Vec<T>::N;
    const int cgs = Cch / V;
    const long long ntile = (total + CONV_TT - 1) / CONV_TT;
    for (long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x; item < ntile * cgs;
         item += (long long)gridDim.x * blockDim.x) {
        const int c0 = (int)(item % cgs) * V;
        const long long t0 = (item / cgs) * CONV_TT;
        float wt[CONV_KMAX][V];
        load_taps<V>(w, c0, K, wt);
        float x0[V], x1[V], x2[V];
        int d0, d1, d2;  // document of each window entry (-1: outside the tensor)
        {
            const long long ta = t0 - 3, tb = t0 - 2, tc = t0 - 1;
#pragma unroll
            for (int i = 0; i < V; ++i) x0[i] = x1[i] = x2[i] = 0.f;
            d0 = d1 = d2 = -1;
            if (ta >= 0) { Vec<T>::load(x + ta * Cch + c0, x0); d0 = doc_of(cu, N, ta, Tlen); }
            if (tb >= 0) { Vec<T>::load(x + tb * Cch + c0, x1); d1 = doc_of(cu, N, tb, Tlen); }
            if (tc >= 0) { Vec<T>::load(x + tc * Cch + c0, x2); d2 = doc_of(cu, N, tc, Tlen); }
        }
#pragma unroll 4
        for (int tt = 0; tt < CONV_TT; ++tt) {
            const long long t = t0 + tt;
            if (t >= total) break;
            float x3[V], out[V];
            Vec<T>::load(x + t * Cch + c0, x3);
            const int d3 = doc_of(cu, N, t, Tlen);
            const float m0 = d0 == d3 ? 1.f : 0.f, m1 = d1 == d3 ? 1.f : 0.f, m2 = d2 == d3 ? 1.f : 0.f;
#pragma unroll
            for (int i = 0; i < V; ++i) {
                const float pre = conv_pre(wt[0][i], wt[1][i], wt[2][i], wt[3][i], m0 * x0[i], m1 * x1[i], m2 * x2[i], x3[i]);
                out[i] = silu_f(pre);
                x0[i] = x1[i];
                x1[i] = x2[i];
                x2[i] = x3[i];
            }
            d0 = d1; d1 = d2; d2 = d3;
            Vec<T>::store(y + t * Cch + c0, out);
        }
    }
}

// dx[t] = sum_j w[j] dpre[t + 3 - j],  dw[j] = sum_t dpre[t] x[t - 3 + j],
// dpre[s] = dy[s] silu'(pre[s]) with pre recomputed from x (four-tap padded filter).
// A block owns 512 bytes of channels and walks token tiles of CONV_BT tokens: the x rows (three
// before the tile, three after) and the dy rows (three after) arrive in shared memory through
// 16-byte asynchronous copies, then thread = channel runs down the tile with its windows in
// registers, writes dx over the consumed dy rows, and the tile leaves again in 16-byte stores.
// The thread's filter gradient stays in registers over all its tiles and goes to
// part[blockIdx.y][C][K] without any reduction inside the block.
constexpr int CONV_BT = 32;
template <typename T>
__global__ void __launch_bounds__(512 / sizeof(T)) short_conv_bwd_kernel(const T* __restrict__ x, const float* __restrict__ w,
                                                                        const T* __restrict__ dy, T* __restrict__ dx,
                                                                        float* __restrict__ part, long long total, int Tlen,
                                                                        int Cch, int K, const int64_t* cu, int N) {
    constexpr int CH = 512 / sizeof(T), V = 16 / sizeof(T), PCS = CH / V, XR = CONV_BT + 6, GR = CONV_BT + 3;
    __shared__ __align__(16) T sx[XR][CH];
    __shared__ __align__(16) T sg[GR][CH];
    __shared__ int sdoc[XR];
    const int tid = threadIdx.x, cbase = blockIdx.x * CH, c = cbase + tid;
    const bool act = c < Cch;
    float wt[CONV_KMAX], dw[CONV_KMAX] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < CONV_KMAX; ++j) wt[j] = (act && j >= CONV_KMAX - K) ? w[(size_t)c * K + j - (CONV_KMAX - K)] : 0.f;
    const long long ntile = (total + CONV_BT - 1) / CONV_BT;
    for (long long tile = blockIdx.y; tile < ntile; tile += gridDim.y) {
        const long long t0 = tile * CONV_BT;
        for (int q = tid; q < XR * PCS; q += CH) {
            const int r = q / PCS, pc = q % PCS;
            const long long t = t0 - 3 + r;
            const bool valid = t >= 0 && t < total && cbase + pc * V < Cch;
            const T* src = x + (valid ? (size_t)t * Cch + cbase + pc * V : 0);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(&sx[r][pc * V])),
                         "l"(src), "r"(valid ? 16 : 0) : "memory");
        }
        for (int q = tid; q < GR * PCS; q += CH) {
            const int r = q / PCS, pc = q % PCS;
            const long long t = t0 + r;
            const bool valid = t < total && cbase + pc * V < Cch;
            const T* src = dy + (valid ? (size_t)t * Cch + cbase + pc * V : 0);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(&sg[r][pc * V])),
                         "l"(src), "r"(valid ? 16 : 0) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (tid < XR) {  // document of every row of the tile (-1: outside the tensor; such rows are all zero)
            const long long t = t0 - 3 + tid;
            sdoc[tid] = (t >= 0 && t < total) ? doc_of(cu, N, t, Tlen) : -1;
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (act) {
            // window: x and dpre of tokens s-3, s-2, s-1 (a, b, c) and the current one (d)
            float xa = (float)sx[0][tid], xb = (float)sx[1][tid], xc = (float)sx[2][tid];
            int da = sdoc[0], db = sdoc[1], dc = sdoc[2];
            float pa = 0.f, pb = 0.f, pc_ = 0.f;
#pragma unroll 7
            for (int sI = 0; sI < GR; ++sI) {
                const float xd = (float)sx[sI + 3][tid], gy = (float)sg[sI][tid];
                const int dd = sdoc[sI + 3];
                const float a0 = da == dd ? xa : 0.f, a1 = db == dd ? xb : 0.f, a2 = dc == dd ? xc : 0.f;
                const float pd = gy * dsilu_f(conv_pre(wt[0], wt[1], wt[2], wt[3], a0, a1, a2, xd));
                if (sI < CONV_BT) {  // the tile's own tokens feed the filter gradient
                    dw[0] = fmaf(pd, a0, dw[0]);
                    dw[1] = fmaf(pd, a1, dw[1]);
                    dw[2] = fmaf(pd, a2, dw[2]);
                    dw[3] = fmaf(pd, xd, dw[3]);
                }
                if (sI >= 3) {  // dx of the oldest window entry; its dy row has been consumed
                    const float out = fmaf(wt[0], dd == da ? pd : 0.f,
                                           fmaf(wt[1], dc == da ? pc_ : 0.f, fmaf(wt[2], db == da ? pb : 0.f, wt[3] * pa)));
                    sg[sI - 3][tid] = (T)out;
                }
                xa = xb; xb = xc; xc = xd;
                da = db; db = dc; dc = dd;
                pa = pb; pb = pc_; pc_ = pd;
            }
        }
        __syncthreads();
        for (int q = tid; q < CONV_BT * PCS; q += CH) {
            const int r = q / PCS, pc = q % PCS;
            const long long t = t0 + r;
            if (t < total && cbase + pc * V < Cch)
                *reinterpret_cast<uint4*>(dx + (size_t)t * Cch + cbase + pc * V) = *reinterpret_cast<const uint4*>(&sg[r][pc * V]);
        }
        __syncthreads();
    }
    if (act) {
#pragma unroll
        for (int j = 0; j < CONV_KMAX; ++j)
            if (j >= CONV_KMAX - K) part[((size_t)blockIdx.y * Cch + c) * K + j - (CONV_KMAX - K)] = dw[j];
    }
}

// out[i] = sum_p part[p][i] in a fixed order: a block takes 32 outputs; its eight warps sum the
// partials p = w, w + 8, ... (independent loads in flight), then warp 0 adds the eight sums in order.
__global__ void __launch_bounds__(256) partial_reduce_kernel(const float* __restrict__ part, float* __restrict__ out,
                                                             int n_partial, int n) {
    __shared__ float sacc[8][33];
    const int x = threadIdx.x & 31, w = threadIdx.x >> 5, i = blockIdx.x * 32 + x;
    float acc = 0.f;
    if (i < n)
        for (int p = w; p < n_partial; p += 8) acc += part[(size_t)p * n + i];
    sacc[w][x] = acc;
    __syncthreads();
    if (w == 0 && i < n) {
        float t = 0.f;
#pragma unroll
        for (int g = 0; g < 8; ++g) t += sacc[g][x];
        out[i] = t;
    }
}

// ---- RMSNorm(x) * w * sigmoid(gate): DIM / 8 (BF16) or DIM / 4 (FP32) lanes per row, 16-byte accesses
template <typename T, int DIM>
__global__ void __launch_bounds__(256) norm_gate_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gate,
                                                            const float* __restrict__ w, T* __restrict__ y,
                                                            float* __restrict__ rstd, long long rows, float eps) {
    constexpr int V = Vec<T>::N, LPR = DIM / V;  // lanes per row: 16 or 32 (8 for DIM = 64 BF16)
    const int lane = threadIdx.x & 31, sub = lane % LPR, rsub = lane / LPR;
    constexpr int RPW = 32 / LPR;  // rows per warp per iteration
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nw = ((long long)gridDim.x * blockDim.x) >> 5;
    float wv[V];
#pragma unroll
    for (int i = 0; i < V; ++i) wv[i] = w[sub * V + i];
    for (long long r0 = warp * RPW; r0 < rows; r0 += nw * RPW) {
        const long long r = r0 + rsub;
        const bool ok = r < rows;
        float xv[V], gv[V], out[V], ss = 0.f;
#pragma unroll
        for (int i = 0; i < V; ++i) xv[i] = gv[i] = 0.f;
        if (ok) {
            Vec<T>::load(x + r * DIM + sub * V, xv);
            Vec<T>::load(gate + r * DIM + sub * V, gv);
        }
#pragma unroll
        for (int i = 0; i < V; ++i) ss += xv[i] * xv[i];
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float rs = rsqrtf(ss / DIM + eps);
        if (ok) {
            if (sub == 0 && rstd) rstd[r] = rs;
#pragma unroll
            for (int i = 0; i < V; ++i) out[i] = xv[i] * rs * wv[i] * sigmoid_f(gv[i]);
            Vec<T>::store(y + r * DIM + sub * V, out);
        }
    }
}

template <typename T, int DIM>
__global__ void __launch_bounds__(256) norm_gate_bwd_kernel(const T* __restrict__ x, const T* __restrict__ gate,
                                                            const float* __restrict__ w, const T* __restrict__ dy,
                                                            T* __restrict__ dx, T* __restrict__ dgate,
                                                            float* __restrict__ part, long long rows, float eps) {
    constexpr int V = Vec<T>::N, LPR = DIM / V, RPW = 32 / LPR;
    __shared__ float sred[8][RPW][DIM];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, sub = lane % LPR, rsub = lane / LPR;
    const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + wib;
    const long long nw = (long long)gridDim.x * (blockDim.x >> 5);
    float wv[V], dwv[V];
#pragma unroll
    for (int i = 0; i < V; ++i) {
        wv[i] = w[sub * V + i];
        dwv[i] = 0.f;
    }
    for (long long r0 = warp * RPW; r0 < rows; r0 += nw * RPW) {
        const long long r = r0 + rsub;
        const bool ok = r < rows;
        float xv[V], gv[V], gy[V], dn[V], ss = 0.f, dot = 0.f;
#pragma unroll
        for (int i = 0; i < V; ++i) xv[i] = gv[i] = gy[i] = 0.f;
        if (ok) {
            Vec<T>::load(x + r * DIM + sub * V, xv);
            Vec<T>::load(gate + r * DIM + sub * V, gv);
            Vec<T>::load(dy + r * DIM + sub * V, gy);
        }
#pragma unroll
        for (int i = 0; i < V; ++i) ss += xv[i] * xv[i];
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float rs = rsqrtf(ss / DIM + eps);
        float dg[V];
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const float sgm = sigmoid_f(gv[i]);
            const float xh = xv[i] * rs;
            dg[i] = gy[i] * xh * wv[i] * sgm * (1.f - sgm);
            dn[i] = gy[i] * sgm;
            dwv[i] += dn[i] * xh;
            dn[i] *= wv[i];
            dot += dn[i] * xh;
        }
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        dot /= DIM;
        if (ok) {
            float out[V];
#pragma unroll
            for (int i = 0; i < V; ++i) out[i] = rs * (dn[i] - xv[i] * rs * dot);
            Vec<T>::store(dx + r * DIM + sub * V, out);
            Vec<T>::store(dgate + r * DIM + sub * V, dg);
        }
    }
#pragma unroll
    for (int i = 0; i < V; ++i) sred[wib][rsub][sub * V + i] = dwv[i];
    __syncthreads();
    for (int d = threadIdx.x; d < DIM; d += blockDim.x) {
        float s = 0.f;
        for (int ww = 0; ww < (int)(blockDim.x >> 5); ++ww)
            for (int rr = 0; rr < RPW; ++rr) s += sred[ww][rr][d];
        part[(size_t)blockIdx.x * DIM + d] = s;
    }
}

// ---------------------------------------------------------------------------------------
// Gate-span statistic (scripts/profile_kda_gate_spans.py:21-56 of the reference): for every
// [16 rows x 32 channels] tile of the within-chunk cumulative log2 decay, the largest drop below
// the tile's first row.  One CTA per (sequence, chunk, head), one thread per channel, so the
// cumulative sum runs in registers and a warp is exactly one channel tile.
// Output order [B][T/64][4][H][d/32], the flattening the reference's function returns.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) gate_tile_spans_kernel(const T* __restrict__ raw, const float* __restrict__ a_log,
                                                              const float* __restrict__ dt_bias, float* __restrict__ out,
                                                              int Tlen, int H, int d) {
    const int ch = threadIdx.x, h = blockIdx.x % H, cidx = blockIdx.x / H;  // cidx = b * (T / 64) + chunk
    const int nct = d / 32;
    const float negA = -expf(a_log[h]) * LOG2E, bias = dt_bias[h * d + ch];
    const T* src = raw + ((size_t)cidx * C * H + h) * d + ch;
    float cum = 0.f;
#pragma unroll 1
    for (int blk = 0; blk < C / 16; ++blk) {
        float first = 0.f, span = 0.f;
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            cum += negA * softplus_f(ldf(src + (size_t)(16 * blk + r) * H * d) + bias);
            if (r == 0) first = cum;
            span = fmaxf(span, first - cum);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) span = fmaxf(span, __shfl_xor_sync(0xffffffffu, span, o));
        if ((ch & 31) == 0) out[(((size_t)cidx * (C / 16) + blk) * H + h) * nct + (ch >> 5)] = span;
    }
}

}  // namespace kda

using namespace kda;

extern "C" {

int kda_gate_tile_spans(const void* raw, const float* a_log, const float* dt_bias, float* out, int32_t B, int32_t T,
                        int32_t H, int32_t d, int32_t dtype, void* stream) {
    if (!raw || !a_log || !dt_bias || !out) return KDA_ERR_NULL;
    if (B <= 0 || T <= 0 || H <= 0 || T % C || d <= 0 || d % 32 || d > 256) return KDA_ERR_SHAPE;
    if (dtype != KDA_DTYPE_BF16 && dtype != KDA_DTYPE_F32) return KDA_ERR_DTYPE;
    const long long grid = (long long)B * (T / C) * H;
    if (grid > 0x7fffffffLL) return KDA_ERR_SHAPE;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == KDA_DTYPE_BF16)
        gate_tile_spans_kernel<__nv_bfloat16><<<(int)grid, d, 0, s>>>((const __nv_bfloat16*)raw, a_log, dt_bias, out, T, H, d);
    else
        gate_tile_spans_kernel<float><<<(int)grid, d, 0, s>>>((const float*)raw, a_log, dt_bias, out, T, H, d);
    return launch_status();
}

int kda_short_conv_fwd(const void* x, const float* weight, void* y, int32_t B, int32_t T, int32_t Cch, int32_t ksize,
                       int32_t dtype, const int64_t* cu_seqlens, int32_t N, void* stream) {
    if (!x || !weight || !y) return KDA_ERR_NULL;
    if (ksize < 1 || ksize > CONV_KMAX || B <= 0 || T <= 0 || (cu_seqlens && B != 1)) return KDA_ERR_SHAPE;
    const int V = dtype == KDA_DTYPE_BF16 ? 8 : 4;
    if (dtype != KDA_DTYPE_BF16 && dtype != KDA_DTYPE_F32) return KDA_ERR_DTYPE;
    if (Cch % V) return KDA_ERR_SHAPE;
    if (((uintptr_t)x | (uintptr_t)y) & 15) return KDA_ERR_ALIGN;
    long long total = (long long)B * T;
    long long items = ((total + CONV_TT - 1) / CONV_TT) * (Cch / V);
    int grid = (int)((items + 127) / 128 < 148 * 16 ? (items + 127) / 128 : 148 * 16);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == KDA_DTYPE_BF16)
        short_conv_fwd_kernel<__nv_bfloat16><<<grid, 128, 0, s>>>((const __nv_bfloat16*)x, weight, (__nv_bfloat16*)y, total,
                                                                  T, Cch, ksize, cu_seqlens, N);
    else
        short_conv_fwd_kernel<float><<<grid, 128, 0, s>>>((const float*)x, weight, (float*)y, total, T, Cch, ksize,
                                                          cu_seqlens, N);
    return launch_status();
}

int kda_short_conv_bwd(const void* x, const float* weight, const void* dy, void* dx, float* dweight,
                       float* partial, int32_t n_partial, int32_t B, int32_t T, int32_t Cch, int32_t ksize,
                       int32_t dtype, const int64_t* cu_seqlens, int32_t N, void* stream) {
    if (!x || !weight || !dy || !dx || !dweight || !partial) return KDA_ERR_NULL;
    if (ksize < 1 || ksize > CONV_KMAX || B <= 0 || T <= 0 || n_partial < 1 || n_partial > 65535 || (cu_seqlens && B != 1))
        return KDA_ERR_SHAPE;  // (n_partial is a grid dimension)
    if (dtype != KDA_DTYPE_BF16 && dtype != KDA_DTYPE_F32) return KDA_ERR_DTYPE;
    const int V = dtype == KDA_DTYPE_BF16 ? 8 : 4;
    if (Cch % V) return KDA_ERR_SHAPE;
    if (((uintptr_t)x | (uintptr_t)dy | (uintptr_t)dx) & 15) return KDA_ERR_ALIGN;
    long long total = (long long)B * T;
    const int chb = dtype == KDA_DTYPE_BF16 ? 256 : 128;  // channels per block (512 bytes)
    dim3 grid((Cch + chb - 1) / chb, n_partial), block(chb);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == KDA_DTYPE_BF16)
        short_conv_bwd_kernel<__nv_bfloat16><<<grid, block, 0, s>>>((const __nv_bfloat16*)x, weight, (const __nv_bfloat16*)dy,
                                                                    (__nv_bfloat16*)dx, partial, total, T, Cch, ksize,
                                                                    cu_seqlens, N);
    else
        short_conv_bwd_kernel<float><<<grid, block, 0, s>>>((const float*)x, weight, (const float*)dy, (float*)dx, partial,
                                                            total, T, Cch, ksize, cu_seqlens, N);
    int n = Cch * ksize;
    partial_reduce_kernel<<<(n + 31) / 32, 256, 0, s>>>(partial, dweight, n_partial, n);
    return launch_status();
}

int kda_norm_gate_fwd(const void* x, const void* gate, const float* weight, void* y, float* rstd, int64_t rows,
                      int32_t dim, float eps, int32_t dtype, void* stream) {
    if (!x || !gate || !weight || !y) return KDA_ERR_NULL;
    if (rows <= 0 || (dim != 64 && dim != 128)) return KDA_ERR_SHAPE;
    if (dtype != KDA_DTYPE_BF16 && dtype != KDA_DTYPE_F32) return KDA_ERR_DTYPE;
    cudaStream_t s = (cudaStream_t)stream;
    int grid = (int)((rows + 15) / 16 < 148 * 8 ? (rows + 15) / 16 : 148 * 8);
#define NG_FWD(TT, DD) \
    norm_gate_fwd_kernel<TT, DD><<<grid, 256, 0, s>>>((const TT*)x, (const TT*)gate, weight, (TT*)y, rstd, rows, eps)
    if (dtype == KDA_DTYPE_BF16) { if (dim == 64) NG_FWD(__nv_bfloat16, 64); else NG_FWD(__nv_bfloat16, 128); }
    else { if (dim == 64) NG_FWD(float, 64); else NG_FWD(float, 128); }
#undef NG_FWD
    return launch_status();
}

int kda_norm_gate_bwd(const void* x, const void* gate, const float* weight, const void* dy, void* dx, void* dgate,
                      float* dweight, float* partial, int32_t n_partial, int64_t rows, int32_t dim, float eps,
                      int32_t dtype, void* stream) {
    if (!x || !gate || !weight || !dy || !dx || !dgate || !dweight || !partial) return KDA_ERR_NULL;
    if (rows <= 0 || (dim != 64 && dim != 128) || n_partial < 1 || n_partial > 65535) return KDA_ERR_SHAPE;
    if (dtype != KDA_DTYPE_BF16 && dtype != KDA_DTYPE_F32) return KDA_ERR_DTYPE;
    cudaStream_t s = (cudaStream_t)stream;
#define NG_BWD(TT, DD)                                                                                               \
    norm_gate_bwd_kernel<TT, DD><<<n_partial, 256, 0, s>>>((const TT*)x, (const TT*)gate, weight, (const TT*)dy, (TT*)dx, \
                                                           (TT*)dgate, partial, rows, eps)
    if (dtype == KDA_DTYPE_BF16) { if (dim == 64) NG_BWD(__nv_bfloat16, 64); else NG_BWD(__nv_bfloat16, 128); }
    else { if (dim == 64) NG_BWD(float, 64); else NG_BWD(float, 128); }
#undef NG_BWD
    partial_reduce_kernel<<<(dim + 31) / 32, 256, 0, s>>>(partial, dweight, n_partial, dim);
    return launch_status();
}

// The variant of kda_short_conv_bwd for callers that must not allocate: same kernels, same
// reduction order (so the same bits as kda_short_conv_bwd with n_partial = 64), but the
// partial sums live in g_conv_static_partial instead of a caller buffer.
int kda_short_conv_bwd_static(const void* x, const float* weight, const void* dy, void* dx, float* dweight, int32_t B,
                              int32_t T, int32_t Cch, int32_t ksize, int32_t dtype, const int64_t* cu_seqlens, int32_t N,
                              void* stream) {
    if (ksize < 1 || Cch < 1) return KDA_ERR_SHAPE;
    if ((int64_t)Cch * ksize > CONV_STATIC_MAX_WEIGHTS) return KDA_ERR_STATIC_LIMIT;
    // One-time set-up per device, with that device current: ask the runtime where this
    // device's copy of the array lives.  The array's name itself is not that address.
    static std::mutex mu;
    static float* dev_ptr[64] = {nullptr};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return fail_cuda(cudaGetLastError());
    if (dev >= 64) return KDA_ERR_STATIC_LIMIT;  // the per-device address table has 64 entries
    float* part = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!dev_ptr[dev]) {
            void* ptr = nullptr;
            const cudaError_t e = cudaGetSymbolAddress(&ptr, g_conv_static_partial);
            if (e != cudaSuccess || !ptr) return fail_cuda(e);
            dev_ptr[dev] = static_cast<float*>(ptr);
        }
        part = dev_ptr[dev];
    }
    return kda_short_conv_bwd(x, weight, dy, dx, dweight, part, CONV_STATIC_PARTIALS, B, T, Cch, ksize, dtype, cu_seqlens,
                              N, stream);
}

}  // extern "C"
