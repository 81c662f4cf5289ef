// HBM-bound companions of the KDA op inside the KimiDeltaAttention sublayer:
// causal depthwise short convolution + SiLU (k3mini/model.py:76-88) and the headwise
// RMSNorm * sigmoid(gate) output stage (k3mini/model.py:91-98).  Both are single passes
// with 16-byte vector accesses; parameter gradients are reduced in a fixed order.
#include <mutex>

#include "kda_common.cuh"

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

// start of the document that contains flattened token t
__device__ __forceinline__ long long doc_start(const int64_t* cu, int N, long long t, int T) {
    if (!cu) return (t / T) * T;
    int lo = 0, hi = N;  // cu[lo] <= t < cu[hi]
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (cu[mid] <= t) lo = mid; else hi = mid;
    }
    return cu[lo];
}
__device__ __forceinline__ long long doc_end(const int64_t* cu, int N, long long t, int T) {
    if (!cu) return (t / T + 1) * T;
    int lo = 0, hi = N;
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (cu[mid] <= t) lo = mid; else hi = mid;
    }
    return cu[hi];
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float dsilu_f(float x) {
    float s = 1.f / (1.f + expf(-x));
    return s * (1.f + x * (1.f - s));
}

// y[t, c] = silu(sum_j w[c][j] * x[t - (K-1) + j, c]), taps before the document start are 0
template <typename T>
__global__ void short_conv_fwd_kernel(const T* __restrict__ x, const float* __restrict__ w, T* __restrict__ y,
                                      long long total, int Tlen, int Cch, int K, const int64_t* cu, int N) {
    constexpr int V = Vec<T>::N;
    const int cgs = Cch / V;
    const long long ntile = (total + CONV_TT - 1) / CONV_TT;
    for (long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x; item < ntile * cgs;
         item += (long long)gridDim.x * blockDim.x) {
        const int cg = (int)(item % cgs);
        const long long t0 = (item / cgs) * CONV_TT;
        const int c0 = cg * V;
        float wt[V][CONV_KMAX];
#pragma unroll
        for (int i = 0; i < V; ++i)
#pragma unroll
            for (int j = 0; j < CONV_KMAX; ++j) wt[i][j] = j < K ? w[(c0 + i) * K + j] : 0.f;
        float win[CONV_KMAX][V];  // win[j] = x[t - (K-1) + j]
        long long ds = doc_start(cu, N, t0, Tlen), de = doc_end(cu, N, t0, Tlen);
#pragma unroll
        for (int j = 0; j < CONV_KMAX; ++j)
#pragma unroll
            for (int i = 0; i < V; ++i) win[j][i] = 0.f;
        for (int j = 0; j < K - 1; ++j) {
            long long ts = t0 - (K - 1) + j;
            if (ts >= ds) Vec<T>::load(x + ts * Cch + c0, win[j]);
        }
        for (int tt = 0; tt < CONV_TT; ++tt) {
            long long t = t0 + tt;
            if (t >= total) break;
            if (t >= de) {  // entered the next document: forget the window
                ds = de;
                de = doc_end(cu, N, t, Tlen);
#pragma unroll
                for (int j = 0; j < CONV_KMAX; ++j)
#pragma unroll
                    for (int i = 0; i < V; ++i) win[j][i] = 0.f;
            }
            Vec<T>::load(x + t * Cch + c0, win[K - 1]);
            float out[V];
#pragma unroll
            for (int i = 0; i < V; ++i) {
                float s = 0.f;
#pragma unroll
                for (int j = 0; j < CONV_KMAX; ++j)
                    if (j < K) s = fmaf(wt[i][j], win[j][i], s);
                out[i] = silu_f(s);
            }
            Vec<T>::store(y + t * Cch + c0, out);
#pragma unroll
            for (int j = 0; j + 1 < CONV_KMAX; ++j)
                if (j + 1 < K) {
#pragma unroll
                    for (int i = 0; i < V; ++i) win[j][i] = win[j + 1][i];
                }
        }
    }
}

// dx[t] = sum_j w[j] dpre[t + (K-1) - j],  dw[j] = sum_t dpre[t] x[t - (K-1) + j],
// dpre[s] = dy[s] silu'(pre[s]) with pre recomputed from x.  blockDim = (32 channel groups,
// 8 token tiles); per-block partial dw in part[blockIdx.y][C][K].
template <typename T>
__global__ void short_conv_bwd_kernel(const T* __restrict__ x, const float* __restrict__ w, const T* __restrict__ dy,
                                      T* __restrict__ dx, float* __restrict__ part, long long total, int Tlen, int Cch,
                                      int K, const int64_t* cu, int N) {
    constexpr int V = Vec<T>::N;
    __shared__ float sred[8][32][V * CONV_KMAX + 1];
    const int cgs = Cch / V;
    const int cg = blockIdx.x * 32 + threadIdx.x;
    const bool active = cg < cgs;
    const int c0 = cg * V;
    const long long ntile = (total + CONV_TT - 1) / CONV_TT;
    float wt[V][CONV_KMAX], dw[V][CONV_KMAX];
#pragma unroll
    for (int i = 0; i < V; ++i)
#pragma unroll
        for (int j = 0; j < CONV_KMAX; ++j) {
            wt[i][j] = (active && j < K) ? w[(c0 + i) * K + j] : 0.f;
            dw[i][j] = 0.f;
        }
    if (active) {
        for (long long tile = (long long)blockIdx.y * 8 + threadIdx.y; tile < ntile; tile += (long long)gridDim.y * 8) {
            const long long t0 = tile * CONV_TT;
            // x window xs[i] = x[t0 - (K-1) + i], i in [0, TT + 2(K-1)); dpre for s in [t0, t0 + TT + K-1)
            constexpr int XW = CONV_TT + 2 * (CONV_KMAX - 1);
            constexpr int PW = CONV_TT + CONV_KMAX - 1;
            float dpre[PW][V];
            {
                float xs[XW][V];
                long long ds0 = doc_start(cu, N, t0, Tlen);
                for (int i = 0; i < XW; ++i) {
                    long long ts = t0 - (K - 1) + i;
#pragma unroll
                    for (int u = 0; u < V; ++u) xs[i][u] = 0.f;
                    if (ts >= ds0 && ts < total && i < CONV_TT + 2 * (K - 1)) Vec<T>::load(x + ts * Cch + c0, xs[i]);
                }
                for (int s = 0; s < PW; ++s) {
                    long long ts = t0 + s;
#pragma unroll
                    for (int u = 0; u < V; ++u) dpre[s][u] = 0.f;
                    if (ts >= total || s >= CONV_TT + K - 1) continue;
                    long long ds = doc_start(cu, N, ts, Tlen);
                    float g[V];
                    Vec<T>::load(dy + ts * Cch + c0, g);
#pragma unroll
                    for (int u = 0; u < V; ++u) {
                        float pre = 0.f;
#pragma unroll
                        for (int j = 0; j < CONV_KMAX; ++j)
                            if (j < K && ts - (K - 1) + j >= ds) pre = fmaf(wt[u][j], xs[s + j][u], pre);
                        dpre[s][u] = g[u] * dsilu_f(pre);
                    }
                    if (s < CONV_TT) {  // this thread owns token ts for the weight gradient
#pragma unroll
                        for (int u = 0; u < V; ++u)
#pragma unroll
                            for (int j = 0; j < CONV_KMAX; ++j)
                                if (j < K && ts - (K - 1) + j >= ds) dw[u][j] = fmaf(dpre[s][u], xs[s + j][u], dw[u][j]);
                    }
                }
            }
            for (int tt = 0; tt < CONV_TT; ++tt) {
                long long t = t0 + tt;
                if (t >= total) break;
                long long de = doc_end(cu, N, t, Tlen);
                float out[V];
#pragma unroll
                for (int u = 0; u < V; ++u) {
                    float s = 0.f;
#pragma unroll
                    for (int j = 0; j < CONV_KMAX; ++j)
                        if (j < K && t + (K - 1) - j < de) s = fmaf(wt[u][j], dpre[tt + (K - 1) - j][u], s);
                    out[u] = s;
                }
                Vec<T>::store(dx + t * Cch + c0, out);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < V; ++i)
#pragma unroll
        for (int j = 0; j < CONV_KMAX; ++j) sred[threadIdx.y][threadIdx.x][i * CONV_KMAX + j] = dw[i][j];
    __syncthreads();
    if (threadIdx.y == 0 && active) {
        for (int i = 0; i < V; ++i)
            for (int j = 0; j < K; ++j) {
                float s = 0.f;
                for (int yy = 0; yy < 8; ++yy) s += sred[yy][threadIdx.x][i * CONV_KMAX + j];
                part[((size_t)blockIdx.y * Cch + c0 + i) * K + j] = s;
            }
    }
}

// out[i] = sum_p part[p][i]
__global__ void partial_reduce_kernel(const float* __restrict__ part, float* __restrict__ out, int n_partial, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float s = 0.f;
    for (int p = 0; p < n_partial; ++p) s += part[(size_t)p * n + i];
    out[i] = s;
}

// ---- RMSNorm(x) * w * sigmoid(gate), one warp per row -----------------------------------
template <typename T, int DIM>
__global__ void norm_gate_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gate, const float* __restrict__ w,
                                     T* __restrict__ y, float* __restrict__ rstd, long long rows, float eps) {
    constexpr int PER = DIM / 32;
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nw = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long r = warp; r < rows; r += nw) {
        float xv[PER], ss = 0.f;
#pragma unroll
        for (int m = 0; m < PER; ++m) {
            xv[m] = ldf(x + r * DIM + lane + 32 * m);
            ss += xv[m] * xv[m];
        }
        ss = warp_sum(ss);
        float rs = rsqrtf(ss / DIM + eps);
        if (lane == 0 && rstd) rstd[r] = rs;
#pragma unroll
        for (int m = 0; m < PER; ++m) {
            int d = lane + 32 * m;
            stf(y + r * DIM + d, xv[m] * rs * w[d] * sigmoid_f(ldf(gate + r * DIM + d)));
        }
    }
}

template <typename T, int DIM>
__global__ void norm_gate_bwd_kernel(const T* __restrict__ x, const T* __restrict__ gate, const float* __restrict__ w,
                                     const T* __restrict__ dy, T* __restrict__ dx, T* __restrict__ dgate,
                                     float* __restrict__ part, long long rows, float eps) {
    constexpr int PER = DIM / 32;
    __shared__ float sred[8][DIM];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + wib;
    const long long nw = (long long)gridDim.x * (blockDim.x >> 5);
    float dwv[PER];
#pragma unroll
    for (int m = 0; m < PER; ++m) dwv[m] = 0.f;
    for (long long r = warp; r < rows; r += nw) {
        float xv[PER], dn[PER], ss = 0.f, dot = 0.f;
#pragma unroll
        for (int m = 0; m < PER; ++m) {
            xv[m] = ldf(x + r * DIM + lane + 32 * m);
            ss += xv[m] * xv[m];
        }
        ss = warp_sum(ss);
        float rs = rsqrtf(ss / DIM + eps);
#pragma unroll
        for (int m = 0; m < PER; ++m) {
            int d = lane + 32 * m;
            float s = sigmoid_f(ldf(gate + r * DIM + d));
            float g = ldf(dy + r * DIM + d);
            float xh = xv[m] * rs;
            stf(dgate + r * DIM + d, g * xh * w[d] * s * (1.f - s));
            dn[m] = g * s;
            dwv[m] += dn[m] * xh;
            dn[m] *= w[d];
            dot += dn[m] * xh;
        }
        dot = warp_sum(dot) / DIM;
#pragma unroll
        for (int m = 0; m < PER; ++m) stf(dx + r * DIM + lane + 32 * m, rs * (dn[m] - xv[m] * rs * dot));
    }
#pragma unroll
    for (int m = 0; m < PER; ++m) sred[wib][lane + 32 * m] = dwv[m];
    __syncthreads();
    for (int d = threadIdx.x; d < DIM; d += blockDim.x) {
        float s = 0.f;
        for (int ww = 0; ww < (int)(blockDim.x >> 5); ++ww) s += sred[ww][d];
        part[(size_t)blockIdx.x * DIM + d] = s;
    }
}

}  // namespace kda

using namespace kda;

extern "C" {

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
    return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

int kda_short_conv_bwd(const void* x, const float* weight, const void* dy, void* dx, float* dweight,
                       float* partial, int32_t n_partial, int32_t B, int32_t T, int32_t Cch, int32_t ksize,
                       int32_t dtype, const int64_t* cu_seqlens, int32_t N, void* stream) {
    if (!x || !weight || !dy || !dx || !dweight || !partial) return KDA_ERR_NULL;
    if (ksize < 1 || ksize > CONV_KMAX || B <= 0 || T <= 0 || n_partial < 1 || (cu_seqlens && B != 1)) return KDA_ERR_SHAPE;
    if (dtype != KDA_DTYPE_BF16 && dtype != KDA_DTYPE_F32) return KDA_ERR_DTYPE;
    const int V = dtype == KDA_DTYPE_BF16 ? 8 : 4;
    if (Cch % V) return KDA_ERR_SHAPE;
    if (((uintptr_t)x | (uintptr_t)dy | (uintptr_t)dx) & 15) return KDA_ERR_ALIGN;
    long long total = (long long)B * T;
    dim3 grid((Cch / V + 31) / 32, n_partial), block(32, 8);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == KDA_DTYPE_BF16)
        short_conv_bwd_kernel<__nv_bfloat16><<<grid, block, 0, s>>>((const __nv_bfloat16*)x, weight, (const __nv_bfloat16*)dy,
                                                                    (__nv_bfloat16*)dx, partial, total, T, Cch, ksize,
                                                                    cu_seqlens, N);
    else
        short_conv_bwd_kernel<float><<<grid, block, 0, s>>>((const float*)x, weight, (const float*)dy, (float*)dx, partial,
                                                            total, T, Cch, ksize, cu_seqlens, N);
    int n = Cch * ksize;
    partial_reduce_kernel<<<(n + 255) / 256, 256, 0, s>>>(partial, dweight, n_partial, n);
    return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

int kda_norm_gate_fwd(const void* x, const void* gate, const float* weight, void* y, float* rstd, int64_t rows,
                      int32_t dim, float eps, int32_t dtype, void* stream) {
    if (!x || !gate || !weight || !y) return KDA_ERR_NULL;
    if (rows <= 0 || (dim != 64 && dim != 128)) return KDA_ERR_SHAPE;
    if (dtype != KDA_DTYPE_BF16 && dtype != KDA_DTYPE_F32) return KDA_ERR_DTYPE;
    cudaStream_t s = (cudaStream_t)stream;
    int grid = (int)((rows + 7) / 8 < 148 * 16 ? (rows + 7) / 8 : 148 * 16);
#define NG_FWD(TT, DD) \
    norm_gate_fwd_kernel<TT, DD><<<grid, 256, 0, s>>>((const TT*)x, (const TT*)gate, weight, (TT*)y, rstd, rows, eps)
    if (dtype == KDA_DTYPE_BF16) { if (dim == 64) NG_FWD(__nv_bfloat16, 64); else NG_FWD(__nv_bfloat16, 128); }
    else { if (dim == 64) NG_FWD(float, 64); else NG_FWD(float, 128); }
#undef NG_FWD
    return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

int kda_norm_gate_bwd(const void* x, const void* gate, const float* weight, const void* dy, void* dx, void* dgate,
                      float* dweight, float* partial, int32_t n_partial, int64_t rows, int32_t dim, float eps,
                      int32_t dtype, void* stream) {
    if (!x || !gate || !weight || !dy || !dx || !dgate || !dweight || !partial) return KDA_ERR_NULL;
    if (rows <= 0 || (dim != 64 && dim != 128) || n_partial < 1) return KDA_ERR_SHAPE;
    if (dtype != KDA_DTYPE_BF16 && dtype != KDA_DTYPE_F32) return KDA_ERR_DTYPE;
    cudaStream_t s = (cudaStream_t)stream;
#define NG_BWD(TT, DD)                                                                                               \
    norm_gate_bwd_kernel<TT, DD><<<n_partial, 256, 0, s>>>((const TT*)x, (const TT*)gate, weight, (const TT*)dy, (TT*)dx, \
                                                           (TT*)dgate, partial, rows, eps)
    if (dtype == KDA_DTYPE_BF16) { if (dim == 64) NG_BWD(__nv_bfloat16, 64); else NG_BWD(__nv_bfloat16, 128); }
    else { if (dim == 64) NG_BWD(float, 64); else NG_BWD(float, 128); }
#undef NG_BWD
    partial_reduce_kernel<<<(dim + 255) / 256, 256, 0, s>>>(partial, dweight, n_partial, dim);
    return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

// The variant of kda_short_conv_bwd for callers that must not allocate: same kernels, same
// reduction order (so the same bits as kda_short_conv_bwd with n_partial = 64), but the
// partial sums live in g_conv_static_partial instead of a caller buffer.
int kda_short_conv_bwd_static(const void* x, const float* weight, const void* dy, void* dx, float* dweight, int32_t B,
                              int32_t T, int32_t Cch, int32_t ksize, int32_t dtype, const int64_t* cu_seqlens, int32_t N,
                              void* stream) {
    if (ksize < 1 || Cch < 1 || (int64_t)Cch * ksize > CONV_STATIC_MAX_WEIGHTS) return KDA_ERR_STATIC_LIMIT;
    // One-time set-up per device, with that device current: ask the runtime where this
    // device's copy of the array lives.  The array's name itself is not that address.
    static std::mutex mu;
    static float* dev_ptr[64] = {nullptr};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return KDA_ERR_LAUNCH;
    float* part = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!dev_ptr[dev]) {
            void* ptr = nullptr;
            if (cudaGetSymbolAddress(&ptr, g_conv_static_partial) != cudaSuccess || !ptr) return KDA_ERR_LAUNCH;
            dev_ptr[dev] = static_cast<float*>(ptr);
        }
        part = dev_ptr[dev];
    }
    return kda_short_conv_bwd(x, weight, dy, dx, dweight, part, CONV_STATIC_PARTIALS, B, T, Cch, ksize, dtype, cu_seqlens,
                              N, stream);
}

}  // extern "C"
