// KDA chunkwise forward and backward with FP32 CUDA-core arithmetic.
//
// This is the "FP32-operand validation mode" of the library: every contraction is an FP32
// FMA loop, every pairwise decay 2^(G_i - G_j) is evaluated exactly (no factorisation, so
// no span guard is needed), and the state is FP32.  The same four stages, with the same
// workspace records, are what the tensor-core kernels implement:
//
//   fwd_intra  (one CTA per chunk x head)   prologue, Aqk, L, T=(I+diag(beta)L)^-1, W, U
//   fwd_state  (one CTA per seq x head x dv-panel, sequential over chunks)  V', O, S
//   bwd_state  (same grid, reverse order)   dV', dS
//   bwd_chunk  (one CTA per chunk x head)   everything else, down to the raw-input grads
//
// The math follows the recurrence of k3mini/model.py:115-129 rewritten per 64-token chunk.
// (the SPLIT instantiation of kda_bwd_chunk returns early by design: no "unreachable loop" remarks)
#pragma nv_diag_suppress 128
#include "kda_common.cuh"
#include "kda_tc.cuh"

namespace kda {

void prof_mark(cudaStream_t s);

constexpr int NTHREADS = 256;
constexpr int KS = 16;  // k-slice of the tile product

// ---------------------------------------------------------------------------------------
// acc[M/16][N/16] += A[M x K] * B[K x N], operands fetched through functors la(m,k), lb(k,n)
// (from global or shared memory, any element type) and staged through shared memory in
// slices of KS.  Thread (ty,tx) = (tid/16, tid%16) owns rows ty+16r and columns tx+16c.
// a_kfast / b_kfast say which index is contiguous in the operand's memory, so that the
// staging loads coalesce.
// ---------------------------------------------------------------------------------------
template <int M, int N, class LA, class LB>
__device__ __forceinline__ void mm_tile(float (&acc)[M / 16][N / 16], int K, LA la, LB lb, float* st,
                                        bool a_kfast, bool b_kfast) {
    float* stA = st;
    float* stB = st + KS * (M + 1);
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    for (int k0 = 0; k0 < K; k0 += KS) {
        __syncthreads();
        for (int idx = tid; idx < M * KS; idx += NTHREADS) {
            int m, k;
            if (a_kfast) { k = idx % KS; m = idx / KS; } else { m = idx % M; k = idx / M; }
            stA[k * (M + 1) + m] = la(m, k0 + k);
        }
        for (int idx = tid; idx < N * KS; idx += NTHREADS) {
            int n, k;
            if (b_kfast) { k = idx % KS; n = idx / KS; } else { n = idx % N; k = idx / N; }
            stB[k * (N + 1) + n] = lb(k0 + k, n);
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < KS; ++k) {
            float a[M / 16], b[N / 16];
#pragma unroll
            for (int r = 0; r < M / 16; ++r) a[r] = stA[k * (M + 1) + ty + 16 * r];
#pragma unroll
            for (int c = 0; c < N / 16; ++c) b[c] = stB[k * (N + 1) + tx + 16 * c];
#pragma unroll
            for (int r = 0; r < M / 16; ++r)
#pragma unroll
                for (int c = 0; c < N / 16; ++c) acc[r][c] = fmaf(a[r], b[c], acc[r][c]);
        }
    }
    __syncthreads();
}

template <int M, int N>
__device__ __forceinline__ void zero_acc(float (&acc)[M][N]) {
#pragma unroll
    for (int r = 0; r < M; ++r)
#pragma unroll
        for (int c = 0; c < N; ++c) acc[r][c] = 0.f;
}

// sum over the 16 lanes that share a row (tx = 0..15 within a half warp)
__device__ __forceinline__ float row16_sum(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---------------------------------------------------------------------------------------
// Prologue of one chunk x head into shared memory:
//   sq, sk  normalised q, k (x / max(||x||, 1e-6), k3mini/model.py:218-219) or raw
//   sG      inclusive cumulative log2-decay of the chunk (rows >= len repeat the last value)
//   sv      v (optional)          sbeta  beta after the optional sigmoid (0 on padding rows)
//   srq,srk 1 / max(||x||, eps) per row (1 when the norm is not applied)
// ---------------------------------------------------------------------------------------
template <typename T, int D>
__device__ __forceinline__ void load_prologue(const KdaParams& p, const ChunkInfo& ci, int h, float* sq, float* sk,
                                              float* sG, float* sv, float* sbeta, float* srq, float* srk) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const T* q = (const T*)p.q;
    const T* k = (const T*)p.k;
    const T* v = (const T*)p.v;
    const T* g = (const T*)p.g;
    const T* beta = (const T*)p.beta;
    const bool l2 = p.flags & KDA_FLAG_QK_L2NORM, gate = p.flags & KDA_FLAG_GATE, sig = p.flags & KDA_FLAG_BETA_SIGMOID;
    const float negA = gate ? -expf(p.A_log[h]) : 0.f;
    for (int r = warp; r < C; r += NTHREADS / 32) {
        const bool valid = r < ci.len;
        const size_t row = (size_t)(ci.tok0 + r) * p.H + h;
        float qv[D / 32], kv[D / 32];
        float ssq = 0.f, ssk = 0.f;
#pragma unroll
        for (int m = 0; m < D / 32; ++m) {
            int d = lane + 32 * m;
            qv[m] = valid ? ldf(q + row * D + d) : 0.f;
            kv[m] = valid ? ldf(k + row * D + d) : 0.f;
            ssq += qv[m] * qv[m];
            ssk += kv[m] * kv[m];
        }
        float rq = 1.f, rk = 1.f;
        if (l2) {
            ssq = warp_sum(ssq);
            ssk = warp_sum(ssk);
            rq = 1.f / fmaxf(sqrtf(ssq), 1e-6f);
            rk = 1.f / fmaxf(sqrtf(ssk), 1e-6f);
        }
#pragma unroll
        for (int m = 0; m < D / 32; ++m) {
            int d = lane + 32 * m;
            sq[r * D + d] = qv[m] * rq;
            sk[r * D + d] = kv[m] * rk;
            float gl = 0.f;
            if (valid) {
                float x = ldf(g + row * D + d);
                if (gate) {
                    if (p.dt_bias) x += p.dt_bias[h * D + d];
                    gl = negA * softplus_f(x);
                } else {
                    gl = x;
                }
            }
            sG[r * D + d] = gl * LOG2E;
            if (sv) sv[r * D + d] = valid ? ldf(v + row * D + d) : 0.f;
        }
        if (lane == 0) {
            float b = 0.f;
            if (valid) {
                b = ldf(beta + row);
                if (sig) b = sigmoid_f(b);
            }
            sbeta[r] = b;
            srq[r] = rq;
            srk[r] = rk;
        }
    }
    __syncthreads();
    for (int d = tid; d < D; d += NTHREADS) {
        float run = 0.f;
        for (int r = 0; r < C; ++r) {
            run += sG[r * D + d];
            sG[r * D + d] = run;
        }
    }
    __syncthreads();
}

// ---------------------------------------------------------------------------------------
// fwd_intra
// ---------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(NTHREADS, 1) kda_fwd_intra_simt(const KdaParams p) {
    extern __shared__ float smem[];
    float* sq = smem;
    float* sk = sq + C * D;
    float* sG = sk + C * D;
    float* sv = sG + C * D;
    float* sA = sv + C * D;       // [64][65]
    float* sL = sA + C * 65;
    float* sT = sL + C * 65;
    float* sbeta = sT + C * 65;
    float* srq = sbeta + C;
    float* srk = srq + C;
    float* st = srk + C;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, ty = tid >> 4, tx = tid & 15;
    const int c = blockIdx.x / p.H, h = blockIdx.x % p.H;
    const ChunkInfo ci = chunk_info(p, c);
    const WsLayout L = ws_layout(p.NT, p.H, p.dk, p.dv, p.dtype);
    char* ws = (char*)p.workspace;
    const size_t rec = (size_t)c * p.H + h;
    T* gW = (T*)(ws + L.W) + rec * C * D;
    T* gU = (T*)(ws + L.U) + rec * C * D;
    T* gA = (T*)(ws + L.Aqk) + rec * C * C;
    T* gQt = (T*)(ws + L.Qt) + rec * C * D;
    T* gKh = (T*)(ws + L.Kh) + rec * C * D;
    T* gT = (T*)(ws + L.Tm) + rec * C * C;
    float* gGam = (float*)(ws + L.gamC) + rec * D;

    load_prologue<T, D>(p, ci, h, sq, sk, sG, sv, sbeta, srq, srk);
    const bool save = !(p.flags & KDA_FLAG_NO_SAVE);  // forward-only calls keep nothing for a backward
    if (save) {  // prologue results kept for the backward
        float* gGc = (float*)(ws + L.Gc) + rec * C * D;
        T* gQn = (T*)(ws + L.Qn) + rec * C * D;
        T* gKn = (T*)(ws + L.Kn) + rec * C * D;
        float* gaux = (float*)(ws + L.aux) + rec * 3 * C;
        for (int idx = tid; idx < C * D; idx += NTHREADS) {
            // d = 128: the chunk-swizzled row layout the tensor-core backward reads (swz_f32 / swz_bf16)
            const int r = idx / D, dd = idx % D;
            gGc[D == 128 ? tc::swz_f32(r, dd) : idx] = sG[idx];
            stf(gQn + (D == 128 ? (sizeof(T) == 2 ? tc::swz_bf16(r, dd) : tc::swz_f32(r, dd)) : idx), sq[idx]);
            stf(gKn + (D == 128 ? (sizeof(T) == 2 ? tc::swz_bf16(r, dd) : tc::swz_f32(r, dd)) : idx), sk[idx]);
        }
        if (tid < C) {
            gaux[tid] = srq[tid];
            gaux[C + tid] = srk[tid];
            gaux[2 * C + tid] = sbeta[tid];
        }
    }

    // exact pairwise products: one warp per (i, j) pair, lanes over channels
    for (int i = warp; i < C; i += NTHREADS / 32) {
        float qi[D / 32], ki[D / 32], gi[D / 32];
#pragma unroll
        for (int m = 0; m < D / 32; ++m) {
            qi[m] = sq[i * D + lane + 32 * m];
            ki[m] = sk[i * D + lane + 32 * m];
            gi[m] = sG[i * D + lane + 32 * m];
        }
        for (int j = 0; j < C; ++j) {
            float a = 0.f, l = 0.f;
            if (j <= i) {
#pragma unroll
                for (int m = 0; m < D / 32; ++m) {
                    float kd = sk[j * D + lane + 32 * m] * exp2f(gi[m] - sG[j * D + lane + 32 * m]);
                    a = fmaf(qi[m], kd, a);
                    l = fmaf(ki[m], kd, l);
                }
                a = warp_sum(a);
                l = warp_sum(l);
            }
            if (lane == 0) {
                sA[i * 65 + j] = (j <= i) ? a * p.scale : 0.f;
                sL[i * 65 + j] = (j < i) ? l : 0.f;
            }
        }
    }
    for (int idx = tid; idx < C * 65; idx += NTHREADS) sT[idx] = 0.f;
    __syncthreads();

    // T = (I + diag(beta) L)^-1 by forward substitution, 4 threads per column
    {
        const int col = tid >> 2, part = tid & 3;
        for (int i = 0; i < C; ++i) {
            float s = 0.f;
            for (int j = part; j < i; j += 4) s = fmaf(sL[i * 65 + j], sT[j * 65 + col], s);
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            if (part == 0 && col <= i) sT[i * 65 + col] = (i == col ? 1.f : 0.f) - sbeta[i] * s;
            __syncthreads();
        }
    }

    // records that depend only on the prologue
    for (int idx = tid; idx < C * C; idx += NTHREADS) {
        int i = idx / C, j = idx % C;
        stf(gA + tc::cm_idx(i, j, C), sA[i * 65 + j]);
        if (save) stf(gT + tc::cm_idx(i, j, C), sT[i * 65 + j]);
    }
    for (int idx = tid; idx < C * D; idx += NTHREADS) {
        int i = idx / D, d = idx % D;
        float G = sG[idx], gl = sG[(C - 1) * D + d];
        float gam = exp2f(G);
        stf(gQt + tc::cm_idx(i, d, D), p.scale * sq[idx] * gam);
        stf(gKh + tc::cm_idx(i, d, D), sk[idx] * exp2f(gl - G));
        if (i == C - 1) gGam[d] = gam;
    }
    __syncthreads();
    // operands of the WY products, in place: beta * k * 2^G and beta * v
    for (int idx = tid; idx < C * D; idx += NTHREADS) {
        int i = idx / D;
        sq[idx] = sbeta[i] * sk[idx] * exp2f(sG[idx]);
        sv[idx] = sbeta[i] * sv[idx];
    }
    __syncthreads();
    {
        float acc[4][D / 16];
        zero_acc(acc);
        mm_tile<C, D>(acc, C, [&](int m, int k) { return sT[m * 65 + k]; }, [&](int k, int n) { return sq[k * D + n]; },
                      st, true, false);
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int cc = 0; cc < D / 16; ++cc) stf(gW + tc::cm_idx(tx + 16 * cc, ty + 16 * r, C), acc[r][cc]);
        zero_acc(acc);
        mm_tile<C, D>(acc, C, [&](int m, int k) { return sT[m * 65 + k]; }, [&](int k, int n) { return sv[k * D + n]; },
                      st, true, false);
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int cc = 0; cc < D / 16; ++cc) stf(gU + tc::cm_idx(tx + 16 * cc, ty + 16 * r, C), acc[r][cc]);
    }
}

// ---------------------------------------------------------------------------------------
// fwd_state: sequential over the chunks of one sequence, for one head and one panel of BV
// state columns.  Writes V' over U, the chunk-entry states, o and the final state.
// ---------------------------------------------------------------------------------------
template <typename T, int D, int BV>
__global__ void __launch_bounds__(NTHREADS) kda_fwd_state_simt(const KdaParams p) {
    extern __shared__ float smem[];
    float* sS = smem;                  // [D][BV+1]
    float* sVn = sS + D * (BV + 1);    // [64][BV+1]
    float* st = sVn + C * (BV + 1);
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int e0 = blockIdx.x * BV, h = blockIdx.y, n = blockIdx.z;
    const WsLayout L = ws_layout(p.NT, p.H, p.dk, p.dv, p.dtype);
    char* ws = (char*)p.workspace;
    int c0, nc;
    seq_chunks(p, n, c0, nc);
    const size_t sbase = ((size_t)n * p.H + h) * D * D;

    for (int idx = tid; idx < D * BV; idx += NTHREADS) {
        int d = idx / BV, e = idx % BV;
        sS[d * (BV + 1) + e] = p.h0 ? p.h0[sbase + state_idx(p, d, e0 + e)] : 0.f;
    }
    __syncthreads();

    for (int lc = 0; lc < nc; ++lc) {
        const int c = c0 + lc;
        const ChunkInfo ci = chunk_info(p, c);
        const size_t rec = (size_t)c * p.H + h;
        const T* gW = (const T*)(ws + L.W) + rec * C * D;
        T* gU = (T*)(ws + L.U) + rec * C * D;
        const T* gA = (const T*)(ws + L.Aqk) + rec * C * C;
        const T* gQt = (const T*)(ws + L.Qt) + rec * C * D;
        const T* gKh = (const T*)(ws + L.Kh) + rec * C * D;
        T* gS0 = (T*)(ws + L.S0) + rec * D * D;
        const float* gGam = (const float*)(ws + L.gamC) + rec * D;
        T* o = (T*)p.o;

        for (int idx = tid; idx < D * BV; idx += NTHREADS) {
            int d = idx / BV, e = idx % BV;
            if (!(p.flags & KDA_FLAG_NO_SAVE)) stf(gS0 + tc::cm_idx(e0 + e, d, D), sS[d * (BV + 1) + e]);
        }
        // V' = U - W S
        {
            float acc[4][BV / 16];
            zero_acc(acc);
            mm_tile<C, BV>(acc, D, [&](int m, int k) { return ldf(gW + tc::cm_idx(k, m, C)); },
                           [&](int k, int nn) { return sS[k * (BV + 1) + nn]; }, st, true, false);
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int cc = 0; cc < BV / 16; ++cc) {
                    int i = ty + 16 * r, e = tx + 16 * cc;
                    float vn = ldf(gU + tc::cm_idx(e0 + e, i, C)) - acc[r][cc];
                    sVn[i * (BV + 1) + e] = vn;
                    if (!(p.flags & KDA_FLAG_NO_SAVE)) stf(gU + tc::cm_idx(e0 + e, i, C), vn);
                }
        }
        // O = Qt S + Aqk V'
        {
            float acc[4][BV / 16];
            zero_acc(acc);
            mm_tile<C, BV>(acc, D, [&](int m, int k) { return ldf(gQt + tc::cm_idx(m, k, D)); },
                           [&](int k, int nn) { return sS[k * (BV + 1) + nn]; }, st, true, false);
            mm_tile<C, BV>(acc, C, [&](int m, int k) { return ldf(gA + tc::cm_idx(m, k, C)); },
                           [&](int k, int nn) { return sVn[k * (BV + 1) + nn]; }, st, true, false);
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int cc = 0; cc < BV / 16; ++cc) {
                    int i = ty + 16 * r, e = tx + 16 * cc;
                    if (i < ci.len) stf(o + ((size_t)(ci.tok0 + i) * p.H + h) * D + e0 + e, acc[r][cc]);
                }
        }
        // S = diag(gamC) S + Kh^T V'
        {
            float acc[D / 16][BV / 16];
            zero_acc(acc);
            mm_tile<D, BV>(acc, C, [&](int m, int k) { return ldf(gKh + tc::cm_idx(k, m, D)); },
                           [&](int k, int nn) { return sVn[k * (BV + 1) + nn]; }, st, false, false);
#pragma unroll
            for (int r = 0; r < D / 16; ++r)
#pragma unroll
                for (int cc = 0; cc < BV / 16; ++cc) {
                    int d = ty + 16 * r, e = tx + 16 * cc;
                    sS[d * (BV + 1) + e] = gGam[d] * sS[d * (BV + 1) + e] + acc[r][cc];
                }
        }
        __syncthreads();
    }
    if (p.ht) {
        for (int idx = tid; idx < D * BV; idx += NTHREADS) {
            int d = idx / BV, e = idx % BV;
            p.ht[sbase + state_idx(p, d, e0 + e)] = sS[d * (BV + 1) + e];
        }
    }
}

// ---------------------------------------------------------------------------------------
// bwd_state: reverse over the chunks.  dV' = Aqk^T dO + Kh dS,
// dS <- diag(gamC) dS + Qt^T dO - W^T dV'.  Stores the dS entering each chunk and dV'.
// ---------------------------------------------------------------------------------------
template <typename T, int D, int BV>
__global__ void __launch_bounds__(NTHREADS) kda_bwd_state_simt(const KdaParams p) {
    extern __shared__ float smem[];
    float* sS = smem;                  // dS [D][BV+1]
    float* sVn = sS + D * (BV + 1);    // dV' [64][BV+1]
    float* st = sVn + C * (BV + 1);
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int e0 = blockIdx.x * BV, h = blockIdx.y, n = blockIdx.z;
    const WsLayout L = ws_layout(p.NT, p.H, p.dk, p.dv, p.dtype);
    const char* ws = (const char*)p.workspace;
    char* sc = (char*)p.bwd_scratch;
    int c0, nc;
    seq_chunks(p, n, c0, nc);
    const size_t sbase = ((size_t)n * p.H + h) * D * D;
    const T* dO = (const T*)p.grad_o;

    for (int idx = tid; idx < D * BV; idx += NTHREADS) {
        int d = idx / BV, e = idx % BV;
        sS[d * (BV + 1) + e] = p.grad_ht ? p.grad_ht[sbase + state_idx(p, d, e0 + e)] : 0.f;
    }
    __syncthreads();

    for (int lc = nc - 1; lc >= 0; --lc) {
        const int c = c0 + lc;
        const ChunkInfo ci = chunk_info(p, c);
        const size_t rec = (size_t)c * p.H + h;
        const T* gW = (const T*)(ws + L.W) + rec * C * D;
        const T* gA = (const T*)(ws + L.Aqk) + rec * C * C;
        const T* gQt = (const T*)(ws + L.Qt) + rec * C * D;
        const T* gKh = (const T*)(ws + L.Kh) + rec * C * D;
        const float* gGam = (const float*)(ws + L.gamC) + rec * D;
        T* gdS = (T*)(sc + L.dS) + rec * D * D;
        T* gdV = (T*)(sc + L.dVn) + rec * C * D;
        auto ldo = [&](int i, int e) {
            return i < ci.len ? ldf(dO + ((size_t)(ci.tok0 + i) * p.H + h) * D + e0 + e) : 0.f;
        };
        for (int idx = tid; idx < D * BV; idx += NTHREADS) {
            int d = idx / BV, e = idx % BV;
            stf(gdS + tc::cm_idx(e0 + e, d, D), sS[d * (BV + 1) + e]);
        }
        {
            float acc[4][BV / 16];
            zero_acc(acc);
            mm_tile<C, BV>(acc, C, [&](int m, int k) { return ldf(gA + tc::cm_idx(k, m, C)); },
                           [&](int k, int nn) { return ldo(k, nn); }, st, false, false);
            mm_tile<C, BV>(acc, D, [&](int m, int k) { return ldf(gKh + tc::cm_idx(m, k, D)); },
                           [&](int k, int nn) { return sS[k * (BV + 1) + nn]; }, st, true, false);
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int cc = 0; cc < BV / 16; ++cc) {
                    int i = ty + 16 * r, e = tx + 16 * cc;
                    sVn[i * (BV + 1) + e] = acc[r][cc];
                    stf(gdV + tc::cm_idx(e0 + e, i, C), acc[r][cc]);
                }
        }
        {
            float acc[D / 16][BV / 16];
            zero_acc(acc);
            mm_tile<D, BV>(acc, C, [&](int m, int k) { return ldf(gQt + tc::cm_idx(k, m, D)); },
                           [&](int k, int nn) { return ldo(k, nn); }, st, false, false);
            mm_tile<D, BV>(acc, C, [&](int m, int k) { return -ldf(gW + tc::cm_idx(m, k, C)); },
                           [&](int k, int nn) { return sVn[k * (BV + 1) + nn]; }, st, false, false);
#pragma unroll
            for (int r = 0; r < D / 16; ++r)
#pragma unroll
                for (int cc = 0; cc < BV / 16; ++cc) {
                    int d = ty + 16 * r, e = tx + 16 * cc;
                    sS[d * (BV + 1) + e] = gGam[d] * sS[d * (BV + 1) + e] + acc[r][cc];
                }
        }
        __syncthreads();
    }
    if (p.grad_h0) {
        for (int idx = tid; idx < D * BV; idx += NTHREADS) {
            int d = idx / BV, e = idx % BV;
            p.grad_h0[sbase + state_idx(p, d, e0 + e)] = sS[d * (BV + 1) + e];
        }
    }
}

// ---------------------------------------------------------------------------------------
// bwd_chunk: all chunk-local adjoints, the exact pairwise intra step, the reverse cumulative
// sum of the gate gradient and the chain rule through gate / L2 norm / sigmoid.
// ---------------------------------------------------------------------------------------
// SPLIT = true stops after the chunk-level adjoints and leaves them in the scratch buffer for
// the separate intra kernel of the BF16 path (used to validate the two halves independently).
// one entry of the hand-over matrices dAqk / dM in the layout bwd_intra reads: three BF16 tiles
// cm(i, j; 64) whose sum is x
__device__ __forceinline__ void store_split3(__nv_bfloat16* base, int i, int j, float x) {
    uint32_t p0, p1, p2;
    split3_bf16(x, 0.f, p0, p1, p2);
    unsigned short* b = reinterpret_cast<unsigned short*>(base) + tc::cm_idx(i, j, C);
    b[0] = (unsigned short)(p0 & 0xffffu);
    b[C * C] = (unsigned short)(p1 & 0xffffu);
    b[2 * C * C] = (unsigned short)(p2 & 0xffffu);
}

template <typename T, int D, bool SPLIT = false>
__global__ void __launch_bounds__(NTHREADS, 1) kda_bwd_chunk_simt(const KdaParams p) {
    extern __shared__ float smem[];
    float* sq = smem;
    float* sk = sq + C * D;
    float* sG = sk + C * D;
    float* sW = sG + C * D;        // dW, later scratch
    float* sT = sW + C * D;        // [64][65]
    float* sdA = sT + C * 65;
    float* sdM = sdA + C * 65;     // first holds dT
    float* sY = sdM + C * 65;
    float* sbeta = sY + C * 65;
    float* srq = sbeta + C;
    float* srk = srq + C;
    float* sdb = srk + C;          // dbeta accumulator
    float* scol = sdb + C;         // [D] last-row term of dG
    float* sred = scol + D;        // [8] block reduction
    float* st = sred + 8;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, ty = tid >> 4, tx = tid & 15;
    const int c = blockIdx.x / p.H, h = blockIdx.x % p.H;
    const ChunkInfo ci = chunk_info(p, c);
    const WsLayout L = ws_layout(p.NT, p.H, p.dk, p.dv, p.dtype);
    const char* ws = (const char*)p.workspace;
    char* sc = (char*)p.bwd_scratch;
    const size_t rec = (size_t)c * p.H + h;
    const T* gVn = (const T*)(ws + L.U) + rec * C * D;
    const T* gT = (const T*)(ws + L.Tm) + rec * C * C;
    const T* gS0 = (const T*)(ws + L.S0) + rec * D * D;
    const float* gGam = (const float*)(ws + L.gamC) + rec * D;
    const T* gdS = (const T*)(sc + L.dS) + rec * D * D;
    const T* gdV = (const T*)(sc + L.dVn) + rec * C * D;
    const T* dO = (const T*)p.grad_o;
    const T* v = (const T*)p.v;
    const float scale = p.scale;

    load_prologue<T, D>(p, ci, h, sq, sk, sG, nullptr, sbeta, srq, srk);
    for (int idx = tid; idx < C * C; idx += NTHREADS) sT[(idx / C) * 65 + idx % C] = ldf(gT + tc::cm_idx(idx / C, idx % C, C));
    if (tid < C) sdb[tid] = 0.f;

    auto ldo = [&](int i, int e) { return i < ci.len ? ldf(dO + ((size_t)(ci.tok0 + i) * p.H + h) * D + e) : 0.f; };
    auto ldv = [&](int i, int e) { return i < ci.len ? ldf(v + ((size_t)(ci.tok0 + i) * p.H + h) * D + e) : 0.f; };

    float dq_a[4][D / 16], dk_a[4][D / 16], dG_a[4][D / 16];
    float db_r[4] = {0.f, 0.f, 0.f, 0.f};
    zero_acc(dq_a);
    zero_acc(dk_a);
    zero_acc(dG_a);

    // 1. dAqk = tril(dO V'^T)
    {
        float acc[4][4];
        zero_acc(acc);
        mm_tile<C, C>(acc, D, [&](int m, int k) { return ldo(m, k); }, [&](int k, int n) { return ldf(gVn + tc::cm_idx(k, n, C)); }, st,
                      true, true);
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                int i = ty + 16 * r, j = tx + 16 * cc;
                sdA[i * 65 + j] = (i >= j) ? acc[r][cc] : 0.f;
                if constexpr (SPLIT) {
                    store_split3((__nv_bfloat16*)(sc + L.dAM) + rec * 6 * C * C, i, j, i > j ? sdA[i * 65 + j] : 0.f);
                    if (i == j) ((float*)(sc + L.dAd))[rec * C + i] = sdA[i * 65 + j];
                }
            }
    }
    // 2. dW = -dV' S0^T
    {
        float acc[4][D / 16];
        zero_acc(acc);
        mm_tile<C, D>(acc, D, [&](int m, int k) { return ldf(gdV + tc::cm_idx(k, m, C)); },
                      [&](int k, int n) { return ldf(gS0 + tc::cm_idx(k, n, D)); }, st, true, true);
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int cc = 0; cc < D / 16; ++cc) sW[(ty + 16 * r) * D + tx + 16 * cc] = -acc[r][cc];
    }
    // 3. dT = tril(dW (beta K~)^T + dV' (beta V)^T)   -> sdM
    {
        float acc[4][4];
        zero_acc(acc);
        mm_tile<C, C>(acc, D, [&](int m, int k) { return sW[m * D + k]; },
                      [&](int k, int n) { return sbeta[n] * sk[n * D + k] * exp2f(sG[n * D + k]); }, st, true, true);
        mm_tile<C, C>(acc, D, [&](int m, int k) { return ldf(gdV + tc::cm_idx(k, m, C)); },
                      [&](int k, int n) { return sbeta[n] * ldv(n, k); }, st, true, true);
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                int i = ty + 16 * r, j = tx + 16 * cc;
                sdM[i * 65 + j] = (i >= j) ? acc[r][cc] : 0.f;
            }
    }
    // 4. dM = -T^T dT T^T (strictly lower part is what the intra step uses)
    {
        float acc[4][4];
        zero_acc(acc);
        mm_tile<C, C>(acc, C, [&](int m, int k) { return sdM[m * 65 + k]; }, [&](int k, int n) { return sT[n * 65 + k]; }, st,
                      true, true);
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) sY[(ty + 16 * r) * 65 + tx + 16 * cc] = acc[r][cc];
        zero_acc(acc);
        mm_tile<C, C>(acc, C, [&](int m, int k) { return sT[k * 65 + m]; }, [&](int k, int n) { return sY[k * 65 + n]; }, st,
                      false, false);
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                int i = ty + 16 * r, j = tx + 16 * cc;
                sdM[i * 65 + j] = (i > j) ? -acc[r][cc] : 0.f;
                if constexpr (SPLIT)
                    store_split3((__nv_bfloat16*)(sc + L.dAM) + rec * 6 * C * C + 3 * C * C, i, j, sdM[i * 65 + j]);
            }
    }
    // 5. d(beta K~) = T^T dW
    {
        float acc[4][D / 16];
        zero_acc(acc);
        mm_tile<C, D>(acc, C, [&](int m, int k) { return sT[k * 65 + m]; }, [&](int k, int n) { return sW[k * D + n]; }, st,
                      false, false);
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int cc = 0; cc < D / 16; ++cc) {
                int i = ty + 16 * r, d = tx + 16 * cc;
                if constexpr (SPLIT) {
                    stf((T*)(sc + L.dKb) + rec * C * D + handover_idx(i, d), acc[r][cc]);
                    continue;
                }
                float gam = exp2f(sG[i * D + d]);
                float kt = sk[i * D + d] * gam;
                float dkt = sbeta[i] * acc[r][cc];
                dk_a[r][cc] += dkt * gam;
                dG_a[r][cc] += dkt * kt;
                db_r[r] += acc[r][cc] * kt;
            }
    }
    // 6. d(beta V) = T^T dV'  -> dv
    {
        float acc[4][D / 16];
        zero_acc(acc);
        mm_tile<C, D>(acc, C, [&](int m, int k) { return sT[k * 65 + m]; }, [&](int k, int n) { return ldf(gdV + tc::cm_idx(n, k, C)); },
                      st, false, false);
        T* dv = (T*)p.grad_v;
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int cc = 0; cc < D / 16; ++cc) {
                int i = ty + 16 * r, e = tx + 16 * cc;
                if (i < ci.len) {
                    stf(dv + ((size_t)(ci.tok0 + i) * p.H + h) * D + e, sbeta[i] * acc[r][cc]);
                    db_r[r] += acc[r][cc] * ldv(i, e);
                }
            }
    }
    // 7. dQt = dO S0^T
    {
        float acc[4][D / 16];
        zero_acc(acc);
        mm_tile<C, D>(acc, D, [&](int m, int k) { return ldo(m, k); }, [&](int k, int n) { return ldf(gS0 + tc::cm_idx(k, n, D)); }, st,
                      true, true);
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int cc = 0; cc < D / 16; ++cc) {
                int i = ty + 16 * r, d = tx + 16 * cc;
                if constexpr (SPLIT) {
                    stf((T*)(sc + L.dQt) + rec * C * D + handover_idx(i, d), acc[r][cc]);
                    continue;
                }
                float gam = exp2f(sG[i * D + d]);
                dq_a[r][cc] += scale * acc[r][cc] * gam;
                dG_a[r][cc] += acc[r][cc] * scale * sq[i * D + d] * gam;
            }
    }
    // 8. dKh = V' dS^T ; its column sums feed the last row of dG
    {
        float acc[4][D / 16];
        zero_acc(acc);
        mm_tile<C, D>(acc, D, [&](int m, int k) { return ldf(gVn + tc::cm_idx(k, m, C)); },
                      [&](int k, int n) { return ldf(gdS + tc::cm_idx(k, n, D)); }, st, true, true);
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int cc = 0; cc < D / 16; ++cc) {
                int i = ty + 16 * r, d = tx + 16 * cc;
                if constexpr (SPLIT) {
                    stf((T*)(sc + L.dKh) + rec * C * D + handover_idx(i, d), acc[r][cc]);
                    sW[i * D + d] = 0.f;
                    continue;
                }
                float dec = exp2f(sG[(C - 1) * D + d] - sG[i * D + d]);
                float kh = sk[i * D + d] * dec;
                dk_a[r][cc] += acc[r][cc] * dec;
                dG_a[r][cc] -= acc[r][cc] * kh;
                sW[i * D + d] = acc[r][cc] * kh;
            }
    }
    __syncthreads();
    for (int d = tid; d < D; d += NTHREADS) {
        float s = 0.f;
        for (int i = 0; i < C; ++i) s += sW[i * D + d];
        scol[d] = s;
    }
    __syncthreads();
    // 9. d(gamC)[d] = sum_e dS[d][e] S0[d][e]
    for (int d = warp; d < D; d += NTHREADS / 32) {
        float s = 0.f;
        for (int e = lane; e < D; e += 32) s = fmaf(ldf(gdS + tc::cm_idx(e, d, D)), ldf(gS0 + tc::cm_idx(e, d, D)), s);
        s = warp_sum(s);
        if (lane == 0) scol[d] += s * gGam[d];
    }
    if constexpr (SPLIT) {  // hand over: beta gradient so far and dGamma_C * Gamma_C
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            float s = row16_sum(db_r[r]);
            if (tx == 0) ((float*)(sc + L.dbp))[rec * C + ty + 16 * r] = s;
        }
        __syncthreads();
        for (int d = tid; d < D; d += NTHREADS) ((float*)(sc + L.gC))[rec * D + d] = scol[d];
        return;
    }
    // 10. intra step with exact pairwise decays
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int i = ty + 16 * r;
#pragma unroll
        for (int cc = 0; cc < D / 16; ++cc) {
            const int d = tx + 16 * cc;
            const float gi = sG[i * D + d], qi = sq[i * D + d], ki = sk[i * D + d];
            // strictly-lower / strictly-upper parts; the diagonal pair (j == i) has decay 1 and
            // contributes equal and opposite amounts to dG, so it is kept out of dG exactly
            float a1 = 0.f, a2 = 0.f;
            for (int j = 0; j < i; ++j) {
                float kd = sk[j * D + d] * exp2f(gi - sG[j * D + d]);
                a1 = fmaf(sdA[i * 65 + j], kd, a1);
                a2 = fmaf(sdM[i * 65 + j], kd, a2);
            }
            float c1 = 0.f;
            for (int ii = i + 1; ii < C; ++ii) {
                float e = exp2f(sG[ii * D + d] - gi);
                float t = scale * sdA[ii * 65 + i] * sq[ii * D + d] + sbeta[ii] * sdM[ii * 65 + i] * sk[ii * D + d];
                c1 = fmaf(t, e, c1);
            }
            const float diag = scale * sdA[i * 65 + i];
            float dq_in = scale * a1, dk_row = sbeta[i] * a2;
            db_r[r] += ki * a2;
            dq_a[r][cc] += dq_in + diag * ki;
            dk_a[r][cc] += dk_row + c1 + diag * qi;
            dG_a[r][cc] += qi * dq_in + ki * dk_row - ki * c1;
        }
    }
    // 11. dbeta rows
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        float s = row16_sum(db_r[r]);
        if (tx == 0) sdb[ty + 16 * r] = s;
    }
    // 12. reverse cumulative sum of dG and the gate chain
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int cc = 0; cc < D / 16; ++cc) sW[(ty + 16 * r) * D + tx + 16 * cc] = dG_a[r][cc];
    __syncthreads();
    {
        const bool gate = p.flags & KDA_FLAG_GATE;
        const float negA = gate ? -expf(p.A_log[h]) : 0.f;
        const T* g = (const T*)p.g;
        T* dg = (T*)p.grad_g;
        float dA = 0.f;
        for (int d = tid; d < D; d += NTHREADS) {
            float run = scol[d], dbias = 0.f;
            for (int i = C - 1; i >= 0; --i) {
                run += sW[i * D + d];
                if (i < ci.len) {
                    size_t off = ((size_t)(ci.tok0 + i) * p.H + h) * D + d;
                    if (gate) {
                        float z = ldf(g + off);
                        if (p.dt_bias) z += p.dt_bias[h * D + d];
                        dA = fmaf(run, negA * softplus_f(z), dA);
                        float dx = run * negA * sigmoid_f(z);
                        dbias += dx;
                        stf(dg + off, dx);
                    } else {
                        stf(dg + off, run);
                    }
                }
            }
            if (gate) ((float*)(sc + L.dbias_part))[rec * D + d] = dbias;
        }
        if (gate) {
            dA = warp_sum(dA);
            if (lane == 0) sred[warp] = dA;
            __syncthreads();
            if (tid == 0) {
                float s = 0.f;
                for (int w = 0; w < NTHREADS / 32; ++w) s += sred[w];
                ((float*)(sc + L.dA_part))[rec] = s;
            }
        }
    }
    // 13. chain through the L2 norm, 14. through the sigmoid
    {
        const bool l2 = p.flags & KDA_FLAG_QK_L2NORM;
        T* dq = (T*)p.grad_q;
        T* dk = (T*)p.grad_k;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int i = ty + 16 * r;
            float dotq = 0.f, dotk = 0.f;
            if (l2) {
#pragma unroll
                for (int cc = 0; cc < D / 16; ++cc) {
                    dotq += sq[i * D + tx + 16 * cc] * dq_a[r][cc];
                    dotk += sk[i * D + tx + 16 * cc] * dk_a[r][cc];
                }
                dotq = row16_sum(dotq);
                dotk = row16_sum(dotk);
            }
            if (i < ci.len) {
#pragma unroll
                for (int cc = 0; cc < D / 16; ++cc) {
                    int d = tx + 16 * cc;
                    size_t off = ((size_t)(ci.tok0 + i) * p.H + h) * D + d;
                    float a = dq_a[r][cc], b = dk_a[r][cc];
                    if (l2) {
                        a = (a - sq[i * D + d] * dotq) * srq[i];
                        b = (b - sk[i * D + d] * dotk) * srk[i];
                    }
                    stf(dq + off, a);
                    stf(dk + off, b);
                }
            }
        }
        if (tid < ci.len) {
            float b = sbeta[tid], db = sdb[tid];
            if (p.flags & KDA_FLAG_BETA_SIGMOID) db *= b * (1.f - b);
            stf((T*)p.grad_beta + (size_t)(ci.tok0 + tid) * p.H + h, db);
        }
    }
}

// deterministic reduction of the per-chunk partial parameter gradients: one block per head,
// 8 groups of 128 threads each sum every 8th chunk in order, then the 8 group sums are added
// in a fixed order
__global__ void __launch_bounds__(1024) kda_param_reduce(const KdaParams p) {
    __shared__ float sb[8][128];
    __shared__ float sa[8][32];
    const WsLayout L = ws_layout(p.NT, p.H, p.dk, p.dv, p.dtype);
    const char* sc = (const char*)p.bwd_scratch;
    const int h = blockIdx.x, d = threadIdx.x & 127, grp = threadIdx.x >> 7;
    const float* pb = (const float*)(sc + L.dbias_part);
    const float* pa = (const float*)(sc + L.dA_part);
    // (sixteen loads in flight per thread, added in chunk order: the loop is a chain of round trips otherwise)
    float s = 0.f;
    if (d < p.dk)
        for (int c0 = grp; c0 < p.NT; c0 += 8 * 16) {
            float v[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const int c = c0 + 8 * u;
                v[u] = c < p.NT ? pb[((size_t)c * p.H + h) * p.dk + d] : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 16; ++u) s += v[u];
        }
    sb[grp][d] = s;
    // dA_log: lanes 0..31 of every group take every 32nd of the group's chunks
    float a = 0.f;
    if (d < 32)
        for (int c = grp + 8 * d; c < p.NT; c += 256) a += pa[(size_t)c * p.H + h];
    if (d < 32) sa[grp][d] = a;
    __syncthreads();
    if (grp == 0) {
        if (d < p.dk && p.grad_dt_bias) {
            float t = 0.f;
            for (int gidx = 0; gidx < 8; ++gidx) t += sb[gidx][d];
            p.grad_dt_bias[h * p.dk + d] = t;
        }
        if (d == 0 && p.grad_A_log) {
            float t = 0.f;
            for (int gidx = 0; gidx < 8; ++gidx)
                for (int l = 0; l < 32; ++l) t += sa[gidx][l];
            p.grad_A_log[h] = t;
        }
    }
}

// ---------------------------------------------------------------------------------------
// host-side launchers
// ---------------------------------------------------------------------------------------
template <int D>
constexpr size_t smem_intra() { return (size_t)(4 * C * D + 3 * C * 65 + 3 * C + KS * (C + 1) + KS * (D + 1)) * 4; }
template <int D, int BV>
constexpr size_t smem_state() { return (size_t)(D * (BV + 1) + C * (BV + 1) + KS * (D + 1) + KS * (BV + 1)) * 4; }
template <int D>
constexpr size_t smem_bwd_chunk() {
    return (size_t)(4 * C * D + 4 * C * 65 + 4 * C + D + 8 + KS * (C + 1) + KS * (D + 1)) * 4;
}

template <typename K>
static cudaError_t set_smem(K kernel, size_t bytes) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

template <typename T, int D>
static cudaError_t launch_stage(const KdaParams& p, int stage, cudaStream_t s) {
    constexpr int BV = 32;
    cudaError_t e = cudaSuccess;
    switch (stage) {
        case 0:
            if ((e = set_smem(kda_fwd_intra_simt<T, D>, smem_intra<D>())) != cudaSuccess) return e;
            kda_fwd_intra_simt<T, D><<<p.NT * p.H, NTHREADS, smem_intra<D>(), s>>>(p);
            break;
        case 1:
            if ((e = set_smem(kda_fwd_state_simt<T, D, BV>, smem_state<D, BV>())) != cudaSuccess) return e;
            kda_fwd_state_simt<T, D, BV><<<dim3(D / BV, p.H, p.N), NTHREADS, smem_state<D, BV>(), s>>>(p);
            break;
        case 2:
            if ((e = set_smem(kda_bwd_state_simt<T, D, BV>, smem_state<D, BV>())) != cudaSuccess) return e;
            kda_bwd_state_simt<T, D, BV><<<dim3(D / BV, p.H, p.N), NTHREADS, smem_state<D, BV>(), s>>>(p);
            break;
        case 3:
            if ((e = set_smem(kda_bwd_chunk_simt<T, D>, smem_bwd_chunk<D>())) != cudaSuccess) return e;
            kda_bwd_chunk_simt<T, D><<<p.NT * p.H, NTHREADS, smem_bwd_chunk<D>(), s>>>(p);
            break;
        case 5:
            if ((e = set_smem(kda_bwd_chunk_simt<T, D, true>, smem_bwd_chunk<D>())) != cudaSuccess) return e;
            kda_bwd_chunk_simt<T, D, true><<<p.NT * p.H, NTHREADS, smem_bwd_chunk<D>(), s>>>(p);
            break;
        default:
            kda_param_reduce<<<p.H, 1024, 0, s>>>(p);
    }
    return cudaGetLastError();
}

// stage: 0 fwd_intra, 1 fwd_state, 2 bwd_state, 3 bwd_chunk, 4 param_reduce, 5 bwd_chunk stopped after the adjoints
cudaError_t simt_stage(const KdaParams& p, int stage, cudaStream_t s) {
    if (p.dtype == KDA_DTYPE_F32)
        return p.dk == 64 ? launch_stage<float, 64>(p, stage, s) : launch_stage<float, 128>(p, stage, s);
    return p.dk == 64 ? launch_stage<__nv_bfloat16, 64>(p, stage, s) : launch_stage<__nv_bfloat16, 128>(p, stage, s);
}

cudaError_t simt_fwd(const KdaParams& p, cudaStream_t s) {
    cudaError_t e;
    for (int st = 0; st < 2; ++st) {
        if ((e = simt_stage(p, st, s)) != cudaSuccess) return e;
        prof_mark(s);
    }
    return cudaSuccess;
}

cudaError_t simt_bwd(const KdaParams& p, cudaStream_t s) {
    cudaError_t e;
    for (int st = 2; st < 5; ++st) {
        if (st == 4 && !(p.flags & KDA_FLAG_GATE)) break;
        if ((e = simt_stage(p, st, s)) != cudaSuccess) return e;
        prof_mark(s);
    }
    return cudaSuccess;
}

}  // namespace kda
