// Shared definitions of the KDA kernels: parameter block, chunk indexing, workspace layout,
// element load/store helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/kda_b200.h"

namespace kda {

constexpr int C = KDA_CHUNK;       // tokens per chunk
constexpr float LOG2E = 1.4426950408889634f;

// records what the CUDA runtime said for kda_last_cuda_error() and returns KDA_ERR_LAUNCH
int fail_cuda(cudaError_t e);
// status of an entry point after its launches: KDA_OK, or KDA_ERR_LAUNCH with the runtime's message kept
inline int launch_status() {
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? KDA_OK : fail_cuda(e);
}
// number of SMs of the current device (grid size of the kernels that walk their units themselves);
// looked up once per device ordinal, 148 where the runtime does not answer
inline int sm_count() {
    static int cached[64] = {0};
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    if (dev >= 0 && dev < 64) cached[dev] = n;
    return n;
}

// The units a CTA of a unit-walking kernel visits: first, first + stride, ...  Unit u is chunk u / H with
// the head skewed by the chunk, (u % H + chunk) % H, so that the units of one CTA cycle through all heads
// whatever the stride (heads differ in cost).  Stepping costs additions only: the integer divisions, which
// are long dependent instruction chains, happen once per kernel.
struct UnitWalk {
    int unit, c, r, cm, stride, dq, dr, dqm, H;
    __device__ __forceinline__ void init(int first, int stride_, int H_) {
        H = H_; stride = stride_; unit = first;
        c = first / H; r = first - c * H; cm = c % H;
        dq = stride / H; dr = stride - dq * H; dqm = dq % H;
    }
    __device__ __forceinline__ int head() const { const int h = r + cm; return h >= H ? h - H : h; }
    __device__ __forceinline__ size_t rec() const { return (size_t)c * H + head(); }  // index of the unit's records
    __device__ __forceinline__ void next() {
        unit += stride; c += dq; r += dr; cm += dqm;
        if (r >= H) { r -= H; ++c; ++cm; }
        if (cm >= H) cm -= H;
    }
};

// Hand-over arrays dQt / dKh / dKb of the backward (BF16, 64 rows x 128 channels per unit): channel-major, so
// that the thread that owns a channel writes and reads 16 consecutive rows as two 16-byte words; the eight
// 16-byte chunks of a channel are XOR-swizzled by the channel, which makes the shared-memory reads of eight
// neighbouring channels hit eight different bank groups.
__host__ __device__ inline int handover_idx(int i, int d) { return d * 64 + ((((i >> 3) ^ (d & 7)) << 3) | (i & 7)); }

// ---------------------------------------------------------------------------------------
// element access
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// ---------------------------------------------------------------------------------------
// chunk indexing.  Chunks never straddle a sequence boundary: with cu_seqlens every
// document restarts its own chunk grid (the last chunk of a document may be partial).
// ---------------------------------------------------------------------------------------
struct ChunkInfo {
    int seq;        // sequence (document) index
    int lc;         // chunk index inside the sequence
    long long tok0; // flattened token index (b * T + t) of the chunk's first row
    int len;        // valid rows, 1..64
};

__device__ __forceinline__ ChunkInfo chunk_info(const KdaParams& p, int c) {
    ChunkInfo ci;
    if (p.cu_seqlens != nullptr && p.chunk_tab != nullptr) {
        const int4 t = reinterpret_cast<const int4*>(p.chunk_tab)[c];
        ci.seq = t.x;
        ci.lc = t.y;
        ci.tok0 = t.z;
        ci.len = t.w;
    } else if (p.cu_seqlens != nullptr) {
        ci.seq = p.chunk_seq[c];
        ci.lc = c - p.seq_chunk_off[ci.seq];
        long long s = p.cu_seqlens[ci.seq], e = p.cu_seqlens[ci.seq + 1];
        ci.tok0 = s + (long long)ci.lc * C;
        long long rem = e - ci.tok0;
        ci.len = rem < C ? (int)rem : C;
    } else {
        int nts = (p.T + C - 1) / C;
        ci.seq = c / nts;
        ci.lc = c - ci.seq * nts;
        ci.tok0 = (long long)ci.seq * p.T + (long long)ci.lc * C;
        int rem = p.T - ci.lc * C;
        ci.len = rem < C ? rem : C;
    }
    return ci;
}

// first chunk and number of chunks of sequence n
__device__ __forceinline__ void seq_chunks(const KdaParams& p, int n, int& c0, int& nc) {
    if (p.cu_seqlens != nullptr) {
        c0 = p.seq_chunk_off[n];
        nc = p.seq_chunk_off[n + 1] - c0;
    } else {
        nc = (p.T + C - 1) / C;
        c0 = n * nc;
    }
}

// first and one-past-last flattened token index of sequence n; chunk lc of the sequence then starts at
// first + lc * C and holds min(C, end - start) rows (what chunk_info returns, without its division / table load:
// for the kernels that walk the chunks of ONE sequence)
__device__ __forceinline__ void seq_tokens(const KdaParams& p, int n, long long& first, long long& end) {
    if (p.cu_seqlens != nullptr) {
        first = p.cu_seqlens[n];
        end = p.cu_seqlens[n + 1];
    } else {
        first = (long long)n * p.T;
        end = first + p.T;
    }
}
__device__ __forceinline__ ChunkInfo chunk_of_seq(int n, int lc, long long first, long long end) {
    ChunkInfo ci;
    ci.seq = n;
    ci.lc = lc;
    ci.tok0 = first + (long long)lc * C;
    const long long rem = end - ci.tok0;
    ci.len = rem < C ? (int)rem : C;
    return ci;
}

// ---------------------------------------------------------------------------------------
// workspace layout (byte offsets).  All per-(chunk, head) records are stored
// [NT][H][...] so that consecutive heads of one chunk are adjacent.  Inside a record the
// elements are in the core-matrix order of kda_tc.cuh (cm_idx), so that a record is a
// ready-made tcgen05 operand after one linear bulk copy into shared memory:
//   W    as W^T   cm(d, i; 64)      U / V'  as V'^T  cm(e, i; 64)     (i = token in chunk)
//   Aqk, Tm       cm(i, j; 64)      Qt, Kh           cm(i, d; dk)
//   S0, dS as S^T cm(e, d; dk)      dVn     as dV'^T cm(e, i; 64)
// gamC is a plain float[dk]; aux is a plain row-major array; Gc, Qn, Kn are row-major with their
// 16-byte chunks XOR-swizzled by the row when dk = 128 (swz_f32 / swz_bf16 in kda_tc.cuh).
// ---------------------------------------------------------------------------------------
struct WsLayout {
    size_t W, U, Aqk, Qt, Kh, gamC, total_nosave;       // what fwd_state consumes (all a forward-only call needs)
    size_t Tm, S0;                                      // kept for the backward only
    size_t Gc, Qn, Kn, aux, total;                      // prologue results kept for the backward
    size_t Vc, total_conv;                              // convolved v rows (fused short convolution only)
    size_t dS, dVn, dA_part, dbias_part;                // backward scratch
    size_t dAM, dAd, dQt, dKh, dKb, dbp, gC, bwd_total; // hand-over from bwd_wy to bwd_intra
    size_t cv_part, cv_head, cv_tail, bwd_total_conv;   // fused short-convolution backward only
};

__host__ __device__ inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

__host__ __device__ inline WsLayout ws_layout(int NT, int H, int dk, int dv, int dtype) {
    size_t es = dtype == KDA_DTYPE_BF16 ? 2 : 4;
    size_t n = (size_t)NT * H;
    WsLayout w;
    size_t off = 0;
    w.W = off;    off = align256(off + n * C * dk * es);
    w.U = off;    off = align256(off + n * C * dv * es);
    w.Aqk = off;  off = align256(off + n * C * C * es);
    w.Qt = off;   off = align256(off + n * C * dk * es);
    w.Kh = off;   off = align256(off + n * C * dk * es);
    w.gamC = off; off = align256(off + n * dk * 4);
    // a forward that nobody differentiates (KDA_FLAG_NO_SAVE) stops here: T, the chunk-entry states,
    // the V' overwrite of U and the kept prologue are written only for the backward
    w.total_nosave = off;
    w.Tm = off;   off = align256(off + n * C * C * es);
    w.S0 = off;   off = align256(off + n * dk * dv * es);
    // kept so that the backward does not redo the prologue: cumulative log2 decay G (float
    // [64][dk]), normalised q and k (element type, [64][dk] row-major), and per row
    // 1/|q|, 1/|k|, beta after the sigmoid (float [3][64])
    w.Gc = off;   off = align256(off + n * C * dk * 4);
    w.Qn = off;   off = align256(off + n * C * dk * es);
    w.Kn = off;   off = align256(off + n * C * dk * es);
    w.aux = off;  off = align256(off + n * 3 * C * 4);
    w.total = off;
    // with the short convolution fused into the load stage the backward needs the convolved v
    // rows ([64][dv] row-major per record); the record sits behind everything else so that the
    // plain call's workspace does not grow
    w.Vc = off;   off = align256(off + n * C * dv * es);
    w.total_conv = off;
    off = 0;
    w.dS = off;         off = align256(off + n * dk * dv * es);
    w.dVn = off;        off = align256(off + n * C * dv * es);
    w.dA_part = off;    off = align256(off + n * 4);
    w.dbias_part = off; off = align256(off + n * dk * 4);
    // Two-kernel backward of the BF16 path: bwd_wy leaves dAqk and dM, each as THREE BF16 tiles
    // cm(i, j; 64) whose sum is the FP32 value (x = p0 + p1 + p2: a 24-bit split, because the gate
    // gradient is a difference of large terms built from them), strictly lower triangle, stored
    // [dAqk p0, p1, p2, dM p0, p1, p2] -- ready-made tensor-core operands of bwd_intra; the diagonal
    // of dAqk (float [64]); the raw products dQt, dKh, d(beta K~) as [64][dk] in the element type
    // (BF16 on the BF16 path: rounding them moves no gradient by more than 3e-4 relative L2); the
    // beta gradient collected so far (float [64]) and dGamma_C * Gamma_C (float [dk]).
    w.dAM = off;  off = align256(off + n * 6 * C * C * 2);
    w.dAd = off;  off = align256(off + n * C * 4);
    w.dQt = off;  off = align256(off + n * C * dk * es);
    w.dKh = off;  off = align256(off + n * C * dk * es);
    w.dKb = off;  off = align256(off + n * C * dk * es);
    w.dbp = off;  off = align256(off + n * C * 4);
    w.gC = off;   off = align256(off + n * dk * 4);
    w.bwd_total = off;
    // fused short-convolution backward (behind everything else, so that the plain call's scratch does not
    // grow): per unit and tensor (q, k, v) the filter-gradient partial sums float [dk][4], and dpre of the
    // chunk's first / last three rows float [3][dk] for the rows whose look-ahead crosses the chunk border
    w.cv_part = off; off = align256(off + n * 3 * dk * 4 * 4);
    w.cv_head = off; off = align256(off + n * 3 * 3 * dk * 4);
    w.cv_tail = off; off = align256(off + n * 3 * 3 * dk * 4);
    w.bwd_total_conv = off;
    return w;
}

// state element index for logical (d, e) of a [dk, dv] state, honouring the v-first layout
__device__ __forceinline__ size_t state_idx(const KdaParams& p, int d, int e) {
    return (p.flags & KDA_FLAG_STATE_V_FIRST) ? (size_t)e * p.dk + d : (size_t)d * p.dv + e;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Three-way BF16 split of two floats: x = p0 + p1 + p2 up to 2^-24 relative (each p is a pair of
// BF16 values, element 0 in the low half).  The split operands let BF16 tensor-core passes
// (p0 q0 + p0 q1 + p1 q0 + p1 q1 + p0 q2 + p2 q0) reach FP32-class products.
__device__ __forceinline__ void split3_bf16(float x0, float x1, uint32_t& p0, uint32_t& p1, uint32_t& p2) {
    __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
    p0 = *reinterpret_cast<uint32_t*>(&h);
    float r0 = x0 - __uint_as_float(p0 << 16), r1 = x1 - __uint_as_float(p0 & 0xffff0000u);
    h = __floats2bfloat162_rn(r0, r1);
    p1 = *reinterpret_cast<uint32_t*>(&h);
    r0 -= __uint_as_float(p1 << 16);
    r1 -= __uint_as_float(p1 & 0xffff0000u);
    h = __floats2bfloat162_rn(r0, r1);
    p2 = *reinterpret_cast<uint32_t*>(&h);
}

// SiLU and the four-tap causal filter shared by the stand-alone convolution kernels and the
// fused load stage; one fixed FMA order so that both produce the same bits
// (branch-free approximate division, 2 ulp: an IEEE division carries a slow-path branch that keeps
// the compiler from interleaving the independent channels of a thread)
__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.f + __expf(-x)); }
__device__ __forceinline__ float conv_pre(float w0, float w1, float w2, float w3, float x0, float x1, float x2, float x3) {
    return fmaf(w3, x3, fmaf(w2, x2, fmaf(w1, x1, w0 * x0)));
}

// softplus with torch's threshold of 20 (F.softplus, k3mini/model.py:220)
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
// softplus for the BF16 path: max(x, 0) + log(1 + e^-|x|) with hardware exp / log; the
// absolute error stays below 1e-7, which is what matters for a log-decay
__device__ __forceinline__ float softplus_fast(float x) {
    const float t = __expf(-fabsf(x));
    const float l = t < 1e-3f ? t * fmaf(t, fmaf(0.33333334f, t, -0.5f), 1.f) : __logf(1.f + t);
    return fmaxf(x, 0.f) + l;
}

}  // namespace kda
