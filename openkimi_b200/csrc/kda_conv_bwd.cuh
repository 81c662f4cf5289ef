// Backward of the causal depthwise short convolution + SiLU (k3mini/model.py:76-88) for one
// 64-row chunk of one head, run INSIDE the KDA backward kernels right after the gradient of the
// convolved rows has been produced (it never goes to HBM).  Arithmetic and summation order of the
// input gradient are those of the stand-alone kernel (short_conv_bwd_kernel), so the fused path
// returns the same bits:
//   dpre[s] = dy[s] silu'(pre[s]),  pre[s] = sum_j w[j] x[s - 3 + j]      (four-tap padded filter)
//   dx[s]   = w0 dpre[s+3] + w1 dpre[s+2] + w2 dpre[s+1] + w3 dpre[s]
//   dw[j]   = sum_s dpre[s] x[s - 3 + j]
// dx of the last three rows of a chunk needs dpre of the next chunk's first three rows, which
// another CTA produces: every chunk leaves dpre of its first and last three rows in a side buffer
// and a small fix-up kernel finishes those rows (same FMA order).
#pragma once

#include "kda_common.cuh"

namespace kda {

__device__ __forceinline__ float dsilu_f(float x) {
    const float s = __fdividef(1.f, 1.f + __expf(-x));
    return s * (1.f + x * (1.f - s));
}

// Thread = (channel ch, 16-row block blk) of a 512-thread CTA.
//   sxh  [3][128] BF16: rows -3 .. -1 of the pre-convolution tensor, sx [64][128]: rows 0 .. 63 (zero where a
//        row does not exist); the two may be one [67][128] array (sx = sxh + 3 * 128)
//   sdy  [64][128] BF16: gradient of the convolved rows (zero past the end of a partial chunk)
//   w    the four padded taps of this channel
// Returns dx of the block's 16 rows in out[] (rows 61..63 are incomplete when the chunk has a
// successor), adds the block's share of dw, and hands dpre of rows 0..2 / 61..63 to head / tail
// ([3][128] FP32 each, written by block 0 / block 3).
__device__ __forceinline__ void conv_bwd_block(const __nv_bfloat16* __restrict__ sxh, const __nv_bfloat16* __restrict__ sx,
                                               const __nv_bfloat16* __restrict__ sdy,
                                               const float (&w)[4], int ch, int blk, float* __restrict__ head,
                                               float* __restrict__ tail, float (&dw)[4], float (&out)[16]) {
    const int b0 = 16 * blk;
    auto X = [&](int r) { return __bfloat162float(r < 0 ? sxh[(r + 3) * 128 + ch] : sx[r * 128 + ch]); };
    float xa = X(b0 - 3), xb = X(b0 - 2), xc = X(b0 - 1), pa = 0.f, pb = 0.f, pc = 0.f;
#pragma unroll
    for (int sI = 0; sI < 19; ++sI) {
        const int s = b0 + sI;
        const bool in = s < 64;  // rows of the next chunk: their dpre arrives through the fix-up
        const float xd = in ? X(in ? s : 0) : 0.f, gy = in ? __bfloat162float(sdy[(in ? s : 0) * 128 + ch]) : 0.f;
        const float pd = gy * dsilu_f(conv_pre(w[0], w[1], w[2], w[3], xa, xb, xc, xd));
        if (sI < 16) {
            dw[0] = fmaf(pd, xa, dw[0]);
            dw[1] = fmaf(pd, xb, dw[1]);
            dw[2] = fmaf(pd, xc, dw[2]);
            dw[3] = fmaf(pd, xd, dw[3]);
            if (blk == 0 && sI < 3) head[sI * 128 + ch] = pd;
            if (blk == 3 && sI >= 13) tail[(sI - 13) * 128 + ch] = pd;
        }
        if (sI >= 3) out[sI - 3] = fmaf(w[0], pd, fmaf(w[1], pc, fmaf(w[2], pb, w[3] * pa)));
        xa = xb; xb = xc; xc = xd;
        pa = pb; pb = pc; pc = pd;
    }
}

// The padded taps of one channel on their way to shared memory (dst: one float4): a 16-byte cp.async when the
// filter has four taps and its array is 16-byte aligned (it joins the caller's next commit group, so the
// latency of the load is not paid where the taps are used), plain loads and a store otherwise.
__device__ __forceinline__ void stage_taps(float4* dst, const float* __restrict__ wsrc, int h, int ch, int K) {
    const float* p = wsrc + (size_t)(h * 128 + ch) * K;
    if (K == 4 && (reinterpret_cast<uintptr_t>(wsrc) & 15) == 0) {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(p) : "memory");
    } else {
        float w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) w[j] = j >= 4 - K ? p[j - (4 - K)] : 0.f;
        *dst = make_float4(w[0], w[1], w[2], w[3]);
    }
}

// the padded taps of channel (head h, ch): tap j multiplies x[s - 3 + j]
__device__ __forceinline__ void conv_taps(const float* __restrict__ wsrc, int h, int ch, int K, float (&w)[4]) {
    const float* p = wsrc + (size_t)(h * 128 + ch) * K;
#pragma unroll
    for (int j = 0; j < 4; ++j) w[j] = j >= 4 - K ? p[j - (4 - K)] : 0.f;
}

}  // namespace kda
