// fwd_intra on tensor cores (BF16 operands, d = 128).  One CTA per SM walks the (chunk, head) units
// (UnitWalk) and requests the inputs of its next unit while it works on the current one.
//
//   0  the unit's gate, q, k, v tiles arrive as bulk-tensor tile copies (tensor maps; row by row for
//      partial chunks).  Gate channel-wise: activation and the within-chunk cumulative sum G (log2);
//      q, k, v, beta row-wise: L2 norm, sigmoid, beta*v operand.
//      The CONV instantiation reads the pre-convolution projections instead (three halo rows
//      before the chunk included) and applies the causal depthwise filter + SiLU of
//      k3mini/model.py:76-88,181-185 in registers before anything else sees the rows
//   1  the four diagonal 16x16 blocks of Aqk and L on the CUDA cores: where all four [16 x 32] tiles
//      of a block pass the span guard, with the FP32 midpoint factorisation (pre-scaled key rows, no
//      exponential per pair), otherwise with exact pairwise decays
//   2  decay-scaled operands: Qt, Kh records; beta*k*2^G; and for every 16-row block I >= 1
//      the factorised operands  k_j 2^(r_I - G_j) (j < 16 I)  and  x_i 2^(G_i - r_I) (i in I),
//      r_I = G at the first row of block I, so that every exponent is <= 0; off-diagonal blocks of
//      Aqk and L as tcgen05 MMAs (M = 64 keys, N = 32 = q and k rows of block I, K = 128)
//   3  T = (I + diag(beta) L)^-1: forward substitution inside the diagonal blocks, block
//      forward substitution for the rest (FP32)
//   4  Aqk and T records; 5  W^T = (beta k 2^G)^T T^T and U^T = (beta v)^T T^T as tcgen05 MMAs
//      (M = 128 channels); 6  W, U, gamC records.
#include "kda_common.cuh"
#include "kda_tc.cuh"
#include "kda_tmap.cuh"

namespace kda {

using namespace tc;

namespace fi {
constexpr int D = 128, NTHR = 512;
constexpr uint32_t SQ = 0;                   // q^  bf16 [64][128] row-major
constexpr uint32_t SK = SQ + 16384;          // k^  bf16 [64][128]
constexpr uint32_t SG = SK + 16384;          // G   f32  [64][128]
constexpr uint32_t KSC = SG + 32768;         // 3 x cm(j, d; 128) bf16; block 0 later holds T (bf16)
constexpr uint32_t XSC = KSC + 3 * 16384;    // 3 x cm(n, d; 128) bf16, 32 rows each
constexpr uint32_t KB = XSC + 3 * 8192;      // beta k 2^G  cm(j, d; 128)
constexpr uint32_t BV = KB + 16384;          // beta v      cm(j, e; 128)
constexpr int LDR = 68;                      // row stride of A, L, T in floats
constexpr uint32_t SA = BV + 16384;          // f32 [64][LDR]
constexpr uint32_t SL = SA + 64 * LDR * 4;
constexpr uint32_t ST = SL + 64 * LDR * 4;
constexpr uint32_t SBETA = ST + 64 * LDR * 4;        // f32 [3][64]: 1/|q|, 1/|k|, beta (the aux record)
constexpr uint32_t STOT = SBETA + 768;       // f32 [4][128] running gate totals of the four 16-row groups
constexpr uint32_t SMIDF = STOT + 2048;      // f32 [4][128] midpoint of every (block, channel) of the cumulative gate
constexpr uint32_t SPASS = SMIDF + 2048;     // int [4][4]: guard decision of every [16 rows x 32 channels] tile
constexpr uint32_t TOTAL = SPASS + 64;
constexpr uint32_t KN = KSC;                 // f32 [64][128] (chunk-swizzled rows): k_j 2^(m - G_j), live only during the diagonal phase
constexpr uint32_t T_D = 0, T_W = 96, T_U = 160, TMEM_COLS = 256;
}  // namespace fi
using fi::LDR;

// One block column J of T = (I + diag(beta) L)^-1 (see stage 3 of the kernel).  sL holds L
// (strictly lower, row stride LDR: rows start on 16-byte boundaries and are read four floats at a time), sT
// receives T; sT must be zero above the diagonal blocks.
// Eight warps work (the column solve is a dependent chain: more lanes only add redundancy):
// warp (J, cw) owns columns 8 cw + lane % 8 of block column J, and its four lane groups (lane / 8)
// split the 16 rows of every block below the diagonal, four rows each.
// J is uniform over the warp; the loops run over all blocks with warp-uniform skips so that the
// register arrays keep compile-time indices in a single copy of the code.
__device__ __forceinline__ void solve_block_column(const float* sL, float* sT, const float* sbeta, int J, int cw, int lane,
                                                   bool active) {
    if (!active) {
        __syncthreads();  // (matches the barrier below)
        return;
    }
    const int col = 8 * cw + (lane & 7), rq = lane >> 3, gc = 16 * J + col;
    float t[4][16];
    // diagonal block: forward substitution down the column (every lane group does all 16 rows)
#pragma unroll
    for (int r = 0; r < 16; ++r) {
        const float* lrow = sL + (16 * J + r) * LDR + 16 * J;
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int j = 0; j < r; j += 4) {
            const float4 l = *reinterpret_cast<const float4*>(lrow + j);
            s0 = fmaf(l.x, t[0][j], s0);
            if (j + 1 < r) s1 = fmaf(l.y, t[0][j + 1], s1);
            if (j + 2 < r) s0 = fmaf(l.z, t[0][j + 2], s0);
            if (j + 3 < r) s1 = fmaf(l.w, t[0][j + 3], s1);
        }
        t[0][r] = (r == col ? 1.f : 0.f) - sbeta[16 * J + r] * (s0 + s1);
        if (r < col) t[0][r] = 0.f;
    }
    if (rq == 0) {
#pragma unroll
        for (int r = 0; r < 16; ++r) sT[(16 * J + r) * LDR + gc] = t[0][r];
    }
    __syncthreads();  // every diagonal block of T is in shared memory
    // t[n] is the column restricted to block J + n.  Lane group rq owns rows rq, rq + 4, rq + 8, rq + 12 of a
    // block: the four rows one load instruction touches are adjacent, LDR floats apart, in four different banks.
#pragma unroll
    for (int n = 1; n < 4; ++n) {
        const int I = J + n;
        if (I > 3) break;
        // y = sum_K (beta L)_IK t_K for my four rows, then all 16 entries from the lane groups
        float y4[4], y[16];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int r = 16 * I + rq + 4 * q;
            float s = 0.f;
#pragma unroll
            for (int kn = 0; kn < n; ++kn)
#pragma unroll
                for (int m = 0; m < 16; m += 4) {
                    const float4 l = *reinterpret_cast<const float4*>(sL + r * LDR + 16 * (J + kn) + m);
                    s = fmaf(l.x, t[kn][m], s);
                    s = fmaf(l.y, t[kn][m + 1], s);
                    s = fmaf(l.z, t[kn][m + 2], s);
                    s = fmaf(l.w, t[kn][m + 3], s);
                }
            y4[q] = sbeta[r] * s;
        }
#pragma unroll
        for (int g4 = 0; g4 < 4; ++g4)
#pragma unroll
            for (int q = 0; q < 4; ++q) y[g4 + 4 * q] = __shfl_sync(0xffffffffu, y4[q], (lane & 7) + 8 * g4);
        // t_I = -T_II y for my four rows, shared the same way
        float n4[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int r = 16 * I + rq + 4 * q;
            float s = 0.f;
#pragma unroll
            for (int m = 0; m < 16; m += 4) {
                const float4 l = *reinterpret_cast<const float4*>(sT + r * LDR + 16 * I + m);
                s = fmaf(l.x, y[m], s);
                s = fmaf(l.y, y[m + 1], s);
                s = fmaf(l.z, y[m + 2], s);
                s = fmaf(l.w, y[m + 3], s);
            }
            n4[q] = -s;
            sT[r * LDR + gc] = -s;
        }
#pragma unroll
        for (int g4 = 0; g4 < 4; ++g4)
#pragma unroll
            for (int q = 0; q < 4; ++q) t[n][g4 + 4 * q] = __shfl_sync(0xffffffffu, n4[q], (lane & 7) + 8 * g4);
    }
}

// Off-diagonal blocks from tensor memory into sA (Aqk, scaled) and sL: accumulator column
// 32 (I - 1) + n holds, for key row j (lane), the product with q row n (n < 16) or k row n - 16 of
// block I.  One call covers the 32 columns of block I = CBASE / 32 + 1; CBASE is a template argument
// so that every block / row index is a constant.
template <int CBASE>
__device__ __forceinline__ void read_offdiag(uint32_t tmem_d, int qd, int lane, float* sA, float* sL, float scale) {
    const int j = 16 * qd + (lane & 15);
#pragma unroll
    for (int cc = 0; cc < 32; cc += 16) {
        uint32_t r[16];
        tmem_ld16(tmem_d + ((uint32_t)(32 * qd) << 16) + CBASE + cc, r);
        tmem_wait_ld();
        if (lane < 16) {
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const int col = CBASE + cc + u, I = (col >> 5) + 1, nn = col & 31;
                if (j < 16 * I) {
                    const float val = __uint_as_float(r[u]);
                    if (nn < 16) sA[(16 * I + nn) * LDR + j] = val * scale;
                    else sL[(16 * I + nn - 16) * LDR + j] = val;
                }
            }
        }
    }
}

template <bool CONV>
__global__ void __launch_bounds__(fi::NTHR, 1) kda_fwd_intra_tc(const KdaParams p, const __grid_constant__ RowMaps maps) {
    using namespace fi;
    extern __shared__ __align__(128) unsigned char dyn[];
    __shared__ uint64_t bar, bar2, rowbar, vbar;
    __shared__ uint32_t tmem_s;
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(dyn + SQ);
    __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(dyn + SK);
    float* sG = reinterpret_cast<float*>(dyn + SG);
    __nv_bfloat16* sKB = reinterpret_cast<__nv_bfloat16*>(dyn + KB);
    __nv_bfloat16* sBV = reinterpret_cast<__nv_bfloat16*>(dyn + BV);
    float* sA = reinterpret_cast<float*>(dyn + SA);
    float* sL = reinterpret_cast<float*>(dyn + SL);
    float* sT = reinterpret_cast<float*>(dyn + ST);
    float* saux = reinterpret_cast<float*>(dyn + SBETA);
    float* sbeta = saux + 2 * C;
    float* stot = reinterpret_cast<float*>(dyn + STOT);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const WsLayout L = ws_layout(p.NT, p.H, p.dk, p.dv, p.dtype);
    char* ws = (char*)p.workspace;
    const __nv_bfloat16* q = (const __nv_bfloat16*)p.q;
    const __nv_bfloat16* k = (const __nv_bfloat16*)p.k;
    const __nv_bfloat16* v = (const __nv_bfloat16*)p.v;
    const __nv_bfloat16* g = (const __nv_bfloat16*)p.g;
    const __nv_bfloat16* beta = (const __nv_bfloat16*)p.beta;
    const bool l2 = p.flags & KDA_FLAG_QK_L2NORM, gate = p.flags & KDA_FLAG_GATE, sig = p.flags & KDA_FLAG_BETA_SIGMOID;
    const bool save = !(p.flags & KDA_FLAG_NO_SAVE);  // forward-only calls keep nothing for a backward

    KDA_PHASE_BEGIN();
    if (warp == 0) {
        tmem_alloc(&tmem_s, TMEM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        mbar_init(&bar, 3);   // three issuing threads commit the off-diagonal products
        mbar_init(&bar2, 2);  // two issuing threads commit the W and U products
        mbar_init(&rowbar, 1);
        mbar_init(&vbar, 1);
        mbar_fence_init();
    }
    __syncthreads();

    // ---- 0: a unit's inputs arrive as bulk-tensor tile copies (row by row for partial chunks), completing on two
    //      mbarriers.  The CTA walks the units blockIdx.x, blockIdx.x + gridDim.x, ... and requests the inputs of
    //      its NEXT unit while it still works on the current one, into space that is dead by then: the gate, q and
    //      k rows (q, k: ROWS each, three halo rows first when the convolution is fused; the halo rows of v too)
    //      go to the operand space behind the first key tile once the off-diagonal products have been read, some
    //      8 us ahead of their use; the v rows, which are needed last, go to the L tile once T is solved; the few
    //      scalars travel in registers.  Rows past the end of the sequence are zero-filled by the thread that
    //      would have requested them.
    constexpr int HALO = CONV ? 3 : 0, ROWS = C + HALO;
    constexpr uint32_t RGATE = KSC + 16384, RQ = RGATE + C * D * 2, RK = RQ + ROWS * D * 2, RVH = RK + ROWS * D * 2, TAPS = ST;
    static_assert(RVH + HALO * D * 2 <= KB, "staging overruns the operand space");
    __nv_bfloat16* sRG = reinterpret_cast<__nv_bfloat16*>(dyn + RGATE);
    __nv_bfloat16* sRq = reinterpret_cast<__nv_bfloat16*>(dyn + RQ);    // rows -HALO .. 63 of q
    __nv_bfloat16* sRk = reinterpret_cast<__nv_bfloat16*>(dyn + RK);
    __nv_bfloat16* sRvh = reinterpret_cast<__nv_bfloat16*>(dyn + RVH);  // rows -3 .. -1 of v (fused convolution only)
    __nv_bfloat16* sRv = reinterpret_cast<__nv_bfloat16*>(dyn + SL);    // rows 0 .. 63 of v
    const int quarter = tid >> 7, dch = tid & 127;  // gate: thread = (16-row group, channel)
    const int hw = tid >> 4, c8 = (tid & 15) * 8;   // rows: half warp = row, lane = 8 channels
    auto zero_row = [&](__nv_bfloat16* dst) {
#pragma unroll
        for (int j = 0; j < 16; ++j) reinterpret_cast<uint4*>(dst)[j] = make_uint4(0, 0, 0, 0);
    };
    const bool tiles = maps.ok != 0;  // whole [64 x 128] tiles with one bulk-tensor copy each (full chunks only)
    auto row_src = [&](const __nv_bfloat16* base, const ChunkInfo& ci, int h, int i) { return base + ((size_t)(ci.tok0 + i) * p.H + h) * D; };
    auto request_rows = [&](const ChunkInfo& ci, int h) {  // gate, q, k (and every halo row)
        // (issued from the last warp, which has no share in the column solve that follows the in-loop request: the
        //  issuing warp is held up while the copy unit works through its requests)
        if (tid == NTHR - 32) mbar_expect_tx(&rowbar, (uint32_t)(3 * ci.len + ((CONV && ci.lc > 0) ? 9 : 0)) * 256u);
        if (tiles && ci.len == C) {
            if (tid == NTHR - 32) tma_load_tile(sRG, &maps.m[3], h * D, (int)ci.tok0, &rowbar);
            if (tid == NTHR - 31) tma_load_tile(sRq + HALO * D, &maps.m[0], h * D, (int)ci.tok0, &rowbar);
            if (tid == NTHR - 30) tma_load_tile(sRk + HALO * D, &maps.m[1], h * D, (int)ci.tok0, &rowbar);
        } else if (tid < 3 * C) {
            const int t3 = tid >> 6, i = tid & 63;
            __nv_bfloat16* dst = (t3 == 0 ? sRG : t3 == 1 ? sRq + HALO * D : sRk + HALO * D) + i * D;
            if (i < ci.len) tma_load_1d(dst, row_src(t3 == 0 ? g : t3 == 1 ? q : k, ci, h, i), 256, &rowbar);
            else zero_row(dst);
        }
        if (CONV && lane == 0 && warp >= 6 && warp < 15) {  // three rows before the chunk (one copy each from nine warps):
            const int t3 = (warp - 6) / 3, r = (warp - 6) % 3;  // they exist unless the chunk starts its sequence
            __nv_bfloat16* dst = (t3 == 0 ? sRq : t3 == 1 ? sRk : sRvh) + r * D;
            if (ci.lc > 0) tma_load_1d(dst, row_src(t3 == 0 ? q : t3 == 1 ? k : v, ci, h, r - 3), 256, &rowbar);
            else zero_row(dst);
        }
    };
    auto request_v = [&](const ChunkInfo& ci, int h) {
        if (tid == 256) mbar_expect_tx(&vbar, (uint32_t)ci.len * 256u);
        if (tiles && ci.len == C) {
            if (tid == 256) tma_load_tile(sRv, &maps.m[2], h * D, (int)ci.tok0, &vbar);
        } else if (tid >= 256 && tid < 256 + C) {
            const int i = tid - 256;
            if (i < ci.len) tma_load_1d(sRv + i * D, row_src(v, ci, h, i), 256, &vbar);
            else zero_row(sRv + i * D);
        }
    };
    struct Scalars {  // (beta stays in its storage type: a conversion here would wait for the load)
        float a_log, bias;
        __nv_bfloat16 rb[2];
        float4 tap;
    };
    auto request_scalars = [&](const ChunkInfo& ci, int h, Scalars& sc) {
        sc.a_log = gate ? p.A_log[h] : 0.f;
        sc.bias = (gate && p.dt_bias) ? p.dt_bias[h * D + dch] : 0.f;
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            const int i = CONV ? 2 * hw + m : hw + 32 * m;
            sc.rb[m] = beta[(size_t)(ci.tok0 + (i < ci.len ? i : 0)) * p.H + h];  // (used by lane 0 of the half warp, rows < len)
        }
        sc.tap = make_float4(0.f, 0.f, 0.f, 0.f);
        if constexpr (CONV) {  // filter taps of this head, padded to four: entry e = tensor * 128 + channel
            const int K = p.conv_ksize;
            if (tid < 3 * D) {
                float t4[4] = {0.f, 0.f, 0.f, 0.f};
                const float* w = (tid < D ? p.conv_q : tid < 2 * D ? p.conv_k : p.conv_v) + (size_t)(h * D + (tid & (D - 1))) * K;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (j >= 4 - K) t4[j] = w[j - (4 - K)];
                sc.tap = make_float4(t4[0], t4[1], t4[2], t4[3]);
            }
        }
    };
    // taps: entry (tensor, channel) at [tensor][channel % 8][channel / 8], so that the sixteen lanes of a
    // half warp read consecutive 16-byte words; they wait in the (dead) T tile for the next unit
    auto park_taps = [&](const Scalars& sc) {
        if constexpr (CONV) {
            float4* sW = reinterpret_cast<float4*>(dyn + TAPS);
            if (tid < 3 * D) sW[(tid & ~(D - 1)) + (tid & 7) * 16 + ((tid & (D - 1)) >> 3)] = sc.tap;
        }
    };
    const int n_units = p.NT * p.H;
    Scalars nx;
    // unit u = (chunk u / H, head (u + chunk) % H): the head is skewed by the chunk index so that the units a
    // CTA visits (stride gridDim.x) cycle through ALL heads even when the stride shares a factor with H
    // (heads differ in cost: the ones whose tiles fail the span guard take the exact path)
    UnitWalk uw;
    uw.init(blockIdx.x, gridDim.x, p.H);
    ChunkInfo ci = chunk_info(p, blockIdx.x / p.H);
    request_rows(ci, uw.head());
    request_v(ci, uw.head());
    request_scalars(ci, uw.head(), nx);
    park_taps(nx);
    __syncthreads();
    uint32_t it = 0;
    bool ok = true, more = false;
    for (; uw.unit < n_units; uw.next(), ++it) {
    const int c = uw.c, h = uw.head();
    const size_t rec = (size_t)c * p.H + h;
    __nv_bfloat16* gW = (__nv_bfloat16*)(ws + L.W) + rec * C * D;
    __nv_bfloat16* gU = (__nv_bfloat16*)(ws + L.U) + rec * C * D;
    __nv_bfloat16* gA = (__nv_bfloat16*)(ws + L.Aqk) + rec * C * C;
    __nv_bfloat16* gQt = (__nv_bfloat16*)(ws + L.Qt) + rec * C * D;
    __nv_bfloat16* gKh = (__nv_bfloat16*)(ws + L.Kh) + rec * C * D;
    __nv_bfloat16* gT = (__nv_bfloat16*)(ws + L.Tm) + rec * C * C;
    float* gGam = (float*)(ws + L.gamC) + rec * D;
    UnitWalk un = uw;  // the next unit of this CTA
    un.next();
    more = un.unit < n_units;
    ChunkInfo ci_nx = ci;
    const float a_log_h = nx.a_log, bias = nx.bias;
    float rb[2];
#pragma unroll
    for (int m = 0; m < 2; ++m)
        rb[m] = ((tid & 15) == 0 && (CONV ? 2 * hw + m : hw + 32 * m) < ci.len) ? __bfloat162float(nx.rb[m]) : 0.f;
    ok = mbar_wait(&rowbar, it & 1, p, 8);
    KDA_PHASE(13);
    // ---- 0a: gate, channel-wise: thread (quarter, d) owns rows 16*quarter .. 16*quarter+15 of channel d
    {
        const float negA = gate ? -expf(a_log_h) : 0.f;
        float run = 0.f;
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            const int i = 16 * quarter + r;
            const float x = __bfloat162float(sRG[i * D + dch]);
            float gl = 0.f;
            if (i < ci.len) gl = gate ? negA * softplus_fast(x + bias) : x;
            run = fmaf(gl, LOG2E, run);  // explicit: both instantiations must round alike
            sG[swz_f32(i, dch)] = run;
        }
        stot[quarter * D + dch] = run;
    }
    KDA_PHASE(0);
    ok = mbar_wait(&vbar, it & 1, p, 8) && ok;
    KDA_PHASE(14);
    // Rows of a half warp: hw and hw + 32 without the convolution; 2 hw and 2 hw + 1 with it, so that
    // the five input rows 2 hw - 3 .. 2 hw + 1 serve the two outputs of one thread.
    uint4 rq4[2], rk4[2], rv4[2];
    if constexpr (CONV) {
        // ---- 0c: y[i] = silu(sum_j tap[j] x[i - 3 + j]) for the thread's two rows, rounded to
        //      BF16 like the stand-alone convolution; the rest of the stage sees only y
        const float4* sW = reinterpret_cast<const float4*>(dyn + TAPS);
        // row x of a tensor's window (x = 0 .. 66 stands for token x - 3 of the chunk); the halo rows of v sit apart
        auto conv_rows = [&](uint4(&out)[2], int tensor) {
            float4 w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) w[j] = sW[tensor * D + j * 16 + (c8 >> 3)];
            float win[5][8];
#pragma unroll
            for (int r = 0; r < 5; ++r) {
                const int x = 2 * hw + r;
                const __nv_bfloat16* row = tensor == 0 ? sRq + x * D : tensor == 1 ? sRk + x * D : (x < 3 ? sRvh + x * D : sRv + (x - 3) * D);
                bf16x8_to_f32(*reinterpret_cast<const uint4*>(row + c8), win[r]);
            }
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                float y[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    y[j] = silu_f(conv_pre(w[j].x, w[j].y, w[j].z, w[j].w, win[m][j], win[m + 1][j], win[m + 2][j], win[m + 3][j]));
                out[m] = 2 * hw + m < ci.len ? f32_to_bf16x8(y) : make_uint4(0, 0, 0, 0);
            }
        };
        conv_rows(rq4, 0);
        conv_rows(rk4, 1);
        conv_rows(rv4, 2);
        if (save) {
            __nv_bfloat16* gVc = (__nv_bfloat16*)(ws + L.Vc) + rec * C * D;
#pragma unroll
            for (int m = 0; m < 2; ++m) *reinterpret_cast<uint4*>(gVc + (2 * hw + m) * D + c8) = rv4[m];
        }
    } else {
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            const int off = (hw + 32 * m) * D + c8;
            rq4[m] = *reinterpret_cast<const uint4*>(sRq + off);
            rk4[m] = *reinterpret_cast<const uint4*>(sRk + off);
            rv4[m] = *reinterpret_cast<const uint4*>(sRv + off);
        }
    }
    // ---- 0b: q, k, v, beta row-wise: a half warp owns two rows, lane c8 the channels 8 c8 ..
    {
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            const int i = CONV ? 2 * hw + m : hw + 32 * m;
            const bool valid = i < ci.len;
            float qf[8], kf[8], vf[8];
            bf16x8_to_f32(rq4[m], qf);
            bf16x8_to_f32(rk4[m], kf);
            bf16x8_to_f32(rv4[m], vf);
            float b = rb[m];
            if ((tid & 15) == 0 && valid && sig) b = sigmoid_f(b);
            b = __shfl_sync(0xffffffffu, b, lane & 16);
            float rq = 1.f, rk = 1.f;
            if (l2) {
                float ssq = 0.f, ssk = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    ssq = fmaf(qf[j], qf[j], ssq);  // explicit: both instantiations must round alike
                    ssk = fmaf(kf[j], kf[j], ssk);
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
#pragma unroll
            for (int j = 0; j < 8; ++j) vf[j] *= b;
            *reinterpret_cast<uint4*>(sQ + swz_bf16(i, c8)) = f32_to_bf16x8(qf);
            *reinterpret_cast<uint4*>(sK + swz_bf16(i, c8)) = f32_to_bf16x8(kf);
            *reinterpret_cast<uint4*>(sBV + cm_idx(i, c8, D)) = f32_to_bf16x8(vf);
            if ((tid & 15) == 0) {
                sbeta[i] = b;
                saux[i] = rq;
                saux[C + i] = rk;
            }
        }
    }
    KDA_PHASE(1);
    tc_fence_before();
    __syncthreads();  // the raw gate, q, k rows (operand space) and the raw v rows (L tile) are consumed
    tc_fence_after();
    // A and T must read zero above the diagonal: the stages below write A for j <= i only and T from the diagonal
    // block down, and the records carry whole 64 x 64 tiles.  Row i is cleared from its diagonal block on, four
    // floats at a time.  (L needs no clearing: the solve reads its diagonal blocks for j < i only, which the
    // diagonal walks write, and the blocks below them whole, which the accumulator read-back writes.)
#pragma unroll
    for (int idx = tid; idx < C * 16; idx += NTHR) {
        const int i = idx >> 4, q4 = idx & 15;
        if (q4 >= 4 * (i >> 4)) {
            *reinterpret_cast<float4*>(sA + i * LDR + 4 * q4) = make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4*>(sT + i * LDR + 4 * q4) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    const uint32_t tmem0 = tmem_s;
    // ---- the later 16-row groups of the cumulative sum pick up the totals of the earlier ones; every thread
    //      keeps the 16 G values of its (block, channel) and evaluates the span guard of its tile (a warp is one
    //      [16 rows x 32 channels] tile, k3mini/backends.py:17-19): where it passes, the diagonal block may use the
    //      midpoint factorisation 2^(G_i - m) 2^(m - G_j) in FP32 (every factor within 2^(+-116)), for which the
    //      thread leaves k_j 2^(m - G_j) of its rows in the (still free) operand space
    float* smidf = reinterpret_cast<float*>(dyn + SMIDF);
    int* spass = reinterpret_cast<int*>(dyn + SPASS);
    float* sKN = reinterpret_cast<float*>(dyn + KN);
    {
        float t = 0.f;
        if (quarter > 0) t = stot[dch];
        if (quarter > 1) t += stot[D + dch];
        if (quarter > 2) t += stot[2 * D + dch];
        float Gr[16], mid;
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            Gr[r] = sG[swz_f32(16 * quarter + r, dch)] + t;
            if (quarter > 0) sG[swz_f32(16 * quarter + r, dch)] = Gr[r];
        }
        const bool tpass = guard_tile(Gr, p.guard_span, mid);
        smidf[quarter * D + dch] = mid;
        if (lane == 0) spass[quarter * 4 + (warp & 3)] = tpass ? 1 : 0;
        if (tpass) {
#pragma unroll
            for (int r = 0; r < 16; ++r)
                sKN[swz_f32(16 * quarter + r, dch)] =
                    __bfloat162float(sK[swz_bf16(16 * quarter + r, dch)]) * ex2_approx(mid - Gr[r]);
        }
    }
    fence_async_smem();
    __syncthreads();
    KDA_PHASE(2);
    // ---- diagonal blocks on the CUDA cores: midpoint-factorised where all four tiles of the block passed the
    //      guard, exact (one exp2 per pair and channel) otherwise.  Thread = (block b, slot, channel slice cs): the eight lanes of a slot split the
    // 128 channels (16 each: 32 u + 4 cs .. +3), keep their row i in registers, walk key rows j four at a
    // time, and the eight slices of a pair meet in three shuffles.  Four warps share a block; the 136
    // pairs (j <= i) of the block are dealt out so that no warp walks more than twelve key rows:
    //   warps 0, 1 (slot s = 0..7):  row 8 + s            against keys 0..7   (all valid)
    //   warps 2, 3 (slot s = 0..7):  row 15 - s           against keys 8..15, then row s against keys 0..7
    // Eight lanes read 128 contiguous bytes of a row: no bank conflicts.
    {
        // (role w4 rotates with the block: the four warps of one scheduler, warp % 4 alike, take the four roles,
        //  two short walks of 8 key rows and two long ones of 12, instead of four of a kind)
        const int cs = lane & 7, b = warp >> 2, w4 = (warp + b) & 3, slot = 4 * (w4 & 1) + (lane >> 3);
        // element offsets of this lane's channels 32 u + 4 cs .. + 3 inside the swizzled row r (swz_f32 / swz_bf16
        // with the row-dependent part computed once per row): FP32 chunk 8 u + cs, BF16 chunk 4 u + cs / 2
        auto goff = [&](int r, int u) { return 32 * u + 4 * (cs ^ (r & 7)); };
        auto boff = [&](int r, int u) { return 8 * (((4 * u + (cs >> 1)) ^ (r & 7))) + 4 * (cs & 1); };
        auto row_against = [&](int i, int jbeg, int jend) {  // jbeg, jend multiples of four, uniform over the warp
            const int ri = 16 * b + i;
            float gi[16], qi[16], ki[16];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float4 g4 = *reinterpret_cast<const float4*>(sG + ri * D + goff(ri, u));
                gi[4 * u] = g4.x; gi[4 * u + 1] = g4.y; gi[4 * u + 2] = g4.z; gi[4 * u + 3] = g4.w;
                const uint2 q2 = *reinterpret_cast<const uint2*>(sQ + ri * D + boff(ri, u));
                const uint2 k2 = *reinterpret_cast<const uint2*>(sK + ri * D + boff(ri, u));
                const float2 qa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q2.x));
                const float2 qb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q2.y));
                const float2 ka = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&k2.x));
                const float2 kb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&k2.y));
                qi[4 * u] = qa.x; qi[4 * u + 1] = qa.y; qi[4 * u + 2] = qb.x; qi[4 * u + 3] = qb.y;
                ki[4 * u] = ka.x; ki[4 * u + 1] = ka.y; ki[4 * u + 2] = kb.x; ki[4 * u + 3] = kb.y;
            }
            // four key rows at a time: their eight sums (a and l of each pair) are reduced over the eight
            // slices by a transposing exchange, 7 shuffles instead of 24, after which lane cs owns sum
            // number cs and stores it
#pragma unroll 1
            for (int j0 = jbeg; j0 < jend; j0 += 4) {
                float v[8];
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const int rj = 16 * b + j0 + jj;
                    float2 av = make_float2(0.f, 0.f), lv = av;  // packed two-wide FMAs: even / odd channels
                    const int gj0 = goff(rj, 0), kj0 = boff(rj, 0), kj1 = boff(rj, 1);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const float4 g4 = *reinterpret_cast<const float4*>(sG + rj * D + gj0 + 32 * u);
                        const uint2 k2 = *reinterpret_cast<const uint2*>(sK + rj * D + ((u & 1) ? kj1 : kj0) + 64 * (u >> 1));
                        const float2 ka = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&k2.x));
                        const float2 kb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&k2.y));
                        // (rows j > i are computed too but never stored; whatever they overflow to is dropped)
                        const float2 k01 = __fmul2_rn(ka, make_float2(ex2_approx(gi[4 * u] - g4.x), ex2_approx(gi[4 * u + 1] - g4.y)));
                        const float2 k23 = __fmul2_rn(kb, make_float2(ex2_approx(gi[4 * u + 2] - g4.z), ex2_approx(gi[4 * u + 3] - g4.w)));
                        av = __ffma2_rn(make_float2(qi[4 * u], qi[4 * u + 1]), k01, __ffma2_rn(make_float2(qi[4 * u + 2], qi[4 * u + 3]), k23, av));
                        lv = __ffma2_rn(make_float2(ki[4 * u], ki[4 * u + 1]), k01, __ffma2_rn(make_float2(ki[4 * u + 2], ki[4 * u + 3]), k23, lv));
                    }
                    v[2 * jj] = av.x + av.y;
                    v[2 * jj + 1] = lv.x + lv.y;
                }
                const bool b2 = cs & 4, b1 = cs & 2, b0 = cs & 1;
                float w4s[4], w2s[2];
#pragma unroll
                for (int t = 0; t < 4; ++t) w4s[t] = (b2 ? v[t + 4] : v[t]) + __shfl_xor_sync(0xffffffffu, b2 ? v[t] : v[t + 4], 4);
#pragma unroll
                for (int t = 0; t < 2; ++t) w2s[t] = (b1 ? w4s[t + 2] : w4s[t]) + __shfl_xor_sync(0xffffffffu, b1 ? w4s[t] : w4s[t + 2], 2);
                const float sum = (b0 ? w2s[1] : w2s[0]) + __shfl_xor_sync(0xffffffffu, b0 ? w2s[0] : w2s[1], 1);
                const int j = j0 + (cs >> 1);
                if (j <= i) {
                    if (!b0) sA[ri * LDR + 16 * b + j] = sum * p.scale;
                    else if (j < i) sL[ri * LDR + 16 * b + j] = sum;
                }
            }
        };
        // guarded variant of the same walk: no exponential in the pair loop, the key rows come pre-scaled
        auto row_against_mid = [&](int i, int jbeg, int jend) {
            const int ri = 16 * b + i;
            float qP[16], kP[16];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int d0 = 32 * u + 4 * cs;
                const float4 g4 = *reinterpret_cast<const float4*>(sG + ri * D + goff(ri, u));
                const float4 m4 = *reinterpret_cast<const float4*>(smidf + b * D + d0);
                const uint2 q2 = *reinterpret_cast<const uint2*>(sQ + ri * D + boff(ri, u));
                const uint2 k2 = *reinterpret_cast<const uint2*>(sK + ri * D + boff(ri, u));
                const float2 qa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q2.x));
                const float2 qb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q2.y));
                const float2 ka = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&k2.x));
                const float2 kb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&k2.y));
                const float p0 = ex2_approx(g4.x - m4.x), p1 = ex2_approx(g4.y - m4.y), p2 = ex2_approx(g4.z - m4.z),
                            p3 = ex2_approx(g4.w - m4.w);
                qP[4 * u] = qa.x * p0; qP[4 * u + 1] = qa.y * p1; qP[4 * u + 2] = qb.x * p2; qP[4 * u + 3] = qb.y * p3;
                kP[4 * u] = ka.x * p0; kP[4 * u + 1] = ka.y * p1; kP[4 * u + 2] = kb.x * p2; kP[4 * u + 3] = kb.y * p3;
            }
#pragma unroll 2
            for (int j0 = jbeg; j0 < jend; j0 += 4) {
                float v[8];
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const int rj = 16 * b + j0 + jj;
                    const int gj0 = goff(rj, 0);
                    float2 av = make_float2(0.f, 0.f), lv = av;
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const float4 kn = *reinterpret_cast<const float4*>(sKN + rj * D + gj0 + 32 * u);
                        const float2 k01 = make_float2(kn.x, kn.y), k23 = make_float2(kn.z, kn.w);
                        av = __ffma2_rn(make_float2(qP[4 * u], qP[4 * u + 1]), k01, __ffma2_rn(make_float2(qP[4 * u + 2], qP[4 * u + 3]), k23, av));
                        lv = __ffma2_rn(make_float2(kP[4 * u], kP[4 * u + 1]), k01, __ffma2_rn(make_float2(kP[4 * u + 2], kP[4 * u + 3]), k23, lv));
                    }
                    v[2 * jj] = av.x + av.y;
                    v[2 * jj + 1] = lv.x + lv.y;
                }
                const bool b2 = cs & 4, b1 = cs & 2, b0 = cs & 1;
                float w4s[4], w2s[2];
#pragma unroll
                for (int t = 0; t < 4; ++t) w4s[t] = (b2 ? v[t + 4] : v[t]) + __shfl_xor_sync(0xffffffffu, b2 ? v[t] : v[t + 4], 4);
#pragma unroll
                for (int t = 0; t < 2; ++t) w2s[t] = (b1 ? w4s[t + 2] : w4s[t]) + __shfl_xor_sync(0xffffffffu, b1 ? w4s[t] : w4s[t + 2], 2);
                const float sum = (b0 ? w2s[1] : w2s[0]) + __shfl_xor_sync(0xffffffffu, b0 ? w2s[0] : w2s[1], 1);
                const int j = j0 + (cs >> 1);
                if (j <= i) {
                    if (!b0) sA[ri * LDR + 16 * b + j] = sum * p.scale;
                    else if (j < i) sL[ri * LDR + 16 * b + j] = sum;
                }
            }
        };
        const bool fast = (spass[4 * b] & spass[4 * b + 1] & spass[4 * b + 2] & spass[4 * b + 3]) != 0;  // uniform over the block
        // warps 0, 1 of a block: row 8 + slot against keys 0..7; warp 2: rows 15 - slot (15..12) against keys 8..15, then
        // rows slot (0..3) against keys 0..3; warp 3: rows 15 - slot (11..8) against keys 8..11, then rows slot (4..7)
        // against keys 0..7.
        if constexpr (CONV) {
            // One rolled loop over the (at most two) segments keeps a single copy of each walk in the code: with the
            // convolution the kernel is ~190 KB of instructions otherwise, every unit fetches them anew, and above
            // that size the fetches started to cost (1.89 -> 1.71 ms on the sublayer workload).
            const int nseg = w4 < 2 ? 1 : 2;
#pragma unroll 1
            for (int sgi = 0; sgi < nseg; ++sgi) {
                int i, jb, je;
                if (w4 < 2) { i = 8 + slot; jb = 0; je = 8; }
                else if (sgi == 0) { i = 15 - slot; jb = 8; je = w4 == 2 ? 16 : 12; }
                else { i = slot; jb = 0; je = w4 == 2 ? 4 : 8; }
                if (fast) row_against_mid(i, jb, je);
                else row_against(i, jb, je);
            }
        } else if (fast) {  // (without the convolution the straight-line form fits and is 0.3 us per unit faster)
            if (w4 < 2) {
                row_against_mid(8 + slot, 0, 8);
            } else {
                row_against_mid(15 - slot, 8, w4 == 2 ? 16 : 12);
                row_against_mid(slot, 0, w4 == 2 ? 4 : 8);
            }
        } else if (w4 < 2) {
            row_against(8 + slot, 0, 8);
        } else {
            row_against(15 - slot, 8, w4 == 2 ? 16 : 12);
            row_against(slot, 0, w4 == 2 ? 4 : 8);
        }
    }
    __syncthreads();  // the pre-scaled key rows are dead: their space becomes operand space
    KDA_PHASE(10);
    // ---- 1: decay-scaled operands.  A warp takes 8 rows x 4 channel groups at a time, so that its
    //      16-byte stores into the core-matrix tiles cover four whole 128-byte core matrices
    //      (no bank conflicts; the row-major loads of q^, k^, G take the conflicts instead, and
    //      there are five times fewer of them)
    {
#pragma unroll 1
        for (int it = 0; it < 2; ++it) {
            const int combo = 2 * warp + it;
            const int i = 8 * (combo >> 2) + (lane & 7), c8 = 8 * (4 * (combo & 3) + (lane >> 3)), m = i >> 4;
            float G8[8], qf[8], kf[8], o8[8], gl[8];
            {
                const float4 a = *reinterpret_cast<const float4*>(sG + swz_f32(C - 1, c8));
                const float4 b = *reinterpret_cast<const float4*>(sG + swz_f32(C - 1, c8 + 4));
                gl[0] = a.x; gl[1] = a.y; gl[2] = a.z; gl[3] = a.w; gl[4] = b.x; gl[5] = b.y; gl[6] = b.z; gl[7] = b.w;
            }
            {
                const float4 a = *reinterpret_cast<const float4*>(sG + swz_f32(i, c8));
                const float4 b = *reinterpret_cast<const float4*>(sG + swz_f32(i, c8 + 4));
                G8[0] = a.x; G8[1] = a.y; G8[2] = a.z; G8[3] = a.w; G8[4] = b.x; G8[5] = b.y; G8[6] = b.z; G8[7] = b.w;
            }
            bf16x8_to_f32(*reinterpret_cast<const uint4*>(sQ + swz_bf16(i, c8)), qf);
            bf16x8_to_f32(*reinterpret_cast<const uint4*>(sK + swz_bf16(i, c8)), kf);
            const float bi = sbeta[i];
            float eg[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) eg[j] = ex2_approx(G8[j]);
#pragma unroll
            for (int j = 0; j < 8; ++j) o8[j] = p.scale * qf[j] * eg[j];
            *reinterpret_cast<uint4*>(gQt + cm_idx(i, c8, D)) = f32_to_bf16x8(o8);
#pragma unroll
            for (int j = 0; j < 8; ++j) o8[j] = bi * kf[j] * eg[j];
            *reinterpret_cast<uint4*>(sKB + cm_idx(i, c8, D)) = f32_to_bf16x8(o8);
#pragma unroll
            for (int j = 0; j < 8; ++j) o8[j] = kf[j] * ex2_approx(gl[j] - G8[j]);
            *reinterpret_cast<uint4*>(gKh + cm_idx(i, c8, D)) = f32_to_bf16x8(o8);
            if (m >= 1) {  // rows of block m as the N operand of block m's products
                float r[8];
                {
                    const float4 a = *reinterpret_cast<const float4*>(sG + swz_f32(16 * m, c8));
                    const float4 b = *reinterpret_cast<const float4*>(sG + swz_f32(16 * m, c8 + 4));
                    r[0] = a.x; r[1] = a.y; r[2] = a.z; r[3] = a.w; r[4] = b.x; r[5] = b.y; r[6] = b.z; r[7] = b.w;
                }
                __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(dyn + XSC + (m - 1) * 8192);
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = ex2_approx(G8[j] - r[j]);
#pragma unroll
                for (int j = 0; j < 8; ++j) o8[j] = qf[j] * f[j];
                *reinterpret_cast<uint4*>(xs + cm_idx(i - 16 * m, c8, D)) = f32_to_bf16x8(o8);
#pragma unroll
                for (int j = 0; j < 8; ++j) o8[j] = kf[j] * f[j];
                *reinterpret_cast<uint4*>(xs + cm_idx(16 + i - 16 * m, c8, D)) = f32_to_bf16x8(o8);
            }
#pragma unroll 1
            for (int I = 1; I <= 3; ++I) {  // keys scaled for the later blocks
                __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(dyn + KSC + (I - 1) * 16384);
                if (m < I) {
                    const float4 a = *reinterpret_cast<const float4*>(sG + swz_f32(16 * I, c8));
                    const float4 b = *reinterpret_cast<const float4*>(sG + swz_f32(16 * I, c8 + 4));
                    const float r[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
                    for (int j = 0; j < 8; ++j) o8[j] = kf[j] * ex2_approx(r[j] - G8[j]);
                    *reinterpret_cast<uint4*>(ks + cm_idx(i, c8, D)) = f32_to_bf16x8(o8);
                } else {
                    *reinterpret_cast<uint4*>(ks + cm_idx(i, c8, D)) = make_uint4(0, 0, 0, 0);
                }
            }
        }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();

    KDA_PHASE(3);
    // ---- 2: off-diagonal blocks on the tensor cores, diagonal blocks exactly on the CUDA cores
    // (lane 0 of warps 0, 1, 2 issues the eight MMAs of block I = warp + 1: the accumulators are
    //  independent, and no warp starts its share of the diagonal work a whole issue sequence late)
    if (warp < 3 && lane == 0) {
        tc_fence_after();
        const uint32_t sb = smem_u32(dyn);
        constexpr uint32_t id = make_idesc(64, 32, false, false);
        const int I = warp + 1;
#pragma unroll
        for (int s = 0; s < 8; ++s)
            mma_ss(tmem0 + T_D + 32 * (I - 1), make_desc(sb + KSC + (I - 1) * 16384 + s * 256, 128, 2048),
                   make_desc(sb + XSC + (I - 1) * 8192 + s * 256, 128, 2048), id, s > 0);
        mma_commit(&bar);
    }
    KDA_PHASE(4);
    ok = mbar_wait(&bar, it & 1, p, 8) && ok;
    tc_fence_after();
    KDA_PHASE(11);
    if (ok) {  // warp (quadrant, group): accumulator columns 32 group .. 32 group + 31 = block I = group + 1
        const int grp = warp >> 2;
        if (grp == 0) read_offdiag<0>(tmem0 + T_D, warp & 3, lane, sA, sL, p.scale);
        else if (grp == 1) read_offdiag<32>(tmem0 + T_D, warp & 3, lane, sA, sL, p.scale);
        else if (grp == 2) read_offdiag<64>(tmem0 + T_D, warp & 3, lane, sA, sL, p.scale);
    }
    KDA_PHASE(12);
    tc_fence_before();
    __syncthreads();
    if (more) {  // the operand tiles of the off-diagonal products are dead; the scalars have the whole solve to arrive
        ci_nx = chunk_info(p, un.c);
        request_rows(ci_nx, un.head());
        request_scalars(ci_nx, un.head(), nx);
    }
    KDA_PHASE(15);

    KDA_PHASE(5);
    // (issued here rather than before the operand stage, whose shared-memory traffic they would share)
    if (tid == NTHR - 64 && save) {  // prologue results for the backward: bulk stores straight from shared memory, issued by a
                                     // thread of a warp that has no share in the solve
        tma_store_1d((float*)(ws + L.Gc) + rec * C * D, sG, C * D * 4);
        tma_store_1d((__nv_bfloat16*)(ws + L.Qn) + rec * C * D, sQ, C * D * 2);
        tma_store_1d((__nv_bfloat16*)(ws + L.Kn) + rec * C * D, sK, C * D * 2);
        tma_store_1d((float*)(ws + L.aux) + rec * 3 * C, saux, 3 * C * 4);
        tma_store_commit();
    }

    // ---- 3: T = (I + diag(beta) L)^-1, column by column.  Column c of T depends only on
    //      column c of the blocks above it, so one lane carries a whole column in registers:
    //      warp w < 8 owns columns 8 (w / 4) + lane % 8 of block column J = w % 4 (w < 4) or 3 - w % 4 (w >= 4),
    //      and its four lane groups (lane / 8) split the 16 rows of every block below the diagonal.  Warps w and
    //      w + 4 issue from the same scheduler: with J and 3 - J they bring it 3 block levels whatever J is.
    solve_block_column(sL, sT, sbeta, (warp & 4) ? 3 - (warp & 3) : (warp & 3), (warp >> 2) & 1, lane, warp < 8);
    fence_async_smem();
    __syncthreads();
    if (more) request_v(ci_nx, un.head());  // L is dead: its tile receives the next unit's v rows

    KDA_PHASE(6);
    // ---- 4: Aqk and T records; T as the B operand of the WY products
    {
        __nv_bfloat16* sTB = reinterpret_cast<__nv_bfloat16*>(dyn + KSC);
        // eight lanes = eight adjacent rows of one 8-column group: one core matrix of the records, 32 distinct banks
        const int i = (tid & 7) | ((tid >> 6) << 3), j8 = ((tid >> 3) & 7) * 8;
        float a8[8], t8[8];
#pragma unroll
        for (int j = 0; j < 8; j += 4) {
            const float4 a = *reinterpret_cast<const float4*>(sA + i * LDR + j8 + j);
            const float4 t = *reinterpret_cast<const float4*>(sT + i * LDR + j8 + j);
            a8[j] = a.x, a8[j + 1] = a.y, a8[j + 2] = a.z, a8[j + 3] = a.w;
            t8[j] = t.x, t8[j + 1] = t.y, t8[j + 2] = t.z, t8[j + 3] = t.w;
        }
        const uint4 tb = f32_to_bf16x8(t8);
        *reinterpret_cast<uint4*>(gA + cm_idx(i, j8, C)) = f32_to_bf16x8(a8);
        if (save) *reinterpret_cast<uint4*>(gT + cm_idx(i, j8, C)) = tb;
        *reinterpret_cast<uint4*>(sTB + cm_idx(i, j8, C)) = tb;
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    KDA_PHASE(7);
    // ---- 5: W^T and U^T (one issuing thread each)
    if (lane == 0 && warp < 2) {
        tc_fence_after();
        const uint32_t sb = smem_u32(dyn);
        constexpr uint32_t id = make_idesc(128, 64, true, false);
        const uint32_t acc = warp == 0 ? T_W : T_U, a_tile = warp == 0 ? KB : BV;
#pragma unroll
        for (int s = 0; s < 4; ++s)
            mma_ss(tmem0 + acc, make_desc(sb + a_tile + s * 4096, 2048, 128), make_desc(sb + KSC + s * 256, 128, 1024), id, s > 0);
        mma_commit(&bar2);
    }
    if (tid < D) gGam[tid] = ex2_approx(sG[swz_f32(C - 1, tid)]);
    ok = mbar_wait(&bar2, it & 1, p, 8) && ok;
    tc_fence_after();

    KDA_PHASE(8);
    // ---- 6: W and U records: warp (quadrant, group) takes token columns 32 (group % 2) .. +31 of W (groups
    //      0, 1) or U (groups 2, 3)
    if (ok) {
        const int qd = warp & 3, dd = 32 * qd + lane, grp = warp >> 2;
        __nv_bfloat16* dst = grp < 2 ? gW : gU;
        const uint32_t src = tmem0 + ((uint32_t)(32 * qd) << 16) + (grp < 2 ? T_W : T_U);
#pragma unroll
        for (int i0 = 32 * (grp & 1); i0 < 32 * (grp & 1) + 32; i0 += 16) {
            uint32_t r[16];
            tmem_ld16(src + i0, r);
            tmem_wait_ld();
            *reinterpret_cast<uint4*>(dst + cm_idx(dd, i0, C)) =
                make_uint4(pack_bf16(__uint_as_float(r[0]), __uint_as_float(r[1])), pack_bf16(__uint_as_float(r[2]), __uint_as_float(r[3])),
                           pack_bf16(__uint_as_float(r[4]), __uint_as_float(r[5])), pack_bf16(__uint_as_float(r[6]), __uint_as_float(r[7])));
            *reinterpret_cast<uint4*>(dst + cm_idx(dd, i0 + 8, C)) =
                make_uint4(pack_bf16(__uint_as_float(r[8]), __uint_as_float(r[9])), pack_bf16(__uint_as_float(r[10]), __uint_as_float(r[11])),
                           pack_bf16(__uint_as_float(r[12]), __uint_as_float(r[13])), pack_bf16(__uint_as_float(r[14]), __uint_as_float(r[15])));
        }
    }
    if (more) park_taps(nx);  // (T has left for its record and its operand tile)
    if (tid == NTHR - 64) tma_store_wait_all();
    tc_fence_before();
    ok = __syncthreads_and(ok);
    KDA_PHASE(9);
    if (!ok) break;  // a wait gave up (recorded in the status word): no further unit is started
    ci = ci_nx;
    }
    if (!ok && more) {  // the next unit's copies are in flight: they must have landed before the CTA leaves
        mbar_wait(&rowbar, (it + 1) & 1, p, 8);
        mbar_wait(&vbar, (it + 1) & 1, p, 8);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_s, TMEM_COLS);
}

cudaError_t launch_fwd_intra_tc(const KdaParams& p, cudaStream_t s) {
    auto kern = p.conv_q ? kda_fwd_intra_tc<true> : kda_fwd_intra_tc<false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fi::TOTAL);
    if (e != cudaSuccess) return e;
    const int units = p.NT * p.H, sms = sm_count();
    RowMaps maps = {};
    const long long tokens = (long long)p.B * p.T;
    maps.ok = !(p.flags & KDA_FLAG_ROW_COPIES) && make_row_map(&maps.m[0], p.q, tokens, p.H, C) && make_row_map(&maps.m[1], p.k, tokens, p.H, C) &&
              make_row_map(&maps.m[2], p.v, tokens, p.H, C) && make_row_map(&maps.m[3], p.g, tokens, p.H, C);
    kern<<<units < sms ? units : sms, fi::NTHR, fi::TOTAL, s>>>(p, maps);
    return cudaGetLastError();
}

}  // namespace kda

KDA_PHASE_EXPORT(kda_debug_phases_fwd_intra)
