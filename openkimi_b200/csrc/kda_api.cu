// C ABI of the KDA library: argument validation and stage dispatch.  No allocation, no
// device synchronisation; every error is a return code.
#include <math.h>
#include <stdio.h>
#include <string.h>

#include "kda_common.cuh"
#include "kda_tmap.cuh"

namespace kda {
cudaError_t simt_fwd(const KdaParams& p, cudaStream_t s);
cudaError_t simt_bwd(const KdaParams& p, cudaStream_t s);
cudaError_t tc_fwd(const KdaParams& p, cudaStream_t s);
cudaError_t tc_bwd(const KdaParams& p, cudaStream_t s);
bool tc_supported(const KdaParams& p);

static thread_local char g_last_error[256] = "";

// records what the runtime said (kda_last_cuda_error) and returns KDA_ERR_LAUNCH
int fail_cuda(cudaError_t e) {
    snprintf(g_last_error, sizeof(g_last_error), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
    return KDA_ERR_LAUNCH;
}

// The tensor-map encoder is a driver function; it is looked up through the runtime so that the library
// has no link-time dependency on the driver.
bool make_row_map(CUtensorMap* out, const void* base, long long tokens, int H, int box_rows) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            fn = (EncodeFn)f;
        tried = true;
    }
    if (!fn || !base || tokens <= 0) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)H * 128, (cuuint64_t)tokens};
    const cuuint64_t strides[1] = {(cuuint64_t)H * 128 * 2};
    const cuuint32_t box[2] = {128, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// ---- optional per-stage timing (benchmark instrumentation) ---------------------------------
// Each kda_fwd / kda_bwd call made while profiling is on takes the next slot and brackets
// its stages with CUDA events on the caller's stream; nothing is synchronised here.
constexpr int PROF_STAGES = 8;
struct ProfSlot { cudaEvent_t ev[PROF_STAGES + 1]; int n; int kind; };
static ProfSlot* g_prof = nullptr;
static int g_prof_cap = 0, g_prof_used = 0;
static bool g_prof_on = false;
static ProfSlot* g_cur = nullptr;

void prof_mark(cudaStream_t s) {
    if (g_cur && g_cur->n <= PROF_STAGES) cudaEventRecord(g_cur->ev[g_cur->n++], s);
}
static void prof_open(int kind, cudaStream_t s) {
    g_cur = nullptr;
    if (g_prof_on && g_prof_used < g_prof_cap) {
        g_cur = &g_prof[g_prof_used++];
        g_cur->n = 0;
        g_cur->kind = kind;
        prof_mark(s);
    }
}

__global__ void status_publish_kernel(const int32_t* status, int32_t* status_host) {
    const int v = *status;
    if (v) *status_host = v;
}

static bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

static int validate(const KdaParams* p, bool bwd) {
    if (!p) return KDA_ERR_NULL;
    if (p->dtype != KDA_DTYPE_F32 && p->dtype != KDA_DTYPE_BF16) return KDA_ERR_DTYPE;
    if (p->B <= 0 || p->T <= 0 || p->H <= 0 || p->N <= 0 || p->NT <= 0) return KDA_ERR_SHAPE;
    if (p->dk != p->dv || (p->dk != 64 && p->dk != 128)) return KDA_ERR_SHAPE;
    if (p->cu_seqlens) {
        if (p->B != 1 || !p->chunk_seq || !p->seq_chunk_off) return KDA_ERR_SHAPE;
    } else {
        if (p->N != p->B || p->NT != p->B * ((p->T + C - 1) / C)) return KDA_ERR_SHAPE;
    }
    if (!p->q || !p->k || !p->v || !p->g || !p->beta || !p->o || !p->workspace) return KDA_ERR_NULL;
    if ((p->flags & KDA_FLAG_GATE) && !p->A_log) return KDA_ERR_NULL;
    if (!(p->guard_span < 0.f) && !(isfinite(p->guard_span) && p->guard_span <= kda_guard_max_span()))
        return KDA_ERR_GUARD;
    const void* ptrs[] = {p->q, p->k, p->v, p->g, p->o, p->workspace, p->h0, p->ht, p->chunk_tab};
    for (const void* x : ptrs)
        if (!aligned16(x)) return KDA_ERR_ALIGN;
    WsLayout L = ws_layout(p->NT, p->H, p->dk, p->dv, p->dtype);
    const bool conv = p->conv_q || p->conv_k || p->conv_v;
    if (conv) {
        if (!p->conv_q || !p->conv_k || !p->conv_v) return KDA_ERR_NULL;
        if (p->conv_ksize < 1 || p->conv_ksize > 4) return KDA_ERR_SHAPE;
        if ((p->flags & (KDA_FLAG_FORCE_SIMT | KDA_FLAG_SIMT_FWD_INTRA | KDA_FLAG_SIMT_BWD_CHUNK | KDA_FLAG_SIMT_BWD_WY)) || !tc_supported(*p))
            return KDA_ERR_UNSUPPORTED;
    }
    const bool nosave = p->flags & KDA_FLAG_NO_SAVE;
    if (bwd && nosave) return KDA_ERR_WORKSPACE;  // the records of a forward-only call do not exist
    if (p->workspace_bytes < (nosave ? L.total_nosave : conv ? L.total_conv : L.total) || ((uintptr_t)p->workspace & 255))
        return KDA_ERR_WORKSPACE;
    if (bwd) {
        if (!p->grad_o || !p->grad_q || !p->grad_k || !p->grad_v || !p->grad_g || !p->grad_beta || !p->bwd_scratch) return KDA_ERR_NULL;
        if ((p->flags & KDA_FLAG_GATE) && !p->grad_A_log) return KDA_ERR_NULL;
        const bool cvb = p->grad_conv_q || p->grad_conv_k || p->grad_conv_v;
        if (cvb && (!conv || !p->grad_conv_q || !p->grad_conv_k || !p->grad_conv_v)) return KDA_ERR_NULL;
        if (p->bwd_scratch_bytes < (cvb ? L.bwd_total_conv : L.bwd_total) || ((uintptr_t)p->bwd_scratch & 255))
            return KDA_ERR_WORKSPACE;
        const void* bp[] = {p->grad_o, p->grad_q, p->grad_k, p->grad_v, p->grad_g, p->grad_ht, p->grad_h0};
        for (const void* x : bp)
            if (!aligned16(x)) return KDA_ERR_ALIGN;
    }
    return KDA_OK;
}
}  // namespace kda

using namespace kda;

extern "C" {

int kda_abi_version(void) { return 4; }

int kda_guard_version(void) { return 1; }
float kda_guard_max_span(void) { return 232.0f; }
const char* kda_guard_dot_precision(void) { return "tf32x3"; }

const char* kda_last_cuda_error(void) { return g_last_error; }

const char* kda_status_string(int s) {
    switch (s) {
        case KDA_OK: return "ok";
        case KDA_ERR_NULL: return "a required pointer is NULL";
        case KDA_ERR_SHAPE: return "unsupported or inconsistent sizes (need dk == dv in {64,128}, chunk 64)";
        case KDA_ERR_DTYPE: return "unsupported element type";
        case KDA_ERR_WORKSPACE: return "workspace too small or not 256-byte aligned";
        case KDA_ERR_ALIGN: return "tensor pointer not 16-byte aligned";
        case KDA_ERR_LAUNCH: return "CUDA launch failed";
        case KDA_ERR_DEVICE_WAIT: return "a bounded device-side wait gave up";
        case KDA_ERR_GUARD: return "guard span must be negative (exact) or a finite value <= 232";
        case KDA_ERR_UNSUPPORTED: return "the fused short convolution needs BF16 tensors with dk = dv = 128 and the tensor-core stages";
        case KDA_ERR_STATIC_LIMIT: return "size exceeds the built-in scratch of the allocation-free entry point (C * ksize <= 8192)";
        default: return "unknown status";
    }
}

int kda_workspace_bytes(const KdaParams* p, size_t* fwd_bytes, size_t* bwd_bytes) {
    if (!p) return KDA_ERR_NULL;
    if (p->NT <= 0 || p->H <= 0 || p->dk <= 0 || p->dv <= 0) return KDA_ERR_SHAPE;
    WsLayout L = ws_layout(p->NT, p->H, p->dk, p->dv, p->dtype);
    if (fwd_bytes) *fwd_bytes = (p->flags & KDA_FLAG_NO_SAVE) ? L.total_nosave : p->conv_q ? L.total_conv : L.total;
    if (bwd_bytes) *bwd_bytes = p->conv_q ? L.bwd_total_conv : L.bwd_total;
    return KDA_OK;
}

int kda_fwd(const KdaParams* p, void* stream) {
    int v = validate(p, false);
    if (v != KDA_OK) return v;
    cudaStream_t s = (cudaStream_t)stream;
    const bool tc = !(p->flags & KDA_FLAG_FORCE_SIMT) && tc_supported(*p);
    prof_open(0, s);
    cudaError_t e = tc ? tc_fwd(*p, s) : simt_fwd(*p, s);
    g_cur = nullptr;
    return e == cudaSuccess ? KDA_OK : fail_cuda(e);
}

int kda_bwd(const KdaParams* p, void* stream) {
    int v = validate(p, true);
    if (v != KDA_OK) return v;
    cudaStream_t s = (cudaStream_t)stream;
    const bool tc = !(p->flags & KDA_FLAG_FORCE_SIMT) && tc_supported(*p);
    prof_open(1, s);
    cudaError_t e = tc ? tc_bwd(*p, s) : simt_bwd(*p, s);
    g_cur = nullptr;
    return e == cudaSuccess ? KDA_OK : fail_cuda(e);
}

int kda_status_publish(const int32_t* status, int32_t* status_host, void* stream) {
    if (!status || !status_host) return KDA_ERR_NULL;
    status_publish_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(status, status_host);
    return launch_status();
}

int kda_profile_begin(int max_calls) {
    if (max_calls < 0) return KDA_ERR_SHAPE;
    if (max_calls > g_prof_cap) {
        ProfSlot* n = new ProfSlot[max_calls];
        for (int i = 0; i < max_calls; ++i)
            for (int j = 0; j <= PROF_STAGES; ++j)
                if (i < g_prof_cap) n[i].ev[j] = g_prof[i].ev[j];
                else if (cudaEventCreate(&n[i].ev[j]) != cudaSuccess) return KDA_ERR_LAUNCH;
        delete[] g_prof;
        g_prof = n;
        g_prof_cap = max_calls;
    }
    g_prof_used = 0;
    g_prof_on = max_calls > 0;
    return KDA_OK;
}

int kda_profile_read(int call, int* kind, float* stage_ms, int max_stages) {
    g_prof_on = false;
    if (call < 0 || call >= g_prof_used || !stage_ms) return -1;
    ProfSlot& sl = g_prof[call];
    if (kind) *kind = sl.kind;
    int n = sl.n - 1 < max_stages ? sl.n - 1 : max_stages;
    for (int i = 0; i < n; ++i)
        if (cudaEventElapsedTime(&stage_ms[i], sl.ev[i], sl.ev[i + 1]) != cudaSuccess) return -1;
    return n;
}

}  // extern "C"
