// Error reporting and device queries shared by every C-ABI entry point.
#include <cstring>
#include <mutex>

#include "cast.cuh"
#include "common.cuh"

namespace mpt {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: %s", what, cudaGetErrorString(e));
        return MPT_ERR_CUDA;
    }
    return MPT_OK;
}

bool convert_format(const char* who, const mpt_format* in, AnyFmt* out) {
    if (in == nullptr) { set_error("%s: null format descriptor", who); return false; }
    AnyFmt a;
    a.kind = in->kind;
    a.bl = a.bu = 1; a.P = 1; a.is_signed = 1; a.policy = 0;
    switch (in->kind) {
        case MPT_FMT_FLOAT:
            if (!valid_format(in->man, in->exp)) { set_error("%s: unsupported float format man=%d exp=%d", who, in->man, in->exp); return false; }
            a.fp = make_fmt(in->man, in->exp, in->subnormals, in->saturate);
            break;
        case MPT_FMT_SUPERFP:
            if (!valid_format(in->man, in->exp) || in->binades_l < 1 || in->binades_u < 1) {
                set_error("%s: unsupported supernormal format man=%d exp=%d binades=(%d,%d)", who, in->man, in->exp, in->binades_l, in->binades_u);
                return false;
            }
            a.fp = make_fmt(in->man, in->exp, 1, in->saturate);
            a.bl = in->binades_l; a.bu = in->binades_u;
            break;
        case MPT_FMT_BINARY8:
            if (in->P < 1 || in->P > 7 || in->overflow_policy < 0 || in->overflow_policy > 2) {
                set_error("%s: unsupported binary8 format P=%d policy=%d", who, in->P, in->overflow_policy);
                return false;
            }
            a.fp = make_fmt(in->P - 1, 8, in->subnormals, 0);
            a.P = in->P; a.is_signed = in->is_signed != 0; a.policy = in->overflow_policy;
            break;
        default:
            set_error("%s: unknown format kind %d", who, in->kind);
            return false;
    }
    *out = a;
    return true;
}

int sm_count() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace mpt

extern "C" {

const char* mpt_last_error(void) { return mpt::g_err; }
int mpt_version(void) { return 100; }

int mpt_stream_priority_range(int* lowest, int* highest) {
    int lo = 0, hi = 0;
    const cudaError_t e = cudaDeviceGetStreamPriorityRange(&lo, &hi);
    if (e != cudaSuccess) { mpt::set_error("stream_priority_range: %s", cudaGetErrorString(e)); return MPT_ERR_CUDA; }
    if (lowest) *lowest = lo;
    if (highest) *highest = hi;
    return MPT_OK;
}

int mpt_copy_columns_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes, size_t rows,
                           void* stream) {
    if (rows == 0 || width_bytes == 0) return MPT_OK;
    if (!dst || !src || width_bytes > dst_pitch || width_bytes > src_pitch) {
        mpt::set_error("copy_columns_async: null pointer or a row wider than its pitch");
        return MPT_ERR_INVALID_ARGUMENT;
    }
    const cudaError_t e = cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyDefault,
                                            static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) { mpt::set_error("copy_columns_async: %s", cudaGetErrorString(e)); return MPT_ERR_CUDA; }
    return MPT_OK;
}

}
