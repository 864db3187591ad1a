// Batched transpose of the last two dimensions: out[b][c][r] = in[b][r][c].
//
// The layers hand the GEMM transposed views (W^T in the forward pass, dY^T and X^T for the weight gradient, K^T in
// attention), and the GEMM wants dense row-major operands; this kernel makes the dense copy at close to the copy
// bandwidth, where a generic strided elementwise copy reads or writes one of the two sides 4 bytes at a time per
// 32-byte sector.  A CTA moves a 64 x 64 tile through shared memory: 16-byte coalesced reads along the input rows,
// 16-byte coalesced writes along the output rows, the row pitch of 65 words keeping the column reads free of bank
// conflicts.  HBM-bound: 8 bytes per element.
#include "common.cuh"

namespace mpt {
namespace {

constexpr int kTile = 64;

__global__ void __launch_bounds__(256) transpose_kernel(const float* __restrict__ in, float* __restrict__ out, int rows, int cols) {
    __shared__ float tile[kTile][kTile + 1];
    const int64_t plane = (int64_t)rows * cols;
    const float* src = in + blockIdx.z * plane;
    float* dst = out + blockIdx.z * plane;
    const int r0 = blockIdx.y * kTile, c0 = blockIdx.x * kTile;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;          // 16 x 16 threads, 4 columns each, 4 row passes
    const bool vec_in = (cols & 3) == 0 && ((reinterpret_cast<uintptr_t>(in) & 15u) == 0);
    const bool vec_out = (rows & 3) == 0 && ((reinterpret_cast<uintptr_t>(out) & 15u) == 0);
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const int r = r0 + ty + 16 * p, c = c0 + 4 * tx;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (r < rows) {
            if (vec_in && c + 3 < cols) {
                const float4 q = *reinterpret_cast<const float4*>(src + (int64_t)r * cols + c);
                v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (c + j < cols) v[j] = src[(int64_t)r * cols + c + j];
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) tile[ty + 16 * p][4 * tx + j] = v[j];
    }
    __syncthreads();
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const int c = c0 + ty + 16 * p, r = r0 + 4 * tx;             // output row c, output columns r .. r + 3
        if (c >= cols) continue;
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = tile[4 * tx + j][ty + 16 * p];
        if (vec_out && r + 3 < rows) *reinterpret_cast<float4*>(dst + (int64_t)c * rows + r) = make_float4(v[0], v[1], v[2], v[3]);
        else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (r + j < rows) dst[(int64_t)c * rows + r + j] = v[j];
        }
    }
}

}  // namespace
}  // namespace mpt

extern "C" int mpt_transpose_last2(const float* in, float* out, int64_t batch, int64_t rows, int64_t cols, void* stream) {
    using namespace mpt;
    if (batch == 0 || rows == 0 || cols == 0) return MPT_OK;
    MPT_REQUIRE(in && out && batch > 0 && rows > 0 && cols > 0, "transpose_last2: bad arguments");
    MPT_REQUIRE(in != out, "transpose_last2: in place is not supported");
    const int64_t gx = (cols + kTile - 1) / kTile, gy = (rows + kTile - 1) / kTile;
    MPT_REQUIRE(rows <= 0x7FFFFFFF && cols <= 0x7FFFFFFF && gy <= 65535 && batch <= 65535,
                "transpose_last2: more than 65535 row tiles or batch entries");
    transpose_kernel<<<dim3((unsigned)gx, (unsigned)gy, (unsigned)batch), 256, 0, static_cast<cudaStream_t>(stream)>>>(in, out, (int)rows, (int)cols);
    return check_launch("transpose_last2");
}
