// Shared host-side helpers of the C ABI: error reporting, argument checks, Philox.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

#include "../../include/mptorch_b200.h"

namespace mpt {

void set_error(const char* fmt, ...);          // defined in api.cu
int check_launch(const char* what);            // cudaGetLastError -> MPT_ERR_CUDA

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

inline bool valid_format(int man, int exp) { return man >= 0 && man <= 23 && exp >= 1 && exp <= 8; }

#define MPT_REQUIRE(cond, ...)                     \
    do {                                           \
        if (!(cond)) {                             \
            ::mpt::set_error(__VA_ARGS__);         \
            return MPT_ERR_INVALID_ARGUMENT;       \
        }                                          \
    } while (0)

struct AnyFmt;
// Validate a public format descriptor and convert it; false (with the error set) if it is malformed.
bool convert_format(const char* who, const mpt_format* in, AnyFmt* out);

// Number of SMs of the current device (cached per device).
int sm_count();

// Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11).
struct Philox {
    uint32_t c[4];
    __host__ __device__ Philox(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3) : c{c0, c1, c2, c3} {}
    __host__ __device__ void run(uint32_t k0, uint32_t k1) {
#pragma unroll
        for (int i = 0; i < 10; ++i) {
            // one 32 x 32 -> 64 multiply per product (a single wide multiply-add on the GPU)
            const uint64_t p0 = (uint64_t)0xD2511F53u * c[0], p1 = (uint64_t)0xCD9E8D57u * c[2];
            const uint32_t h0 = (uint32_t)(p0 >> 32), l0 = (uint32_t)p0, h1 = (uint32_t)(p1 >> 32), l1 = (uint32_t)p1;
            const uint32_t n0 = h1 ^ c[1] ^ k0, n2 = h0 ^ c[3] ^ k1;
            c[0] = n0; c[1] = l1; c[2] = n2; c[3] = l0;
            k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
        }
    }
};

}  // namespace mpt
