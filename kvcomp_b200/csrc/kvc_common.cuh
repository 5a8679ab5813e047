// Shared device/host helpers of libkvcomp_b200 (sm_100a).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/kvcomp_b200.h"

#define KVC_VEC_LEN 128       // symbols per vector (kernels.h:12,18)
#define KVC_VEC_PER_BLK 64    // vectors per block  (kernels.h:13,19)
#define KVC_LUT_SIZE (1 << KVC_LUT_BITS)
#define KVC_TREE_LEAF 0xFFFFu   // wide-tree node: low half == LEAF -> high half is the symbol
#define KVC_TREE_NONE 0xFFFEu   // wide-tree child that does not exist

void kvc_set_error(const char *fmt, ...);

#define KVC_REQUIRE(cond, ...)                      \
    do {                                            \
        if (!(cond)) {                              \
            kvc_set_error(__VA_ARGS__);             \
            return KVC_ERR_ARG;                     \
        }                                           \
    } while (0)

#define KVC_CUDA_OK(call)                                                              \
    do {                                                                               \
        cudaError_t e_ = (call);                                                       \
        if (e_ != cudaSuccess) {                                                       \
            kvc_set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_),      \
                          __FILE__, __LINE__);                                         \
            return KVC_ERR_CUDA;                                                       \
        }                                                                              \
    } while (0)

#define KVC_LAUNCH_OK() KVC_CUDA_OK(cudaGetLastError())

static inline cudaStream_t kvc_cu(kvc_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

int kvc_sm_count();

// ---- device helpers ---------------------------------------------------------------
struct kvc_qmeta_dev {          // kvc_qmeta with typed pointers, passed by value to kernels
    const void *min_int;
    const __half *scale;
    int min_bytes;
    int tok_div;
    long long sj, sb, sh, sc;
};

static inline kvc_qmeta_dev kvc_to_dev(const kvc_qmeta &q) {
    kvc_qmeta_dev d;
    d.min_int = q.min_int; d.scale = reinterpret_cast<const __half *>(q.scale);
    d.min_bytes = q.min_bytes; d.tok_div = q.tok_div;
    d.sj = q.sj; d.sb = q.sb; d.sh = q.sh; d.sc = q.sc;
    return d;
}

// t / tok_div without the emulated 64-bit division: token indices fit 32 bits in every real cache
__device__ __forceinline__ long long kvc_tok_unit(long long t, int tok_div) {
    if (tok_div == 1) return t;
    if ((unsigned long long)t <= 0xffffffffull) return (long long)((uint32_t)t / (uint32_t)tok_div);
    return t / tok_div;
}

__device__ __forceinline__ int kvc_load_min(const kvc_qmeta_dev &m, long long u) {
    int r;                      // one sign-extending load either way: nothing consumes the value here
    if (m.min_bytes == 1) r = reinterpret_cast<const int8_t *>(m.min_int)[u];
    else r = reinterpret_cast<const int16_t *>(m.min_int)[u];
    return r;
}
__device__ __forceinline__ unsigned short kvc_load_scale_bits(const kvc_qmeta_dev &m, long long u) {
    return reinterpret_cast<const unsigned short *>(m.scale)[u];
}
__device__ __forceinline__ float kvc_scale_value(unsigned short bits) { return __half2float(__ushort_as_half(bits)); }

__device__ __forceinline__ uint32_t kvc_bswap(uint32_t x) { return __byte_perm(x, 0, 0x0123); }

// 4x4 byte transpose: in a, b, c, d = rows; out a = {a0,b0,c0,d0}, b = {a1,b1,c1,d1}, ...
__device__ __forceinline__ void kvc_transpose4x4(uint32_t &a, uint32_t &b, uint32_t &c, uint32_t &d) {
    const uint32_t t0 = __byte_perm(a, b, 0x5140), t1 = __byte_perm(c, d, 0x5140);
    const uint32_t t2 = __byte_perm(a, b, 0x7362), t3 = __byte_perm(c, d, 0x7362);
    a = __byte_perm(t0, t1, 0x5410); b = __byte_perm(t0, t1, 0x7632);
    c = __byte_perm(t2, t3, 0x5410); d = __byte_perm(t2, t3, 0x7632);
}

__device__ __forceinline__ float kvc_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float kvc_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
