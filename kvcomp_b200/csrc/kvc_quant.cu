// Error-bounded quantiser, dequantiser and the dense q.k baseline.
//
// Follows utils/compute.py:93-106 (quant) as torch evaluates it on fp16 tensors: every
// elementwise op widens to fp32, computes, and rounds to nearest-even back to fp16; the
// Python scalar `rel` stays fp32.  Explicit round-to-nearest intrinsics are used so that no
// contraction or fast-math rewrite can change a bit.
#include <algorithm>

#include "kvc_common.cuh"

namespace {

struct UnitParam { float sf; float mi; float rcp; };   // scale, min_int and 1/scale as floats

__device__ __forceinline__ UnitParam unit_param(float mn, float mx, float rel, __half *scale_out, int *flags) {
    __half range = __float2half_rn(__fsub_rn(mx, mn));
    __half sc = __float2half_rn(__fmul_rn(__half2float(range), rel));
    UnitParam p;
    p.sf = __half2float(sc);
    p.rcp = 0.0f;
    if (p.sf == 0.0f || p.sf != p.sf) { p.mi = 0.0f; *flags |= KVC_FLAG_ZERO_SCALE; }
    else { p.mi = rintf(__half2float(__float2half_rn(__fdiv_rn(mn, p.sf)))); p.rcp = __frcp_rn(p.sf); }
    *scale_out = sc;
    return p;
}

__device__ __forceinline__ void store_min(void *min_int, int min_bytes, long long u, float mi, int *flags) {
    int v = (int)mi;
    if (min_bytes == 1) {
        if (v < -128 || v > 127) *flags |= KVC_FLAG_MIN_OVERFLOW;
        reinterpret_cast<int8_t *>(min_int)[u] = (int8_t)v;      // wraps like the reference's .to(int8)
    } else {
        if (v < -32768 || v > 32767) *flags |= KVC_FLAG_MIN_OVERFLOW;
        reinterpret_cast<int16_t *>(min_int)[u] = (int16_t)v;
    }
}

// fp16(x / scale) without the full IEEE division: q1 = x*r corrected once by the exact residual is within
// 2^-24 (relative) of the true quotient t.  x and scale carry 11 significant bits, so t is at least
// 2^-23 (relative) away from every midpoint between two fp16 values (t = m would need m*scale = x with a
// 12-bit m); hence q1, the correctly rounded fp32 quotient and t all round to the same fp16 value.
// rint(v) for |v| < 2^22 without the conversion pipe: adding 1.5 * 2^23 rounds to an integer (to nearest
// even, the mode rintf uses) and leaves that integer in the low mantissa bits.
#define KVC_RINT_MAGIC 12582912.0f
__device__ __forceinline__ uint32_t quant_one(__half x, const UnitParam &p, int *flags) {
    if (p.sf == 0.0f || p.sf != p.sf) return 0u;
    const float xf = __half2float(x);
    const float q0 = __fmul_rn(xf, p.rcp);
    const float q1 = __fmaf_rn(__fmaf_rn(-q0, p.sf, xf), p.rcp, q0);
    const float qh = __half2float(__float2half_rn(q1));                      // |qh| <= 65504 (or inf)
    const float q = __fsub_rn(__fadd_rn(qh, KVC_RINT_MAGIC), KVC_RINT_MAGIC);  // = rintf(qh) for finite qh
    const float d = __fsub_rn(q, p.mi);
    if (d >= 0.0f && d <= 255.0f)            // an integer that fp16 holds exactly: the code, read from the mantissa
        return (uint32_t)__float_as_int(__fadd_rn(d, KVC_RINT_MAGIC)) & 0xffu;
    // out of range (or not finite): follow the fp16 arithmetic to the end, as the reference's tensors do
    const float qs = rintf(qh);
    const float c = __half2float(__float2half_rn(__fsub_rn(qs, p.mi)));
    if (!(c >= 0.0f && c <= 255.0f)) { *flags |= KVC_FLAG_CODE_OVERFLOW; }
    return (uint32_t)(int)c & 0xffu;
}

// quantise 8 halves held in a uint4 -> 8 code bytes in a uint2; optional smem histogram.
// PS: 0 = the eight values share one unit (p[0]), 1 = value i belongs to unit p[i].
//
// Packed path, for units whose min_int lies in -255..255 (`small_min`; mi2 holds the min_ints as fp16 pairs):
// after the fp32 product q0 = x * (1 / scale) everything is done on two values per instruction in fp16, which
// is what the reference's tensors hold anyway.
//  * fp16(q0) equals the reference's fp16(x / scale) except on exact ties between two fp16 subnormals, where
//    both round to the integer 0 (checked over every pair of fp16 values).
//  * (qh + 1536) - 1536 in fp16 is rint(qh) for |qh| <= 512; beyond that the result stays beyond 511 in
//    magnitude or is no integer, and with |min_int| <= 255 such a value fails the range test below.
//  * d = r - min_int, then d + 1024 has the bit pattern 0x6400 + d for the integers 0 <= d < 1024: the code is
//    read from the mantissa, and one mask over all eight tells whether every code is in 0..255.
// Anything else (a value out of range, not finite, a unit with a large min_int) takes the fp32 path below it,
// which follows the reference's arithmetic to the end.
template <int PS>
__device__ __forceinline__ uint2 quant_eight(const uint4 &v, const UnitParam *p, bool small_min, const __half2 *mi2,
                                             int *flags, unsigned int *hist) {
    const __half *h = reinterpret_cast<const __half *>(&v);
    uint2 o;
    if (small_min) {
        const __half2 *h2 = reinterpret_cast<const __half2 *>(&v);
        const __half2 big = __float2half2_rn(1536.0f), nbig = __float2half2_rn(-1536.0f), k1024 = __float2half2_rn(1024.0f);
        uint32_t u[4], odd = 0;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float2 xf = __half22float2(h2[k]);
            const __half2 qh = __floats2half2_rn(__fmul_rn(xf.x, p[2 * k * PS].rcp), __fmul_rn(xf.y, p[(2 * k + 1) * PS].rcp));
            const __half2 r = __hadd2(__hadd2(qh, big), nbig);
            const __half2 t = __hadd2(__hsub2(r, mi2[k * PS]), k1024);
            u[k] = *reinterpret_cast<const uint32_t *>(&t) - 0x64006400u;
            odd |= u[k];
        }
        if ((odd & 0xff00ff00u) == 0) {
            if (hist) {
#pragma unroll
                for (int k = 0; k < 4; k++) { atomicAdd(&hist[u[k] & 0xffu], 1u); atomicAdd(&hist[u[k] >> 16], 1u); }
            }
            o.x = __byte_perm(u[0], u[1], 0x6420);
            o.y = __byte_perm(u[2], u[3], 0x6420);
            return o;
        }
    }
    uint32_t c[8];
    uint32_t odd = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const UnitParam &u = p[i * PS];
        const float xf = __half2float(h[i]);
        const float q0 = __fmul_rn(xf, u.rcp);
        const float q1 = __fmaf_rn(__fmaf_rn(-q0, u.sf, xf), u.rcp, q0);
        const float qh = __half2float(__float2half_rn(q1));
        const float q = __fsub_rn(__fadd_rn(qh, KVC_RINT_MAGIC), KVC_RINT_MAGIC);
        const float d = __fsub_rn(q, u.mi);
        // d as an integer, read from the mantissa: in range exactly when 0 <= d <= 255
        const uint32_t t = (uint32_t)__float_as_int(__fadd_rn(d, KVC_RINT_MAGIC)) - 0x4B400000u;
        odd |= t;
        c[i] = t & 0xffu;
    }
    if (odd > 255u) {
#pragma unroll
        for (int i = 0; i < 8; i++) c[i] = quant_one(h[i], p[i * PS], flags);
    }
    if (hist) {
#pragma unroll
        for (int i = 0; i < 8; i++) atomicAdd(&hist[c[i]], 1u);
    }
    o.x = c[0] | (c[1] << 8) | (c[2] << 16) | (c[3] << 24);
    o.y = c[4] | (c[5] << 8) | (c[6] << 16) | (c[7] << 24);
    return o;
}
__device__ __forceinline__ bool small_min_int(float mi) { return mi >= -255.0f && mi <= 255.0f; }

// The CTA's bins are private to each warp (sh[warp][256]): fewer lanes meet on a counter.
__device__ __forceinline__ void hist_clear(unsigned int *sh, int tid, int nthr) {
    for (int i = tid; i < (nthr / 32) * 256; i += nthr) sh[i] = 0;
    __syncthreads();
}
__device__ __forceinline__ void hist_flush(const unsigned int *sh, unsigned long long *gh, int tid, int nthr) {
    __syncthreads();
    for (int i = tid; i < 256; i += nthr) {
        unsigned int c = 0;
        for (int w = 0; w < nthr / 32; w++) c += sh[w * 256 + i];
        if (c) atomicAdd(&gh[i], (unsigned long long)c);
    }
}

// extremes of 8 halves: packed fp16 min / max (exact, a NaN operand yields the other one, as fminf does),
// widened once at the end
__device__ __forceinline__ void minmax8(const uint4 &v, float &mn, float &mx) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&v);
    const __half2 lo = __hmin2(__hmin2(h[0], h[1]), __hmin2(h[2], h[3]));
    const __half2 hi = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
    mn = fminf(mn, fminf(__low2float(lo), __high2float(lo)));
    mx = fmaxf(mx, fmaxf(__low2float(hi), __high2float(hi)));
}

// ---- ChannelQuant (utils/compute.py:140): one unit per (token block, b, h, channel) -------------
// CTA = one (j, b, h) tile of blk tokens x 128 channels; thread = 8 channels x every 8th token.
// (Measured slower: several tiles per CTA with one flush of the bins; tiles of two or four heads; the tile's
// rows held in registers between the two passes; four rows in flight per thread in either pass.)
__global__ void __launch_bounds__(128) quant_channel_kernel(
    const __half *__restrict__ x, long long B, long long H, int blk, float rel,
    uint8_t *__restrict__ codes, void *__restrict__ min_int, int min_bytes, __half *__restrict__ scale,
    unsigned long long *__restrict__ ghist, int *__restrict__ status) {
    __shared__ float smn[8][128], smx[8][128];
    __shared__ unsigned int shist[256];
    const int tid = threadIdx.x, cg = tid & 15, r = tid >> 4;
    const long long row_stride = B * H * 128;
    if (ghist) { for (int i = tid; i < 256; i += 128) shist[i] = 0; }      // a barrier follows before the first count
    int flags = 0;
    const long long tile = blockIdx.x;                 // (j * B + b) * H + h
    const long long h = tile % H, b = (tile / H) % B, j = tile / (H * B);
    const long long base = ((j * blk) * B + b) * H * 128 + h * 128 + cg * 8;
    __half2 mn2[4], mx2[4];                                 // extremes of the thread's 8 channels, two per register
#pragma unroll
    for (int i = 0; i < 4; i++) { mn2[i] = __float2half2_rn(INFINITY); mx2[i] = __float2half2_rn(-INFINITY); }
    for (int i = r; i < blk; i += 8) {
        uint4 v = *reinterpret_cast<const uint4 *>(x + base + i * row_stride);
        const __half2 *hv = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
        for (int k = 0; k < 4; k++) { mn2[k] = __hmin2(mn2[k], hv[k]); mx2[k] = __hmax2(mx2[k], hv[k]); }
    }
#pragma unroll
    for (int k = 0; k < 4; k++) {
        smn[r][cg * 8 + 2 * k] = __low2float(mn2[k]); smn[r][cg * 8 + 2 * k + 1] = __high2float(mn2[k]);
        smx[r][cg * 8 + 2 * k] = __low2float(mx2[k]); smx[r][cg * 8 + 2 * k + 1] = __high2float(mx2[k]);
    }
    __syncthreads();
    {   // thread = channel: fold the 8 partials, derive the unit's parameters once, share them
        float a = smn[0][tid], z = smx[0][tid];
#pragma unroll
        for (int rr = 1; rr < 8; rr++) { a = fminf(a, smn[rr][tid]); z = fmaxf(z, smx[rr][tid]); }
        __half sc;
        const UnitParam q = unit_param(a, z, rel, &sc, &flags);
        const long long u = tile * 128 + tid;
        scale[u] = sc;
        store_min(min_int, min_bytes, u, q.mi, &flags);
        __syncthreads();                                   // every partial is read before the rows are reused
        smn[0][tid] = q.sf; smn[1][tid] = q.mi; smn[2][tid] = q.rcp;
    }
    __syncthreads();
    UnitParam p[8];
#pragma unroll
    for (int k = 0; k < 8; k++) { p[k].sf = smn[0][cg * 8 + k]; p[k].mi = smn[1][cg * 8 + k]; p[k].rcp = smn[2][cg * 8 + k]; }
    bool small = true;
    __half2 mi2[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        small = small && small_min_int(p[2 * k].mi) && small_min_int(p[2 * k + 1].mi);
        mi2[k] = __floats2half2_rn(p[2 * k].mi, p[2 * k + 1].mi);
    }
    for (int i = r; i < blk; i += 8) {
        uint4 v = *reinterpret_cast<const uint4 *>(x + base + i * row_stride);
        uint2 o = quant_eight<1>(v, p, small, mi2, &flags, ghist ? shist : nullptr);
        *reinterpret_cast<uint2 *>(codes + base + i * row_stride) = o;
    }
    if (flags) atomicOr(status, flags);
    if (ghist) {
        __syncthreads();
        for (int i = tid; i < 256; i += 128)
            if (shist[i]) atomicAdd(&ghist[i], (unsigned long long)shist[i]);
    }
}

// ---- units that are contiguous runs of `ulen` elements -----------------------------------------
// TokenQuant (all of a token's [B,]H,D values) and VectorQuant (one head's D values).
// GROUP threads share one unit: a warp for short units, the whole CTA (256) for long ones.
template <int GROUP>
__global__ void __launch_bounds__(256) quant_contig_kernel(
    const __half *__restrict__ x, long long n_units, long long ulen, float rel,
    uint8_t *__restrict__ codes, void *__restrict__ min_int, int min_bytes, __half *__restrict__ scale,
    unsigned long long *__restrict__ ghist, int *__restrict__ status) {
    __shared__ float red[2][8];
    __shared__ unsigned int shist[8 * 256];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int UNITS_PER_CTA = 256 / GROUP;
    const long long u = (long long)blockIdx.x * UNITS_PER_CTA + (GROUP == 256 ? 0 : warp);
    const int gl = GROUP == 256 ? tid : lane;          // index inside the group
    if (ghist) hist_clear(shist, tid, 256);
    const bool active = u < n_units;
    const long long chunks = ulen / 8;
    const __half *xu = x + u * ulen;
    float mn = INFINITY, mx = -INFINITY;
    if (active)
        for (long long k = gl; k < chunks; k += GROUP) {
            uint4 v = *reinterpret_cast<const uint4 *>(xu + k * 8);
            minmax8(v, mn, mx);
        }
    mn = -kvc_warp_max(-mn); mx = kvc_warp_max(mx);
    if (GROUP == 256) {
        if (lane == 0) { red[0][warp] = mn; red[1][warp] = mx; }
        __syncthreads();
        mn = red[0][0]; mx = red[1][0];
#pragma unroll
        for (int w = 1; w < 8; w++) { mn = fminf(mn, red[0][w]); mx = fmaxf(mx, red[1][w]); }
    }
    int flags = 0;
    if (active) {
        __half sc;
        UnitParam p = unit_param(mn, mx, rel, &sc, &flags);
        if (gl == 0) { scale[u] = sc; store_min(min_int, min_bytes, u, p.mi, &flags); }
        const bool small = small_min_int(p.mi);
        const __half2 mi2 = __float2half2_rn(p.mi);
        for (long long k = gl; k < chunks; k += GROUP) {
            uint4 v = *reinterpret_cast<const uint4 *>(xu + k * 8);
            uint2 o = quant_eight<0>(v, &p, small, &mi2, &flags, ghist ? shist + warp * 256 : nullptr);
            *reinterpret_cast<uint2 *>(codes + u * ulen + k * 8) = o;
        }
    }
    if (flags) atomicOr(status, flags);
    if (ghist) hist_flush(shist, ghist, tid, 256);
}

// Units of CH * WARPS * 256 elements held in registers between the min/max pass and the quantising
// pass (CH 16-byte chunks per thread).  WARPS = 1: a warp per unit, 8 units per 256-thread CTA, nothing
// but shuffles shared.  WARPS > 1: a CTA of WARPS warps per unit, one barrier to join their extremes.
template <int CH, int WARPS>
__global__ void __launch_bounds__(WARPS == 1 ? 256 : WARPS * 32) quant_contig_reg_kernel(
    const __half *__restrict__ x, long long n_units, float rel,
    uint8_t *__restrict__ codes, void *__restrict__ min_int, int min_bytes, __half *__restrict__ scale,
    unsigned long long *__restrict__ ghist, int *__restrict__ status) {
    constexpr int NT = WARPS == 1 ? 256 : WARPS * 32;       // threads per CTA
    constexpr int GT = WARPS * 32;                          // threads per unit
    constexpr long long ULEN = (long long)CH * GT * 8;
    __shared__ unsigned int shist[(NT / 32) * 256];
    __shared__ float red[2][WARPS];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gt = WARPS == 1 ? lane : tid;                 // index inside the unit
    if (ghist) hist_clear(shist, tid, NT);
    int flags = 0;
    const long long u_step = WARPS == 1 ? (long long)gridDim.x * 8 : (long long)gridDim.x;
    // every thread of the CTA runs the same number of rounds (the barrier below), units past the end idle
    for (long long u0 = WARPS == 1 ? (long long)blockIdx.x * 8 : (long long)blockIdx.x; u0 < n_units; u0 += u_step) {
    const long long u = WARPS == 1 ? u0 + warp : u0;
    const bool active = u < n_units;
    const __half *xu = x + u * ULEN;
    uint4 v[CH];
    float mn = INFINITY, mx = -INFINITY;
    if (active) {
#pragma unroll
        for (int i = 0; i < CH; i++) v[i] = *reinterpret_cast<const uint4 *>(xu + (long long)(i * GT + gt) * 8);
#pragma unroll
        for (int i = 0; i < CH; i++) minmax8(v[i], mn, mx);
    }
    mn = -kvc_warp_max(-mn); mx = kvc_warp_max(mx);
    if (WARPS > 1) {
        if (lane == 0) { red[0][warp] = mn; red[1][warp] = mx; }
        __syncthreads();
        mn = red[0][0]; mx = red[1][0];
#pragma unroll
        for (int w = 1; w < WARPS; w++) { mn = fminf(mn, red[0][w]); mx = fmaxf(mx, red[1][w]); }
    }
    if (active) {
        __half sc;
        const UnitParam p = unit_param(mn, mx, rel, &sc, &flags);
        if (gt == 0) { scale[u] = sc; store_min(min_int, min_bytes, u, p.mi, &flags); }
        const bool small = small_min_int(p.mi);
        const __half2 mi2 = __float2half2_rn(p.mi);
#pragma unroll
        for (int i = 0; i < CH; i++) {
            const uint2 o = quant_eight<0>(v[i], &p, small, &mi2, &flags, ghist ? shist + warp * 256 : nullptr);
            *reinterpret_cast<uint2 *>(codes + u * ULEN + (long long)(i * GT + gt) * 8) = o;
        }
    }
    if (WARPS > 1) __syncthreads();                         // the extremes are read before the next unit's
    }
    if (flags) atomicOr(status, flags);
    if (ghist) hist_flush(shist, ghist, tid, NT);
}

// ---- BlockQuant: one unit per token block (x sequence), far larger than a CTA ------------------
// Three launches: per-row min/max folded into the unit with atomics on order-preserving keys,
// a per-unit finalise, and the elementwise pass.  A row is one (token, b): H*D contiguous values.
// The same three serve the two-call form (kvc_quant_minmax / kvc_quantize_ranged) for every unit made of
// whole rows: `blk` is then the unit's token divisor (the block for BlockQuant, 1 for TokenQuant).
__device__ __forceinline__ unsigned int half_key(float f) {      // monotone in the value
    unsigned int h = __half_as_ushort(__float2half_rn(f));
    return (h & 0x8000u) ? (~h & 0xffffu) : (h | 0x8000u);
}
__device__ __forceinline__ float key_half(unsigned int k) {
    unsigned int h = (k & 0x8000u) ? (k & 0x7fffu) : (~k & 0xffffu);
    return __half2float(__ushort_as_half((unsigned short)h));
}

__global__ void __launch_bounds__(256) quant_block_minmax_kernel(
    const __half *__restrict__ x, long long B, long long row_len, int blk, int batch_shared,
    unsigned int *__restrict__ ws) {
    __shared__ float red[2][8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long row = blockIdx.x, t = row / B, b = row % B;
    const long long u = batch_shared ? t / blk : (t / blk) * B + b;
    const __half *xr = x + row * row_len;
    float mn = INFINITY, mx = -INFINITY;
    for (long long k = tid; k < row_len / 8; k += 256) {
        uint4 v = *reinterpret_cast<const uint4 *>(xr + k * 8);
        minmax8(v, mn, mx);
    }
    mn = -kvc_warp_max(-mn); mx = kvc_warp_max(mx);
    if (lane == 0) { red[0][warp] = mn; red[1][warp] = mx; }
    __syncthreads();
    if (tid == 0) {
#pragma unroll
        for (int w = 1; w < 8; w++) { mn = fminf(mn, red[0][w]); mx = fmaxf(mx, red[1][w]); }
        atomicMax(&ws[2 * u], 0xffffu - half_key(mn));     // max of the inverted key == min of the value
        atomicMax(&ws[2 * u + 1], half_key(mx));
    }
}

// keys -> the units' extremes as fp16 (what ranks exchange when a unit spans the heads of several of them)
__global__ void quant_minmax_export_kernel(const unsigned int *__restrict__ ws, long long n_units,
                                           __half *__restrict__ mn_out, __half *__restrict__ mx_out) {
    long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= n_units) return;
    mn_out[u] = __float2half_rn(key_half(0xffffu - ws[2 * u]));
    mx_out[u] = __float2half_rn(key_half(ws[2 * u + 1]));
}

// mn_in / mx_in (optional): the units' extremes given by the caller instead of the keys in ws
__global__ void quant_block_finalize_kernel(unsigned int *__restrict__ ws, long long n_units, float rel,
                                            void *__restrict__ min_int, int min_bytes,
                                            __half *__restrict__ scale, int *__restrict__ status,
                                            const __half *__restrict__ mn_in, const __half *__restrict__ mx_in) {
    long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= n_units) return;
    float mn, mx;
    if (mn_in) { mn = __half2float(mn_in[u]); mx = __half2float(mx_in[u]); }
    else { mn = key_half(0xffffu - ws[2 * u]); mx = key_half(ws[2 * u + 1]); }
    int flags = 0;
    __half sc;
    UnitParam p = unit_param(mn, mx, rel, &sc, &flags);
    scale[u] = sc;
    store_min(min_int, min_bytes, u, p.mi, &flags);
    // leave the unit parameters where the elementwise pass reads them
    ws[2 * u] = __float_as_uint(p.sf);
    ws[2 * u + 1] = __float_as_uint(p.mi);
    if (flags) atomicOr(status, flags);
}

__global__ void __launch_bounds__(256) quant_block_apply_kernel(
    const __half *__restrict__ x, long long B, long long row_len, int blk, int batch_shared,
    const unsigned int *__restrict__ ws, uint8_t *__restrict__ codes,
    unsigned long long *__restrict__ ghist, int *__restrict__ status) {
    __shared__ unsigned int shist[8 * 256];
    const int tid = threadIdx.x;
    const long long row = blockIdx.x, t = row / B, b = row % B;
    const long long u = batch_shared ? t / blk : (t / blk) * B + b;
    if (ghist) hist_clear(shist, tid, 256);
    UnitParam p;
    p.sf = __uint_as_float(ws[2 * u]); p.mi = __uint_as_float(ws[2 * u + 1]);
    p.rcp = (p.sf == 0.0f || p.sf != p.sf) ? 0.0f : __frcp_rn(p.sf);
    int flags = 0;
    const bool small = small_min_int(p.mi);
    const __half2 mi2 = __float2half2_rn(p.mi);
    for (long long k = tid; k < row_len / 8; k += 256) {
        uint4 v = *reinterpret_cast<const uint4 *>(x + row * row_len + k * 8);
        uint2 o = quant_eight<0>(v, &p, small, &mi2, &flags, ghist ? shist + (tid >> 5) * 256 : nullptr);
        *reinterpret_cast<uint2 *>(codes + row * row_len + k * 8) = o;
    }
    if (flags) atomicOr(status, flags);
    if (ghist) hist_flush(shist, ghist, tid, 256);
}

// ---- dequantise: fp16((code + min_int) * scale), models/cache/kvcomp_encode.py:146 -------------
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t *__restrict__ codes, kvc_qmeta_dev m,
                                                      long long rows, long long B, long long H, int D,
                                                      __half *__restrict__ out) {
    // one thread = 8 consecutive channels of one (t, b, h) row
    const long long per_row = D / 8;
    long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= rows * per_row) return;
    const long long row = i / per_row; const int c0 = (int)(i % per_row) * 8;
    const long long h = row % H, b = (row / H) % B, t = row / (H * B);
    const long long ub = kvc_tok_unit(t, m.tok_div) * m.sj + b * m.sb + h * m.sh;
    uint2 cv = *reinterpret_cast<const uint2 *>(codes + row * D + c0);
    const uint8_t *cb = reinterpret_cast<const uint8_t *>(&cv);
    uint4 o; __half *oh = reinterpret_cast<__half *>(&o);
#pragma unroll
    for (int k = 0; k < 8; k++) {
        long long u = ub + (long long)(c0 + k) * m.sc;
        float s = __half2float(__float2half_rn((float)((int)cb[k] + kvc_load_min(m, u))));
        oh[k] = __float2half_rn(__fmul_rn(s, __half2float(m.scale[u])));
    }
    *reinterpret_cast<uint4 *>(out + row * D + c0) = o;
}

// ---- dense q.k over uncompressed K (kernels.cu:1192-1219), fp32 accumulation --------------------
// One warp per (token, head) row of 128 fp16 values; lane = 4 channels.
__global__ void __launch_bounds__(256) k_matvec_kernel(const __half *__restrict__ k, const __half *__restrict__ q,
                                                       __half *__restrict__ out, long long rows, long long H) {
    const int lane = threadIdx.x & 31;
    long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    uint2 kv = *reinterpret_cast<const uint2 *>(k + row * 128 + lane * 4);
    uint2 qv = *reinterpret_cast<const uint2 *>(q + (row % H) * 128 + lane * 4);
    const __half2 *k2 = reinterpret_cast<const __half2 *>(&kv), *q2 = reinterpret_cast<const __half2 *>(&qv);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 2; i++) {
        float2 a = __half22float2(k2[i]), c = __half22float2(q2[i]);
        acc = fmaf(a.x, c.x, acc); acc = fmaf(a.y, c.y, acc);
    }
    acc = kvc_warp_sum(acc);
    if (lane == 0) out[row] = __float2half_rn(acc);
}

}  // namespace

extern "C" int kvc_qmeta_make(int mode, int batch_shared, int64_t T, int64_t B, int64_t H, int64_t D,
                              int64_t block, kvc_qmeta *q, int64_t *n_units) {
    KVC_REQUIRE(q != nullptr, "kvc_qmeta_make: q is null");
    KVC_REQUIRE(T >= 0 && B > 0 && H > 0 && D > 0, "kvc_qmeta_make: bad shape");
    const int64_t nb = batch_shared ? 1 : B;
    int64_t n = 0;
    q->sj = q->sb = q->sh = q->sc = 0;
    switch (mode) {
    case KVC_MODE_BLOCK:
        KVC_REQUIRE(block > 0 && T % block == 0, "kvc_qmeta_make: T=%lld is not a multiple of block=%lld", (long long)T, (long long)block);
        q->tok_div = (int32_t)block; q->sj = nb; q->sb = batch_shared ? 0 : 1; n = (T / block) * nb; break;
    case KVC_MODE_CHANNEL:
        KVC_REQUIRE(block > 0 && T % block == 0, "kvc_qmeta_make: T=%lld is not a multiple of block=%lld", (long long)T, (long long)block);
        q->tok_div = (int32_t)block; q->sj = B * H * D; q->sb = H * D; q->sh = D; q->sc = 1; n = (T / block) * B * H * D; break;
    case KVC_MODE_TOKEN:
        q->tok_div = 1; q->sj = nb; q->sb = batch_shared ? 0 : 1; n = T * nb; break;
    case KVC_MODE_VECTOR:
        q->tok_div = 1; q->sj = B * H; q->sb = H; q->sh = 1; n = T * B * H; break;
    default:
        KVC_REQUIRE(false, "kvc_qmeta_make: unknown mode %d", mode);
    }
    if (n_units) *n_units = n;
    return KVC_OK;
}

extern "C" int64_t kvc_quantize_workspace(int mode, int batch_shared, int64_t T, int64_t B, int64_t block) {
    if (mode != KVC_MODE_BLOCK || block <= 0) return 0;
    return (T / block) * (batch_shared ? 1 : B) * 8;
}

extern "C" int kvc_quantize(const void *x, int64_t T, int64_t B, int64_t H, int64_t D,
                            int mode, int batch_shared, int64_t block, float rel,
                            uint8_t *codes, void *min_int, int min_bytes, void *scale,
                            unsigned long long *hist, void *workspace, int64_t workspace_bytes,
                            int32_t *status, kvc_stream_t stream) {
    KVC_REQUIRE(x && codes && min_int && scale && status, "kvc_quantize: null pointer");
    KVC_REQUIRE(T >= 0 && B > 0 && H > 0 && D > 0 && D % 8 == 0, "kvc_quantize: bad shape T=%lld B=%lld H=%lld D=%lld", (long long)T, (long long)B, (long long)H, (long long)D);
    KVC_REQUIRE(min_bytes == 1 || min_bytes == 2, "kvc_quantize: min_bytes must be 1 or 2");
    KVC_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(codes) & 7) == 0,
                "kvc_quantize: x must be 16-byte and codes 8-byte aligned");
    if (T == 0) return KVC_OK;
    cudaStream_t s = kvc_cu(stream);
    const __half *xh = reinterpret_cast<const __half *>(x);
    __half *sc = reinterpret_cast<__half *>(scale);
    switch (mode) {
    case KVC_MODE_CHANNEL: {
        KVC_REQUIRE(D == 128, "kvc_quantize: ChannelQuant needs head_dim 128");
        KVC_REQUIRE(block > 0 && T % block == 0, "kvc_quantize: T=%lld is not a multiple of block=%lld", (long long)T, (long long)block);
        long long tiles = (T / block) * B * H;
        KVC_REQUIRE(tiles < (1ll << 31), "kvc_quantize: too many tiles");
        quant_channel_kernel<<<(unsigned)tiles, 128, 0, s>>>(xh, B, H, (int)block, rel, codes, min_int, min_bytes, sc, hist, status);
        break;
    }
    case KVC_MODE_TOKEN:
    case KVC_MODE_VECTOR: {
        long long ulen = mode == KVC_MODE_VECTOR ? D : (batch_shared ? B * H * D : H * D);
        long long n_units = T * B * H * D / ulen;
#define KVC_QR(CH_, W_) quant_contig_reg_kernel<CH_, W_><<<(unsigned)std::min<long long>((W_) == 1 ? (n_units + 7) / 8 : n_units, (long long)kvc_sm_count() * (2048 / ((W_) == 1 ? 256 : (W_) * 32))), (W_) == 1 ? 256 : (W_) * 32, 0, s>>>( \
        xh, n_units, rel, codes, min_int, min_bytes, sc, hist, status)
        if (n_units < (1ll << 31) && (ulen == 256 || ulen == 512 || ulen == 1024 || ulen == 2048 || ulen == 4096 || ulen == 8192)) {
            switch (ulen) {
            case 256: KVC_QR(1, 1); break;
            case 512: KVC_QR(2, 1); break;
            case 1024: KVC_QR(4, 1); break;
            case 2048: KVC_QR(4, 2); break;
            case 4096: KVC_QR(4, 4); break;
            default: KVC_QR(4, 8); break;
            }
        } else
#undef KVC_QR
        if (ulen >= 2048) {
            KVC_REQUIRE(n_units < (1ll << 31), "kvc_quantize: too many units");
            quant_contig_kernel<256><<<(unsigned)n_units, 256, 0, s>>>(xh, n_units, ulen, rel, codes, min_int, min_bytes, sc, hist, status);
        } else {
            long long ctas = (n_units + 7) / 8;
            KVC_REQUIRE(ctas < (1ll << 31), "kvc_quantize: too many units");
            quant_contig_kernel<32><<<(unsigned)ctas, 256, 0, s>>>(xh, n_units, ulen, rel, codes, min_int, min_bytes, sc, hist, status);
        }
        break;
    }
    case KVC_MODE_BLOCK: {
        KVC_REQUIRE(block > 0 && T % block == 0, "kvc_quantize: T=%lld is not a multiple of block=%lld", (long long)T, (long long)block);
        long long n_units = (T / block) * (batch_shared ? 1 : B);
        KVC_REQUIRE(workspace && workspace_bytes >= n_units * 8, "kvc_quantize: BlockQuant needs %lld bytes of workspace", n_units * 8);
        KVC_REQUIRE(T * B < (1ll << 31), "kvc_quantize: too many rows");
        unsigned int *ws = reinterpret_cast<unsigned int *>(workspace);
        KVC_CUDA_OK(cudaMemsetAsync(ws, 0, n_units * 8, s));
        quant_block_minmax_kernel<<<(unsigned)(T * B), 256, 0, s>>>(xh, B, H * D, (int)block, batch_shared, ws);
        quant_block_finalize_kernel<<<(unsigned)((n_units + 127) / 128), 128, 0, s>>>(ws, n_units, rel, min_int, min_bytes, sc, status, nullptr, nullptr);
        quant_block_apply_kernel<<<(unsigned)(T * B), 256, 0, s>>>(xh, B, H * D, (int)block, batch_shared, ws, codes, hist, status);
        break;
    }
    default:
        KVC_REQUIRE(false, "kvc_quantize: unknown mode %d", mode);
    }
    KVC_LAUNCH_OK();
    return KVC_OK;
}

extern "C" int kvc_dequant(const uint8_t *codes, const kvc_qmeta *q, int64_t T, int64_t B, int64_t H, int64_t D,
                           void *out, kvc_stream_t stream) {
    KVC_REQUIRE(codes && q && q->min_int && q->scale && out, "kvc_dequant: null pointer");
    KVC_REQUIRE(D > 0 && D % 8 == 0 && q->tok_div > 0, "kvc_dequant: bad shape");
    KVC_REQUIRE(q->min_bytes == 1 || q->min_bytes == 2, "kvc_dequant: min_bytes must be 1 or 2");
    long long rows = T * B * H, n = rows * (D / 8);
    if (n == 0) return KVC_OK;
    dequant_kernel<<<(unsigned)((n + 255) / 256), 256, 0, kvc_cu(stream)>>>(codes, kvc_to_dev(*q), rows, B, H, (int)D,
                                                                            reinterpret_cast<__half *>(out));
    KVC_LAUNCH_OK();
    return KVC_OK;
}

extern "C" int kvc_k_matvec(const void *k, const void *q, void *out, int64_t ctx, int64_t H, kvc_stream_t stream) {
    KVC_REQUIRE(k && q && out, "kvc_k_matvec: null pointer");
    KVC_REQUIRE(ctx >= 0 && H > 0, "kvc_k_matvec: bad shape");
    long long rows = ctx * H;
    if (rows == 0) return KVC_OK;
    k_matvec_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, kvc_cu(stream)>>>(
        reinterpret_cast<const __half *>(k), reinterpret_cast<const __half *>(q), reinterpret_cast<__half *>(out), rows, H);
    KVC_LAUNCH_OK();
    return KVC_OK;
}

// ---- rotary embedding of new keys on their way into the cache -------------------------------------
// models/cache/kvcomp_quant.py:43-48 rotates the new keys (utils/compute.py:25-33: t * cos + rotate_half(t) * sin,
// every op a rounded fp16 tensor op) before they enter the recent window; the cache keeps tokens token-major.
// One pass does both: x [B, H, t, D] -> out [t, B, H, D], same bits as torch's four ops and the transposing copy.
// blockIdx.y = 1 (kvc_kv_store): the same rows of a second tensor xv -> outv without rotation (the new values)
__global__ void __launch_bounds__(256) rope_store_kernel(const __half *__restrict__ x, const __half *__restrict__ cs,
                                                         const __half *__restrict__ sn, __half *__restrict__ out,
                                                         long long B, long long H, long long t, int D, long long cs_bstride,
                                                         const __half *__restrict__ xv, __half *__restrict__ outv) {
    // A kernel launched behind this one with programmatic stream serialisation (the fused attention) may set up
    // while these few rows are written: it touches them only after its own grid-dependency wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (blockIdx.y == 1) { x = xv; out = outv; cs = nullptr; }
    const int per_row = D / 16;                                  // a thread: 8 channels of the lower half and their partners
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= t * B * H * per_row) return;
    const int c0 = (int)(i % per_row) * 8, half = D / 2;
    const long long row = i / per_row, h = row % H, b = (row / H) % B, tok = row / (H * B);
    const __half *xr = x + ((b * H + h) * t + tok) * D;
    __half *orow = out + ((tok * B + b) * H + h) * D;
    const uint4 xa = *reinterpret_cast<const uint4 *>(xr + c0), xb = *reinterpret_cast<const uint4 *>(xr + c0 + half);
    if (cs == nullptr) {                                         // no rotation (values): the transposition alone
        *reinterpret_cast<uint4 *>(orow + c0) = xa;
        *reinterpret_cast<uint4 *>(orow + c0 + half) = xb;
        return;
    }
    const __half *cr = cs + b * cs_bstride + tok * D, *sr = sn + b * cs_bstride + tok * D;
    const uint4 ca = *reinterpret_cast<const uint4 *>(cr + c0), cb = *reinterpret_cast<const uint4 *>(cr + c0 + half);
    const uint4 sa = *reinterpret_cast<const uint4 *>(sr + c0), sb = *reinterpret_cast<const uint4 *>(sr + c0 + half);
    const __half *x1 = reinterpret_cast<const __half *>(&xa), *x2 = reinterpret_cast<const __half *>(&xb);
    const __half *c1 = reinterpret_cast<const __half *>(&ca), *c2 = reinterpret_cast<const __half *>(&cb);
    const __half *s1 = reinterpret_cast<const __half *>(&sa), *s2 = reinterpret_cast<const __half *>(&sb);
    uint4 oa, ob;
    __half *o1 = reinterpret_cast<__half *>(&oa), *o2 = reinterpret_cast<__half *>(&ob);
    auto mul = [](__half a, __half b2) { return __half2float(__float2half_rn(__fmul_rn(__half2float(a), __half2float(b2)))); };
#pragma unroll
    for (int k = 0; k < 8; k++) {
        // rotate_half: the lower half meets -x2, the upper half x1
        o1[k] = __float2half_rn(__fadd_rn(mul(x1[k], c1[k]), mul(__hneg(x2[k]), s1[k])));
        o2[k] = __float2half_rn(__fadd_rn(mul(x2[k], c2[k]), mul(x1[k], s2[k])));
    }
    *reinterpret_cast<uint4 *>(orow + c0) = oa;
    *reinterpret_cast<uint4 *>(orow + c0 + half) = ob;
}

extern "C" int kvc_rope_store(const void *x, const void *cos_, const void *sin_, void *out, int64_t B, int64_t H, int64_t t,
                              int64_t D, int64_t cos_batch_stride, kvc_stream_t stream) {
    KVC_REQUIRE(x && out && ((cos_ == nullptr) == (sin_ == nullptr)), "kvc_rope_store: null pointer");
    KVC_REQUIRE(B > 0 && H > 0 && t >= 0 && D > 0 && D % 16 == 0, "kvc_rope_store: bad shape");
    KVC_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(cos_) | reinterpret_cast<uintptr_t>(sin_) |
                  reinterpret_cast<uintptr_t>(out)) & 15) == 0, "kvc_rope_store: pointers must be 16-byte aligned");
    KVC_REQUIRE(cos_batch_stride == 0 || cos_batch_stride == t * D, "kvc_rope_store: cos/sin must be [B, t, D] or [1, t, D]");
    const long long n = t * B * H * (D / 16);
    if (n == 0) return KVC_OK;
    KVC_REQUIRE((n + 255) / 256 < (1ll << 31), "kvc_rope_store: too many elements");
    rope_store_kernel<<<(unsigned)((n + 255) / 256), 256, 0, kvc_cu(stream)>>>(
        reinterpret_cast<const __half *>(x), reinterpret_cast<const __half *>(cos_), reinterpret_cast<const __half *>(sin_),
        reinterpret_cast<__half *>(out), B, H, t, (int)D, cos_batch_stride, nullptr, nullptr);
    KVC_LAUNCH_OK();
    return KVC_OK;
}

extern "C" int kvc_kv_store(const void *k, const void *v, const void *cos_, const void *sin_, void *kout, void *vout,
                            int64_t B, int64_t H, int64_t t, int64_t D, int64_t cos_batch_stride, kvc_stream_t stream) {
    KVC_REQUIRE(k && v && cos_ && sin_ && kout && vout, "kvc_kv_store: null pointer");
    KVC_REQUIRE(B > 0 && H > 0 && t >= 0 && D > 0 && D % 16 == 0, "kvc_kv_store: bad shape");
    KVC_REQUIRE(((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(cos_) |
                  reinterpret_cast<uintptr_t>(sin_) | reinterpret_cast<uintptr_t>(kout) | reinterpret_cast<uintptr_t>(vout)) & 15) == 0,
                "kvc_kv_store: pointers must be 16-byte aligned");
    KVC_REQUIRE(cos_batch_stride == 0 || cos_batch_stride == t * D, "kvc_kv_store: cos/sin must be [B, t, D] or [1, t, D]");
    const long long n = t * B * H * (D / 16);
    if (n == 0) return KVC_OK;
    KVC_REQUIRE((n + 255) / 256 < (1ll << 31), "kvc_kv_store: too many elements");
    rope_store_kernel<<<dim3((unsigned)((n + 255) / 256), 2), 256, 0, kvc_cu(stream)>>>(
        reinterpret_cast<const __half *>(k), reinterpret_cast<const __half *>(cos_), reinterpret_cast<const __half *>(sin_),
        reinterpret_cast<__half *>(kout), B, H, t, (int)D, cos_batch_stride,
        reinterpret_cast<const __half *>(v), reinterpret_cast<__half *>(vout));
    KVC_LAUNCH_OK();
    return KVC_OK;
}

// ---- the quantiser in two calls: extremes first, codes later --------------------------------------
// For units made of whole (token, sequence) rows -- BlockQuant and TokenQuant, whose units span the heads
// (models/cache/kvcomp_encode.py:10-13, utils/compute.py:138-143).  When the heads of a cache are split
// over several GPUs, every rank takes the extremes of its own heads, the ranks exchange them (elementwise
// min and max), and every rank quantises with the joint extremes: same scale, min_int and codes as one GPU
// holding all heads would produce.
static int ranged_units(int mode, int batch_shared, int64_t T, int64_t B, int64_t block, long long *n_units, int *tok_div) {
    KVC_REQUIRE(mode == KVC_MODE_BLOCK || mode == KVC_MODE_TOKEN, "units of mode %d do not span heads: use kvc_quantize", mode);
    if (mode == KVC_MODE_BLOCK) KVC_REQUIRE(block > 0 && T % block == 0, "T=%lld is not a multiple of block=%lld", (long long)T, (long long)block);
    *tok_div = mode == KVC_MODE_BLOCK ? (int)block : 1;
    *n_units = (T / *tok_div) * (batch_shared ? 1 : B);
    return KVC_OK;
}

extern "C" int kvc_quant_minmax(const void *x, int64_t T, int64_t B, int64_t H, int64_t D, int mode, int batch_shared,
                                int64_t block, void *mn_out, void *mx_out, void *workspace, int64_t workspace_bytes,
                                kvc_stream_t stream) {
    KVC_REQUIRE(x && mn_out && mx_out, "kvc_quant_minmax: null pointer");
    KVC_REQUIRE(T >= 0 && B > 0 && H > 0 && D > 0 && (H * D) % 8 == 0, "kvc_quant_minmax: bad shape");
    KVC_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0, "kvc_quant_minmax: x must be 16-byte aligned");
    long long n_units; int tok_div;
    if (int rc = ranged_units(mode, batch_shared, T, B, block, &n_units, &tok_div)) return rc;
    if (T == 0) return KVC_OK;
    KVC_REQUIRE(workspace && workspace_bytes >= n_units * 8, "kvc_quant_minmax: needs %lld bytes of workspace", n_units * 8);
    KVC_REQUIRE(T * B < (1ll << 31), "kvc_quant_minmax: too many rows");
    cudaStream_t s = kvc_cu(stream);
    unsigned int *ws = reinterpret_cast<unsigned int *>(workspace);
    KVC_CUDA_OK(cudaMemsetAsync(ws, 0, n_units * 8, s));
    quant_block_minmax_kernel<<<(unsigned)(T * B), 256, 0, s>>>(reinterpret_cast<const __half *>(x), B, H * D, tok_div, batch_shared, ws);
    quant_minmax_export_kernel<<<(unsigned)((n_units + 127) / 128), 128, 0, s>>>(ws, n_units, reinterpret_cast<__half *>(mn_out),
                                                                                  reinterpret_cast<__half *>(mx_out));
    KVC_LAUNCH_OK();
    return KVC_OK;
}

extern "C" int kvc_quantize_ranged(const void *x, int64_t T, int64_t B, int64_t H, int64_t D, int mode, int batch_shared,
                                   int64_t block, float rel, const void *mn_in, const void *mx_in,
                                   uint8_t *codes, void *min_int, int min_bytes, void *scale, unsigned long long *hist,
                                   void *workspace, int64_t workspace_bytes, int32_t *status, kvc_stream_t stream) {
    KVC_REQUIRE(x && mn_in && mx_in && codes && min_int && scale && status, "kvc_quantize_ranged: null pointer");
    KVC_REQUIRE(T >= 0 && B > 0 && H > 0 && D > 0 && (H * D) % 8 == 0, "kvc_quantize_ranged: bad shape");
    KVC_REQUIRE(min_bytes == 1 || min_bytes == 2, "kvc_quantize_ranged: min_bytes must be 1 or 2");
    KVC_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(codes) & 7) == 0,
                "kvc_quantize_ranged: x must be 16-byte and codes 8-byte aligned");
    long long n_units; int tok_div;
    if (int rc = ranged_units(mode, batch_shared, T, B, block, &n_units, &tok_div)) return rc;
    if (T == 0) return KVC_OK;
    KVC_REQUIRE(workspace && workspace_bytes >= n_units * 8, "kvc_quantize_ranged: needs %lld bytes of workspace", n_units * 8);
    KVC_REQUIRE(T * B < (1ll << 31), "kvc_quantize_ranged: too many rows");
    cudaStream_t s = kvc_cu(stream);
    unsigned int *ws = reinterpret_cast<unsigned int *>(workspace);
    quant_block_finalize_kernel<<<(unsigned)((n_units + 127) / 128), 128, 0, s>>>(
        ws, n_units, rel, min_int, min_bytes, reinterpret_cast<__half *>(scale), status,
        reinterpret_cast<const __half *>(mn_in), reinterpret_cast<const __half *>(mx_in));
    quant_block_apply_kernel<<<(unsigned)(T * B), 256, 0, s>>>(reinterpret_cast<const __half *>(x), B, H * D, tok_div, batch_shared,
                                                               ws, codes, hist, status);
    KVC_LAUNCH_OK();
    return KVC_OK;
}
