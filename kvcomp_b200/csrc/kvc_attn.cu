// Fused decompress + mat-vec kernels: q.K^T scores, P.V partials, and the one-pass decode
// attention (q.K^T -> online softmax -> P.V) straight from the compressed streams.
//
// Reference kernels restated: huffman_decode_and_mat_vec_mul (kernels.cu:721-776),
// v_huffman_decode_and_mat_vec_mul (kernels.cu:778-861); attention semantics of
// eager_attention_forward (models/llama.py:211-234).
//
// Work layout (all three kernels): CTA = 256 threads working on 256 tokens of one (b, kv head).
//   K phase: thread = token; its vector holds the token's 128 channel codes.
//            score = sum_c code_c * w[c] + zp, with w[c] = q[c]*scale[c] staged per 64-token block
//            (dequantisation folded into the weights, the min_int term summed once per block).
//   V phase: thread = (128-token group, channel); its vector holds 128 tokens of that channel.
//            out[ch] = sum_t code_t * ps[t] + zpv, with ps[t] = p[t]*scale[t] staged per group.
// Both phases are "decode 128 symbols and dot them with a shared 128-vector", so they share one
// decoder.  With grouped-query attention the G query heads of a KV head share every decode: the
// weights are stored [position][G] and each symbol feeds G accumulators.
// Accumulation is fp32 throughout (the reference accumulates in fp16).
#include <math_constants.h>

#include "kvc_decode.cuh"

namespace {

constexpr int SLOT_BYTES = 8192 + 32;
constexpr int WROW = 132;                 // weight rows: 128 positions + zeroed overrun
constexpr int NTHR = 256;

struct CacheDev {
    const uint8_t *encoded;
    long long encoded_bytes;
    const uint2 *block_info;
    const uint16_t *thread_info;
    const void *book;
    kvc_qmeta_dev q;
};

CacheDev to_dev(const kvc_cache &c) {
    CacheDev d;
    d.encoded = c.encoded; d.encoded_bytes = c.encoded_bytes;
    d.block_info = reinterpret_cast<const uint2 *>(c.block_info); d.thread_info = c.thread_info;
    d.book = c.book; d.q = kvc_to_dev(c.q);
    return d;
}

// acc[g] += f0*w[c][g] + f1*w[c+1][g] + f2*w[c+2][g]
template <int G> __device__ __forceinline__ void fma3(float (&acc)[G], const float *wp, float f0, float f1, float f2);
template <> __device__ __forceinline__ void fma3<1>(float (&acc)[1], const float *wp, float f0, float f1, float f2) {
    acc[0] = fmaf(f0, wp[0], fmaf(f1, wp[1], fmaf(f2, wp[2], acc[0])));
}
template <> __device__ __forceinline__ void fma3<2>(float (&acc)[2], const float *wp, float f0, float f1, float f2) {
    float2 a = *reinterpret_cast<const float2 *>(wp), b = *reinterpret_cast<const float2 *>(wp + 2),
           c = *reinterpret_cast<const float2 *>(wp + 4);
    acc[0] = fmaf(f0, a.x, fmaf(f1, b.x, fmaf(f2, c.x, acc[0])));
    acc[1] = fmaf(f0, a.y, fmaf(f1, b.y, fmaf(f2, c.y, acc[1])));
}
template <> __device__ __forceinline__ void fma3<4>(float (&acc)[4], const float *wp, float f0, float f1, float f2) {
    float4 a = *reinterpret_cast<const float4 *>(wp), b = *reinterpret_cast<const float4 *>(wp + 4),
           c = *reinterpret_cast<const float4 *>(wp + 8);
    acc[0] = fmaf(f0, a.x, fmaf(f1, b.x, fmaf(f2, c.x, acc[0])));
    acc[1] = fmaf(f0, a.y, fmaf(f1, b.y, fmaf(f2, c.y, acc[1])));
    acc[2] = fmaf(f0, a.z, fmaf(f1, b.z, fmaf(f2, c.z, acc[2])));
    acc[3] = fmaf(f0, a.w, fmaf(f1, b.w, fmaf(f2, c.w, acc[3])));
}

// decode the thread's vector and dot it with the weight rows at w ([WROW][G])
template <int G>
__device__ __forceinline__ bool decode_dot(const uint8_t *slot, uint32_t byte_pos, const KvcBookSmem &book,
                                           const float *w, float (&acc)[G]) {
    return kvc_decode_vector(reinterpret_cast<const uint32_t *>(slot), byte_pos, SLOT_BYTES / 4 - 1, book,
                             [&](uint32_t s0, uint32_t s1, uint32_t s2, uint32_t, int c) {
                                 fma3<G>(acc, w + c * G, (float)s0, (float)s1, (float)s2);
                             });
}

// stage the block `blk` of cache `kc` into `slot` with the 64 threads of a sub-group
__device__ __forceinline__ bool stage(const CacheDev &kc, long long blk, uint8_t *slot, uint32_t *lead, int v) {
    const uint2 bi = kc.block_info[blk];
    const uint32_t nbytes = bi.y & 0xffffu;
    if (nbytes == 0 || nbytes > 8191u || (long long)bi.x + nbytes > kc.encoded_bytes) { *lead = 0; return false; }
    *lead = kvc_stage_block(slot, kc.encoded, kc.encoded_bytes, bi.x, nbytes, v, 64);
    return true;
}

__device__ __forceinline__ uint32_t vec_start(const uint16_t *thread_info, long long blk, int v) {
    return v ? (uint32_t)(thread_info[blk * 64 + v - 1] >> 3) : 0u;
}

// K weights of the 4 blocks of a 256-token tile: w[sub][c][g] and zp[sub][g].
// Units that depend on the channel (sc != 0) need tok_div % 64 == 0 so that a block shares them;
// otherwise scale and min_int are per-token scalars applied after the dot product.
template <int G>
__device__ __forceinline__ void k_weights(float *w, float *zp, const float *qf, const kvc_qmeta_dev &m,
                                          long long tok0, long long T, long long b, long long h, int tid) {
    for (int idx = tid; idx < 4 * WROW * G; idx += NTHR) {
        const int sub = idx / (WROW * G), rem = idx - sub * (WROW * G), c = rem / G, g = rem - c * G;
        const long long t = tok0 + sub * 64;
        float val = 0.f;
        if (c < 128 && t < T) {
            val = qf[g * 128 + c];
            if (m.sc != 0) {
                const long long u = (t / m.tok_div) * m.sj + b * m.sb + h * m.sh + (long long)c * m.sc;
                val *= __half2float(m.scale[u]);
            }
        }
        w[idx] = val;
    }
    if (m.sc != 0) {
        const int lane = tid & 31, warp = tid >> 5;
        for (int pair = warp; pair < 4 * G; pair += NTHR / 32) {
            const int sub = pair / G, g = pair - sub * G;
            const long long t = tok0 + sub * 64;
            float s = 0.f;
            if (t < T)
                for (int c = lane; c < 128; c += 32) {
                    const long long u = (t / m.tok_div) * m.sj + b * m.sb + h * m.sh + (long long)c * m.sc;
                    s = fmaf((float)kvc_load_min(m, u) * __half2float(m.scale[u]), qf[g * 128 + c], s);
                }
            s = kvc_warp_sum(s);
            if (lane == 0) zp[pair] = s;
        }
    }
}

template <int G>
__device__ __forceinline__ void load_q(float *qf, float *qsum, const __half *q, long long b, long long Hq,
                                       long long hq0, float scaling, int tid) {
    for (int i = tid; i < G * 128; i += NTHR) {
        const int g = i >> 7, c = i & 127;
        qf[i] = __half2float(q[(b * Hq + hq0 + g) * 128 + c]) * scaling;
    }
    __syncthreads();
    if (tid < G * 32) {           // one warp per query head
        const int g = tid >> 5, lane = tid & 31;
        float s = qf[g * 128 + lane] + qf[g * 128 + lane + 32] + qf[g * 128 + lane + 64] + qf[g * 128 + lane + 96];
        s = kvc_warp_sum(s);
        if (lane == 0) qsum[g] = s;
    }
}

// score of the thread's token from its decoded dot products
template <int G>
__device__ __forceinline__ void k_finish(float (&acc)[G], const float *zp_sub, const float *qsum,
                                         const kvc_qmeta_dev &m, long long t, long long b, long long h) {
    if (m.sc != 0) {
#pragma unroll
        for (int g = 0; g < G; g++) acc[g] += zp_sub[g];
    } else {
        const long long u = (t / m.tok_div) * m.sj + b * m.sb + h * m.sh;
        const float sc = __half2float(m.scale[u]), mi = (float)kvc_load_min(m, u);
#pragma unroll
        for (int g = 0; g < G; g++) acc[g] = sc * fmaf(mi, qsum[g], acc[g]);
    }
}

// ---- fused K: raw scores ------------------------------------------------------------------------
template <int G>
struct QkSmem {
    KvcBookSmem book;
    uint8_t slot[4][SLOT_BYTES];
    float w[4 * WROW * G];
    float zp[4 * G];
    float qf[G * 128];
    float qsum[G];
    uint32_t lead[4];
    int ok[4];
};

template <int G>
__global__ void __launch_bounds__(NTHR) fused_qk_kernel(CacheDev kc, long long T, long long B, long long Hkv, long long Hq,
                                                        long long g0, const __half *__restrict__ q, void *__restrict__ out,
                                                        int out_f32, int *__restrict__ status) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    QkSmem<G> &sm = *reinterpret_cast<QkSmem<G> *>(smem_raw);
    const int tid = threadIdx.x, sub = tid >> 6, v = tid & 63;
    const long long cols = B * Hkv, col = blockIdx.y, b = col / Hkv, h = col % Hkv;
    const long long Gt = Hq / Hkv, hq0 = h * Gt + g0;
    const long long tok0 = (long long)blockIdx.x * 256, t = tok0 + tid;
    kvc_load_book(sm.book, kc.book, tid, NTHR);
    load_q<G>(sm.qf, sm.qsum, q, b, Hq, hq0, 1.0f, tid);
    const long long blk = (tok0 / 64 + sub) * cols + col;
    const bool active = t < T;
    if (active) { uint32_t ld; bool ok = stage(kc, blk, sm.slot[sub], &ld, v); if (v == 0) { sm.lead[sub] = ld; sm.ok[sub] = ok; } }
    __syncthreads();
    k_weights<G>(sm.w, sm.zp, sm.qf, kc.q, tok0, T, b, h, tid);
    __syncthreads();
    if (!active) return;
    float acc[G];
#pragma unroll
    for (int g = 0; g < G; g++) acc[g] = 0.f;
    bool ok = sm.ok[sub];
    if (ok) ok = decode_dot<G>(sm.slot[sub], sm.lead[sub] + vec_start(kc.thread_info, blk, v), sm.book, sm.w + sub * WROW * G, acc);
    if (!ok) atomicOr(status, KVC_FLAG_BAD_STREAM);
    k_finish<G>(acc, sm.zp + sub * G, sm.qsum, kc.q, t, b, h);
#pragma unroll
    for (int g = 0; g < G; g++) {
        const long long o = (b * Hq + hq0 + g) * T + t;
        if (out_f32) reinterpret_cast<float *>(out)[o] = acc[g];
        else reinterpret_cast<__half *>(out)[o] = __float2half_rn(acc[g]);
    }
}

// ---- fused V: per-group partial outputs ----------------------------------------------------------
// V weights of the 2 token groups of a tile: ps[grp][t][g] = P[t] * scale[t], zpv[grp][g].
template <int G>
struct PvSmem {
    KvcBookSmem book;
    uint8_t slot[4][SLOT_BYTES];
    float ps[2 * WROW * G];
    float zpv[2 * G];
    float red[8 * G];
    uint32_t lead[4];
    int ok[4];
};

template <int G>
__global__ void __launch_bounds__(NTHR) fused_pv_kernel(CacheDev vc, long long T, long long B, long long Hkv, long long Hq,
                                                        long long g0, const __half *__restrict__ P, __half *__restrict__ out,
                                                        int *__restrict__ status) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    PvSmem<G> &sm = *reinterpret_cast<PvSmem<G> *>(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, sub = tid >> 6, v = tid & 63;
    const int grp = tid >> 7, ch = tid & 127;
    const long long cols = B * Hkv, col = blockIdx.y, b = col / Hkv, h = col % Hkv;
    const long long Gt = Hq / Hkv, hq0 = h * Gt + g0;
    const long long tok0 = (long long)blockIdx.x * 256, t = tok0 + tid;
    const kvc_qmeta_dev &m = vc.q;
    kvc_load_book(sm.book, vc.book, tid, NTHR);
    const long long gI = tok0 / 128 + grp;
    const long long blk = gI * (cols * 2) + col * 2 + (ch >> 6);
    const bool active = gI * 128 < T;
    if (active) { uint32_t ld; bool ok = stage(vc, blk, sm.slot[sub], &ld, v); if (v == 0) { sm.lead[sub] = ld; sm.ok[sub] = ok; } }
    // weights: thread = token
    float zl[G];
    {
        float sc = 0.f, mi = 0.f;
        if (t < T) {
            const long long u = (t / m.tok_div) * m.sj + b * m.sb + h * m.sh;
            sc = __half2float(m.scale[u]); mi = (float)kvc_load_min(m, u);
        }
#pragma unroll
        for (int g = 0; g < G; g++) {
            float p = t < T ? __half2float(P[(b * Hq + hq0 + g) * T + t]) : 0.f;
            float w = p * sc;
            sm.ps[(grp * WROW + ch) * G + g] = w;
            zl[g] = kvc_warp_sum(w * mi);
        }
        if (ch < 4) for (int g = 0; g < G; g++) sm.ps[(grp * WROW + 128 + ch) * G + g] = 0.f;
        if (lane == 0) for (int g = 0; g < G; g++) sm.red[warp * G + g] = zl[g];
    }
    __syncthreads();
    if (tid < 2 * G) {
        const int gg = tid / G, g = tid - gg * G;
        sm.zpv[tid] = sm.red[(gg * 4 + 0) * G + g] + sm.red[(gg * 4 + 1) * G + g] + sm.red[(gg * 4 + 2) * G + g] + sm.red[(gg * 4 + 3) * G + g];
    }
    __syncthreads();
    if (!active) return;
    float acc[G];
#pragma unroll
    for (int g = 0; g < G; g++) acc[g] = 0.f;
    bool ok = sm.ok[sub];
    if (ok) ok = decode_dot<G>(sm.slot[sub], sm.lead[sub] + vec_start(vc.thread_info, blk, v), sm.book, sm.ps + grp * WROW * G, acc);
    if (!ok) atomicOr(status, KVC_FLAG_BAD_STREAM);
#pragma unroll
    for (int g = 0; g < G; g++)
        out[((gI * B + b) * Hq + hq0 + g) * 128 + ch] = __float2half_rn(acc[g] + sm.zpv[grp * G + g]);
}

// ---- one-pass decode attention -------------------------------------------------------------------
template <int G>
struct AttnSmem {
    KvcBookSmem bookK, bookV;
    uint8_t slotK[4][SLOT_BYTES];
    uint8_t slotV[4][SLOT_BYTES];
    float w[4 * WROW * G];        // K weights; reused for the final cross-group sum
    float ps[2 * WROW * G];
    float zp[4 * G];
    float zpv[2 * G];
    float qf[G * 128];
    float qsum[G];
    float red[3][8 * G];          // per-warp max, sum, zpv partials
    float alpha[G];
    uint32_t leadK[4], leadV[4];
    int okK[4], okV[4];
    int last;
};

struct AttnParams {
    CacheDev k, v;
    long long T, B, Hkv, Hq, g0, Tr;
    const __half *q, *ktail, *vtail;
    __half *out;
    float scaling;
    int splits, tiles_per_split;
    float *ws_part;               // [B*Hq][splits][130]: m, l, acc[128]
    int *ws_count;                // [B*Hq]
    int *status;
};

template <int G>
__global__ void __launch_bounds__(NTHR, 2) attn_decode_kernel(AttnParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    AttnSmem<G> &sm = *reinterpret_cast<AttnSmem<G> *>(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, sub = tid >> 6, v = tid & 63;
    const int grp = tid >> 7, ch = tid & 127;
    const long long T = p.T, B = p.B, Hkv = p.Hkv, Hq = p.Hq;
    const long long cols = B * Hkv, col = blockIdx.y, b = col / Hkv, h = col % Hkv;
    const long long Gt = Hq / Hkv, hq0 = h * Gt + p.g0;
    const int split = blockIdx.x;
    const long long n_tiles = (T + 255) / 256;
    const long long tile_lo = (long long)split * p.tiles_per_split;
    long long tile_hi = tile_lo + p.tiles_per_split;
    if (tile_hi > n_tiles) tile_hi = n_tiles;
    const kvc_qmeta_dev &km = p.k.q, &vm = p.v.q;

    kvc_load_book(sm.bookK, p.k.book, tid, NTHR);
    kvc_load_book(sm.bookV, p.v.book, tid, NTHR);
    load_q<G>(sm.qf, sm.qsum, p.q, b, Hq, hq0, p.scaling, tid);

    float m_run[G], l_run[G], acc[G];
#pragma unroll
    for (int g = 0; g < G; g++) { m_run[g] = -CUDART_INF_F; l_run[g] = 0.f; acc[g] = 0.f; }
    int flags = 0;

    for (long long tile = tile_lo; tile < tile_hi; tile++) {
        const long long tok0 = tile * 256, t = tok0 + tid;
        const long long blkK = (tok0 / 64 + sub) * cols + col;
        const long long gI = tok0 / 128 + grp;
        const long long blkV = gI * (cols * 2) + col * 2 + (ch >> 6);
        const bool actK = t < T, actV = gI * 128 < T;
        __syncthreads();                                   // slots, weights and reductions are free
        if (actK) { uint32_t ld; bool ok = stage(p.k, blkK, sm.slotK[sub], &ld, v); if (v == 0) { sm.leadK[sub] = ld; sm.okK[sub] = ok; } }
        if (actV) { uint32_t ld; bool ok = stage(p.v, blkV, sm.slotV[sub], &ld, v); if (v == 0) { sm.leadV[sub] = ld; sm.okV[sub] = ok; } }
        k_weights<G>(sm.w, sm.zp, sm.qf, km, tok0, T, b, h, tid);
        __syncthreads();
        // ---- K: scores of this tile's tokens
        float s[G];
#pragma unroll
        for (int g = 0; g < G; g++) s[g] = 0.f;
        if (actK) {
            bool ok = sm.okK[sub];
            if (ok) ok = decode_dot<G>(sm.slotK[sub], sm.leadK[sub] + vec_start(p.k.thread_info, blkK, v), sm.bookK, sm.w + sub * WROW * G, s);
            if (!ok) flags |= KVC_FLAG_BAD_STREAM;
            k_finish<G>(s, sm.zp + sub * G, sm.qsum, km, t, b, h);
        } else {
#pragma unroll
            for (int g = 0; g < G; g++) s[g] = -CUDART_INF_F;
        }
        // ---- online softmax over the tile
#pragma unroll
        for (int g = 0; g < G; g++) { float mx = kvc_warp_max(s[g]); if (lane == 0) sm.red[0][warp * G + g] = mx; }
        __syncthreads();
        float vsc = 0.f, vmi = 0.f;
        if (actK) {
            const long long u = (t / vm.tok_div) * vm.sj + b * vm.sb + h * vm.sh;
            vsc = __half2float(vm.scale[u]); vmi = (float)kvc_load_min(vm, u);
        }
        float alpha[G];
#pragma unroll
        for (int g = 0; g < G; g++) {
            float mt = sm.red[0][g];
#pragma unroll
            for (int w8 = 1; w8 < 8; w8++) mt = fmaxf(mt, sm.red[0][w8 * G + g]);
            const float m_new = fmaxf(m_run[g], mt);
            alpha[g] = __expf(m_run[g] - m_new);           // exp(-inf) = 0 on the first tile
            const float pr = actK ? __expf(s[g] - m_new) : 0.f;
            m_run[g] = m_new;
            const float wv = pr * vsc;
            sm.ps[(grp * WROW + ch) * G + g] = wv;
            const float ssum = kvc_warp_sum(pr), zsum = kvc_warp_sum(wv * vmi);
            if (lane == 0) { sm.red[1][warp * G + g] = ssum; sm.red[2][warp * G + g] = zsum; }
        }
        if (ch < 4) for (int g = 0; g < G; g++) sm.ps[(grp * WROW + 128 + ch) * G + g] = 0.f;
        __syncthreads();
#pragma unroll
        for (int g = 0; g < G; g++) {
            float lt = 0.f;
#pragma unroll
            for (int w8 = 0; w8 < 8; w8++) lt += sm.red[1][w8 * G + g];
            l_run[g] = l_run[g] * alpha[g] + lt;
        }
        // ---- V: accumulate this tile's contribution for the thread's (group, channel)
        float dv[G];
#pragma unroll
        for (int g = 0; g < G; g++) dv[g] = 0.f;
        if (actV) {
            bool ok = sm.okV[sub];
            if (ok) ok = decode_dot<G>(sm.slotV[sub], sm.leadV[sub] + vec_start(p.v.thread_info, blkV, v), sm.bookV, sm.ps + grp * WROW * G, dv);
            if (!ok) flags |= KVC_FLAG_BAD_STREAM;
#pragma unroll
            for (int g = 0; g < G; g++)
                dv[g] += sm.red[2][(grp * 4 + 0) * G + g] + sm.red[2][(grp * 4 + 1) * G + g] +
                         sm.red[2][(grp * 4 + 2) * G + g] + sm.red[2][(grp * 4 + 3) * G + g];
        }
#pragma unroll
        for (int g = 0; g < G; g++) acc[g] = fmaf(acc[g], alpha[g], dv[g]);
    }

    // ---- uncompressed tail (the recent window), handled by the last split: dense fp16 rows
    if (p.Tr > 0 && split == p.splits - 1) {
        for (long long r0 = 0; r0 < p.Tr; r0 += 256) {
            const long long r = r0 + tid;
            const bool act = r < p.Tr;
            __syncthreads();
            float s[G];
#pragma unroll
            for (int g = 0; g < G; g++) s[g] = act ? 0.f : -CUDART_INF_F;
            if (act) {
                const __half *kr = p.ktail + ((r * B + b) * Hkv + h) * 128;
                for (int c8 = 0; c8 < 16; c8++) {
                    uint4 kv = *reinterpret_cast<const uint4 *>(kr + c8 * 8);
                    const __half *kh = reinterpret_cast<const __half *>(&kv);
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        const float kf = __half2float(kh[k]);
#pragma unroll
                        for (int g = 0; g < G; g++) s[g] = fmaf(kf, sm.qf[g * 128 + c8 * 8 + k], s[g]);
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < G; g++) { float mx = kvc_warp_max(s[g]); if (lane == 0) sm.red[0][warp * G + g] = mx; }
            __syncthreads();
            float alpha[G];
            float *pt = sm.w;                                  // p[t][g] for the 256 rows
#pragma unroll
            for (int g = 0; g < G; g++) {
                float mt = sm.red[0][g];
#pragma unroll
                for (int w8 = 1; w8 < 8; w8++) mt = fmaxf(mt, sm.red[0][w8 * G + g]);
                const float m_new = fmaxf(m_run[g], mt);
                alpha[g] = __expf(m_run[g] - m_new);
                const float pr = act ? __expf(s[g] - m_new) : 0.f;
                m_run[g] = m_new;
                pt[tid * G + g] = pr;
                const float ssum = kvc_warp_sum(pr);
                if (lane == 0) sm.red[1][warp * G + g] = ssum;
            }
            __syncthreads();
            float dv[G];
#pragma unroll
            for (int g = 0; g < G; g++) {
                float lt = 0.f;
#pragma unroll
                for (int w8 = 0; w8 < 8; w8++) lt += sm.red[1][w8 * G + g];
                l_run[g] = l_run[g] * alpha[g] + lt;
                dv[g] = 0.f;
            }
            // thread (grp, ch) sums rows r0 + 128*grp .. +127 of its channel
            for (int i = 0; i < 128; i++) {
                const long long rr = r0 + grp * 128 + i;
                if (rr >= p.Tr) break;
                const float vf = __half2float(p.vtail[((rr * B + b) * Hkv + h) * 128 + ch]);
#pragma unroll
                for (int g = 0; g < G; g++) dv[g] = fmaf(pt[(grp * 128 + i) * G + g], vf, dv[g]);
            }
#pragma unroll
            for (int g = 0; g < G; g++) acc[g] = fmaf(acc[g], alpha[g], dv[g]);
        }
    }
    if (flags) atomicOr(p.status, flags);

    // ---- combine the two token groups of the CTA, then the splits
    __syncthreads();
    float *sumbuf = sm.w;                                      // [2][128][G]
#pragma unroll
    for (int g = 0; g < G; g++) sumbuf[(grp * 128 + ch) * G + g] = acc[g];
    __syncthreads();
    const long long head0 = b * Hq + hq0;
    if (p.splits == 1) {
        if (tid < 128) {
#pragma unroll
            for (int g = 0; g < G; g++) {
                const float o = (sumbuf[tid * G + g] + sumbuf[(128 + tid) * G + g]) / l_run[g];
                p.out[(head0 + g) * 128 + tid] = __float2half_rn(o);
            }
        }
        return;
    }
    if (tid < 128) {
#pragma unroll
        for (int g = 0; g < G; g++) {
            float *part = p.ws_part + ((head0 + g) * p.splits + split) * 130;
            part[2 + tid] = sumbuf[tid * G + g] + sumbuf[(128 + tid) * G + g];
            if (tid == 0) { part[0] = m_run[g]; part[1] = l_run[g]; }
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int done = atomicAdd(&p.ws_count[head0], 1);
        sm.last = (done == p.splits - 1);
    }
    __syncthreads();
    if (!sm.last) return;
    __threadfence();
    if (tid < 128) {
#pragma unroll
        for (int g = 0; g < G; g++) {
            const float *part = p.ws_part + (head0 + g) * p.splits * 130;
            float M = -CUDART_INF_F;
            for (int s2 = 0; s2 < p.splits; s2++) M = fmaxf(M, __ldcg(part + s2 * 130));
            float L = 0.f, O = 0.f;
            for (int s2 = 0; s2 < p.splits; s2++) {
                const float m2 = __ldcg(part + s2 * 130);
                const float e = m2 == -CUDART_INF_F ? 0.f : __expf(m2 - M);
                L = fmaf(__ldcg(part + s2 * 130 + 1), e, L);
                O = fmaf(__ldcg(part + s2 * 130 + 2 + tid), e, O);
            }
            p.out[(head0 + g) * 128 + tid] = __float2half_rn(O / L);
        }
    }
    if (tid == 0) p.ws_count[head0] = 0;                       // leave the counters zeroed for the next call
}

template <class K>
int set_smem(K kernel, size_t bytes) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) { kvc_set_error("cudaFuncSetAttribute(%zu bytes) failed: %s", bytes, cudaGetErrorString(e)); return KVC_ERR_CUDA; }
    return KVC_OK;
}

int check_cache(const kvc_cache *c, const char *who, bool is_k) {
    KVC_REQUIRE(c && c->encoded && c->block_info && c->thread_info && c->book && c->q.min_int && c->q.scale,
                "%s: null pointer in the %s cache", who, is_k ? "K" : "V");
    KVC_REQUIRE(c->q.min_bytes == 1 || c->q.min_bytes == 2, "%s: min_bytes must be 1 or 2", who);
    KVC_REQUIRE(c->q.tok_div > 0, "%s: tok_div must be positive", who);
    KVC_REQUIRE((reinterpret_cast<uintptr_t>(c->book) & 15) == 0 && (reinterpret_cast<uintptr_t>(c->block_info) & 7) == 0,
                "%s: book must be 16-byte and block_info 8-byte aligned", who);
    if (is_k) KVC_REQUIRE(c->q.sc == 0 || c->q.tok_div % 64 == 0,
                          "%s: K units that depend on the channel must cover whole 64-token blocks", who);
    else KVC_REQUIRE(c->q.sc == 0, "%s: V units that depend on the channel are not supported by the fused kernels", who);
    return KVC_OK;
}

// the G query heads of a KV head are processed in chunks of 4, 2 or 1
int next_chunk(long long remaining) { return remaining >= 4 ? 4 : (remaining >= 2 ? 2 : 1); }

}  // namespace

extern "C" int kvc_fused_qk(const kvc_cache *k, int64_t T, int64_t B, int64_t Hkv, int64_t Hq,
                            const void *q, void *out, int out_f32, int32_t *status, kvc_stream_t stream) {
    if (int rc = check_cache(k, "kvc_fused_qk", true)) return rc;
    KVC_REQUIRE(q && out && status, "kvc_fused_qk: null pointer");
    KVC_REQUIRE(B > 0 && Hkv > 0 && Hq > 0 && Hq % Hkv == 0 && T >= 0 && T % 64 == 0, "kvc_fused_qk: bad shape");
    KVC_REQUIRE(B * Hkv <= 65535, "kvc_fused_qk: B*Hkv exceeds the grid limit");
    if (T == 0) return KVC_OK;
    const CacheDev kc = to_dev(*k);
    const dim3 grid((unsigned)((T + 255) / 256), (unsigned)(B * Hkv));
    const long long Gt = Hq / Hkv;
    for (long long g0 = 0; g0 < Gt;) {
        const int G = next_chunk(Gt - g0);
#define KVC_QK(GG)                                                                                              \
    {                                                                                                           \
        if (int rc = set_smem(fused_qk_kernel<GG>, sizeof(QkSmem<GG>))) return rc;                              \
        fused_qk_kernel<GG><<<grid, NTHR, sizeof(QkSmem<GG>), kvc_cu(stream)>>>(                                \
            kc, T, B, Hkv, Hq, g0, reinterpret_cast<const __half *>(q), out, out_f32, status);                  \
    }
        if (G == 4) KVC_QK(4) else if (G == 2) KVC_QK(2) else KVC_QK(1)
#undef KVC_QK
        g0 += G;
    }
    KVC_LAUNCH_OK();
    return KVC_OK;
}

extern "C" int kvc_fused_pv(const kvc_cache *v, int64_t T, int64_t B, int64_t Hkv, int64_t Hq,
                            const void *P, void *out, int32_t *status, kvc_stream_t stream) {
    if (int rc = check_cache(v, "kvc_fused_pv", false)) return rc;
    KVC_REQUIRE(P && out && status, "kvc_fused_pv: null pointer");
    KVC_REQUIRE(B > 0 && Hkv > 0 && Hq > 0 && Hq % Hkv == 0 && T >= 0 && T % 128 == 0, "kvc_fused_pv: bad shape");
    KVC_REQUIRE(B * Hkv <= 65535, "kvc_fused_pv: B*Hkv exceeds the grid limit");
    if (T == 0) return KVC_OK;
    const CacheDev vc = to_dev(*v);
    const dim3 grid((unsigned)((T + 255) / 256), (unsigned)(B * Hkv));
    const long long Gt = Hq / Hkv;
    for (long long g0 = 0; g0 < Gt;) {
        const int G = next_chunk(Gt - g0);
#define KVC_PV(GG)                                                                                              \
    {                                                                                                           \
        if (int rc = set_smem(fused_pv_kernel<GG>, sizeof(PvSmem<GG>))) return rc;                              \
        fused_pv_kernel<GG><<<grid, NTHR, sizeof(PvSmem<GG>), kvc_cu(stream)>>>(                                \
            vc, T, B, Hkv, Hq, g0, reinterpret_cast<const __half *>(P), reinterpret_cast<__half *>(out), status); \
    }
        if (G == 4) KVC_PV(4) else if (G == 2) KVC_PV(2) else KVC_PV(1)
#undef KVC_PV
        g0 += G;
    }
    KVC_LAUNCH_OK();
    return KVC_OK;
}

extern "C" int kvc_attn_splits(int64_t T, int64_t B, int64_t Hkv, int sm_count) {
    if (T <= 0 || B <= 0 || Hkv <= 0) return 1;
    if (sm_count <= 0) sm_count = kvc_sm_count();
    const long long n_tiles = (T + 255) / 256, cols = B * Hkv;
    long long want = (4ll * sm_count + cols - 1) / cols;           // about two waves of two CTAs per SM
    if (want < 1) want = 1;
    if (want > n_tiles) want = n_tiles;
    const long long tps = (n_tiles + want - 1) / want;
    return (int)((n_tiles + tps - 1) / tps);
}

extern "C" int64_t kvc_attn_workspace(int64_t B, int64_t Hq, int splits) {
    if (splits < 1) splits = 1;
    int64_t counters = ((B * Hq * 4 + 255) / 256) * 256;
    return counters + B * Hq * (int64_t)splits * 130 * 4;
}

extern "C" int kvc_attn_decode(const kvc_cache *k, const kvc_cache *v, int64_t T, int64_t B, int64_t Hkv, int64_t Hq,
                               const void *q, float scaling, const void *ktail, const void *vtail, int64_t Tr,
                               void *out, int splits, void *workspace, int64_t workspace_bytes,
                               int32_t *status, kvc_stream_t stream) {
    if (int rc = check_cache(k, "kvc_attn_decode", true)) return rc;
    if (int rc = check_cache(v, "kvc_attn_decode", false)) return rc;
    KVC_REQUIRE(q && out && status, "kvc_attn_decode: null pointer");
    KVC_REQUIRE(B > 0 && Hkv > 0 && Hq > 0 && Hq % Hkv == 0, "kvc_attn_decode: bad head counts");
    KVC_REQUIRE(T >= 0 && T % 128 == 0, "kvc_attn_decode: the compressed length must be a multiple of 128, got %lld", (long long)T);
    KVC_REQUIRE(Tr >= 0 && (Tr == 0 || (ktail && vtail)), "kvc_attn_decode: tail pointers missing");
    KVC_REQUIRE(T + Tr > 0, "kvc_attn_decode: empty cache");
    KVC_REQUIRE(B * Hkv <= 65535, "kvc_attn_decode: B*Hkv exceeds the grid limit");
    KVC_REQUIRE(Tr == 0 || ((reinterpret_cast<uintptr_t>(ktail) & 15) == 0), "kvc_attn_decode: ktail must be 16-byte aligned");
    const long long n_tiles = (T + 255) / 256;
    if (splits <= 0) splits = kvc_attn_splits(T, B, Hkv, 0);
    if (splits > n_tiles) splits = (int)(n_tiles > 0 ? n_tiles : 1);
    int tps = (int)((n_tiles + splits - 1) / splits);
    if (tps < 1) tps = 1;
    splits = n_tiles > 0 ? (int)((n_tiles + tps - 1) / tps) : 1;
    if (splits > 1) {
        KVC_REQUIRE(workspace && workspace_bytes >= kvc_attn_workspace(B, Hq, splits),
                    "kvc_attn_decode: workspace needs %lld bytes for %d splits", (long long)kvc_attn_workspace(B, Hq, splits), splits);
        KVC_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 15) == 0, "kvc_attn_decode: workspace must be 16-byte aligned");
    }
    AttnParams p;
    p.k = to_dev(*k); p.v = to_dev(*v);
    p.T = T; p.B = B; p.Hkv = Hkv; p.Hq = Hq; p.Tr = Tr;
    p.q = reinterpret_cast<const __half *>(q);
    p.ktail = reinterpret_cast<const __half *>(ktail); p.vtail = reinterpret_cast<const __half *>(vtail);
    p.out = reinterpret_cast<__half *>(out);
    p.scaling = scaling; p.splits = splits; p.tiles_per_split = tps;
    p.ws_count = reinterpret_cast<int *>(workspace);
    p.ws_part = workspace ? reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(workspace) + ((B * Hq * 4 + 255) / 256) * 256) : nullptr;
    p.status = status;
    const dim3 grid((unsigned)splits, (unsigned)(B * Hkv));
    const long long Gt = Hq / Hkv;
    for (long long g0 = 0; g0 < Gt;) {
        const int G = next_chunk(Gt - g0);
        p.g0 = g0;
#define KVC_AT(GG)                                                                                              \
    {                                                                                                           \
        if (int rc = set_smem(attn_decode_kernel<GG>, sizeof(AttnSmem<GG>))) return rc;                         \
        attn_decode_kernel<GG><<<grid, NTHR, sizeof(AttnSmem<GG>), kvc_cu(stream)>>>(p);                        \
    }
        if (G == 4) KVC_AT(4) else if (G == 2) KVC_AT(2) else KVC_AT(1)
#undef KVC_AT
        g0 += G;
    }
    KVC_LAUNCH_OK();
    return KVC_OK;
}
